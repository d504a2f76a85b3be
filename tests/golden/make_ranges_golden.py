"""Generate ``ranges_golden.npz``: outputs of the reference's own band code on seeded inputs.

Runs the reference's ``native/ranges/ranges.cpp`` compiled UNMODIFIED by ``oracle/build_ref.py``
(module ``km_ref_ranges``), in the container that holds the reference tree.  The fixture pins
the oracle's restatement (``oracle/km_oracle.c``) and, through it, the device kernels.

Usage:  python oracle/build_ref.py --only ranges && python tests/golden/make_ranges_golden.py
"""
from __future__ import annotations

import importlib.util
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_ref():
    path = os.path.join(ROOT, "oracle", "_ref", "km_ref_ranges", "km_ref_ranges.so")
    spec = importlib.util.spec_from_file_location("km_ref_ranges", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cases():
    """(name, x1 (B,m), x2 (B,n), cutoff, block, align) -- the input family of the reference's
    tests/test_ranges.py:10-74 (offsets, gaps, batches, block sizes 1 and 3) plus 128-row blocks
    at the sizes of the native tests and of the smallest benchmark configuration."""
    g = torch.Generator().manual_seed(1234)
    out = []
    idx = 0
    for offset in (-1.0, 0.0, 1.5):
        for gap1 in (None, 0, 10):
            for gap2 in (None, 10):
                for B in (1, 3):
                    x1 = torch.sort(torch.rand(B, 50, generator=g) * 10)[0]
                    x2 = torch.sort(torch.rand(B, 55, generator=g) * 10)[0] + offset
                    if gap1 is not None:
                        x1[:, gap1:] += 20
                    if gap2 is not None:
                        x2[:, gap2:] += 20
                    for cutoff in (0.1, 1.0, 11.0):
                        for block in (1, 3):
                            for align in (0, 1):
                                out.append((f"t{idx}", x1, x2, cutoff, block, align))
                                idx += 1
    for (m, n, B, cutoff) in [(128, 128, 1, 2.0), (600, 800, 1, 2.0), (500, 500, 3, 2.0), (301, 199, 2, 2.0),
                              (129, 130, 1, 2.0), (100, 37, 1, 0.5)]:
        x1 = torch.sort(torch.rand(B, m, generator=g) * 10)[0]
        x2 = torch.sort(torch.rand(B, n, generator=g) * 10)[0]
        for align in (0, 1):
            out.append((f"t{idx}", x1, x2, cutoff, 128, align))
            idx += 1
    x = torch.sort(torch.rand(1, 4096, generator=g) * 40)[0]
    out.append((f"t{idx}", x, x, 2.0, 128, 1))
    return out


FIELDS = ("start", "end", "start_t", "end_t", "sym_start", "sym_end")


def main() -> None:
    """Layout of the .npz: ``in<i>_x1`` / ``in<i>_x2`` input sets; ``meta`` (N, 4) =
    cutoff, block, align, input set; per field one flat int32 array with the outputs of all
    cases back to back (shapes follow from the inputs: (B, ceil(m / block)) for start / end and
    the symmetric pair, (B, ceil(n / block)) for the transposed pair, which is present only for
    aligned cases)."""
    ref = load_ref()
    store = {}
    flat = {f: [] for f in FIELDS}
    meta = []
    inputs: dict[int, int] = {}
    for _, x1, x2, cutoff, block, align in cases():
        if id(x1) not in inputs:
            inputs[id(x1)] = len(inputs)
            store[f"in{inputs[id(x1)]}_x1"] = x1.numpy()
            store[f"in{inputs[id(x1)]}_x2"] = x2.numpy()
        meta.append([cutoff, block, align, inputs[id(x1)]])
        s, e = ref.make_ranges(x1, x2, float(cutoff), int(block), bool(align))
        flat["start"].append(s.numpy().ravel())
        flat["end"].append(e.numpy().ravel())
        if align:
            st, et = ref.transpose_ranges(s, e, x1.shape[1], x2.shape[1], int(block))
            flat["start_t"].append(st.numpy().ravel())
            flat["end_t"].append(et.numpy().ravel())
        ss, se = ref.make_ranges_symmetric(x1, float(cutoff), int(block))
        flat["sym_start"].append(ss.numpy().ravel())
        flat["sym_end"].append(se.numpy().ravel())
    store["meta"] = np.array(meta, dtype=np.float64)
    for f in FIELDS:
        store[f] = np.concatenate(flat[f]).astype(np.int32)
    out = os.path.join(HERE, "ranges_golden.npz")
    np.savez_compressed(out, **store)
    print(f"wrote {out}: {len(meta)} cases, {os.path.getsize(out) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
