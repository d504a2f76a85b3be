"""Generate ``cuda_golden.npz``: outputs of the reference's own CUDA kernels on seeded inputs.

Needs a GPU and the modules built by ``oracle/build_ref.py`` (the reference's native ops
compiled UNMODIFIED for sm_100 with the define sets of its single configurations,
kernel_matmul/configurations.py).  Writes inputs and the reference's fp32 outputs; the CPU
test ``tests/test_oracle_cpu.py::test_oracle_matches_reference_cuda_golden`` then pins the fp64
oracle against them.

Usage (on a GPU box):  python tests/golden/make_cuda_golden.py [output.npz]
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

KERNEL_TYPES = ("rbf", "spectral", "locally_periodic")


def load(modname: str):
    path = os.path.join(ROOT, "oracle", "_ref", modname, modname + ".so")
    spec = importlib.util.spec_from_file_location(modname, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "cuda_golden.npz")
    dev = torch.device("cuda:0")
    ranges = load("km_ref_ranges")
    g = torch.Generator().manual_seed(20240607)
    B, m, n, k, kb = 2, 300, 260, 8, 5
    store = {}
    for kt in KERNEL_TYPES:
        P = {"rbf": 2, "spectral": 3, "locally_periodic": 4}[kt]
        x1 = torch.sort(torch.rand(B, m, generator=g) * 10)[0]
        x2 = torch.sort(torch.rand(B, n, generator=g) * 10)[0]
        params = 1 + torch.rand(B, P, generator=g)
        if kt == "spectral":
            params[:, 1] = 0.5 + 0.5 * torch.rand(B, generator=g)
        rhs = torch.randn(B, n, k, generator=g)
        og = torch.randn(B, m, k, generator=g)
        left = torch.randn(B, m, kb, generator=g)
        right = torch.randn(B, n, kb, generator=g)
        # the dense ops run on a smaller problem (their inputs / outputs are full matrices), and
        # out_grad takes values k/8 so that the fixture compresses
        md, nd = 160, 150
        x1d, x2d = x1[:, :md].contiguous(), x2[:, :nd].contiguous()
        dg = torch.randint(-8, 9, (B, md, nd), generator=g).float() / 8
        dstart, dend = ranges.make_ranges(x1d, x2d, 2.0, 128, False)
        start, end = ranges.make_ranges(x1, x2, 2.0, 128, False)
        # square inputs for the gather ops (the reference tests them on square matrices only)
        sstart, send = ranges.make_ranges_symmetric(x1, 2.0, 128)
        # index tensors of rank 2: the modules are built with INDEX_BATCH_DIM = 1
        ishape = (4, 100)
        bidx = torch.randint(0, B, ishape, generator=g, dtype=torch.int32)
        row = torch.randint(0, m, ishape, generator=g, dtype=torch.int32)
        col = torch.randint(0, m, ishape, generator=g, dtype=torch.int32)
        ig = torch.randn(ishape, generator=g)

        d = lambda t: t.to(dev)  # noqa: E731
        res = {
            "matmul": load(f"km_ref_matmul_{kt}_k{k}").call(d(x1), d(x2), d(rhs), d(params), d(start), d(end)),
            "matmul_bwd": load(f"km_ref_matmul_bwd_{kt}").call(d(x1), d(x2), d(rhs), d(params), d(start), d(end), d(og)),
            "bilinear": load(f"km_ref_bilinear_derivative_{kt}").call(d(x1), d(x2), d(left), d(right), d(params), d(start), d(end)),
            "dense": load(f"km_ref_dense_{kt}").call(d(x1d), d(x2d), d(params), d(dstart), d(dend)),
            "dense_bwd": load(f"km_ref_dense_bwd_{kt}").call(d(x1d), d(x2d), d(params), d(dstart), d(dend), d(dg)),
            "index": load(f"km_ref_index_{kt}").call(d(x1), d(x1), d(params), d(sstart), d(send), [d(bidx)], d(row), d(col)),
            "index_bwd": load(f"km_ref_index_bwd_{kt}").call(d(x1), d(x1), d(params), d(sstart), d(send), [d(bidx)], d(row), d(col), d(ig)),
        }
        torch.cuda.synchronize()
        for name, t in dict(x1=x1, x2=x2, params=params, rhs=rhs, og=og, left=left, right=right, dg=dg,
                            start=start, end=end, dstart=dstart, dend=dend, sstart=sstart, send=send,
                            bidx=bidx, row=row, col=col, ig=ig).items():
            store[f"{kt}_{name}"] = t.numpy()
        for name, t in res.items():
            store[f"{kt}_ref_{name}"] = t.detach().cpu().numpy()
    np.savez_compressed(out_path, **store)
    print(f"wrote {out_path}: {os.path.getsize(out_path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
