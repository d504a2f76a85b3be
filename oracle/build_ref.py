"""Build the UNMODIFIED reference sources into ``oracle/_ref/`` (test infrastructure only).

The reference (Turakar/kernel-matmul) ships one pybind11 torch extension per op and per
set of ``-DKM_*`` defines (``kernel_matmul/compile.py:49-125``).  This recipe compiles those
sources where they lie (nothing is copied into this repository) with the same flags the
reference's ``load_native`` would pass, for a fixed list of define sets, cross-compiling the
CUDA ops for sm_100 so that the resulting ``.so`` files can be loaded on a B200 box that
does not hold the reference tree.

Outputs go to ``oracle/_ref/<module name>/<module name>.so`` only.  ``oracle/_ref`` is
git-ignored.  Nothing under ``kernel_matmul_b200/`` may import this file or its outputs:
the built modules are used by ``tests/`` (to pin the CPU oracle against the real reference)
and by ``bench.py`` (to time the reference kernels beside ours).

Usage:  python oracle/build_ref.py [--reference /path/to/kernel-matmul] [--only ranges] [-j 4]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# where the reference project lies (read-only): the environment variable KM_REFERENCE_DIR or --reference
REFERENCE_DIR = os.environ.get("KM_REFERENCE_DIR", "")

KERNEL_DEFINE = {
    "rbf": "KERNEL_RBF",
    "spectral": "KERNEL_SPECTRAL",
    "locally_periodic": "KERNEL_LOCALLY_PERIODIC",
}


def module_specs() -> list[tuple[str, str, dict]]:
    """(module name, native op directory, defines) for every module we build.

    Define sets follow ``kernel_matmul/configurations.py`` (the single, non-autotuned
    configurations) for a flattened batch rank of 1.
    """
    specs: list[tuple[str, str, dict]] = [("km_ref_ranges", "ranges", {})]
    for kt, kdef in KERNEL_DEFINE.items():
        base = {"BLOCK_SIZE": 128, "BATCH_DIM": 1, kdef: None}
        for kb in (1, 8, 16, 32):
            # MatmulSingleConfiguration (configurations.py:58-80): 64 threads x 2 rows.
            specs.append(
                (
                    f"km_ref_matmul_{kt}_k{kb}",
                    "matmul",
                    base
                    | {
                        "MATMUL_K_BLOCK_SIZE": kb,
                        "MATMUL_THREADS": 64,
                        "MATMUL_PER_THREAD": 2,
                        "MATMUL_COL_BLOCKS": 1,
                        "MATMUL_USE_SHM": 1,
                    },
                )
            )
        specs.append(
            (
                f"km_ref_matmul_bwd_{kt}",
                "matmul_bwd",
                base | {"MATMUL_BWD_THREAD_DIM": 16, "MATMUL_BWD_PER_THREAD": 8},
            )
        )
        specs.append(
            (
                f"km_ref_bilinear_derivative_{kt}",
                "bilinear_derivative",
                base
                | {"BILINEAR_DERIVATIVE_THREAD_DIM": 16, "BILINEAR_DERIVATIVE_PER_THREAD": 8},
            )
        )
        specs.append((f"km_ref_dense_{kt}", "dense", base | {"DENSE_THREAD_DIM": 16}))
        specs.append(
            (f"km_ref_dense_bwd_{kt}", "dense_bwd", base | {"DENSE_BWD_THREAD_DIM": 16})
        )
        specs.append(
            (
                f"km_ref_index_{kt}",
                "index",
                base | {"INDEX_THREAD_DIM": 64, "INDEX_BATCH_DIM": 1},
            )
        )
        specs.append(
            (
                f"km_ref_index_bwd_{kt}",
                "index_bwd",
                base | {"INDEX_BWD_THREAD_DIM": 64, "INDEX_BWD_BATCH_DIM": 1},
            )
        )
    return specs


# (kernel type, rhs columns) of the benchmark configurations whose forward product the reference's
# autotuner would tune: small RBF (k = 1), spectral mixture (k = 16), one component of the CG
# operator (k = 8), unbanded RBF (k = 128).
TUNED_PRODUCTS = [("rbf", 1), ("spectral", 16), ("spectral", 8), ("rbf", 128)]


def tuned_matmul_specs() -> list[tuple[str, str, dict]]:
    """The candidates ``MatmulAutotuneConfiguration.make_candidates`` would time
    (kernel_matmul/configurations.py:94-118): 3 thread shapes x 4 COL_BLOCKS, and for k > 32
    three K_BLOCK sizes.  bench.py times them all on the GPU and quotes the fastest."""
    specs = []
    for kt, k in TUNED_PRODUCTS:
        base = {"BLOCK_SIZE": 128, "BATCH_DIM": 1, KERNEL_DEFINE[kt]: None, "MATMUL_USE_SHM": 1}
        k_blocks = [k] if k <= 32 else [16, 32, 64]
        for threads, per in ((32, 4), (64, 2), (128, 1)):
            for cb in (1, 4, 8, 16):
                for kb in k_blocks:
                    if (threads, per, cb) == (64, 2, 1) and kb == k:
                        continue  # the single configuration, built as km_ref_matmul_<kt>_k<k>
                    specs.append((
                        f"km_ref_matmul_{kt}_k{k}_t{threads}x{per}_c{cb}_kb{kb}", "matmul",
                        base | {"MATMUL_K_BLOCK_SIZE": kb, "MATMUL_THREADS": threads, "MATMUL_PER_THREAD": per,
                                "MATMUL_COL_BLOCKS": cb},
                    ))
    return specs


def build_one(reference: str, name: str, op: str, defines: dict) -> str:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "2")
    import torch.utils.cpp_extension as ext

    native = os.path.join(reference, "native")
    sources = []
    for d in ("common", op):
        p = os.path.join(native, d)
        sources += [os.path.join(p, f) for f in sorted(os.listdir(p)) if f.endswith((".cpp", ".cu"))]
    flags = []
    for key in sorted(defines):
        val = defines[key]
        flags.append(f"-DKM_{key}" if val is None else f"-DKM_{key}={val}")
    build_dir = os.path.join(OUT, name)
    os.makedirs(build_dir, exist_ok=True)
    if os.path.exists(os.path.join(build_dir, name + ".so")):
        return name + " (cached)"
    ext.load(
        name=name,
        sources=sources,
        extra_cflags=["-O3"] + flags,
        extra_cuda_cflags=flags,
        build_directory=build_dir,
        is_python_module=True,
        verbose=False,
    )
    return name


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=REFERENCE_DIR)
    ap.add_argument("--only", default=None, help="substring filter on module names")
    ap.add_argument("--tuned", action="store_true",
                    help="also build the reference's autotune candidates of the forward product for the benchmark widths")
    ap.add_argument("-j", type=int, default=4)
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.reference, "native")):
        print(f"reference tree not found at {args.reference}; nothing built")
        return 0
    specs = module_specs() + (tuned_matmul_specs() if args.tuned else [])
    specs = [s for s in specs if args.only is None or args.only in s[0]]
    failed = []
    with concurrent.futures.ProcessPoolExecutor(max_workers=args.j) as pool:
        futs = {pool.submit(build_one, args.reference, *s): s[0] for s in specs}
        for fut in concurrent.futures.as_completed(futs):
            try:
                print("built", fut.result(), flush=True)
            except Exception as exc:  # noqa: BLE001 - report and carry on with the others
                failed.append(futs[fut])
                print("FAILED", futs[fut], str(exc)[-800:], flush=True)
    if failed:
        print("failed modules:", failed)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
