"""Host-side logic that needs no GPU: the C-ABI library loads and exports every declared
symbol, argument validation of the entry points and of the Python layer, the shims that keep
the reference's names."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from kernel_matmul_b200 import _lib

    header = open(os.path.join(ROOT, "include", "km_b200.h")).read()
    declared = set(re.findall(r"KM_API\s+[\w\s\*]+?\b(km_\w+)\s*\(", header))
    assert len(declared) >= 17
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in include/km_b200.h but not exported"
    assert declared == set(_lib.EXPORTED)


def test_version_and_num_params():
    from kernel_matmul_b200._lib import lib

    assert b"sm_100a" in lib.km_version()
    assert [lib.km_num_params(i) for i in range(4)] == [2, 3, 4, -1]


def test_entry_points_validate_before_launch():
    """Bad arguments give an error code and a message; nothing is launched (no GPU needed)."""
    from kernel_matmul_b200._lib import KmBatch, KmView, lib

    b = KmBatch()
    b.ndim = 0
    v = KmView()
    rc = lib.km_matmul_f32(7, b, 10, 10, 1, v, v, v, v, v, v, v, None)
    assert rc == 1 and b"unknown kernel type" in lib.km_last_error()
    rc = lib.km_matmul_f32(0, b, 10, 10, 1, v, v, v, v, v, v, v, None)
    assert rc == 1 and b"null data pointer" in lib.km_last_error()
    b.ndim = 9
    rc = lib.km_matmul_f32(0, b, 10, 10, 1, v, v, v, v, v, v, v, None)
    assert rc == 1 and b"batch rank" in lib.km_last_error()
    b.ndim = 1
    b.size[0] = 4
    assert lib.km_grad_workspace_bytes(0, b, 300) == 4 * 3 * 4 * 4
    rc = lib.km_bilinear_derivative_f32(1, b, 300, 300, 2, v, v, v, v, v, v, v, v, None, 0, None)
    assert rc == 1  # null data pointers are reported before the workspace is looked at
    rc = lib.km_make_ranges_f32(1, 10, 10, None, None, 1.0, 0, 0, None, None, None, None)
    assert rc == 1 and b"block_size" in lib.km_last_error()


def test_ops_reject_cpu_and_wrong_dtype():
    from kernel_matmul_b200 import ops

    x = torch.rand(10)
    s = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="x must be a CUDA tensor"):
        ops.matmul("rbf", x, x, torch.rand(10, 1), torch.ones(2), s, s)
    with pytest.raises(ValueError, match="Unknown kernel type"):
        ops.matmul("matern", x, x, torch.rand(10, 1), torch.ones(2), s, s)


def test_shims_keep_reference_names():
    from kernel_matmul_b200 import _BLOCK_SIZE
    from kernel_matmul_b200.compile import compile_pool, kernel_type_from_defines, load_native
    from kernel_matmul_b200.configurations import (
        BilinearDerivativeConfiguration, DenseBwdConfiguration, DenseConfiguration, IndexBwdConfiguration,
        IndexConfiguration, MatmulAutotuneConfiguration, MatmulBwdConfiguration, MatmulSingleConfiguration,
    )
    from kernel_matmul_b200.native_function import NativeFunction

    assert _BLOCK_SIZE == 128
    x = torch.rand(3, 10)
    args = (x, x, torch.rand(3, 10, 5), torch.ones(3, 2), None, None)
    cfg = MatmulSingleConfiguration("rbf")
    d = cfg.make_config(args)
    assert d["BATCH_DIM"] == 1 and d["BLOCK_SIZE"] == 128 and "KERNEL_RBF" in d and "MATMUL_COL_BLOCKS" in d
    d["MATMUL_COL_BLOCKS"] = 2  # callers of the reference overwrite tuning keys; they are ignored here
    mod = load_native("matmul", d)
    assert mod.kernel_type == "rbf" and callable(mod.call)
    assert len(MatmulAutotuneConfiguration("spectral").make_candidates(args)) == 1
    assert kernel_type_from_defines({"KERNEL_LOCALLY_PERIODIC": None, "BATCH_DIM": 0}) == "locally_periodic"
    with pytest.raises(ValueError):
        load_native("matmul", {"BATCH_DIM": 1})
    with pytest.raises(NotImplementedError):
        load_native("matmul", {"KERNEL_COMPACT": None})
    for cls in (MatmulBwdConfiguration, BilinearDerivativeConfiguration, DenseConfiguration, DenseBwdConfiguration):
        assert "KERNEL_SPECTRAL" in cls("spectral").make_config(args)
    idx = torch.zeros(4, 7, dtype=torch.int32)
    iargs = (x, x, torch.ones(3, 2), None, None, (idx,), idx, idx)
    assert IndexConfiguration("rbf").make_config(iargs)["INDEX_BATCH_DIM"] == 1
    assert IndexBwdConfiguration("rbf").cache_key(iargs + (None,)) == "1_1"
    f = NativeFunction("matmul", MatmulAutotuneConfiguration("rbf"))
    assert f.defines is None
    with compile_pool(4):
        pass


def test_operator_argument_checks():
    from kernel_matmul_b200.linear_operator import KernelMatmulOperator

    x = torch.rand(10, 1)
    s = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(ValueError, match="kernel_type must be specified"):
        KernelMatmulOperator(x, x, torch.ones(2), s, s)
    with pytest.raises(ValueError, match="must have shapes"):
        KernelMatmulOperator(x.squeeze(-1), x, torch.ones(2), s, s, kernel_type="rbf")
    op = KernelMatmulOperator(x, x, torch.ones(3, 2), s, s, kernel_type="rbf")
    assert op.shape == (3, 10, 10) and op.batch_shape == (3,)
    assert op.transpose() is op  # symmetric: x1 == x2


def test_workload_generators_are_deterministic():
    from kernel_matmul_b200 import workloads

    a, b = workloads.rbf_small(), workloads.rbf_small()
    assert torch.equal(a.x, b.x) and torch.equal(a.rhs, b.rhs)
    w = workloads.spectral_mixture(n=1024, components=4, k=2)
    assert w.params.shape == (4, 3) and len(w.cutoffs) == 4 and w.extra["out_grad"].shape == (4, 1024, 2)
    assert bool((w.x[1:] >= w.x[:-1]).all())


def test_torch_extension_exports_the_ten_reference_functions():
    """The ahead-of-time PyTorch extension loads without a GPU and refuses CPU tensors with the
    reference's message (native/common/entrypoint.h:3-5)."""
    import kernel_matmul_b200  # noqa: F401  (loads libkm_b200.so, which the extension links against)
    from kernel_matmul_b200 import _C

    for name in ("matmul", "matmul_bwd", "bilinear_derivative", "dense", "dense_bwd", "index", "index_bwd",
                 "make_ranges", "make_ranges_symmetric", "transpose_ranges"):
        assert callable(getattr(_C, name)), name
    assert (_C.KERNEL_RBF, _C.KERNEL_SPECTRAL, _C.KERNEL_LOCALLY_PERIODIC) == (0, 1, 2)
    x = torch.rand(10)
    s = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="x must be a CUDA tensor"):
        _C.matmul(0, x, x, torch.rand(10, 1), torch.ones(2), s, s)
    with pytest.raises(RuntimeError, match="x must be a CUDA tensor"):
        _C.make_ranges_symmetric(x[None], 1.0, 128)
