"""The tcgen05 (tensor-core) product against the fp64 oracle and against the FMA path."""
import pytest
import torch

from conftest import KERNEL_TYPES, make_params, rel_err

pytestmark = pytest.mark.gpu


def _run(kt, m, n, k, batch=(), cutoff=2.0, shared_rhs=False, square=False):
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    x1 = torch.sort(torch.rand(*batch, m) * 10)[0]
    x2 = x1 if square else torch.sort(torch.rand(*batch, n) * 10)[0]
    n = x2.shape[-1]
    params = make_params(kt, batch)
    if square:
        start, end = O.make_ranges(cutoff, x1)
    else:
        start, end = O.make_ranges(cutoff, x1, x2)
    rhs = torch.randn(n, k).expand(*batch, n, k) if shared_rhs else torch.randn(*batch, n, k)
    ref = O.matmul(kt, x1, x2, rhs, params, start, end)
    d = lambda t: t.cuda()  # noqa: E731
    rhs_d = d(rhs[(0,) * len(batch)]).expand(*batch, n, k) if shared_rhs else d(rhs)
    args = (kt, d(x1), d(x2), rhs_d, d(params), d(start), d(end))
    out = ops.matmul(*args, path="tc")
    assert ops.tc_status(out) == 0
    assert out.shape == ref.shape
    assert rel_err(out, ref) <= 1e-5
    fma = ops.matmul(*args, path="fma")
    assert rel_err(out, fma) <= 1e-5
    return out


@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("k", [16, 64, 128, 200])
def test_tc_product_matches_oracle(kt, k):
    _run(kt, 600, 800, k)


@pytest.mark.parametrize("k", [8, 65, 130, 300])
def test_tc_product_ragged_sizes_and_k_blocks(k):
    # m, n not multiples of 128 / 32; k not a multiple of 16; k > 256 takes two column blocks
    _run("spectral", 301, 199, k, batch=(3,))


def test_tc_product_batched_shared_and_private_rhs():
    _run("rbf", 500, 500, 64, batch=(2, 3), shared_rhs=True, square=True)
    _run("rbf", 500, 500, 64, batch=(4,), shared_rhs=False, square=True)


def test_tc_product_unbanded_and_empty_bands():
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    _run("locally_periodic", 257, 2000, 96, cutoff=None)
    # a band that is empty for some row blocks
    x1 = torch.sort(torch.rand(700) * 10)[0]
    x2 = torch.sort(torch.rand(640) * 3)[0]  # rows beyond ~3 + cutoff see nothing
    start, end = O.make_ranges(0.5, x1, x2)
    assert bool((start == end).any())
    params = torch.tensor([0.8, 1.2])
    rhs = torch.randn(640, 64)
    out = ops.matmul("rbf", x1.cuda(), x2.cuda(), rhs.cuda(), params.cuda(), start.cuda(), end.cuda(), path="tc")
    assert ops.tc_status(out) == 0
    assert rel_err(out, O.matmul("rbf", x1, x2, rhs, params, start, end)) <= 1e-5


def test_auto_path_uses_tensor_cores_from_64_columns():
    from kernel_matmul_b200 import ops

    assert ops.TENSOR_CORE_MIN_K == 64
    out = _run("rbf", 300, 300, 64, square=True)
    assert hasattr(out, "_km_workspace")
