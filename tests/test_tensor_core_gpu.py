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


def test_tc_product_says_that_it_ran_on_the_tensor_cores():
    from kernel_matmul_b200 import ops

    out = _run("rbf", 300, 300, 64, square=True)
    assert ops.used_tensor_cores(out)
    ops.check()


# ------------------------------------------------------------------ GEMM widths 16 / 32 / 64 / 128


@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("k", [1, 5, 12, 16, 17, 30, 32, 33, 50, 64])
def test_tc_narrow_product_matches_oracle(kt, k):
    # GEMM widths 16 (k <= 16), 32 and 64
    _run(kt, 600, 800, k)


def test_tc_narrow_long_bands_many_accumulator_groups():
    # unbanded with n = 3000: 188 tiles of 16 columns = 24 accumulator groups, 47 slot refills
    _run("spectral", 257, 3000, 16, cutoff=None)
    _run("rbf", 128, 2049, 7, cutoff=None)
    _run("locally_periodic", 257, 3000, 32, cutoff=None)
    _run("spectral", 130, 2049, 64, cutoff=None)


def test_tc_narrow_batched_shared_and_private_rhs():
    _run("spectral", 500, 500, 16, batch=(2, 3), shared_rhs=True, square=True)
    _run("locally_periodic", 301, 199, 9, batch=(4,), shared_rhs=False)
    _run("rbf", 301, 199, 40, batch=(3,), shared_rhs=False)


def test_tc_narrow_strided_operands_and_empty_bands():
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    x1 = torch.sort(torch.rand(700) * 10)[0]
    x2 = torch.sort(torch.rand(640) * 3)[0]
    start, end = O.make_ranges(0.5, x1, x2)
    assert bool((start == end).any())
    params = torch.tensor([0.8, 0.7, 1.2])
    rhs_wide = torch.randn(640, 40)
    rhs = rhs_wide[:, 3:33:2]  # 15 columns, column stride 2
    x2_wide = torch.stack([x2, -x2], dim=-1).cuda()
    out = ops.matmul("spectral", x1.cuda(), x2_wide[:, 0], rhs_wide.cuda()[:, 3:33:2], params.cuda(), start.cuda(),
                     end.cuda(), path="tc")
    assert ops.tc_status(out) == 0
    assert rel_err(out, O.matmul("spectral", x1, x2, rhs.contiguous(), params, start, end)) <= 1e-5


# --------------------------------------------------------------------- tensor-core gradients


def _run_grad(kt, m, n, k, batch=(), cutoff=2.0, square=False, which="bilinear_derivative"):
    from conftest import assert_grad_close
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    x1 = torch.sort(torch.rand(*batch, m) * 10)[0]
    x2 = x1 if square else torch.sort(torch.rand(*batch, n) * 10)[0]
    n = x2.shape[-1]
    params = make_params(kt, batch)
    start, end = O.make_ranges(cutoff, x1) if square else O.make_ranges(cutoff, x1, x2)
    left = torch.randn(*batch, m, k)
    right = torch.randn(*batch, n, k)
    d = lambda t: t.cuda()  # noqa: E731
    if which == "bilinear_derivative":
        ref = O.bilinear_derivative(kt, x1, x2, left, right, params, start, end)
        scale = O.bilinear_derivative(kt, x1, x2, left, right, params, start, end, absolute=True)
        out = ops.bilinear_derivative(kt, d(x1), d(x2), d(left), d(right), d(params), d(start), d(end), path="tc")
        fma = ops.bilinear_derivative(kt, d(x1), d(x2), d(left), d(right), d(params), d(start), d(end), path="fma")
    else:
        ref = O.matmul_bwd(kt, x1, x2, right, params, start, end, left)
        scale = O.matmul_bwd(kt, x1, x2, right, params, start, end, left, absolute=True)
        out = ops.matmul_bwd(kt, d(x1), d(x2), d(right), d(params), d(start), d(end), d(left), path="tc")
        fma = ops.matmul_bwd(kt, d(x1), d(x2), d(right), d(params), d(start), d(end), d(left), path="fma")
    assert ops.tc_status(out) == 0
    assert out.shape == ref.shape
    assert_grad_close(out, ref, scale)
    assert_grad_close(fma, ref, scale)


@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("k", [1, 8, 11, 16, 17, 32])
def test_tc_gradient_matches_oracle(kt, k):
    _run_grad(kt, 600, 800, k)


@pytest.mark.parametrize("which", ["bilinear_derivative", "matmul_bwd"])
def test_tc_gradient_batched_ragged(which):
    _run_grad("spectral", 301, 199, 16, batch=(3,), which=which)
    _run_grad("locally_periodic", 500, 500, 32, batch=(2, 2), square=True, which=which)


def test_tc_gradient_unbanded_long_bands():
    _run_grad("spectral", 257, 3000, 16, cutoff=None)
    _run_grad("rbf", 130, 2049, 24, cutoff=None)


@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("k", [33, 40, 48, 56, 64, 65, 100, 130])
def test_tc_gradient_wide_operands(kt, k):
    # up to 64 columns: four consumer groups; beyond: column blocks of 64
    _run_grad(kt, 400, 500, k)


def test_tc_narrow_column_scales():
    # the narrow kernel scales every rhs column by a power of two: columns of very different
    # magnitude (and a zero column) must each keep fp32-level accuracy
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    x = torch.sort(torch.rand(700) * 10)[0]
    start, end = O.make_ranges(2.0, x)
    params = torch.tensor([1.3, 0.6, 0.9])
    rhs = torch.randn(700, 12)
    mags = torch.tensor([1e-30, 1e-12, 1e-3, 1.0, 7.0, 1e4, 1e12, 1e30, 0.0, 3e-5, 2e5, 1.0])
    rhs = rhs * mags
    rhs[:, 11] = torch.randn(700).abs() * torch.logspace(-20, 0, 700)  # wide range inside one column
    out = ops.matmul("spectral", x.cuda(), x.cuda(), rhs.cuda(), params.cuda(), start.cuda(), end.cuda(), path="tc")
    assert ops.tc_status(out) == 0
    ref = O.matmul("spectral", x, x, rhs, params, start, end)
    for c in range(12):
        if mags[c] == 0:
            assert bool((out[:, c] == 0).all())
        else:
            assert rel_err(out[:, c], ref[:, c]) <= 1e-5, c


def test_auto_path_selection_for_narrow_operands():
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    batch = (4,)
    x = torch.sort(torch.rand(8192) * 100)[0]
    start, end = O.make_ranges(2.0, x)
    params = make_params("spectral", batch)
    xd, sd, ed, pd = x.cuda(), start.cuda(), end.cuda(), params.cuda()
    for k, expect_tc in [(16, True), (9, True), (4, False)]:
        rhs = torch.randn(8192, k).cuda()
        out = ops.matmul("spectral", xd.expand(4, -1), xd.expand(4, -1), rhs.expand(4, -1, -1), pd, sd, ed)
        assert ops.used_tensor_cores(out) == expect_tc
        assert ops.tc_status(out) == 0
        fma = ops.matmul("spectral", xd.expand(4, -1), xd.expand(4, -1), rhs.expand(4, -1, -1), pd, sd, ed, path="fma")
        assert rel_err(out, fma) <= 1e-5
    left = torch.randn(4, 8192, 16).cuda()
    right = torch.randn(4, 8192, 16).cuda()
    g = ops.bilinear_derivative("spectral", xd.expand(4, -1), xd.expand(4, -1), left, right, pd, sd, ed)
    assert ops.used_tensor_cores(g) and ops.tc_status(g) == 0
    g4 = ops.bilinear_derivative("spectral", xd.expand(4, -1), xd.expand(4, -1), left[..., :4], right[..., :4], pd, sd, ed)
    assert not ops.used_tensor_cores(g4)
    # small problems stay on the FMA pipe whatever the width
    xs = xd[:300]
    ss, es = O.make_ranges(2.0, x[:300])
    small = ops.matmul("spectral", xs, xs, torch.randn(300, 16).cuda(), pd[0], ss.cuda(), es.cuda())
    assert not ops.used_tensor_cores(small)


@pytest.mark.parametrize("k", [13, 40])
def test_tc_product_row_window(k):
    """km_matmul_tc_rows_f32: a window of row blocks equals the rows of the full product."""
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    B, n = 3, 1500
    x = torch.sort(torch.rand(n) * 20)[0]
    params = make_params("spectral", (B,))
    start, end = O.make_ranges(2.0, x)
    rhs = torch.randn(B, n, k)
    ref = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs, params, start.expand(B, -1), end.expand(B, -1))
    d = lambda t: t.cuda()  # noqa: E731
    args = ("spectral", d(x).expand(B, n), d(x).expand(B, n), d(rhs), d(params), d(start).expand(B, -1), d(end).expand(B, -1))
    out = ops.matmul_rows(*args, row_block_begin=3, row_block_count=4, path="tc")
    assert ops.tc_status(out) == 0 and out.shape == (B, 512, k)
    assert rel_err(out, ref[:, 384:896]) <= 1e-5
    tail = ops.matmul_rows(*args, row_block_begin=10, path="tc")  # ragged last block
    assert rel_err(tail, ref[:, 1280:]) <= 1e-5
    full = ops.matmul(*args, path="tc")
    assert torch.equal(out, full[:, 384:896])


# ------------------------------------------------------------------ separable phases and their guard


@pytest.mark.parametrize("kt", ["spectral", "locally_periodic"])
@pytest.mark.parametrize("rows", ["unsorted", "sorted"])
def test_tc_phase_factors_far_rows_and_offsets(kt, rows):
    # The tensor-core kernels factor cos / sin(W (x1_i - x2_j)) into per-row and per-column values
    # around the row block's middle point.  Unsorted rows spread a block over the whole range (the
    # kernels must then keep the per-entry evaluation); sorted rows far from zero keep the factored
    # form, whose arguments are differences to a nearby origin.
    from conftest import assert_grad_close
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    m, n, k = 500, 700, 16
    x1 = torch.rand(m) * 60 + 300
    if rows == "sorted":
        x1 = torch.sort(x1)[0]
    x2 = torch.sort(torch.rand(n) * 60 + 300)[0]
    params = make_params(kt, ())
    start, end = O.make_ranges(None if rows == "unsorted" else 4.0, x1, x2)
    rhs, og = torch.randn(n, k), torch.randn(m, k)
    d = lambda t: t.cuda()  # noqa: E731
    args = (kt, d(x1), d(x2), d(rhs), d(params), d(start), d(end))
    out = ops.matmul(*args, path="tc")
    assert ops.tc_status(out) == 0
    assert rel_err(out, O.matmul(kt, x1, x2, rhs, params, start, end)) <= 1e-5
    grad = ops.matmul_bwd(*args, d(og), path="tc")
    assert ops.tc_status(grad) == 0
    ref = O.matmul_bwd(kt, x1, x2, rhs, params, start, end, og)
    scale = O.matmul_bwd(kt, x1, x2, rhs, params, start, end, og, absolute=True)
    assert_grad_close(grad, ref, scale)
