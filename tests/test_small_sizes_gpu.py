"""All seven ops on an exhaustive grid of tiny sizes: m, n in {1, 127, 129, 257} and
k in {1, 3, 16, 65, 128}, both kernel families (FMA pipe and tensor cores), rectangular and
symmetric bands.  These are the sizes where every edge of the kernels is hit at once: a single
row or column, one row short of / one row past a block boundary, bands narrower than one tile,
and the symmetric pattern of fewer than 128 points, whose first range end is 128 > n in the
reference (native/ranges/ranges.cpp:83,93) and has to be clamped.

Tolerances as in ``test_ops_gpu.py``.
"""
import pytest
import torch

from conftest import KERNEL_TYPES, assert_grad_close, make_params, rel_err

pytestmark = pytest.mark.gpu

SIZES = [1, 127, 129, 257]
WIDTHS = [1, 3, 16, 65, 128]
TOL = 1e-5


@pytest.fixture(scope="module")
def O():
    from oracle import oracle

    return oracle


def _inputs(O, kt, m, n, symmetric, cutoff=2.0):
    x1 = torch.sort(torch.rand(m) * 10)[0]
    if symmetric:
        x2 = x1
        start, end = O.make_ranges(cutoff, x1)
    else:
        x2 = torch.sort(torch.rand(n) * 10)[0]
        start, end = O.make_ranges(cutoff, x1, x2)
    return x1, x2, make_params(kt, ()), start, end


def _shapes():
    for m in SIZES:
        for n in SIZES:
            yield pytest.param(m, n, False, id=f"{m}x{n}")
    for n in SIZES:
        yield pytest.param(n, n, True, id=f"sym{n}")


@pytest.mark.parametrize("path", ["fma", "tc"])
@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("m,n,symmetric", list(_shapes()))
def test_products_and_gradients_on_tiny_sizes(O, kt, m, n, symmetric, path):
    from kernel_matmul_b200 import ops

    x1, x2, params, start, end = _inputs(O, kt, m, n, symmetric)
    if symmetric and n < 128:
        assert int(end[0]) == 128 > n  # the unclamped end of the reference's scan
    d = [t.cuda() for t in (x1, x2, params, start, end)]
    for k in WIDTHS:
        rhs = torch.randn(x2.shape[0], k)
        out = ops.matmul(kt, d[0], d[1], rhs.cuda(), d[2], d[3], d[4], path=path)
        ref = O.matmul(kt, x1, x2, rhs, params, start, end)
        assert out.shape == ref.shape
        if float(ref.abs().max()) > 0:
            assert rel_err(out, ref) <= TOL, (k, "matmul")
        else:
            assert bool((out == 0).all())
        og = torch.randn(m, k)
        g = ops.matmul_bwd(kt, d[0], d[1], rhs.cuda(), d[2], d[3], d[4], og.cuda(), path=path)
        gref = O.matmul_bwd(kt, x1, x2, rhs, params, start, end, og)
        gscale = O.matmul_bwd(kt, x1, x2, rhs, params, start, end, og, absolute=True)
        assert_grad_close(g, gref, gscale)
        b = ops.bilinear_derivative(kt, d[0], d[1], og.cuda(), rhs.cuda(), d[2], d[3], d[4], path=path)
        assert_grad_close(b, gref, gscale)  # the same contraction with left = out_grad, right = rhs
    ops.check()


@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("m,n,symmetric", list(_shapes()))
def test_dense_and_gather_on_tiny_sizes(O, kt, m, n, symmetric):
    from kernel_matmul_b200 import ops

    x1, x2, params, start, end = _inputs(O, kt, m, n, symmetric)
    d = [t.cuda() for t in (x1, x2, params, start, end)]
    n = x2.shape[0]
    dense = ops.dense(kt, *d)
    ref = O.dense(kt, x1, x2, params, start, end)
    assert dense.shape == ref.shape == (m, n)
    assert rel_err(dense, ref) <= TOL or float(ref.abs().max()) == 0
    assert torch.equal(dense.cpu() != 0, ref != 0)
    og = torch.randn(m, n)
    g = ops.dense_bwd(kt, *d, og.cuda())
    assert_grad_close(g, O.dense_bwd(kt, x1, x2, params, start, end, og), O.dense_bwd(kt, x1, x2, params, start, end, og, absolute=True))
    # every entry once, plus out-of-band ones
    row = torch.arange(m, dtype=torch.int32).repeat_interleave(n)
    col = torch.arange(n, dtype=torch.int32).repeat(m)
    vals = ops.index(kt, *d, (), row.cuda(), col.cuda())
    assert torch.equal(vals.reshape(m, n) != 0, dense != 0)  # gather and materialise see the same band
    assert rel_err(vals.reshape(m, n), ref) <= TOL or float(ref.abs().max()) == 0
    w = torch.randn(m * n)
    gi = ops.index_bwd(kt, *d, (), row.cuda(), col.cuda(), w.cuda())
    assert_grad_close(gi, O.index_bwd(kt, x1, x2, params, start, end, (), row, col, w),
                      O.index_bwd(kt, x1, x2, params, start, end, (), row, col, w, absolute=True))


@pytest.mark.parametrize("n", [1, 127, 129, 257])
def test_band_construction_on_tiny_sizes(O, n):
    from kernel_matmul_b200 import ranges

    x = torch.sort(torch.rand(n) * 10)[0]
    x2 = torch.sort(torch.rand(257 - n + 1) * 10)[0]
    for cutoff in (0.0, 0.5, 2.0, 100.0):
        s, e = ranges.make_ranges(cutoff, x.cuda())
        rs, re = O.make_ranges(cutoff, x)
        assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)
        for align in (False, True):
            s, e = ranges.make_ranges(cutoff, x.cuda(), x2.cuda(), align=align)
            rs, re = O.make_ranges(cutoff, x, x2, align=align)
            assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)
            if align:
                st, et = ranges.transpose_ranges(s, e, n, x2.shape[0])
                rst, ret = O.transpose_ranges(rs, re, n, x2.shape[0])
                assert torch.equal(st.cpu(), rst) and torch.equal(et.cpu(), ret)
