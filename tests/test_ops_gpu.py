"""Parity of the CUDA ops against the fp64 oracle on the reference's test input family.

Tolerances, fp32 path vs fp64 oracle.  Products, dense and gathered entries: <= 1e-5 relative,
measured as max |err| / max |ref| per result (outputs cross zero).  Gradients: <= 1e-5 relative
per element, or <= 1e-7 of the sum of term magnitudes where the terms cancel
(``conftest.assert_grad_close``).  The reference's own tests accept atol 2e-4 for products and
atol = rtol = 2e-3 for gradients (tests/native/test_matmul.py:30, test_matmul_bwd.py:48).
"""
import pytest
import torch

from conftest import KERNEL_TYPES, SHAPES, assert_grad_close, device_example, make_example, rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-5

CASES = [pytest.param(s, kt, id=f"shape{i}-{kt}") for i, s in enumerate(SHAPES) for kt in KERNEL_TYPES]


@pytest.fixture(scope="module")
def km():
    import kernel_matmul_b200 as km

    return km


@pytest.fixture(scope="module")
def O():
    from oracle import oracle

    return oracle


@pytest.mark.parametrize("shape,kt", CASES)
def test_matmul(km, O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    out = km.ops.matmul(kt, d.x1, d.x2, d.rhs, d.params, d.start, d.end)
    ref = O.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    assert out.shape == ref.shape
    assert rel_err(out, ref) <= TOL


@pytest.mark.parametrize("shape,kt", CASES)
def test_matmul_bwd(km, O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    batch = ex.params.shape[:-1]
    og = torch.randn(*batch, ex.x1.shape[-1], ex.rhs.shape[-1])
    og = og / torch.linalg.norm(og, dim=(-2, -1), keepdim=True)
    out = km.ops.matmul_bwd(kt, d.x1, d.x2, d.rhs, d.params, d.start, d.end, og.cuda())
    ref = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og)
    assert out.shape == ref.shape
    scale = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og, absolute=True)
    assert_grad_close(out, ref, scale)


@pytest.mark.parametrize("shape,kt", CASES)
def test_bilinear_derivative(km, O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    left = torch.randn(*ex.x1.shape, 5)
    right = torch.randn(*ex.x2.shape, 5)
    out = km.ops.bilinear_derivative(kt, d.x1, d.x2, left.cuda(), right.cuda(), d.params, d.start, d.end)
    ref = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end)
    assert out.shape == ref.shape
    scale = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end, absolute=True)
    assert_grad_close(out, ref, scale)


@pytest.mark.parametrize("shape,kt", CASES)
def test_dense(km, O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    out = km.ops.dense(kt, d.x1, d.x2, d.params, d.start, d.end)
    ref = O.dense(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end)
    assert out.shape == ref.shape
    assert rel_err(out, ref) <= TOL
    # exact zeros outside the band
    assert bool((out.cpu()[ref == 0] == 0).all())


@pytest.mark.parametrize("shape,kt", CASES)
def test_dense_bwd(km, O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    batch = ex.params.shape[:-1]
    og = torch.randn(*batch, ex.x1.shape[-1], ex.x2.shape[-1])
    out = km.ops.dense_bwd(kt, d.x1, d.x2, d.params, d.start, d.end, og.cuda())
    ref = O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, og)
    scale = O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, og, absolute=True)
    assert_grad_close(out, ref, scale)


@pytest.mark.parametrize("index_shape", [(100,), (5, 101)])
@pytest.mark.parametrize("shape,kt", CASES)
def test_index_and_bwd(km, O, shape, kt, index_shape):
    ex = make_example(shape, kt, square=True)
    d = device_example(ex)
    batch = ex.params.shape[:-1]
    m = ex.x1.shape[-1]
    bidx = tuple(torch.randint(0, s, index_shape, dtype=torch.int32) for s in batch)
    row = torch.randint(0, m, index_shape, dtype=torch.int32)
    col = torch.randint(0, m, index_shape, dtype=torch.int32)
    out = km.ops.index(kt, d.x1, d.x2, d.params, d.start, d.end, tuple(b.cuda() for b in bidx), row.cuda(), col.cuda())
    ref = O.index(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, bidx, row, col)
    assert out.shape == ref.shape
    assert rel_err(out, ref) <= TOL
    assert torch.equal(out.cpu() != 0, ref != 0)  # band membership is exact
    og = torch.randn(index_shape)
    g = km.ops.index_bwd(kt, d.x1, d.x2, d.params, d.start, d.end, tuple(b.cuda() for b in bidx), row.cuda(), col.cuda(), og.cuda())
    gref = O.index_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, bidx, row, col, og)
    assert g.shape == gref.shape
    gscale = O.index_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, bidx, row, col, og, absolute=True)
    assert_grad_close(g, gref, gscale)
