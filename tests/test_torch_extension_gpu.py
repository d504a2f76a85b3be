"""``kernel_matmul_b200._C``, the ahead-of-time PyTorch C++ extension over the C ABI: its ten
functions (the reference's per-op ``call`` and the three ``ranges`` functions,
native/<op>/<op>.cpp, native/ranges/ranges.cpp:152-156) against the fp64 oracle on the reference's
test input family.  Tolerances as in ``test_ops_gpu.py``."""
import pytest
import torch

from conftest import KERNEL_TYPES, SHAPES, assert_grad_close, device_example, make_example, rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-5
CASES = [pytest.param(s, kt, id=f"shape{i}-{kt}") for i, s in enumerate(SHAPES) for kt in KERNEL_TYPES]
KID = {"rbf": 0, "spectral": 1, "locally_periodic": 2}


@pytest.fixture(scope="module")
def C():
    import kernel_matmul_b200  # noqa: F401
    from kernel_matmul_b200 import _C

    return _C


@pytest.fixture(scope="module")
def O():
    from oracle import oracle

    return oracle


@pytest.mark.parametrize("shape,kt", CASES)
def test_extension_products_and_gradients(C, O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    out = C.matmul(KID[kt], d.x1, d.x2, d.rhs, d.params, d.start, d.end)
    ref = O.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    assert out.shape == ref.shape and rel_err(out, ref) <= TOL
    og = torch.randn(ref.shape)
    og = og / torch.linalg.norm(og, dim=(-2, -1), keepdim=True)
    g = C.matmul_bwd(KID[kt], d.x1, d.x2, d.rhs, d.params, d.start, d.end, og.cuda())
    gref = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og)
    assert g.shape == gref.shape
    assert_grad_close(g, gref, O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og, absolute=True))
    left, right = torch.randn(*ex.x1.shape, 5), torch.randn(*ex.x2.shape, 5)
    b = C.bilinear_derivative(KID[kt], d.x1, d.x2, left.cuda(), right.cuda(), d.params, d.start, d.end)
    bref = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end)
    assert_grad_close(b, bref, O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end, absolute=True))


@pytest.mark.parametrize("shape,kt", CASES)
def test_extension_dense_and_gather(C, O, shape, kt):
    ex = make_example(shape, kt, square=True)
    d = device_example(ex)
    dense = C.dense(KID[kt], d.x1, d.x2, d.params, d.start, d.end)
    ref = O.dense(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end)
    assert dense.shape == ref.shape and rel_err(dense, ref) <= TOL
    assert torch.equal(dense.cpu() != 0, ref != 0)
    og = torch.randn(ref.shape)
    g = C.dense_bwd(KID[kt], d.x1, d.x2, d.params, d.start, d.end, og.cuda())
    assert_grad_close(g, O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, og),
                      O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, og, absolute=True))
    batch, m = ex.params.shape[:-1], ex.x1.shape[-1]
    shape_i = (7, 41)
    bidx = [torch.randint(0, s, shape_i, dtype=torch.int32) for s in batch]
    row = torch.randint(0, m, shape_i, dtype=torch.int32)
    col = torch.randint(0, m, (41,), dtype=torch.int32)  # broadcast against the others
    vals = C.index(KID[kt], d.x1, d.x2, d.params, d.start, d.end, [b.cuda() for b in bidx], row.cuda(), col.cuda())
    vref = O.index(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, tuple(bidx), row, col.expand(shape_i))
    assert vals.shape == vref.shape and rel_err(vals, vref) <= TOL
    w = torch.randn(shape_i)
    gi = C.index_bwd(KID[kt], d.x1, d.x2, d.params, d.start, d.end, [b.cuda() for b in bidx], row.cuda(), col.cuda(), w.cuda())
    giref = O.index_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, tuple(bidx), row, col.expand(shape_i), w)
    assert_grad_close(gi, giref, O.index_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, tuple(bidx), row,
                                             col.expand(shape_i), w, absolute=True))


def test_extension_tensor_core_product(C, O):
    """Large enough for the tensor-core path (>= 256 work items, k >= 9)."""
    B, n, k = 4, 8192, 16
    x = torch.sort(torch.rand(n) * 100)[0]
    start, end = O.make_ranges(2.0, x)
    params = torch.stack([1 + torch.rand(B), 0.5 + 0.5 * torch.rand(B), 1 + torch.rand(B)], dim=-1)
    rhs = torch.randn(n, k)
    xd = x.cuda().expand(B, n)
    args = (xd, xd, rhs.cuda().expand(B, n, k), params.cuda(), start.cuda().expand(B, -1), end.cuda().expand(B, -1))
    out = C.matmul(1, *args)
    fma = C.matmul(1, *args, tensor_cores_auto=False)
    ref = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params, start.expand(B, -1), end.expand(B, -1))
    assert rel_err(out, ref) <= TOL and rel_err(fma, ref) <= TOL
    assert not torch.equal(out, fma)  # two different kernels ran


@pytest.mark.parametrize("cutoff", [0.5, 2.0])
def test_extension_band_construction(C, O, cutoff):
    x1 = torch.sort(torch.rand(3, 700) * 10)[0]
    x2 = torch.sort(torch.rand(3, 900) * 10)[0]
    for align in (False, True):
        s, e = C.make_ranges(x1.cuda(), x2.cuda(), cutoff, 128, align)
        rs, re = O.make_ranges(cutoff, x1, x2, align=align)
        assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)
    st, et = C.transpose_ranges(s, e, 700, 900, 128)
    rst, ret = O.transpose_ranges(rs, re, 700, 900)
    assert torch.equal(st.cpu(), rst) and torch.equal(et.cpu(), ret)
    s, e = C.make_ranges_symmetric(x1.cuda(), cutoff, 128)
    rs, re = O.make_ranges(cutoff, x1)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re)


def test_extension_raises_the_reference_messages(C):
    x = torch.rand(300, device="cuda")
    s = torch.zeros(3, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="x must be a CUDA tensor"):
        C.matmul(0, x.cpu(), x, torch.rand(300, 2, device="cuda"), torch.ones(2, device="cuda"), s, s)
    with pytest.raises(RuntimeError, match="x must be int32"):
        C.matmul(0, x, x, torch.rand(300, 2, device="cuda"), torch.ones(2, device="cuda"), s.long(), s)
    with pytest.raises(RuntimeError, match="Unknown kernel type"):
        C.dense(7, x, x, torch.ones(2, device="cuda"), s, s)
