"""The drop-in Python surface on a GPU: autograd Functions, ``KernelMatmulOperator``,
``load_native(...).call`` and ``NativeFunction`` against the fp64 oracle.

These are the call paths of the reference's ``kernel_matmul/linear_operator.py:22-76,185-289``
and ``tests/native/test_native_function.py:9-44``; the inputs are the reference's own test
family (``conftest.SHAPES``: ragged last blocks, expanded batches, k = 1 / 11 / 65).
Tolerances as in ``test_ops_gpu.py``: products, dense and gathered entries <= 1e-5 relative
(max-norm per result), gradients by ``conftest.assert_grad_close``.
"""
import pytest
import torch

from conftest import KERNEL_TYPES, SHAPES, assert_grad_close, device_example, make_example, make_params, rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-5
CASES = [pytest.param(s, kt, id=f"shape{i}-{kt}") for i, s in enumerate(SHAPES) for kt in KERNEL_TYPES]


@pytest.fixture(scope="module")
def O():
    from oracle import oracle

    return oracle


def _operator(d, **kw):
    from kernel_matmul_b200.linear_operator import KernelMatmulOperator

    return KernelMatmulOperator(d.x1.unsqueeze(-1), d.x2.unsqueeze(-1), d.params, d.start, d.end,
                                kernel_type=d.kernel_type, **kw)


@pytest.mark.parametrize("shape,kt", CASES)
def test_operator_matmul_forward_and_backward(O, shape, kt):
    """``op.matmul(rhs)`` through ``_MatmulOperator.apply`` and ``.backward``: the product and
    the gradient that reaches ``params`` (and only ``params``)."""
    ex = make_example(shape, kt)
    d = device_example(ex)
    params = d.params.clone().requires_grad_(True)
    d.params = params
    rhs = d.rhs.clone().requires_grad_(True) if not any(s == 0 for s in d.rhs.stride()) else d.rhs
    op = _operator(d)
    assert tuple(op.shape) == (*ex.params.shape[:-1], ex.x1.shape[-1], ex.x2.shape[-1])
    out = op.matmul(rhs)
    ref = O.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    assert out.shape == ref.shape and rel_err(out, ref) <= TOL
    og = torch.randn(out.shape)
    og = og / torch.linalg.norm(og, dim=(-2, -1), keepdim=True)
    out.backward(og.cuda())
    gref = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og)
    scale = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og, absolute=True)
    assert params.grad is not None and params.grad.shape == gref.shape
    assert_grad_close(params.grad, gref, scale)
    if rhs.requires_grad:
        assert rhs.grad is None  # as in the reference: a gradient for params only


@pytest.mark.parametrize("shape,kt", CASES)
def test_operator_matmul_vector_and_operator_syntax(O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    op = _operator(d)
    ref = O.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    assert rel_err(op @ d.rhs, ref) <= TOL
    if ex.params.dim() == 1:  # a single vector (the reference's LinearOperator accepts 1-D rhs)
        v = op.matmul(d.rhs[..., 0].contiguous())
        assert v.shape == ref.shape[:-1] and rel_err(v, ref[..., 0]) <= TOL


@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_operator_matmul_broadcasts_extra_rhs_batch_dims(O, kt):
    """An rhs with leading dims the operator does not have: the operator is expanded to the
    broadcast batch shape (reference ``linear_operator.py:185-199``)."""
    ex = make_example(SHAPES[2], kt)  # batch (3,)
    d = device_example(ex)
    n, k = ex.x2.shape[-1], 4
    rhs = torch.randn(2, 3, n, k)
    out = _operator(d).matmul(rhs.cuda())
    assert out.shape == (2, 3, ex.x1.shape[-1], k)
    for lead in range(2):
        ref = O.matmul(kt, ex.x1, ex.x2, rhs[lead], ex.params, ex.start, ex.end)
        assert rel_err(out[lead], ref) <= TOL
    # and an operator without batch dims against a batched rhs
    ex0 = make_example(SHAPES[1], kt)
    d0 = device_example(ex0)
    rhs0 = torch.randn(4, ex0.x2.shape[-1], 3)
    out0 = _operator(d0).matmul(rhs0.cuda())
    assert out0.shape == (4, ex0.x1.shape[-1], 3)
    for lead in range(4):
        assert rel_err(out0[lead], O.matmul(kt, ex0.x1, ex0.x2, rhs0[lead], ex0.params, ex0.start, ex0.end)) <= TOL


@pytest.mark.parametrize("shape,kt", CASES)
def test_operator_to_dense_forward_and_backward(O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    params = d.params.clone().requires_grad_(True)
    d.params = params
    dense = _operator(d).to_dense()
    ref = O.dense(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end)
    assert dense.shape == ref.shape and rel_err(dense, ref) <= TOL
    assert bool((dense.detach().cpu()[ref == 0] == 0).all())
    og = torch.randn(ref.shape)
    dense.backward(og.cuda())
    gref = O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, og)
    scale = O.dense_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, og, absolute=True)
    assert_grad_close(params.grad, gref, scale)


@pytest.mark.parametrize("index_shape", [(50,), (4, 33)])
@pytest.mark.parametrize("shape,kt", CASES)
def test_operator_get_indices_forward_and_backward(O, shape, kt, index_shape):
    """``get_indices(row, col, *batch_indices)`` WITH batch indices present and its backward: the
    case the reference's ``_IndexOperator.backward`` cannot run (it unpacks eight saved tensors
    into seven names, ``linear_operator.py:71-72``).  Index tensors are int64 on the CPU, as a
    LinearOperator caller passes them; the operator converts them."""
    ex = make_example(shape, kt, square=True)
    d = device_example(ex)
    params = d.params.clone().requires_grad_(True)
    d.params = params
    batch = ex.params.shape[:-1]
    m = ex.x1.shape[-1]
    bidx = tuple(torch.randint(0, s, index_shape) for s in batch)
    row = torch.randint(0, m, index_shape)
    col = torch.randint(0, m, index_shape)
    out = _operator(d).get_indices(row, col, *bidx)
    to32 = lambda t: t.to(torch.int32)  # noqa: E731
    ref = O.index(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, tuple(map(to32, bidx)), to32(row), to32(col))
    assert out.shape == ref.shape and rel_err(out, ref) <= TOL
    assert torch.equal(out.detach().cpu() != 0, ref != 0)
    og = torch.randn(index_shape)
    out.backward(og.cuda())
    gref = O.index_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, tuple(map(to32, bidx)), to32(row), to32(col), og)
    scale = O.index_bwd(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end, tuple(map(to32, bidx)), to32(row), to32(col), og,
                        absolute=True)
    assert params.grad.shape == gref.shape
    assert_grad_close(params.grad, gref, scale)


@pytest.mark.parametrize("shape,kt", CASES)
def test_operator_bilinear_derivative(O, shape, kt):
    ex = make_example(shape, kt)
    d = device_example(ex)
    left = torch.randn(*ex.x1.shape, 5)
    right = torch.randn(*ex.x2.shape, 5)
    out = _operator(d).bilinear_derivative(left.cuda(), right.cuda())
    ref = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end)
    scale = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end, absolute=True)
    assert out.shape == ref.shape
    assert_grad_close(out, ref, scale)


@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_operator_bilinear_derivative_broadcasts_vector_batch(O, kt):
    """Vectors with a leading dim the operator lacks (reference ``linear_operator.py:248-263``)."""
    ex = make_example(SHAPES[1], kt)
    d = device_example(ex)
    left = torch.randn(3, ex.x1.shape[-1], 4)
    right = torch.randn(3, ex.x2.shape[-1], 4)
    out = _operator(d).bilinear_derivative(left.cuda(), right.cuda())
    assert out.shape == (3, ex.params.shape[-1])
    for b in range(3):
        ref = O.bilinear_derivative(kt, ex.x1, ex.x2, left[b], right[b], ex.params, ex.start, ex.end)
        scale = O.bilinear_derivative(kt, ex.x1, ex.x2, left[b], right[b], ex.params, ex.start, ex.end, absolute=True)
        assert_grad_close(out[b], ref, scale)


@pytest.mark.parametrize("shape,kt", CASES)
def test_operator_transpose_of_a_rectangular_aligned_operator(O, shape, kt):
    """``transpose()`` of a non-symmetric, block-aligned operator equals the transposed matrix
    (``_transpose_nonbatch``, reference ``linear_operator.py:201-215``)."""
    ex = make_example(shape, kt, align=True)
    d = device_example(ex)
    op = _operator(d)
    opt = op.transpose()
    m, n = ex.x1.shape[-1], ex.x2.shape[-1]
    assert tuple(opt.shape[-2:]) == (n, m)
    ref = O.dense(kt, ex.x1, ex.x2, ex.params, ex.start, ex.end).transpose(-1, -2)
    dense_t = opt.to_dense()
    assert rel_err(dense_t, ref) <= TOL
    assert torch.equal(dense_t.cpu() != 0, ref != 0)
    v = torch.randn(*ex.params.shape[:-1], m, 3)
    assert rel_err(opt.matmul(v.cuda()), ref @ v.double()) <= TOL


def test_operator_transpose_refuses_unaligned_ranges():
    ex = make_example(SHAPES[1], "rbf", align=False)
    d = device_example(ex)
    with pytest.raises(ValueError, match="Ranges must be block-aligned"):
        _operator(d).transpose()


@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_operator_symmetric_detection_and_expand_batch(O, kt):
    ex = make_example(SHAPES[2], kt, square=True)  # batch (3,)
    d = device_example(ex)
    op = _operator(d)
    assert op.transpose() is op  # x1 == x2: detected with torch.equal, as the reference does
    big = op.expand_batch((2, 3))
    assert big.batch_shape == (2, 3) and tuple(big.shape) == (2, 3, ex.x1.shape[-1], ex.x1.shape[-1])
    rhs = torch.randn(ex.x1.shape[-1], 2)
    out = big.matmul(rhs.cuda())
    ref = O.matmul(kt, ex.x1, ex.x2, rhs.expand(3, -1, -1), ex.params, ex.start, ex.end)
    assert out.shape == (2, 3, *ref.shape[-2:])
    assert rel_err(out[0], ref) <= TOL and torch.equal(out[0], out[1])
    # not symmetric when told so or when the inputs differ
    ex2 = make_example(SHAPES[1], kt, align=True)
    assert _operator(device_example(ex2)).transpose() is not None
    assert _operator(d, symmetric=False).transpose() is not op


@pytest.mark.parametrize("shape,kt", CASES)
def test_load_native_and_native_function(O, shape, kt):
    """``load_native(name, defines).call(...)`` and ``NativeFunction(name, config)(...)``, the two
    ways the reference reaches a native op (``compile.py:49-125``, ``native_function.py:51-75``;
    its tests: ``tests/native/test_native_function.py:9-44``)."""
    from kernel_matmul_b200.compile import load_native
    from kernel_matmul_b200.configurations import (
        BilinearDerivativeConfiguration, MatmulAutotuneConfiguration, MatmulBwdConfiguration, MatmulSingleConfiguration,
    )
    from kernel_matmul_b200.native_function import NativeFunction

    ex = make_example(shape, kt)
    d = device_example(ex)
    args = (d.x1, d.x2, d.rhs, d.params, d.start, d.end)
    ref = O.matmul(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end)
    defines = MatmulSingleConfiguration(kt).make_config(args)
    assert rel_err(load_native("matmul", defines).call(*args), ref) <= TOL
    for cfg in (MatmulSingleConfiguration(kt), MatmulAutotuneConfiguration(kt)):
        native = NativeFunction("matmul", cfg, verbose=False)
        assert rel_err(native(*args), ref) <= TOL
        assert native.defines is not None and native.defines["BATCH_DIM"] == d.x1.dim() - 1
    og = torch.randn(ref.shape)
    g = NativeFunction("matmul_bwd", MatmulBwdConfiguration(kt))(*args, og.cuda())
    gref = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og)
    assert_grad_close(g, gref, O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, ex.params, ex.start, ex.end, og, absolute=True))
    left, right = torch.randn(*ex.x1.shape, 3), torch.randn(*ex.x2.shape, 3)
    bd = NativeFunction("bilinear_derivative", BilinearDerivativeConfiguration(kt))(
        d.x1, d.x2, left.cuda(), right.cuda(), d.params, d.start, d.end)
    bref = O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end)
    assert_grad_close(bd, bref, O.bilinear_derivative(kt, ex.x1, ex.x2, left, right, ex.params, ex.start, ex.end,
                                                      absolute=True))


def test_native_calls_reject_what_the_reference_rejects():
    """CPU tensors and wrong index dtypes raise the reference's messages
    (``native/common/entrypoint.h:3-14``) on a machine that has a GPU as well."""
    from kernel_matmul_b200 import ops

    ex = make_example(SHAPES[1], "rbf", square=True)
    d = device_example(ex)
    with pytest.raises(RuntimeError, match="x must be a CUDA tensor"):
        ops.matmul("rbf", ex.x1, d.x2, d.rhs, d.params, d.start, d.end)
    with pytest.raises(RuntimeError, match="x must be int32"):
        ops.matmul("rbf", d.x1, d.x2, d.rhs, d.params, d.start.long(), d.end)
    row = torch.zeros(4, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="x must be int32"):
        ops.index("rbf", d.x1, d.x2, d.params, d.start, d.end, (), row, row)


@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_training_step_through_the_operator(O, kt):
    """Two optimiser-style steps: ``loss = sum(w * (K(theta) @ rhs))`` -> ``backward`` -> update
    theta -> again.  The second forward sees the new parameters (nothing is cached across calls)."""
    ex = make_example(SHAPES[2], kt, square=True)
    d = device_example(ex)
    theta = d.params.clone().requires_grad_(True)
    w = torch.randn(*ex.params.shape[:-1], ex.x1.shape[-1], ex.rhs.shape[-1])
    for _ in range(2):
        d.params = theta
        out = _operator(d).matmul(d.rhs)
        loss = (out * w.cuda()).sum()
        (g,) = torch.autograd.grad(loss, theta)
        cpu_theta = theta.detach().cpu()
        gref = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, cpu_theta, ex.start, ex.end, w)
        scale = O.matmul_bwd(kt, ex.x1, ex.x2, ex.rhs, cpu_theta, ex.start, ex.end, w, absolute=True)
        assert_grad_close(g, gref, scale)
        assert rel_err(out, O.matmul(kt, ex.x1, ex.x2, ex.rhs, cpu_theta, ex.start, ex.end)) <= TOL
        theta = (theta.detach() * (1 + 0.05 * torch.rand_like(theta))).requires_grad_(True)
