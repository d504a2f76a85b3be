"""What happens when a hand-off wait inside a tensor-core kernel runs out.

Every such wait has a poll limit.  The tests shorten it from the host
(``km_selftest_set_wait_polls(0)``: a wait that is not already complete at its first test gives
up at once), so the kernels stop at their first hand-off -- nothing faults, traps or hangs.  A
kernel that gave up must: return (the launch completes), set the status word, write NaN results,
and leave the device usable, which the correct re-run after restoring the limit shows.
"""
import ctypes

import pytest
import torch

from conftest import make_params, rel_err

pytestmark = pytest.mark.gpu


def test_a_wait_that_nobody_answers_gives_up_with_a_status():
    from kernel_matmul_b200._lib import lib

    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.km_selftest_bounded_wait(4096, ctypes.c_void_p(status.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert int(status) == 1  # gave up, reported, returned
    assert lib.km_selftest_bounded_wait(1 << 20, ctypes.c_void_p(status.data_ptr()), stream) == 1  # limit too large: refused


@pytest.fixture
def short_waits():
    from kernel_matmul_b200._lib import lib

    assert lib.km_selftest_set_wait_polls(0) == 0
    try:
        yield
    finally:
        assert lib.km_selftest_set_wait_polls(-1) == 0


def _problem(kt, k, B=3, n=2000):
    from oracle import oracle as O

    x = torch.sort(torch.rand(n) * 30)[0]
    params = make_params(kt, (B,))
    start, end = O.make_ranges(2.5, x)
    rhs = torch.randn(n, k)
    cpu = (x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params, start.expand(B, -1), end.expand(B, -1))
    dev = (x.cuda().expand(B, n), x.cuda().expand(B, n), rhs.cuda().expand(B, n, k), params.cuda(),
           start.cuda().expand(B, -1), end.cuda().expand(B, -1))
    return cpu, dev


@pytest.mark.parametrize("kt,k", [("rbf", 16), ("spectral", 40), ("locally_periodic", 128)])
def test_product_that_gives_up_reports_and_poisons_its_output(kt, k, short_waits):
    from kernel_matmul_b200 import ops
    from kernel_matmul_b200._lib import lib
    from oracle import oracle as O

    cpu, dev = _problem(kt, k)
    out = ops.matmul(kt, *dev, path="tc")
    torch.cuda.synchronize()  # the launch ends by itself
    assert bool(torch.isnan(out).all())  # every CTA stopped at its first hand-off
    with pytest.raises(ops.KernelGaveUpError, match="gave up"):
        ops.check()
    ops.check()  # reported once
    # the next op call notices a failed launch without being asked
    out = ops.matmul(kt, *dev, path="tc")
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelGaveUpError):
        ops.dense(kt, dev[0][0, :256], dev[1][0, :256], dev[3][0], dev[4][0, :2], dev[5][0, :2])
    # with the normal limit the same call is correct: the device and the library are fine
    assert lib.km_selftest_set_wait_polls(-1) == 0
    out = ops.matmul(kt, *dev, path="tc")
    ops.check()
    assert rel_err(out, O.matmul(kt, *cpu)) <= 1e-5


@pytest.mark.parametrize("kt,k", [("rbf", 8), ("spectral", 24), ("locally_periodic", 64)])
def test_gradient_that_gives_up_reports_and_is_nan(kt, k, short_waits):
    from kernel_matmul_b200 import ops
    from kernel_matmul_b200._lib import lib
    from oracle import oracle as O
    from conftest import assert_grad_close

    cpu, dev = _problem(kt, k)
    B, n = cpu[0].shape
    left = torch.randn(B, n, k)
    g = ops.bilinear_derivative(kt, dev[0], dev[1], left.cuda(), dev[2], dev[3], dev[4], dev[5], path="tc")
    torch.cuda.synchronize()
    assert bool(torch.isnan(g).all())
    assert ops.tc_status(g) == 1 and ops.tc_status(g) == 0
    assert lib.km_selftest_set_wait_polls(-1) == 0
    g = ops.bilinear_derivative(kt, dev[0], dev[1], left.cuda(), dev[2], dev[3], dev[4], dev[5], path="tc")
    ops.check()
    ref = O.bilinear_derivative(kt, cpu[0], cpu[1], left, cpu[2], cpu[3], cpu[4], cpu[5])
    scale = O.bilinear_derivative(kt, cpu[0], cpu[1], left, cpu[2], cpu[3], cpu[4], cpu[5], absolute=True)
    assert_grad_close(g, ref, scale)


def test_batch_sum_that_gives_up_writes_nan_and_the_solver_notices(short_waits):
    from kernel_matmul_b200 import ops, ranges
    from kernel_matmul_b200._lib import lib
    from kernel_matmul_b200.cg import CGSolver, ShardedOperator

    B, n, k = 16, 3000, 8
    x = torch.sort(torch.rand(n) * 60)[0].cuda()
    params = torch.stack([torch.full((B,), 1.2), torch.rand(B), torch.full((B,), 1.0 / B)], dim=-1).cuda()
    start, end = ranges.make_ranges(5.0, x)
    rhs = torch.randn(n, k).cuda()
    args = ("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params, start.expand(B, -1), end.expand(B, -1))
    out = ops.matmul_rows(*args, sum_batches=True)
    torch.cuda.synchronize()
    assert bool(torch.isnan(out).all())
    # the form with precomputed phase vectors (bulk copies in flight when its waits run out)
    ws = ops.prepare_sum_phases("spectral", x, x, params)
    out = ops.matmul_rows(*args, sum_batches=True, phases=ws)
    torch.cuda.synchronize()
    assert bool(torch.isnan(out).all())
    solver = CGSolver(ShardedOperator.from_kernel("spectral", x, params, start, end, 0.1), rhs)
    solver.step()
    with pytest.raises(RuntimeError, match="non-finite residual"):
        solver.check_finite()
    assert lib.km_selftest_set_wait_polls(-1) == 0
    out = ops.matmul_rows(*args, sum_batches=True)
    out_ph = ops.matmul_rows(*args, sum_batches=True, phases=ws)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out).all()) and bool(torch.isfinite(out_ph).all())
