"""Row-window / batch-sum product and the CG solve on the GPU against the fp64 oracle."""
import math

import pytest
import torch

from conftest import KERNEL_TYPES, make_params, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kt", KERNEL_TYPES)
@pytest.mark.parametrize("k", [1, 8, 11, 40])
def test_row_window_and_batch_sum(kt, k):
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    B, n = 5, 1000
    x = torch.sort(torch.rand(n) * 12)[0]
    params = make_params(kt, (B,))
    start, end = O.make_ranges(1.7, x)
    rhs = torch.randn(n, k)
    ref = O.matmul(kt, x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params, start.expand(B, -1), end.expand(B, -1))
    d = lambda t: t.cuda()  # noqa: E731
    xb = d(x).expand(B, n)
    args = (kt, xb, xb, d(rhs).expand(B, n, k), d(params), d(start).expand(B, -1), d(end).expand(B, -1))
    R = -(-n // 128)
    # window of row blocks, per batch
    out = ops.matmul_rows(*args, row_block_begin=2, row_block_count=3)
    assert out.shape == (B, 384, k)
    assert rel_err(out, ref[:, 256:640]) <= 1e-5
    # last (ragged) window
    out = ops.matmul_rows(*args, row_block_begin=R - 2)
    assert out.shape == (B, n - (R - 2) * 128, k)
    assert rel_err(out, ref[:, (R - 2) * 128:]) <= 1e-5
    # sum over the batch inside the kernel
    out = ops.matmul_rows(*args, sum_batches=True)
    assert out.shape == (n, k)
    assert rel_err(out, ref.sum(0)) <= 1e-5
    buf = torch.full((256, k), float("nan"), device="cuda")
    ops.matmul_rows(*args, row_block_begin=4, row_block_count=2, sum_batches=True, out=buf)
    assert rel_err(buf, ref.sum(0)[512:768]) <= 1e-5
    # the full window equals the plain product bit for bit
    assert torch.equal(ops.matmul_rows(*args), ops.matmul(*args))


def test_cg_solve_matches_dense_fp64():
    from kernel_matmul_b200 import ranges
    from kernel_matmul_b200.cg import ShardedOperator, conjugate_gradient
    from oracle import oracle as O

    n, k, B = 1500, 4, 6
    x = torch.sort(torch.rand(n) * 40)[0]
    params = torch.stack([torch.full((B,), 0.9), torch.rand(B), torch.full((B,), 1.0 / B)], dim=-1)
    params[0, 1] = 0.0  # component 0 is the plain RBF term
    y = torch.randn(n, k)
    xd = x.cuda()
    start, end = ranges.make_ranges(4.0, xd)
    op = ShardedOperator.from_kernel("spectral", xd, params.cuda(), start, end, sigma2=0.1)
    res = conjugate_gradient(op, y.cuda(), iterations=250)
    K = O.dense("spectral", x.expand(B, n), x.expand(B, n), params, start.cpu().expand(B, -1), end.cpu().expand(B, -1)).sum(0)
    ref = torch.linalg.solve(K + 0.1 * torch.eye(n, dtype=torch.float64), y.double())
    # fp32 CG on a system with condition number ~1e3: residual and solution to ~1e-4
    assert float(res.residual_norms[-1].max()) < 2e-4, res.residual_norms[-1]
    assert rel_err(res.solution, ref) <= 1e-3
    # one application of the operator against the oracle
    v = torch.randn(n, k)
    Av = op.apply(v.cuda())
    assert rel_err(Av, K @ v.double() + 0.1 * v.double()) <= 1e-5


@pytest.mark.parametrize("k", [1, 8, 11])
@pytest.mark.parametrize("shared_lengthscale", [True, False])
def test_spectral_mixture_sum_shared_envelope(k, shared_lengthscale):
    """Sum over spectral components sharing x, band and rhs: with one common lengthscale the
    kernel evaluates the envelope once per entry (shared-envelope walk), otherwise it adds the
    components one by one; both against the oracle."""
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    B, n = 37, 900
    x = torch.sort(torch.rand(n) * 15)[0]
    ell = torch.full((B,), 0.7) if shared_lengthscale else 0.5 + torch.rand(B)
    params = torch.stack([ell, torch.rand(B) * 1.5, torch.randn(B)], dim=-1)  # signed scales
    start, end = O.make_ranges(2.8, x)
    rhs = torch.randn(n, k)
    ref = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params,
                   start.expand(B, -1), end.expand(B, -1)).sum(0)
    xd = x.cuda().expand(B, n)
    out = ops.matmul_rows("spectral", xd, xd, rhs.cuda().expand(B, n, k), params.cuda(),
                          start.cuda().expand(B, -1), end.cuda().expand(B, -1), sum_batches=True)
    # the components cancel partly (signed scales): compare against the sum of magnitudes
    scale = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params,
                     start.expand(B, -1), end.expand(B, -1)).abs().sum(0).max()
    assert float((out.cpu().double() - ref).abs().max() / scale) <= 1e-5


def test_host_buffers_step_matches_the_ops():
    """kernel_matmul_b200.host: overlapped copies + product + gradient == the plain ops."""
    from kernel_matmul_b200 import host, ops, ranges

    dev = torch.device("cuda:0")
    B, n, k = 3, 3000, 16
    x = torch.sort(torch.rand(n) * 50)[0].pin_memory()
    rhs = torch.randn(n, k).pin_memory()
    params = torch.stack([1 + torch.rand(B), 0.5 + 0.5 * torch.rand(B), 1 + torch.rand(B)], dim=-1).pin_memory()
    og = torch.randn(B, n, k).pin_memory()
    out = torch.empty(B, n, k).pin_memory()
    grad = torch.empty(B, 3).pin_memory()
    streams = host.HostStreams(dev)
    band = lambda dx: ranges.make_ranges(3.0, dx)  # noqa: E731
    for _ in range(2):  # twice: buffers and streams are reused
        host.matmul_and_grad_from_host("spectral", x, rhs, params, og, band, out, grad, streams)
        torch.cuda.current_stream(dev).synchronize()
        dx = x.to(dev)
        start, end = band(dx)
        ref = ops.matmul("spectral", dx.expand(B, -1), dx.expand(B, -1), rhs.to(dev).expand(B, -1, -1), params.to(dev), start, end)
        gref = ops.matmul_bwd("spectral", dx.expand(B, -1), dx.expand(B, -1), rhs.to(dev).expand(B, -1, -1), params.to(dev),
                              start, end, og.to(dev))
        assert torch.equal(out, ref.cpu())
        assert torch.equal(grad, gref.cpu())
        out.zero_()
        grad.zero_()


@pytest.mark.parametrize("kt", ["rbf", "spectral"])
def test_marginal_likelihood_gradient_matches_dense_fp64(kt):
    """gp.mll_gradient (batched CG + one bilinear_derivative) against the same estimator evaluated
    with dense fp64 algebra and autograd on the band-masked kernel matrix."""
    from kernel_matmul_b200 import gp
    from oracle import dense_reference as D
    from oracle import oracle as O

    n, t, sigma2, cutoff = 1200, 12, 0.5, 8.0  # cutoff >= 4 l: the truncated matrix stays positive definite
    x = torch.sort(torch.rand(n) * 120)[0]
    y = torch.randn(n)
    params = make_params(kt, ())
    probes = torch.randint(0, 2, (n, t)).float() * 2 - 1
    out = gp.mll_gradient(kt, x.cuda(), params.cuda(), sigma2, y.cuda(), cutoff=cutoff, probes=probes.cuda(),
                          cg_iterations=300, path="tc")
    assert float(out.residual_norms[-1].max()) < 1e-4

    start, end = O.make_ranges(cutoff, x)
    theta = params.double().clone().requires_grad_(True)
    K = D.masked_kernel(kt, x, x, theta, start, end)
    Khat = K + sigma2 * torch.eye(n, dtype=torch.float64)
    V = torch.linalg.solve(Khat.detach(), torch.cat([y.reshape(n, 1), probes], dim=-1).double())
    # the CG solves (fp32, residual 1e-4) against the exact ones
    u, w = out.solve.cpu().double(), out.probe_solves.cpu().double()
    assert float((u - V[:, 0]).norm() / V[:, 0].norm()) < 1e-2
    assert float((w - V[:, 1:]).norm() / V[:, 1:].norm()) < 1e-2
    # the estimator as a scalar whose theta-gradient is the wanted vector (u, w, z held fixed):
    # evaluated with the driver's own solves this pins the assembly of the gradient call
    est = -0.5 * (u @ K @ u) + (0.5 / t) * (w * (K @ probes.double())).sum()
    (g_ref,) = torch.autograd.grad(est, theta, retain_graph=True)
    g_sigma_ref = -0.5 * (u @ u) + (0.5 / t) * (w * probes.double()).sum()
    g = out.grad_params.cpu().double()
    assert torch.allclose(g, g_ref, rtol=1e-4, atol=1e-4 * float(g_ref.abs().max())), (g, g_ref)
    assert abs(float(out.grad_sigma2) - float(g_sigma_ref)) <= 1e-4 * abs(float(g_sigma_ref))
    assert abs(float(out.inv_quad) - float(y.double() @ u)) <= 1e-4 * abs(float(y.double() @ u))
    # log det: the Lanczos estimate from the CG coefficients against the same estimator with the exact
    # matrix logarithm, (1 / t) sum_i z_i^T log(Khat) z_i, and that against the true log-determinant
    evals, evecs = torch.linalg.eigh(Khat.detach())
    proj = evecs.T @ probes.double()
    exact_estimator = float(((proj ** 2) * torch.log(evals)[:, None]).sum() / t)
    assert abs(float(out.logdet) - exact_estimator) <= 2e-3 * abs(exact_estimator), (float(out.logdet), exact_estimator)
    true_logdet = float(torch.log(evals).sum())
    assert abs(exact_estimator - true_logdet) <= 0.1 * abs(true_logdet)  # 12 probes: a noisy but unbiased estimate
    nll = 0.5 * float(y.double() @ V[:, 0]) + 0.5 * float(out.logdet) + 0.5 * n * math.log(2 * math.pi)
    assert abs(float(out.nll) - nll) <= 1e-3 * abs(nll)
    # and with exact solves the same estimator agrees to the accuracy of the CG solves
    u, w = V[:, 0], V[:, 1:]
    est = -0.5 * (u @ K @ u) + (0.5 / t) * (w * (K @ probes.double())).sum()
    (g_exact,) = torch.autograd.grad(est, theta)
    assert torch.allclose(g, g_exact, rtol=5e-2, atol=5e-2 * float(g_exact.abs().max())), (g, g_exact)


@pytest.fixture(params=["both contractions on the tensor cores", "second contraction on the FMA pipe",
                        "second contraction on the FMA pipe, one row group", "two row blocks per CTA",
                        "second contraction on the warp-level tensor path"])
def sum_kernel_variant(request, monkeypatch):
    """The five forms of the tensor-core batch sum (the library reads the switches at every launch)."""
    variant = "3" if request.param.startswith("two row blocks") else ("1" if request.param.startswith("second") else "2")
    monkeypatch.setenv("KM_SUM_TC_VARIANT", variant)
    monkeypatch.setenv("KM_SUM_TC_WARP_MMA", "1" if request.param.endswith("warp-level tensor path") else "0")
    if request.param.endswith("one row group"):
        monkeypatch.setenv("KM_SUM_TC_GROUPS", "1")
    return request.param


def test_phase_entry_points_validate_their_arguments():
    """The C entry points of the phase workspace refuse what they cannot do, with a message and
    without launching anything."""
    import ctypes

    from kernel_matmul_b200 import ops
    from kernel_matmul_b200._lib import lib

    B, n = 4, 300
    x = torch.sort(torch.rand(n) * 30)[0].cuda()
    params = torch.stack([torch.full((B,), 1.3), torch.rand(B), torch.full((B,), 0.25)], dim=-1).cuda()
    kb = ops._km_batch((B,))
    xe = x.expand(B, n)
    need = lib.km_sum_phases_workspace_bytes(kb, n, n)
    assert need == -(-n // 64) * 8 * 512 + -(-(n * 8 * 8) // 256) * 256  # psi tiles of 8 padded components, phi rows
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    ws = ws[(-ws.data_ptr()) % 256:]
    args = (kb, n, n, ops._view(xe, 1), ops._view(xe, 1), ops._view(params, 1))
    # too small, misaligned, null
    assert lib.km_sum_phases_prepare_f32(*args, 0, -1, 0, -1, ctypes.c_void_p(ws.data_ptr()), need - 1, None) == 3
    assert b"workspace" in lib.km_last_error()
    assert lib.km_sum_phases_prepare_f32(*args, 0, -1, 0, -1, ctypes.c_void_p(ws.data_ptr() + 16), need, None) == 3
    assert lib.km_sum_phases_prepare_f32(*args, 0, -1, 0, -1, None, need, None) == 3
    # ranges outside the operator
    assert lib.km_sum_phases_prepare_f32(*args, 0, n + 1, 0, -1, ctypes.c_void_p(ws.data_ptr()), need, None) == 1
    assert lib.km_sum_phases_prepare_f32(*args, 10, 5, 0, -1, ctypes.c_void_p(ws.data_ptr()), need, None) == 1
    assert b"rows" in lib.km_last_error()
    # inputs that differ between the components
    xb = torch.rand(B, n).cuda()
    assert lib.km_sum_phases_prepare_f32(kb, n, n, ops._view(xb, 1), ops._view(xe, 1), ops._view(params, 1), 0, -1, 0, -1,
                                         ctypes.c_void_p(ws.data_ptr()), need, None) == 2
    assert b"shared by all components" in lib.km_last_error()
    # more components than the sum kernel takes: no workspace size
    assert lib.km_sum_phases_workspace_bytes(ops._km_batch((2000,)), n, n) == 0
    # a good call
    assert lib.km_sum_phases_prepare_f32(*args, 0, -1, 0, -1, ctypes.c_void_p(ws.data_ptr()), need, None) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("contraction", ["FMA pipe", "warp-level tensor path"])
@pytest.mark.parametrize("B,k", [(2, 1), (7, 8), (64, 8), (33, 11), (64, 16), (100, 8), (130, 3)])
def test_batch_sum_with_precomputed_phases(B, k, contraction, monkeypatch):
    """The same sum with the per-point phase vectors written once per operator
    (km_matmul_sum_ph.cu: ``ops.prepare_sum_phases`` + ``matmul_rows(..., phases=...)``) against the
    fp64 oracle: large input offsets (the phases are taken at the points themselves, in fp64),
    row windows bit-identical to the full product, reuse of the workspace for several right-hand
    sides, and the fallback for different lengthscales."""
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    monkeypatch.setenv("KM_SUM_TC_WARP_MMA", "1" if contraction.startswith("warp") else "0")
    n = 1400  # ragged last row block
    x = torch.sort(torch.rand(n) * 300 + 50000)[0]
    params = torch.stack([torch.full((B,), 1.3), torch.rand(B) * 1.5, (torch.rand(B) + 0.5) / B], dim=-1)
    params[0, 1] = 0.0
    start, end = O.make_ranges(5.0, x)
    d = lambda t: t.cuda()  # noqa: E731
    xd, pd = d(x), d(params)
    ws = ops.prepare_sum_phases("spectral", xd, xd, pd)
    assert ws is not None and ws.data_ptr() % 256 == 0
    for trial in range(2):  # one workspace, several right-hand sides
        rhs = torch.randn(n, k)
        ref = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params, start.expand(B, -1),
                       end.expand(B, -1)).sum(0)
        args = ("spectral", xd.expand(B, n), xd.expand(B, n), d(rhs).expand(B, n, k), pd, d(start).expand(B, -1),
                d(end).expand(B, -1))
        out = ops.matmul_rows(*args, sum_batches=True, phases=ws)
        assert out.shape == (n, k) and bool(torch.isfinite(out).all())
        assert rel_err(out, ref) <= 1e-5
        win = ops.matmul_rows(*args, sum_batches=True, row_block_begin=3, row_block_count=5, phases=ws)
        assert torch.equal(win, out[384:1024])
    # images written for one window's rows and columns only (a rank of a row-sharded solve)
    ws_part = ops.prepare_sum_phases("spectral", xd, xd, pd, rows=(384, 1024), cols=(int(start[3:8].min()), int(end[3:8].max())))
    win = ops.matmul_rows(*args, sum_batches=True, row_block_begin=3, row_block_count=5, phases=ws_part)
    assert torch.equal(win, out[384:1024])
    # different lengthscales: the FMA-pipe kernel computes the sum (the tensor-core CTAs leave at once)
    params2 = params.clone()
    params2[-1, 0] = 1.1
    ref2 = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params2, start.expand(B, -1),
                    end.expand(B, -1)).sum(0)
    out2 = ops.matmul_rows(args[0], args[1], args[2], args[3], d(params2), args[5], args[6], sum_batches=True, phases=ws)
    assert rel_err(out2, ref2) <= 1e-5
    ops.check()
    # other kernels and single components have no phase workspace
    assert ops.prepare_sum_phases("rbf", xd, xd, torch.rand(B, 2).cuda()) is None
    assert ops.prepare_sum_phases("spectral", xd, xd, pd[0]) is None


@pytest.mark.parametrize("B,k", [(2, 1), (7, 8), (64, 8), (33, 11), (64, 16), (100, 8), (130, 3)])
def test_batch_sum_on_tensor_cores(B, k, sum_kernel_variant):
    """Spectral components with one lengthscale: the batch sum as a tensor-core dot product of
    per-point phase vectors (km_matmul_sum_tc.cu) against the fp64 oracle, incl. row windows."""
    from kernel_matmul_b200 import ops
    from oracle import oracle as O

    n = 1400  # ragged last row block
    x = torch.sort(torch.rand(n) * 300 + 5000)[0]  # large offsets: phases are taken relative to the row block
    params = torch.stack([torch.full((B,), 1.3), torch.rand(B) * 1.5, (torch.rand(B) + 0.5) / B], dim=-1)
    params[0, 1] = 0.0
    start, end = O.make_ranges(5.0, x)
    rhs = torch.randn(n, k)
    ref = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params, start.expand(B, -1),
                   end.expand(B, -1)).sum(0)
    d = lambda t: t.cuda()  # noqa: E731
    args = ("spectral", d(x).expand(B, n), d(x).expand(B, n), d(rhs).expand(B, n, k), d(params), d(start).expand(B, -1),
            d(end).expand(B, -1))
    out = ops.matmul_rows(*args, sum_batches=True)
    assert out.shape == (n, k) and bool(torch.isfinite(out).all())
    assert rel_err(out, ref) <= 1e-5
    win = ops.matmul_rows(*args, sum_batches=True, row_block_begin=3, row_block_count=5)
    assert rel_err(win, ref[384:1024]) <= 1e-5
    assert torch.equal(win, out[384:1024])
    # different lengthscales: the FMA-pipe kernel computes the sum (the tensor-core CTAs leave at once)
    params2 = params.clone()
    params2[-1, 0] = 1.1
    ref2 = O.matmul("spectral", x.expand(B, n), x.expand(B, n), rhs.expand(B, n, k), params2, start.expand(B, -1),
                    end.expand(B, -1)).sum(0)
    out2 = ops.matmul_rows(args[0], args[1], args[2], args[3], d(params2), args[5], args[6], sum_batches=True)
    assert rel_err(out2, ref2) <= 1e-5
