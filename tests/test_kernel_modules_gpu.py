"""The kernel modules (``kernel_matmul_b200/kernels.py``): learnable parameters -> band -> operator
-> product -> gradients back to the raw parameters, the training-step path of the reference's
GPyTorch kernels (kernel_matmul/gpytorch/base.py:47-84, examples/fit_sine.py:54-61), checked
against the fp64 oracle and -- with PyTorch's synchronisation debug mode -- for the absence of
any host synchronisation."""
import math

import pytest
import torch

from conftest import KERNEL_TYPES, assert_grad_close, rel_err

pytestmark = pytest.mark.gpu

VALUES = {
    "rbf": dict(lengthscale=[0.9, 1.4], outputscale=[1.3, 0.7]),
    "spectral": dict(lengthscale=[0.9, 1.4], frequency=[0.6, 0.8], outputscale=[1.3, 0.7]),
    "locally_periodic": dict(lengthscale_rbf=[0.9, 1.4], lengthscale_periodic=[1.1, 1.6], period_length=[1.2, 1.9],
                             outputscale=[1.3, 0.7]),
}


def _module(kt, **kw):
    from kernel_matmul_b200 import kernels

    cls = {"rbf": kernels.RBFKernelMatmulModule, "spectral": kernels.SpectralKernelMatmulModule,
           "locally_periodic": kernels.LocallyPeriodicKernelMatmulModule}[kt]
    m = cls(batch_shape=(2,), **kw).cuda()
    return m.initialize(**{k: torch.tensor(v) for k, v in VALUES[kt].items()})


@pytest.mark.parametrize("cutoff_kw", [dict(cutoff=3.0), dict(epsilon=1e-4)], ids=["fixed", "epsilon"])
@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_training_step_without_host_synchronisation(kt, cutoff_kw):
    from oracle import oracle as O

    n, k = 3000, 16
    x = torch.sort(torch.rand(n) * 100)[0]
    rhs, w = torch.randn(n, k), torch.randn(2, n, k)
    xd, rhsd, wd = x.cuda().unsqueeze(-1), rhs.cuda(), w.cuda()
    module = _module(kt, **cutoff_kw)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")  # any synchronising call below raises
    try:
        op = module(xd, xd)
        out = op.matmul(rhsd)
        loss = (out * wd).sum()
        loss.backward()
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()

    params = module.params().detach().cpu()
    if "epsilon" in cutoff_kw:
        largest = module.value("lengthscale_rbf" if kt == "locally_periodic" else "lengthscale").detach().max().cpu()
        z = math.sqrt(2.0) * torch.special.erfinv(torch.tensor(1.0 - 1e-4, dtype=torch.float64)).item()
        cutoff = float((largest.double() * z).float())  # the reference's host value (gpytorch/base.py:59-64)
    else:
        cutoff = 3.0
    start, end = O.make_ranges(cutoff, x)
    assert torch.equal(op._start.cpu()[0], start) and torch.equal(op._end.cpu()[0], end)  # the band, bit for bit
    xb = x.expand(2, n)
    ref = O.matmul(kt, xb, xb, rhs.expand(2, n, k), params, start.expand(2, -1), end.expand(2, -1))
    assert rel_err(out, ref) <= 1e-5
    g = O.matmul_bwd(kt, xb, xb, rhs.expand(2, n, k), params, start.expand(2, -1), end.expand(2, -1), w)
    gs = O.matmul_bwd(kt, xb, xb, rhs.expand(2, n, k), params, start.expand(2, -1), end.expand(2, -1), w, absolute=True)
    for i, name in enumerate(module._PARAMS):
        raw = getattr(module, f"raw_{name}")
        chain = torch.sigmoid(raw.detach().double().cpu())  # d softplus(raw) / d raw
        assert raw.grad is not None and raw.grad.shape == (2,)
        assert_grad_close(raw.grad, g[:, i] * chain, gs[:, i] * chain)


@pytest.mark.parametrize("kt", KERNEL_TYPES)
def test_rectangular_inputs_and_equal_values_in_different_tensors(kt):
    from oracle import oracle as O

    x1 = torch.sort(torch.rand(700) * 30)[0]
    x2 = torch.sort(torch.rand(900) * 30)[0]
    module = _module(kt, cutoff=2.5)
    params = module.params().detach().cpu()
    op = module(x1.cuda().unsqueeze(-1), x2.cuda().unsqueeze(-1))
    assert tuple(op.shape) == (2, 700, 900)
    start, end = O.make_ranges(2.5, x1, x2, align=True)
    v = torch.randn(900, 3)
    ref = O.matmul(kt, x1.expand(2, -1), x2.expand(2, -1), v.expand(2, -1, -1), params, start.expand(2, -1), end.expand(2, -1))
    assert rel_err(op.matmul(v.cuda()), ref) <= 1e-5
    # the transpose of the aligned pattern
    u = torch.randn(700, 3)
    dense = O.dense(kt, x1.expand(2, -1), x2.expand(2, -1), params, start.expand(2, -1), end.expand(2, -1))
    assert rel_err(op.transpose().matmul(u.cuda()), dense.transpose(-1, -2) @ u.double()) <= 1e-5
    # two tensors with the same values are recognised as one input set (by comparing them)
    a, b = x1.cuda().unsqueeze(-1), x1.clone().cuda().unsqueeze(-1)
    sym = module(a, b)
    assert sym.transpose() is sym
    s2, e2 = O.make_ranges(2.5, x1)
    assert torch.equal(sym._start.cpu()[0], s2) and torch.equal(sym._end.cpu()[0], e2)


def test_cutoff_and_epsilon_are_exclusive():
    from kernel_matmul_b200 import kernels

    with pytest.raises(ValueError, match="Cannot have both"):
        kernels.RBFKernelMatmulModule(cutoff=1.0, epsilon=1e-3)
