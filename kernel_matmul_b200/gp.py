"""Gradient of the Gaussian-process marginal likelihood through the banded kernel operator.

The end-to-end training step that the ops exist for (the reference reaches it through GPyTorch:
``ExactMarginalLogLikelihood`` -> ``inv_quad_logdet`` of ``KernelMatmulLinearOperator``,
examples/fit_sine.py:54-61).  For ``Khat = K(x, x; theta) + sigma^2 I`` and targets ``y``

    NLL(theta, sigma^2) = 1/2 y^T Khat^-1 y + 1/2 log det Khat + n/2 log 2 pi
    d NLL / d theta  = -1/2 u^T (dK/dtheta) u + 1/2 tr(Khat^-1 dK/dtheta),     u = Khat^-1 y
    d NLL / d sigma2 = -1/2 u^T u + 1/2 tr(Khat^-1)

with the traces estimated from ``t`` probe vectors ``z_i`` (Hutchinson):
``tr(Khat^-1 A) ~ 1/t sum_i (Khat^-1 z_i)^T A z_i``.  One batched CG solve with the right-hand
sides ``[y, z_1 .. z_t]`` (``cg.conjugate_gradient`` on the banded product) gives ``u`` and
``w_i = Khat^-1 z_i``; ONE ``bilinear_derivative`` call with ``left = [-u/2, w_1/2t ..]`` and
``right = [u, z_1 ..]`` (``1 + t`` columns: the width the tensor-core gradient kernel is built
for) gives every ``d / d theta``.

The value of ``log det Khat`` comes from the same solve (stochastic Lanczos quadrature, what
``linear_operator``'s ``inv_quad_logdet`` does): the step lengths ``alpha_j`` and direction updates
``beta_j`` of the CG run on ``z_i`` are the entries of the Lanczos tridiagonal ``T_i`` of ``Khat``
started at ``z_i`` (``T[j,j] = 1/alpha_j + beta_{j-1}/alpha_{j-1}``, ``T[j,j+1] = sqrt(beta_j)/alpha_j``),
and ``z^T log(Khat) z ~ |z|^2 e_1^T log(T) e_1``; the mean over the probes estimates the trace.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import Tensor

from . import ops, ranges
from .cg import ShardedOperator, conjugate_gradient


def lanczos_log_quadratic_forms(alphas: Tensor, betas: Tensor, residual_norms: Tensor, z_norm2: Tensor,
                                converged: float = 1e-7) -> Tensor:
    """``z_c^T log(A) z_c`` for every column ``c`` of a batched CG run ``A V = Z`` from ``x0 = 0``.

    ``alphas``, ``betas`` ``(m, k)`` and ``residual_norms`` ``(m + 1, k)`` are what the solve recorded,
    ``z_norm2 (k,)`` the squared norms of the right-hand sides.  A column's recurrence is cut where
    its relative residual falls below ``converged`` (its later coefficients are rounding noise).
    Runs in fp64 on the CPU: the tridiagonals are ``m x m`` with ``m`` the iteration count."""
    a = alphas.detach().double().cpu()
    b = betas.detach().double().cpu()
    res = residual_norms.detach().double().cpu()
    z2 = z_norm2.detach().double().cpu()
    m, k = a.shape
    out = torch.zeros(k, dtype=torch.float64)
    for c in range(k):
        steps = m
        for j in range(1, m + 1):
            if not bool(torch.isfinite(res[j, c])) or res[j, c] <= converged:
                steps = j
                break
        steps = max(1, steps)
        T = torch.zeros(steps, steps, dtype=torch.float64)
        for j in range(steps):
            T[j, j] = 1.0 / a[j, c] + (b[j - 1, c] / a[j - 1, c] if j > 0 else 0.0)
            if j + 1 < steps:
                T[j, j + 1] = T[j + 1, j] = torch.sqrt(b[j, c]) / a[j, c]
        evals, evecs = torch.linalg.eigh(T)
        out[c] = z2[c] * (evecs[0] ** 2 * torch.log(evals.clamp_min(1e-300))).sum()
    return out


@dataclass
class MllGradient:
    grad_params: Tensor      # (P,) d NLL / d theta
    grad_sigma2: Tensor      # ()   d NLL / d sigma^2
    inv_quad: Tensor         # ()   y^T Khat^-1 y
    logdet: Tensor           # ()   log det Khat (stochastic Lanczos quadrature over the probes)
    nll: Tensor              # ()   1/2 inv_quad + 1/2 logdet + n/2 log 2 pi
    solve: Tensor            # (n,) u = Khat^-1 y
    probe_solves: Tensor     # (n, t) w_i = Khat^-1 z_i
    residual_norms: Tensor   # (iterations + 1, 1 + t) relative CG residuals


def mll_gradient(kernel_type: str, x: Tensor, params: Tensor, sigma2: float, y: Tensor, *, cutoff: float | None,
                 probes: Tensor | None = None, num_probes: int = 15, cg_iterations: int = 100, group=None,
                 path: str = "auto") -> MllGradient:
    """Gradient of the negative log marginal likelihood wrt ``params`` (``(P,)``) and ``sigma2``.

    ``x (n,)`` sorted inputs and ``y (n,)`` targets on a CUDA device; ``probes (n, t)`` fixes the
    trace probes (default: ``num_probes`` Rademacher vectors from torch's current generator).
    With an initialised process group the CG products are sharded by rows over its ranks.
    """
    n = x.shape[-1]
    start, end = ranges.make_ranges(cutoff, x)
    if probes is None:
        probes = torch.randint(0, 2, (n, num_probes), device=x.device, dtype=torch.float32) * 2.0 - 1.0
    t = probes.shape[-1]
    rhs = torch.cat([y.reshape(n, 1), probes], dim=-1).contiguous()
    op = ShardedOperator.from_kernel(kernel_type, x, params, start, end, sigma2, group=group)
    res = conjugate_gradient(op, rhs, cg_iterations)
    v = res.solution
    u, w = v[:, 0], v[:, 1:]
    scale = torch.cat([torch.full((1,), -0.5, device=x.device), torch.full((t,), 0.5 / t, device=x.device)])
    left = (v * scale).contiguous()
    right = torch.cat([u.reshape(n, 1), probes], dim=-1).contiguous()
    grad_params = ops.bilinear_derivative(kernel_type, x, x, left, right, params, start, end, path=path)
    grad_sigma2 = -0.5 * (u * u).sum() + (0.5 / t) * (w * probes).sum()
    inv_quad = (y * u).sum()
    # log det Khat from the Lanczos coefficients of the probe columns (columns 1 .. t of the solve)
    quad = lanczos_log_quadratic_forms(res.alphas[:, 1:], res.betas[:, 1:], res.residual_norms[:, 1:],
                                       (probes * probes).sum(dim=0))
    logdet = quad.mean().to(device=x.device, dtype=torch.float32)
    nll = 0.5 * inv_quad + 0.5 * logdet + 0.5 * n * math.log(2.0 * math.pi)
    return MllGradient(grad_params, grad_sigma2, inv_quad, logdet, nll, u, w, res.residual_norms)
