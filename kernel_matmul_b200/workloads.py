"""Seeded synthetic inputs of the benchmark configurations.

Everything is drawn on the CPU with ``torch.manual_seed(0)`` in a fixed order and as fp32, so
that a CPU checker and the GPU see identical bits; tensors are returned on the CPU and moved
by the caller.  Expanded (shared) operands are returned as stride-0 views.  The reference has
no datasets: its own tests and example draw the same kind of data
(tests/conftest.py:89-105, examples/matmul.py:61-82).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import Tensor


@dataclass
class Workload:
    name: str
    kernel_type: str
    x: Tensor  # (n,) shared by all batches
    params: Tensor  # (B, P) or (P,)
    cutoffs: list[float | None]  # one per batch row of params (a single entry if shared)
    rhs: Tensor | None = None
    extra: dict = field(default_factory=dict)

    @property
    def n(self) -> int:
        return self.x.shape[-1]


def rbf_small(n: int = 4096) -> Workload:
    """RBF forward, batch 1: x sorted U[0,40], lengthscale 0.5, outputscale 1, cutoff 4 l, k = 1."""
    torch.manual_seed(0)
    x = torch.sort(torch.rand(n) * 40)[0]
    rhs = torch.randn(n, 1)
    return Workload("rbf_n4096_k1", "rbf", x, torch.tensor([0.5, 1.0]), [2.0], rhs)


def spectral_mixture(n: int = 65536, components: int = 16, k: int = 16, span: float = 500.0) -> Workload:
    """Spectral mixture, `components` batches sharing x and rhs: l ~ LogUniform[0.5, 5],
    f ~ U[0, 2], outputscale 1, cutoff 4 l per component; out_grad for matmul_bwd."""
    torch.manual_seed(0)
    x = torch.sort(torch.rand(n) * span)[0]
    ell = torch.exp(torch.rand(components) * math.log(10.0) + math.log(0.5))
    f = torch.rand(components) * 2
    s = torch.ones(components)
    rhs = torch.randn(n, k)
    out_grad = torch.randn(components, n, k)
    params = torch.stack([ell, f, s], dim=-1)
    return Workload(
        f"spectral_b{components}_n{n}_k{k}", "spectral", x, params, [4.0 * float(v) for v in ell], rhs,
        {"out_grad": out_grad},
    )


def locally_periodic_bilinear(n: int = 262144, batch: int = 4, k: int = 32, span: float = 2000.0) -> Workload:
    """Locally periodic bilinear_derivative: l_rbf 3, l_per 0.8, period 1.3, cutoff 12."""
    torch.manual_seed(0)
    x = torch.sort(torch.rand(n) * span)[0]
    lhs = torch.randn(batch, n, k)
    rhs = torch.randn(batch, n, k)
    params = torch.tensor([3.0, 0.8, 1.3, 1.0]).expand(batch, 4)
    return Workload(f"locally_periodic_b{batch}_n{n}_k{k}", "locally_periodic", x, params, [12.0], rhs, {"lhs": lhs})


def rbf_unbanded(n: int = 131072, k: int = 128, lookups: int = 1 << 24) -> Workload:
    """Unbanded RBF (full K), lengthscale 2, plus `lookups` random (row, col) gathers."""
    torch.manual_seed(0)
    x = torch.rand(n) * 100
    rhs = torch.randn(n, k)
    row = torch.randint(0, n, (lookups,), dtype=torch.int32)
    col = torch.randint(0, n, (lookups,), dtype=torch.int32)
    return Workload(f"rbf_unbanded_n{n}_k{k}", "rbf", x, torch.tensor([2.0, 1.0]), [None], rhs, {"row": row, "col": col})


def cg_sum_kernel(n: int = 1 << 22, components: int = 64, k: int = 8, span: float = 20000.0) -> Workload:
    """(K + sigma^2 I) v = y with K the sum of `components` spectral kernels sharing l = 1.5
    (component 0 has f = 0, i.e. it is the RBF term), outputscale 1 / components, cutoff 6."""
    torch.manual_seed(0)
    x = torch.sort(torch.rand(n) * span)[0]
    f = torch.rand(components)
    f[0] = 0.0
    y = torch.randn(n, k)
    params = torch.stack([torch.full((components,), 1.5), f, torch.full((components,), 1.0 / components)], dim=-1)
    return Workload(f"cg_sum_b{components}_n{n}_k{k}", "spectral", x, params, [6.0], y, {"sigma2": 0.01, "iterations": 50})


def band(workload: Workload, x_dev: Tensor) -> tuple[Tensor, Tensor]:
    """start/end on x_dev's device, shape (B, R) with one row per entry of ``cutoffs`` (or (R,)
    for an unbatched workload)."""
    from . import ranges

    if len(workload.cutoffs) > 1 and all(c is not None for c in workload.cutoffs):
        # one band per component, all built by one set of launches
        key = ("cutoffs", str(x_dev.device))
        if key not in workload.extra:
            workload.extra[key] = torch.tensor(workload.cutoffs, dtype=torch.float32, device=x_dev.device)
        return ranges.make_ranges_symmetric_cutoffs(workload.extra[key], x_dev)
    rows = [ranges.make_ranges(c, x_dev) for c in workload.cutoffs]
    if workload.params.dim() == 1:
        return rows[0]
    B = workload.params.shape[0]
    if len(rows) == 1:
        return rows[0][0].expand(B, -1), rows[0][1].expand(B, -1)
    return torch.stack([r[0] for r in rows]), torch.stack([r[1] for r in rows])
