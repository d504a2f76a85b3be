"""Row-sharded conjugate-gradient solve of ``(K + sigma^2 I) V = Y`` with the banded kernel operator.

``K`` is a ``KernelMatmulOperator``-style tuple ``(x, params, start, end, kernel_type)``; when
``params`` has a leading batch dim the operator is the SUM over that batch (a mixture of
components, the reference's ``SumKernel``, kernel_matmul/gpytorch/sum.py), evaluated inside one
kernel launch (``ops.matmul_rows(..., sum_batches=True)``).

Sharding.  The product has no dependence between 128-row blocks, so every rank computes the row
blocks of its own contiguous window against the full search direction and the windows are put
together with one ``all_gather_into_tensor`` per iteration; nothing else is communicated.  All
vector updates and inner products then run redundantly on the full vectors on every rank, in
the same order, so the iterates are bit-identical on all ranks and do not depend on the number
of ranks (a row block is always computed by one CTA in the same order, whichever rank owns it).

The reference itself has no CG: it inherits ``LinearOperator.solve`` from the third-party
``linear_operator`` package (tests/test_linear_operator.py:9-38).  This is a standard batched
CG (one independent alpha / beta per right-hand-side column), checked against a dense fp64
solve in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
from torch import Tensor

BLOCK_SIZE = 128


def row_block_window(num_row_blocks: int, rank: int, world_size: int) -> tuple[int, int]:
    """(first row block, count) of ``rank``: equal windows of ceil(R / world) blocks (the last
    ranks may get fewer or none).  Equal windows keep the all-gather a single collective."""
    per = -(-num_row_blocks // world_size)
    begin = min(rank * per, num_row_blocks)
    return begin, min(per, num_row_blocks - begin)


@dataclass
class CGResult:
    solution: Tensor  # (n, k)
    residual_norms: Tensor  # (iterations + 1, k): ||r_i|| / ||y||
    iterations: int


class ShardedOperator:
    """``v -> (K + sigma^2 I) v`` with rows sharded over the ranks of a process group.

    ``matvec_rows(v, row_block_begin, row_block_count, out)`` computes the rows of ``K v`` inside
    the window into ``out`` (shape ``(rows_in_window, k)``); the default is the km_b200 kernel.
    """

    def __init__(self, n: int, sigma2: float, matvec_rows: Callable[[Tensor, int, int, Tensor], None],
                 group=None, device: torch.device | None = None):
        import torch.distributed as dist

        self.n = n
        self.sigma2 = float(sigma2)
        self.matvec_rows = matvec_rows
        self.group = group
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.rank = self.dist.get_rank(group) if self.dist else 0
        self.world = self.dist.get_world_size(group) if self.dist else 1
        self.R = -(-n // BLOCK_SIZE)
        self.per = -(-self.R // self.world)  # row blocks per rank (padded)
        self.begin, self.count = row_block_window(self.R, self.rank, self.world)
        self.device = device
        self._gather: Tensor | None = None
        self._mine: Tensor | None = None

    @classmethod
    def from_kernel(cls, kernel_type: str, x: Tensor, params: Tensor, start: Tensor, end: Tensor, sigma2: float,
                    group=None) -> "ShardedOperator":
        """Operator backed by ``ops.matmul_rows`` (sum over the batch of ``params`` if batched)."""
        from . import ops

        n = x.shape[-1]
        batched = params.dim() > 1
        B = params.shape[:-1]
        xb = x.expand(*B, n) if batched else x
        sb = start.expand(*B, start.shape[-1]) if batched else start
        eb = end.expand(*B, end.shape[-1]) if batched else end

        def matvec_rows(v: Tensor, rb_begin: int, rb_count: int, out: Tensor) -> None:
            rhs = v.expand(*B, *v.shape) if batched else v
            ops.matmul_rows(kernel_type, xb, xb, rhs, params, sb, eb, row_block_begin=rb_begin,
                            row_block_count=rb_count, sum_batches=batched, out=out)

        return cls(n, sigma2, matvec_rows, group=group, device=x.device)

    def apply(self, v: Tensor) -> Tensor:
        """Full ``(K + sigma^2 I) v`` on every rank."""
        k = v.shape[-1]
        rows_per_rank = self.per * BLOCK_SIZE
        if self._gather is None or self._gather.shape != (self.world * rows_per_rank, k) or self._gather.device != v.device:
            self._gather = torch.zeros(self.world * rows_per_rank, k, device=v.device, dtype=v.dtype)
            self._mine = torch.zeros(rows_per_rank, k, device=v.device, dtype=v.dtype)
        rows = max(0, min(self.n, (self.begin + self.count) * BLOCK_SIZE) - self.begin * BLOCK_SIZE)
        if self.world == 1:
            self.matvec_rows(v, self.begin, self.count, self._gather[:rows])
        else:
            if rows > 0:
                self.matvec_rows(v, self.begin, self.count, self._mine[:rows])
            # the only collective of the solve: every rank's window lands at its row offset
            self.dist.all_gather_into_tensor(self._gather, self._mine, group=self.group)
        return torch.add(self._gather[: self.n], v, alpha=self.sigma2)


def conjugate_gradient(op: ShardedOperator, y: Tensor, iterations: int, tol: float = 0.0) -> CGResult:
    """Batched CG from x0 = 0: every column of ``y`` is its own system sharing the operator.
    Stops after ``iterations`` steps (or earlier when every column's relative residual is below
    ``tol``, which costs one host synchronisation per iteration and is off for ``tol == 0``)."""
    x = torch.zeros_like(y)
    r = y.clone()
    p = r.clone()
    rs = (r * r).sum(dim=0)
    y_norm = rs.sqrt().clamp_min(torch.finfo(y.dtype).tiny)
    history = [torch.ones_like(rs)]
    done = 0
    for _ in range(iterations):
        Ap = op.apply(p)
        pAp = (p * Ap).sum(dim=0)
        alpha = rs / pAp.clamp_min(torch.finfo(y.dtype).tiny)
        x.addcmul_(p, alpha)
        r.addcmul_(Ap, -alpha)
        rs_new = (r * r).sum(dim=0)
        beta = rs_new / rs.clamp_min(torch.finfo(y.dtype).tiny)
        p.mul_(beta).add_(r)
        rs = rs_new
        history.append(rs.sqrt() / y_norm)
        done += 1
        if tol > 0 and bool((history[-1] <= tol).all()):
            break
    return CGResult(x, torch.stack(history), done)
