"""Row-sharded conjugate-gradient solve of ``(K + sigma^2 I) V = Y`` with the banded kernel operator.

``K`` is a ``KernelMatmulOperator``-style tuple ``(x, params, start, end, kernel_type)``; when
``params`` has a leading batch dim the operator is the SUM over that batch (a mixture of
components, the reference's ``SumKernel``, kernel_matmul/gpytorch/sum.py), evaluated inside one
kernel launch (``ops.matmul_rows(..., sum_batches=True)``).

Sharding.  The product has no dependence between 128-row blocks, so every rank owns a contiguous
window of row blocks: it computes those rows of ``K p`` against the full search direction and
keeps ITS rows of the iterate, the residual and the search direction.  Per iteration the ranks
exchange
  * the new search direction (one ``all_gather_into_tensor`` of the row windows), and
  * two small arrays of per-row-block partial inner products (``p . Ap`` and ``r . r``), which
    every rank then adds up in the same fixed order.
An inner product is always formed as "one partial per 128-row block, then the sum over all row
blocks in index order", whichever rank owns a block, so the iterates do not depend on the number
of ranks (bit for bit wherever the per-block sums are computed in a size-independent order, which
holds for the CPU reductions the tests run; a row block's product is always computed by one CTA
in the same order).

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
        self.row0 = self.begin * BLOCK_SIZE
        self.rows = max(0, min(n, (self.begin + self.count) * BLOCK_SIZE) - self.row0)  # rows of this rank
        self.device = device

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

    # ---- pieces of a sharded iteration

    def local(self, v: Tensor) -> Tensor:
        """This rank's rows of a full vector (a view)."""
        return v[self.row0 : self.row0 + self.rows]

    def apply_rows(self, v: Tensor) -> Tensor:
        """This rank's rows of ``(K + sigma^2 I) v`` for a full ``v`` -> ``(rows, k)``."""
        out = torch.empty(self.rows, v.shape[-1], device=v.device, dtype=v.dtype)
        if self.rows > 0:
            self.matvec_rows(v, self.begin, self.count, out)
            out.add_(self.local(v), alpha=self.sigma2)
        return out

    def gather_rows(self, mine: Tensor) -> Tensor:
        """Full ``(n, k)`` vector from every rank's rows (the collective of the solve)."""
        if self.world == 1:
            return mine
        k = mine.shape[-1]
        rows_per_rank = self.per * BLOCK_SIZE
        padded = torch.zeros(rows_per_rank, k, device=mine.device, dtype=mine.dtype)
        padded[: self.rows] = mine
        full = torch.empty(self.world * rows_per_rank, k, device=mine.device, dtype=mine.dtype)
        self.dist.all_gather_into_tensor(full, padded, group=self.group)
        return full[: self.n]

    def dot(self, a: Tensor, b: Tensor) -> Tensor:
        """Column-wise inner products ``(k,)`` of two row-sharded vectors: one partial per 128-row
        block, all partials gathered, then added in block order on every rank."""
        k = a.shape[-1]
        blocks = self.count
        prod = torch.zeros(max(blocks, 0) * BLOCK_SIZE, k, device=a.device, dtype=a.dtype)
        prod[: self.rows] = a * b
        partial = prod.view(blocks, BLOCK_SIZE, k).sum(dim=1)  # (blocks, k)
        if self.world > 1:
            padded = torch.zeros(self.per, k, device=a.device, dtype=a.dtype)
            padded[:blocks] = partial
            every = torch.empty(self.world * self.per, k, device=a.device, dtype=a.dtype)
            self.dist.all_gather_into_tensor(every, padded, group=self.group)
            partial = every[: self.R]
        return partial.sum(dim=0)

    def apply(self, v: Tensor) -> Tensor:
        """Full ``(K + sigma^2 I) v`` on every rank."""
        return self.gather_rows(self.apply_rows(v))


class CGSolver:
    """State of a running solve; ``step()`` is one CG iteration."""

    def __init__(self, op: ShardedOperator, y: Tensor):
        self.op = op
        self.tiny = torch.finfo(y.dtype).tiny
        self.x = torch.zeros(op.rows, y.shape[-1], device=y.device, dtype=y.dtype)  # this rank's rows
        self.r = op.local(y).clone()
        self.p_local = self.r.clone()
        self.p = y.clone() if op.world > 1 else self.p_local  # full search direction
        self.rs = op.dot(self.r, self.r)
        self.y_norm = self.rs.sqrt().clamp_min(self.tiny)

    def step(self) -> Tensor:
        """One iteration; returns the relative residual norms ``(k,)``."""
        op = self.op
        Ap = op.apply_rows(self.p)
        alpha = self.rs / op.dot(self.p_local, Ap).clamp_min(self.tiny)
        self.x.addcmul_(self.p_local, alpha)
        self.r.addcmul_(Ap, -alpha)
        rs_new = op.dot(self.r, self.r)
        beta = rs_new / self.rs.clamp_min(self.tiny)
        self.p_local.mul_(beta).add_(self.r)
        self.p = op.gather_rows(self.p_local)
        self.rs = rs_new
        return rs_new.sqrt() / self.y_norm

    def solution(self) -> Tensor:
        """The full iterate on every rank."""
        return self.op.gather_rows(self.x)


def conjugate_gradient(op: ShardedOperator, y: Tensor, iterations: int, tol: float = 0.0) -> CGResult:
    """Batched CG from x0 = 0: every column of ``y`` is its own system sharing the operator.
    Stops after ``iterations`` steps (or earlier when every column's relative residual is below
    ``tol``, which costs one host synchronisation per iteration and is off for ``tol == 0``)."""
    solver = CGSolver(op, y)
    history = [torch.ones_like(solver.rs)]
    done = 0
    for _ in range(iterations):
        history.append(solver.step())
        done += 1
        if tol > 0 and bool((history[-1] <= tol).all()):
            break
    return CGResult(solver.solution(), torch.stack(history), done)
