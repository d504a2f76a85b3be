"""Row-sharded conjugate-gradient solve of ``(K + sigma^2 I) X = Y`` with the banded kernel operator.

``K`` is a ``KernelMatmulOperator``-style tuple ``(x, params, start, end, kernel_type)``; when
``params`` has a leading batch dim the operator is the SUM over that batch (a mixture of
components, the reference's ``SumKernel``, kernel_matmul/gpytorch/sum.py), evaluated inside one
kernel launch (``ops.matmul_rows(..., sum_batches=True)``).

Sharding.  The product has no dependence between 128-row blocks, so every rank owns a contiguous
window of row blocks: it computes those rows of ``K p`` and owns those rows of the iterate.  The
row blocks are grouped into at most 64 SEGMENTS of equal length aligned at row block 0, and a
window is a whole number of segments; every inner product is formed as "one fp32 partial per
128-row block, an fp64 sum per segment, then the fp64 sum over all segments in order", so the
iterates do not depend on the number of ranks.

An iteration on one rank (all vector work in the kernels of ``csrc/km_cg.cu``, no allocation):

    K p on the own rows                                  (the banded product kernel)
    q = K p + sigma^2 p, partials of p.q, segment sums   (km_cg_q_dots_f32, km_cg_segment_sums_f32)
    ALL-GATHER #1                                        (NCCL)
    alpha; x += alpha p; r -= alpha q; partials of r.r   (km_cg_update_xr_f32, km_cg_segment_sums_f32)
    ALL-GATHER #2  (segment sums of r.r, a few hundred bytes per rank)
    beta; p = r + beta p                                 (km_cg_update_p_f32)

What all-gather #1 carries decides the mode:

* ``"halo"`` -- the operator is banded, so the next product of a rank reads ``p`` only on the
  columns ``[lo, hi)`` of its own row blocks' bands: its own rows plus a halo on each side.  The
  rank keeps ``r`` and ``p`` up to date on ALL of ``[lo, hi)`` by applying the same ``alpha`` and
  ``beta`` there, for which it needs ``q`` on the halo rows: every rank contributes the first and
  the last ``H`` rows of its ``q`` (``H`` = the largest halo, ~1.6 k rows = 51 KB at k = 8 for the
  benchmark's band) together with its segment sums -- ONE small all-gather, and ``p`` itself is
  never exchanged.
* ``"allgather"`` -- every rank contributes all its rows of ``q`` (one all-gather of the
  ``(n, k)`` vector, 134 MB at n = 2^22, k = 8, plus the small one for the sums) and updates
  ``r`` and ``p`` on all ``n`` rows redundantly: the layout for operators without a band, or
  whose halo is wider than a neighbour's window.

The reference itself has no CG: it inherits ``LinearOperator.solve`` from the third-party
``linear_operator`` package (tests/test_linear_operator.py:9-38).  This is a standard batched
CG (one independent alpha / beta per right-hand-side column), checked against a dense fp64
solve in the tests.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable

import torch
from torch import Tensor

BLOCK_SIZE = 128
MAX_SEGMENTS = 64


def segment_layout(num_row_blocks: int, world_size: int) -> tuple[int, int, int]:
    """``(row blocks per segment, segments, segments per rank)``: at most ``MAX_SEGMENTS`` segments
    of equal length (the last may be shorter), dealt out in equal counts (the last ranks may get
    fewer or none)."""
    seg_blocks = max(1, -(-num_row_blocks // MAX_SEGMENTS))
    nseg = -(-num_row_blocks // seg_blocks) if num_row_blocks > 0 else 0
    segs_per_rank = max(1, -(-nseg // world_size))
    return seg_blocks, nseg, segs_per_rank


def row_block_window(num_row_blocks: int, rank: int, world_size: int) -> tuple[int, int]:
    """(first row block, count) of ``rank``: whole segments, equal counts of them per rank."""
    seg_blocks, _, segs_per_rank = segment_layout(num_row_blocks, world_size)
    per = segs_per_rank * seg_blocks
    begin = min(rank * per, num_row_blocks)
    return begin, min(per, num_row_blocks - begin)


@dataclass
class CGResult:
    solution: Tensor  # (n, k)
    residual_norms: Tensor  # (iterations + 1, k): ||r_i|| / ||y||
    iterations: int
    alphas: Tensor | None = None  # (iterations, k) step lengths
    betas: Tensor | None = None  # (iterations, k) direction updates
    y_norms: Tensor | None = None  # (k,) ||y||


class ShardMismatchError(RuntimeError):
    """The ranks of a sharded solve do not describe the same system (size, columns or band)."""


def _ptr(t: Tensor, byte_offset: int = 0) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() + byte_offset)


class CudaVectorOps:
    """The vector steps of an iteration as calls into ``libkm_b200.so`` (fp32 CUDA tensors).
    ``tests/cg_vector_ops.py`` has a PyTorch stand-in with the same methods, which the CPU
    (gloo) tests of the sharding logic use; the product has no other implementation."""

    def __init__(self, device: torch.device):
        from ._lib import check, lib

        self.lib, self.check, self.device = lib, check, device

    def _stream(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def block_dots(self, a, b, row0, row1, block_partials) -> None:
        self.check(self.lib.km_cg_block_dots_f32(a.shape[-1], _ptr(a), _ptr(b), row0, row1, _ptr(block_partials), self._stream()))

    def q_dots(self, kp, p, sigma2, row0, row1, block_partials, send, top_off, top_rows, bottom_off, bottom_rows) -> None:
        self.check(self.lib.km_cg_q_dots_f32(
            p.shape[-1], _ptr(kp), _ptr(p), float(sigma2), row0, row1, _ptr(block_partials),
            _ptr(send, top_off) if top_rows else None, top_rows, _ptr(send, bottom_off) if bottom_rows else None,
            bottom_rows, self._stream()))

    def segment_sums(self, k, block_partials, blocks, seg_blocks, out, out_off) -> None:
        self.check(self.lib.km_cg_segment_sums_f32(k, _ptr(block_partials), blocks, seg_blocks, _ptr(out, out_off), self._stream()))

    def init_scalars(self, k, gathered, rank_stride, ranks, slots, rs, ynorm) -> None:
        self.check(self.lib.km_cg_init_scalars_f32(k, _ptr(gathered), rank_stride, ranks, slots, _ptr(rs), _ptr(ynorm), self._stream()))

    def update_xr(self, x, r, p, q_own, q_below, q_above, row0, row1, lo, hi, gathered, rank_stride, ranks, slots, rs,
                  block_partials, alpha_row=None) -> None:
        (tb, ob, gb), (ta, oa, ga) = q_below, q_above
        self.check(self.lib.km_cg_update_xr_f32(
            p.shape[-1], _ptr(x), _ptr(r), _ptr(p), _ptr(q_own), _ptr(tb, ob) if tb is not None else None, gb,
            _ptr(ta, oa) if ta is not None else None, ga, row0, row1, lo, hi, _ptr(gathered), rank_stride, ranks, slots,
            _ptr(rs), _ptr(block_partials), _ptr(alpha_row) if alpha_row is not None else None, self._stream()))

    def update_p(self, p, r, lo, hi, gathered, rank_stride, ranks, slots, rs_old, rs_new, ynorm, history_row,
                 beta_row=None) -> None:
        self.check(self.lib.km_cg_update_p_f32(
            p.shape[-1], _ptr(p), _ptr(r), lo, hi, _ptr(gathered), rank_stride, ranks, slots, _ptr(rs_old), _ptr(rs_new),
            _ptr(ynorm), _ptr(history_row), _ptr(beta_row) if beta_row is not None else None, self._stream()))


class ShardedOperator:
    """``v -> (K + sigma^2 I) v`` with rows sharded over the ranks of a process group.

    ``matvec_rows(v, row_block_begin, row_block_count, out)`` computes the rows of ``K v`` inside
    the window into ``out`` (shape ``(rows_in_window, k)``) from a full-length ``v`` of which only
    the rows ``col_range = (lo, hi)`` are guaranteed to be current; ``col_range=None`` means all of
    ``v`` is read.  The default is the km_b200 kernel (``from_kernel``).
    """

    def __init__(self, n: int, sigma2: float, matvec_rows: Callable[[Tensor, int, int, Tensor], None],
                 group=None, device: torch.device | None = None, col_range: tuple[int, int] | None = None,
                 band_checksum: int = 0, vector_ops=None, mode: str = "auto"):
        import torch.distributed as dist

        if mode not in ("auto", "halo", "allgather"):
            raise ValueError(f"unknown mode {mode!r}")
        self.n = n
        self.sigma2 = float(sigma2)
        self.matvec_rows = matvec_rows
        self.group = group
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.rank = self.dist.get_rank(group) if self.dist else 0
        self.world = self.dist.get_world_size(group) if self.dist else 1
        self.R = -(-n // BLOCK_SIZE)
        self.seg_blocks, self.nseg, self.segs_per_rank = segment_layout(self.R, self.world)
        self.per = self.segs_per_rank * self.seg_blocks  # row blocks per rank (padded)
        self.per_rows = self.per * BLOCK_SIZE
        self.begin, self.count = row_block_window(self.R, self.rank, self.world)
        self.row0 = self.begin * BLOCK_SIZE
        self.row1 = min(n, (self.begin + self.count) * BLOCK_SIZE)
        self.rows = max(0, self.row1 - self.row0)  # rows of this rank
        self.device = device
        self.vector_ops = vector_ops
        lo, hi = (0, n) if col_range is None else col_range
        # what the product reads, rounded to row-block boundaries, never less than the own rows
        lo = min((max(0, lo) // BLOCK_SIZE) * BLOCK_SIZE, self.row0)
        hi = max(min(n, -(-hi // BLOCK_SIZE) * BLOCK_SIZE), self.row1)
        if self.rows == 0:
            lo = hi = self.row0 = self.row1 = min(self.row0, n)
        self._agree(lo, hi, band_checksum, col_range is not None, mode)

    # ---- set-up: the ranks compare what they were given and settle the exchange layout

    def _agree(self, lo: int, hi: int, band_checksum: int, banded: bool, mode: str) -> None:
        mine = [self.n, self.R, int(band_checksum), lo, hi, self.row0, self.row1, int(banded)]
        if self.world > 1:
            t = torch.tensor(mine, dtype=torch.int64, device=self.device if self.device is not None else "cpu")
            every = torch.empty(self.world * len(mine), dtype=torch.int64, device=t.device)
            self.dist.all_gather_into_tensor(every, t, group=self.group)
            table = every.view(self.world, len(mine)).tolist()
        else:
            table = [mine]
        for rk, row in enumerate(table):
            if row[:3] != table[0][:3]:
                raise ShardMismatchError(
                    f"rank {rk} describes a different system than rank 0: (n, row blocks, band checksum) = "
                    f"{tuple(row[:3])} against {tuple(table[0][:3])}")
        below = max(row[5] - row[3] for row in table)  # most rows any rank needs from the rank before it
        above = max(row[4] - row[6] for row in table)  # ... from the rank after it
        owned = [row[6] - row[5] for row in table]
        # Halo exchange: every rank contributes its first `above` and last `below` rows of q, so each
        # rank that owns rows must own at least that many, and a halo must not reach past the
        # direct neighbour (implied by the same condition).
        halo_possible = (self.world > 1 and all(row[7] for row in table)
                         and all(rows_ == 0 or rows_ >= max(below, above) for rows_ in owned))
        if mode == "halo" and self.world > 1 and not halo_possible:
            raise ValueError("halo exchange needs a band whose halo fits into the neighbouring rank's window")
        if self.world == 1:
            self.mode = "single"
        else:
            self.mode = "halo" if (mode != "allgather" and halo_possible) else "allgather"
        if self.mode == "halo":
            self.lo, self.hi, self.halo_below, self.halo_above = lo, hi, below, above
        else:  # r and p are kept on all rows
            self.lo, self.hi, self.halo_below, self.halo_above = 0, self.n, 0, 0

    @classmethod
    def from_kernel(cls, kernel_type: str, x: Tensor, params: Tensor, start: Tensor, end: Tensor, sigma2: float,
                    group=None, mode: str = "auto", phases: bool | None = None) -> "ShardedOperator":
        """Operator backed by ``ops.matmul_rows`` (sum over the batch of ``params`` if batched);
        ``start`` / ``end`` are one band ``(R,)`` shared by all components.

        ``phases``: for a sum of spectral components, write the per-point phase vectors once now
        (``ops.prepare_sum_phases``: about ``16 B n`` bytes for ``B`` components) so that every product
        of the solve copies them instead of evaluating them again; default: yes, unless the
        environment variable ``KM_SUM_PHASES`` is ``0``."""
        import os

        from . import ops

        n = x.shape[-1]
        batched = params.dim() > 1
        B = params.shape[:-1]
        xb = x.expand(*B, n) if batched else x
        sb = start.expand(*B, start.shape[-1]) if batched else start
        eb = end.expand(*B, end.shape[-1]) if batched else end

        if phases is None:
            phases = os.environ.get("KM_SUM_PHASES", "1") != "0"
        phase_ws = None  # set below, once this rank's rows and columns are known
        prepared: dict = {}  # (buffers, window) -> launch with all arguments already marshalled

        def matvec_rows(v: Tensor, rb_begin: int, rb_count: int, out: Tensor) -> None:
            # a solve calls this with the same two buffers every iteration: validate and marshal once
            key = (v.data_ptr(), tuple(v.shape), tuple(v.stride()), out.data_ptr(), tuple(out.shape), rb_begin, rb_count)
            call = prepared.get(key)
            if call is None:
                rhs = v.expand(*B, *v.shape) if batched else v
                # (the phase images cover this rank's own row blocks only)
                ws = phase_ws if (rb_begin >= begin and rb_begin + rb_count <= begin + count) else None
                call = ops.prepare_matmul_rows(kernel_type, xb, xb, rhs, params, sb, eb, row_block_begin=rb_begin,
                                               row_block_count=rb_count, sum_batches=batched, out=out, phases=ws)
                if call is None:  # (a product that needs a workspace: the unprepared call)
                    def call(rhs=rhs, out=out, ws=ws):
                        ops.matmul_rows(kernel_type, xb, xb, rhs, params, sb, eb, row_block_begin=rb_begin,
                                        row_block_count=rb_count, sum_batches=batched, out=out, phases=ws)
                if len(prepared) >= 8:
                    prepared.clear()
                prepared[key] = call
            call()

        import torch.distributed as dist

        world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        rank = dist.get_rank(group) if world > 1 else 0
        R = -(-n // BLOCK_SIZE)
        begin, count = row_block_window(R, rank, world)
        # the columns this rank's row blocks read, and a checksum of the whole band (one host
        # synchronisation, at set-up only)
        s64, e64 = start.reshape(-1)[:R].to(torch.int64), end.reshape(-1)[:R].to(torch.int64)
        weights = torch.arange(1, R + 1, device=start.device, dtype=torch.int64)
        checksum = ((s64 * weights).sum() * 31 + (e64 * weights).sum()) % (2**61 - 1)
        if count > 0:
            mine = torch.stack([s64[begin:begin + count].min(), e64[begin:begin + count].max(), checksum])
        else:
            mine = torch.stack([torch.zeros((), dtype=torch.int64, device=start.device)] * 2 + [checksum])
        lo, hi, checksum = (int(v) for v in mine.tolist())
        if phases and batched and count > 0:
            phase_ws = ops.prepare_sum_phases(kernel_type, x, x, params, rows=(begin * BLOCK_SIZE, min(n, (begin + count) * BLOCK_SIZE)),
                                              cols=(max(0, min(lo, n)), max(0, min(hi, n))))
        op = cls(n, sigma2, matvec_rows, group=group, device=x.device, col_range=(lo, hi) if count > 0 else (0, 0),
                 band_checksum=checksum, mode=mode)
        op.phase_workspace = phase_ws  # (None: the products evaluate the phase vectors themselves)
        return op

    # ---- the operator applied to a full vector (tests, diagnostics)

    def local(self, v: Tensor) -> Tensor:
        """This rank's rows of a full vector (a view)."""
        return v[self.row0: self.row0 + self.rows]

    def apply_rows(self, v: Tensor) -> Tensor:
        """This rank's rows of ``(K + sigma^2 I) v`` for a full ``v`` -> ``(rows, k)``."""
        out = torch.empty(self.rows, v.shape[-1], device=v.device, dtype=v.dtype)
        if self.rows > 0:
            self.matvec_rows(v, self.begin, self.count, out)
            out.add_(self.local(v), alpha=self.sigma2)
        return out

    def gather_rows(self, mine: Tensor) -> Tensor:
        """Full ``(n, k)`` vector from every rank's rows."""
        if self.world == 1:
            return mine
        k = mine.shape[-1]
        padded = torch.zeros(self.per_rows, k, device=mine.device, dtype=mine.dtype)
        padded[: self.rows] = mine
        full = torch.empty(self.world * self.per_rows, k, device=mine.device, dtype=mine.dtype)
        self.dist.all_gather_into_tensor(full, padded, group=self.group)
        return full[: self.n]

    def apply(self, v: Tensor) -> Tensor:
        """Full ``(K + sigma^2 I) v`` on every rank."""
        return self.gather_rows(self.apply_rows(v))


def _round_up(v: int, to: int) -> int:
    return -(-v // to) * to


class CGSolver:
    """State of a running solve; ``step()`` is one CG iteration.  All buffers are allocated here;
    ``step()`` allocates nothing and never synchronises with the host.

    ``y`` is the full ``(n, k)`` right-hand side, on the operator's device or in (pinned) host
    memory; only the rows this rank keeps current, ``[op.lo, op.hi)``, are read (and, from host
    memory, copied)."""

    def __init__(self, op: ShardedOperator, y: Tensor, max_iterations: int = 256):
        if y.dim() != 2 or y.shape[0] != op.n:
            raise ValueError(f"y must be (n, k) = ({op.n}, k), got {tuple(y.shape)}")
        self.op = op
        self.k = k = y.shape[-1]
        dev, dt = y.device, y.dtype
        if not y.is_cuda and op.device is not None and op.device.type == "cuda":
            dev = op.device  # right-hand side in host memory
        self.V = op.vector_ops
        if self.V is None:
            if dev.type != "cuda" or dt != torch.float32:
                raise RuntimeError("the CG kernels need float32 CUDA tensors (there is no CPU path)")
            self.V = CudaVectorOps(dev)
        esz = y.element_size()
        n_pad = max(op.n, op.world * op.per_rows)  # every rank's padded window exists in every vector
        self.x = torch.zeros(n_pad, k, device=dev, dtype=dt)
        self.r = torch.zeros(n_pad, k, device=dev, dtype=dt)
        self.p = torch.zeros(n_pad, k, device=dev, dtype=dt)
        self.kp = torch.zeros(n_pad, k, device=dev, dtype=dt)
        if op.hi > op.lo:
            self.r[op.lo: op.hi].copy_(y[op.lo: op.hi], non_blocking=True)
            self.p[op.lo: op.hi].copy_(self.r[op.lo: op.hi])
        self.bp = torch.zeros(max(op.count, 1), k, device=dev, dtype=dt)
        self.rs = torch.zeros(2, k, device=dev, dtype=dt)
        self.ynorm = torch.ones(k, device=dev, dtype=dt)
        self.max_iterations = max_iterations
        self.history = torch.ones(max_iterations + 1, k, device=dev, dtype=dt)
        # alpha and beta of every iteration: the Lanczos coefficients of the solve (gp.py turns them
        # into log-determinant estimates)
        self.alphas = torch.zeros(max_iterations, k, device=dev, dtype=dt)
        self.betas = torch.zeros(max_iterations, k, device=dev, dtype=dt)
        self.it = 0
        #: set to a callable ``mark(name)`` to be told where the phases of ``step()`` begin
        #: (bench.py records CUDA events there for its per-phase breakdown)
        self.mark = None
        # exchange buffers: [segment sums (fp64)] [first halo_above rows of q] [last halo_below rows of q]
        self.seg_bytes = _round_up(op.segs_per_rank * k * 8, 256)
        top, bottom = (op.halo_above, op.halo_below) if op.mode == "halo" else (0, 0)
        self.top_rows, self.bottom_rows = top, bottom
        self.top_off = self.seg_bytes
        self.bottom_off = self.top_off + _round_up(top * k * esz, 256)
        self.packed = self.bottom_off + _round_up(bottom * k * esz, 256)
        self.send1 = torch.zeros(self.packed, device=dev, dtype=torch.uint8)
        self.send2 = torch.zeros(self.seg_bytes, device=dev, dtype=torch.uint8)
        if op.world > 1:
            self.g1 = torch.zeros(op.world * self.packed, device=dev, dtype=torch.uint8)
            self.g2 = torch.zeros(op.world * self.seg_bytes, device=dev, dtype=torch.uint8)
            self.gq = torch.zeros(op.world * op.per_rows, k, device=dev, dtype=dt) if op.mode == "allgather" else None
        else:
            self.g1, self.g2, self.gq = self.send1, self.send2, None
        # where q of the rows below / above the own window is found: (buffer, byte offset, row of its first element)
        none = (None, 0, 0)
        if op.mode == "halo":
            self.q_below = (self.g1, (op.rank - 1) * self.packed + self.bottom_off, op.row0 - bottom) if op.lo < op.row0 else none
            self.q_above = (self.g1, (op.rank + 1) * self.packed + self.top_off, op.row1) if op.hi > op.row1 else none
        elif op.mode == "allgather":
            self.q_below = self.q_above = (self.gq, 0, 0)
        else:
            self.q_below = self.q_above = none
        # ||y||^2 through the same partial sums as every later inner product
        self.V.block_dots(self.r, self.r, op.row0, op.row1, self.bp)
        self.V.segment_sums(k, self.bp, op.count, op.seg_blocks, self.send2, 0)
        self._gather(self.g2, self.send2)
        self.V.init_scalars(k, self.g2, self.seg_bytes, op.world, op.segs_per_rank, self.rs[0], self.ynorm)

    def _gather(self, full: Tensor, mine: Tensor) -> None:
        if self.op.world > 1:
            self.op.dist.all_gather_into_tensor(full, mine, group=self.op.group)

    def step(self) -> Tensor:
        """One iteration; returns the relative residual norms ``(k,)`` (a view of the history)."""
        op, V, k = self.op, self.V, self.k
        if self.it >= self.max_iterations:
            raise RuntimeError(f"more than max_iterations = {self.max_iterations} steps")
        rs_old, rs_new = self.rs[self.it & 1], self.rs[(self.it + 1) & 1]
        mark = self.mark or (lambda name: None)
        mark("product")
        if op.rows > 0:
            op.matvec_rows(self.p[: op.n], op.begin, op.count, self.kp[op.row0: op.row1])
        mark("q_dots")
        V.q_dots(self.kp, self.p, op.sigma2, op.row0, op.row1, self.bp, self.send1, self.top_off, self.top_rows,
                 self.bottom_off, self.bottom_rows)
        V.segment_sums(k, self.bp, op.count, op.seg_blocks, self.send1, 0)
        mark("gather1")
        self._gather(self.g1, self.send1)
        if self.gq is not None:
            self._gather(self.gq, self.kp[op.rank * op.per_rows: (op.rank + 1) * op.per_rows])
        mark("update_xr")
        V.update_xr(self.x, self.r, self.p, self.kp, self.q_below, self.q_above, op.row0, op.row1, op.lo, op.hi,
                    self.g1, self.packed, op.world, op.segs_per_rank, rs_old, self.bp, self.alphas[self.it])
        V.segment_sums(k, self.bp, op.count, op.seg_blocks, self.send2, 0)
        mark("gather2")
        self._gather(self.g2, self.send2)
        self.it += 1
        mark("update_p")
        V.update_p(self.p, self.r, op.lo, op.hi, self.g2, self.seg_bytes, op.world, op.segs_per_rank, rs_old, rs_new,
                   self.ynorm, self.history[self.it], self.betas[self.it - 1])
        mark("end")
        return self.history[self.it]

    def residual_norms(self) -> Tensor:
        """``(iterations + 1, k)``: relative residual norms after 0, 1, ... iterations."""
        return self.history[: self.it + 1]

    def check_finite(self) -> None:
        """Raises on EVERY rank if any rank's residual norm is not finite (a product kernel that gave
        up writes NaN into its rows).  One host synchronisation and, with ranks, one all-gather."""
        bad = (~torch.isfinite(self.history[self.it])).any().to(torch.int64).reshape(1)
        if self.op.world > 1:
            every = torch.empty(self.op.world, dtype=torch.int64, device=bad.device)
            self.op.dist.all_gather_into_tensor(every, bad, group=self.op.group)
            bad = every
        flags = bad.tolist()
        if any(flags):
            raise RuntimeError(f"non-finite residual after {self.it} iterations on rank(s) {[i for i, f in enumerate(flags) if f]}")

    def solution_rows(self) -> Tensor:
        """This rank's rows ``[op.row0, op.row1)`` of the iterate (a view; no communication)."""
        return self.x[self.op.row0: self.op.row1]

    def solution(self) -> Tensor:
        """The full iterate on every rank."""
        op = self.op
        if op.world == 1:
            return self.x[: op.n]
        full = torch.empty(op.world * op.per_rows, self.k, device=self.x.device, dtype=self.x.dtype)
        self._gather(full, self.x[op.rank * op.per_rows: (op.rank + 1) * op.per_rows])
        return full[: op.n]


def conjugate_gradient(op: ShardedOperator, y: Tensor, iterations: int, tol: float = 0.0) -> CGResult:
    """Batched CG from x0 = 0: every column of ``y`` is its own system sharing the operator.
    Stops after ``iterations`` steps (or earlier when every column's relative residual is below
    ``tol``, which costs one host synchronisation per iteration and is off for ``tol == 0``)."""
    solver = CGSolver(op, y, max_iterations=max(iterations, 1))
    done = 0
    for _ in range(iterations):
        res = solver.step()
        done += 1
        if tol > 0 and bool((res <= tol).all()):
            break
    return CGResult(solver.solution(), solver.residual_norms().clone(), done, solver.alphas[:done].clone(),
                    solver.betas[:done].clone(), solver.ynorm.clone())
