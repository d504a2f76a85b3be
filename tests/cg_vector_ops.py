"""PyTorch stand-in for ``kernel_matmul_b200.cg.CudaVectorOps`` (TEST INFRASTRUCTURE ONLY).

Same methods, same buffers and byte offsets, any device and dtype: it lets the CPU (gloo) tests
run the sharding, exchange and bookkeeping code of ``cg.py`` without a GPU, and the GPU tests
check the CUDA kernels against it step by step.  Inner products keep the structure of the
kernels (one partial per 128-row block, one fp64 sum per segment, the gathered segment sums added
in order), so results do not depend on the number of ranks here either.
"""
from __future__ import annotations

import torch

BLOCK = 128


def _doubles(buf: torch.Tensor, byte_off: int, count: int) -> torch.Tensor:
    return buf[byte_off: byte_off + 8 * count].view(torch.float64)


def _values(buf: torch.Tensor, byte_off: int, rows: int, k: int, dtype) -> torch.Tensor:
    esz = torch.empty((), dtype=dtype).element_size()
    return buf[byte_off: byte_off + rows * k * esz].view(dtype).view(rows, k)


def _block_partials(prod: torch.Tensor, out: torch.Tensor) -> None:
    rows, k = prod.shape
    blocks = -(-rows // BLOCK)
    if blocks == 0:
        return
    padded = torch.zeros(blocks * BLOCK, k, dtype=prod.dtype, device=prod.device)
    padded[:rows] = prod
    out[:blocks] = padded.view(blocks, BLOCK, k).sum(dim=1)


def _total(gathered: torch.Tensor, rank_stride: int, ranks: int, slots: int, k: int) -> torch.Tensor:
    t = torch.zeros(k, dtype=torch.float64, device=gathered.device)
    for rk in range(ranks):
        seg = _doubles(gathered, rk * rank_stride, slots * k).view(slots, k)
        for s in range(slots):
            t = t + seg[s]
    return t


class TorchVectorOps:
    def block_dots(self, a, b, row0, row1, block_partials) -> None:
        _block_partials(a[row0:row1] * b[row0:row1], block_partials)

    def q_dots(self, kp, p, sigma2, row0, row1, block_partials, send, top_off, top_rows, bottom_off, bottom_rows) -> None:
        if row1 == row0:
            return
        k = p.shape[-1]
        q = kp[row0:row1] + sigma2 * p[row0:row1]
        kp[row0:row1] = q
        _block_partials(p[row0:row1] * q, block_partials)
        if top_rows:
            _values(send, top_off, top_rows, k, q.dtype).copy_(q[:top_rows])
        if bottom_rows:
            _values(send, bottom_off, bottom_rows, k, q.dtype).copy_(q[q.shape[0] - bottom_rows:])

    def segment_sums(self, k, block_partials, blocks, seg_blocks, out, out_off) -> None:
        segs = -(-blocks // seg_blocks) if blocks else 0
        dst = _doubles(out, out_off, segs * k).view(segs, k) if segs else None
        for s in range(segs):
            dst[s] = block_partials[s * seg_blocks: min((s + 1) * seg_blocks, blocks)].double().sum(dim=0)

    def init_scalars(self, k, gathered, rank_stride, ranks, slots, rs, ynorm) -> None:
        t = _total(gathered, rank_stride, ranks, slots, k).to(rs.dtype)
        rs.copy_(t)
        ynorm.copy_(t.sqrt().clamp_min(torch.finfo(rs.dtype).tiny))

    def update_xr(self, x, r, p, q_own, q_below, q_above, row0, row1, lo, hi, gathered, rank_stride, ranks, slots, rs,
                  block_partials, alpha_row=None) -> None:
        if hi == lo:
            return
        k = p.shape[-1]
        tiny = torch.finfo(rs.dtype).tiny
        alpha = rs / _total(gathered, rank_stride, ranks, slots, k).to(rs.dtype).clamp_min(tiny)
        if alpha_row is not None:
            alpha_row.copy_(alpha)
        x[row0:row1] += alpha * p[row0:row1]
        r[row0:row1] -= alpha * q_own[row0:row1]
        if lo < row0:
            buf, off, origin = q_below
            src = _values(buf, off, row0 - origin, k, r.dtype) if buf.dtype == torch.uint8 else buf[origin:] if origin else buf
            r[lo:row0] -= alpha * src[lo - origin: row0 - origin]
        if hi > row1:
            buf, off, origin = q_above
            src = _values(buf, off, hi - origin, k, r.dtype) if buf.dtype == torch.uint8 else buf
            r[row1:hi] -= alpha * src[row1 - origin: hi - origin]
        _block_partials(r[row0:row1] * r[row0:row1], block_partials)

    def update_p(self, p, r, lo, hi, gathered, rank_stride, ranks, slots, rs_old, rs_new, ynorm, history_row,
                 beta_row=None) -> None:
        k = p.shape[-1]
        tiny = torch.finfo(rs_old.dtype).tiny
        new = _total(gathered, rank_stride, ranks, slots, k).to(rs_old.dtype)
        beta = new / rs_old.clamp_min(tiny)
        if beta_row is not None:
            beta_row.copy_(beta)
        p[lo:hi] = r[lo:hi] + beta * p[lo:hi]
        rs_new.copy_(new)
        if history_row is not None:
            history_row.copy_(new.sqrt() / ynorm)
