"""Band (sparsity pattern) construction: start/end column per row block.

Same functions and semantics as the reference's ``kernel_matmul/ranges.py:39-156``; the scans
run as CUDA kernels (``csrc/km_ranges.cu``) without leaving the device or synchronising, where
the reference copies ``x`` to the host and scans on one CPU thread
(native/ranges/ranges.cpp:8-101).  Integer results are bit-identical to the reference's.
"""
from __future__ import annotations

import ctypes
import math

import torch
from torch import Tensor

from . import _BLOCK_SIZE
from ._lib import check, lib


def _device_for(x: Tensor) -> torch.device:
    if x.is_cuda:
        return x.device
    if not torch.cuda.is_available():
        raise RuntimeError("kernel_matmul_b200.ranges needs a CUDA device (there is no CPU path)")
    return torch.device("cuda", torch.cuda.current_device())


def _ptr(t: Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def make_ranges(
    cutoff: float | None,
    x1: Tensor,
    x2: Tensor | None = None,
    *,
    block_size: int = _BLOCK_SIZE,
    align: bool = False,
) -> tuple[Tensor, Tensor]:
    """Compute the sparsity pattern for a given cutoff and input.

    Args:
        cutoff: cutoff distance; ``None`` gives the dense pattern ``[0, n)``.
        x1: ``(batch..., n1)``.
        x2: ``(batch..., n2)``; ``None`` gives the symmetric, block-aligned pattern of ``x1``.
        block_size: rows per block.
        align: round starts and ends to multiples of ``block_size`` so that the pattern can be
            transposed exactly (asymmetric case only; the symmetric pattern is always aligned).

    Returns:
        ``(start, end)`` int32 tensors of shape ``(batch..., ceil(n1 / block_size))`` on
        ``x1``'s device.
    """
    out_device = x1.device
    batch_shape = x1.shape[:-1]
    m = x1.shape[-1]
    rows = int(math.ceil(m / block_size))
    if cutoff is None:
        n = x2.shape[-1] if x2 is not None else m
        start = torch.zeros(*batch_shape, rows, dtype=torch.int32, device=out_device)
        end = torch.full((*batch_shape, rows), n, dtype=torch.int32, device=out_device)
        return start, end

    dev = _device_for(x1)
    x1d = x1.detach().to(device=dev, dtype=torch.float32).reshape(-1, m).contiguous()
    B = x1d.shape[0]
    start = torch.empty(B, rows, dtype=torch.int32, device=dev)
    end = torch.empty(B, rows, dtype=torch.int32, device=dev)
    flags = torch.empty(max(B, 1), dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    with torch.cuda.device(dev):
        if x2 is None:
            check(lib.km_make_ranges_symmetric_f32(B, m, _ptr(x1d), float(cutoff), block_size, _ptr(start),
                                                   _ptr(end), _ptr(flags), stream))
        else:
            if x2.shape[:-1] != batch_shape:
                raise RuntimeError("x1 and x2 must share their batch dimensions")
            n = x2.shape[-1]
            x2d = x2.detach().to(device=dev, dtype=torch.float32).reshape(-1, n).contiguous()
            check(lib.km_make_ranges_f32(B, m, n, _ptr(x1d), _ptr(x2d), float(cutoff), block_size,
                                         1 if align else 0, _ptr(start), _ptr(end), _ptr(flags), stream))
    start = start.reshape(*batch_shape, rows).to(out_device)
    end = end.reshape(*batch_shape, rows).to(out_device)
    return start, end


def make_ranges_symmetric_cutoffs(cutoffs: Tensor, x: Tensor, *, block_size: int = _BLOCK_SIZE) -> tuple[Tensor, Tensor]:
    """The symmetric, block-aligned patterns of ``B`` kernels with their own cutoffs in one call.

    ``cutoffs``: ``(B,)`` float tensor; ``x``: ``(n,)`` (shared by all) or ``(B, n)``.  Returns
    ``(start, end)`` of shape ``(B, ceil(n / block_size))``, equal to stacking
    ``make_ranges(cutoffs[b], x[b])``.  A mixture of components with different lengthscales over
    the same inputs builds its bands with one set of launches instead of ``B`` (the reference
    takes one cutoff per call, kernel_matmul/ranges.py:14-60).
    """
    if cutoffs.dim() != 1 or x.dim() not in (1, 2) or (x.dim() == 2 and x.shape[0] != cutoffs.shape[0]):
        raise RuntimeError("cutoffs must be (B,) and x (n,) or (B, n)")
    out_device = x.device
    dev = _device_for(x)
    B, n = cutoffs.shape[0], x.shape[-1]
    rows = int(math.ceil(n / block_size))
    xd = x.detach().to(device=dev, dtype=torch.float32).contiguous()
    cd = cutoffs.detach().to(device=dev, dtype=torch.float32).contiguous()
    start = torch.empty(B, rows, dtype=torch.int32, device=dev)
    end = torch.empty(B, rows, dtype=torch.int32, device=dev)
    flags = torch.empty(max(B, 1), dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    with torch.cuda.device(dev):
        check(lib.km_make_ranges_symmetric_cutoffs_f32(B, n, _ptr(xd), n if x.dim() == 2 else 0, _ptr(cd), block_size,
                                                       _ptr(start), _ptr(end), _ptr(flags), stream))
    return start.to(out_device), end.to(out_device)


def transpose_ranges(
    start: Tensor, end: Tensor, x1_size: int, x2_size: int, *, block_size: int = _BLOCK_SIZE
) -> tuple[Tensor, Tensor]:
    """Transpose a block-aligned sparsity pattern.

    Raises:
        ValueError: if the pattern is not block-aligned (as the reference does,
            kernel_matmul/ranges.py:110-113).
    """
    if torch.any(torch.logical_and(start % block_size != 0, start != x2_size)) or torch.any(
        torch.logical_and(end % block_size != 0, end != x2_size)
    ):
        raise ValueError("Ranges must be block-aligned")

    out_device = start.device
    dev = _device_for(start)
    batch_shape = start.shape[:-1]
    R = start.shape[-1]
    s = start.detach().to(device=dev, dtype=torch.int32).reshape(-1, R).contiguous()
    e = end.detach().to(device=dev, dtype=torch.int32).reshape(-1, R).contiguous()
    B = s.shape[0]
    C = int(math.ceil(x2_size / block_size))
    start_t = torch.empty(B, C, dtype=torch.int32, device=dev)
    end_t = torch.empty(B, C, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    with torch.cuda.device(dev):
        check(lib.km_transpose_ranges_i32(B, R, _ptr(s), _ptr(e), x1_size, x2_size, block_size, _ptr(start_t),
                                          _ptr(end_t), stream))
    return (start_t.reshape(*batch_shape, C).to(out_device), end_t.reshape(*batch_shape, C).to(out_device))


class RangesCache:
    """Cache of sparsity patterns for a fixed ``x = x1 = x2`` and variable cutoff; indexable by
    cutoff like a dictionary (kernel_matmul/ranges.py:130-156)."""

    _cache: dict[float | None, tuple[Tensor, Tensor]]

    def __init__(self, x: Tensor, align: bool = False):
        self._x = x
        self._cache = {}
        self._align = align

    @property
    def x(self):
        return self._x

    @property
    def align(self):
        return self._align

    def __getitem__(self, cutoff: float | None) -> tuple[Tensor, Tensor]:
        entry = self._cache.get(cutoff)
        if entry is None:
            entry = make_ranges(cutoff, self._x, align=self._align)
            self._cache[cutoff] = entry
        return entry
