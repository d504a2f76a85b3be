"""ctypes front end of the C oracle (``km_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Every function takes CPU tensors (or anything ``torch.as_tensor`` accepts) shaped like the
arguments of the reference's native ops (arbitrary leading batch dims, possibly expanded with
stride 0) and returns fp64 / int32 torch tensors.  Only ``tests/``, the smoke check and the
CPU-baseline leg of ``bench.py`` may import this module.
"""
from __future__ import annotations

import ctypes
import math
from typing import Sequence

import numpy as np
import torch

from . import build as _build

KERNEL_TYPES = {"rbf": 0, "spectral": 1, "locally_periodic": 2}
NUM_PARAMS = {"rbf": 2, "spectral": 3, "locally_periodic": 4}
BLOCK_SIZE = 128

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
        _lib.kmo_count_entries.restype = ctypes.c_int64
    return _lib


def _f32p(a: np.ndarray):
    assert a.dtype == np.float32
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _i32p(a: np.ndarray):
    assert a.dtype == np.int32
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))


def _i64p(a: np.ndarray):
    assert a.dtype == np.int64
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))


def _f64p(a: np.ndarray):
    assert a.dtype == np.float64
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def _flat(t, batch_shape: Sequence[int], nonbatch: int, dtype) -> tuple[np.ndarray, int]:
    """Return (contiguous numpy array, batch stride in elements) for a tensor whose leading
    dims broadcast to ``batch_shape``.  A tensor that is constant along every batch dim is
    passed once with stride 0; anything else is materialised as (B, ...)."""
    t = torch.as_tensor(t).detach().cpu()
    core = t.shape[t.dim() - nonbatch :]
    lead = t.shape[: t.dim() - nonbatch]
    if all(s == 1 for s in lead) or all(
        st == 0 or sz == 1 for st, sz in zip(t.stride()[: len(lead)], lead)
    ):
        idx = (0,) * len(lead)
        single = t[idx].contiguous().to(dtype).numpy()
        return np.ascontiguousarray(single), 0
    full = t.expand(*batch_shape, *core).reshape(-1, *core).contiguous().to(dtype).numpy()
    return np.ascontiguousarray(full), int(np.prod(core)) if len(core) else 1


def _batch_shape(*pairs) -> tuple[int, ...]:
    shapes = [torch.as_tensor(t).shape[: torch.as_tensor(t).dim() - nb] for t, nb in pairs]
    return tuple(torch.broadcast_shapes(*shapes))


def matmul(kernel_type, x1, x2, rhs, params, start, end, *, block=BLOCK_SIZE, row_blocks=None):
    """fp64 K_masked @ rhs.  With ``row_blocks`` (list of row-block indices) only those blocks
    are computed and the result has shape (*batch, len(row_blocks), block, k)."""
    kt = KERNEL_TYPES[kernel_type]
    bs = _batch_shape((x1, 1), (x2, 1), (rhs, 2), (params, 1), (start, 1), (end, 1))
    B = int(np.prod(bs)) if bs else 1
    m, n, k = torch.as_tensor(x1).shape[-1], torch.as_tensor(x2).shape[-1], torch.as_tensor(rhs).shape[-1]
    a1, s1 = _flat(x1, bs, 1, torch.float32)
    a2, s2 = _flat(x2, bs, 1, torch.float32)
    ar, sr = _flat(rhs, bs, 2, torch.float32)
    ap, sp = _flat(params, bs, 1, torch.float32)
    # start and end share one stride: materialise both the same way
    st = torch.as_tensor(start).detach().cpu()
    en = torch.as_tensor(end).detach().cpu()
    R = st.shape[-1]
    assert R == math.ceil(m / block), (R, m, block)
    ast = st.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    aen = en.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    if row_blocks is None:
        out = np.zeros((B, m, k), dtype=np.float64)
        rbp, nrb = None, 0
    else:
        rb = np.ascontiguousarray(np.asarray(row_blocks, dtype=np.int32))
        out = np.zeros((B, len(rb), block, k), dtype=np.float64)
        rbp, nrb = _i32p(rb), len(rb)
    lib().kmo_matmul(
        ctypes.c_int(kt), ctypes.c_int64(B), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k),
        ctypes.c_int(block),
        _f32p(a1), ctypes.c_int64(s1), _f32p(a2), ctypes.c_int64(s2),
        _f32p(ar), ctypes.c_int64(sr), _f32p(ap), ctypes.c_int64(sp),
        _i32p(ast), _i32p(aen), ctypes.c_int64(R),
        rbp, ctypes.c_int(nrb), _f64p(out),
    )
    return torch.from_numpy(out).reshape(*bs, *out.shape[1:])


def bilinear_derivative(kernel_type, x1, x2, left, right, params, start, end, *, block=BLOCK_SIZE, absolute=False):
    """fp64 d/dtheta sum_c left[:,c]^T K_masked right[:,c]  ->  (*batch, P).
    With left = out_grad and right = rhs this is the reference's matmul_bwd.
    ``absolute=True`` returns the sum of the magnitudes of the terms instead (error scale)."""
    kt = KERNEL_TYPES[kernel_type]
    P = NUM_PARAMS[kernel_type]
    bs = _batch_shape((x1, 1), (x2, 1), (left, 2), (right, 2), (params, 1), (start, 1), (end, 1))
    B = int(np.prod(bs)) if bs else 1
    m, n, k = torch.as_tensor(x1).shape[-1], torch.as_tensor(x2).shape[-1], torch.as_tensor(left).shape[-1]
    a1, s1 = _flat(x1, bs, 1, torch.float32)
    a2, s2 = _flat(x2, bs, 1, torch.float32)
    al, sl = _flat(left, bs, 2, torch.float32)
    ar, sr = _flat(right, bs, 2, torch.float32)
    ap, sp = _flat(params, bs, 1, torch.float32)
    st = torch.as_tensor(start).detach().cpu()
    R = st.shape[-1]
    ast = st.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    aen = torch.as_tensor(end).detach().cpu().expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    out = np.zeros((B, P), dtype=np.float64)
    lib().kmo_bilinear_derivative(
        ctypes.c_int(kt), ctypes.c_int64(B), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k),
        ctypes.c_int(block),
        _f32p(a1), ctypes.c_int64(s1), _f32p(a2), ctypes.c_int64(s2),
        _f32p(al), ctypes.c_int64(sl), _f32p(ar), ctypes.c_int64(sr),
        _f32p(ap), ctypes.c_int64(sp),
        _i32p(ast), _i32p(aen), ctypes.c_int64(R), ctypes.c_int(1 if absolute else 0), _f64p(out),
    )
    return torch.from_numpy(out).reshape(*bs, P)


def matmul_bwd(kernel_type, x1, x2, rhs, params, start, end, out_grad, *, block=BLOCK_SIZE, absolute=False):
    return bilinear_derivative(kernel_type, x1, x2, out_grad, rhs, params, start, end, block=block, absolute=absolute)


def dense(kernel_type, x1, x2, params, start, end, *, block=BLOCK_SIZE):
    kt = KERNEL_TYPES[kernel_type]
    bs = _batch_shape((x1, 1), (x2, 1), (params, 1), (start, 1), (end, 1))
    B = int(np.prod(bs)) if bs else 1
    m, n = torch.as_tensor(x1).shape[-1], torch.as_tensor(x2).shape[-1]
    a1, s1 = _flat(x1, bs, 1, torch.float32)
    a2, s2 = _flat(x2, bs, 1, torch.float32)
    ap, sp = _flat(params, bs, 1, torch.float32)
    st = torch.as_tensor(start).detach().cpu()
    R = st.shape[-1]
    ast = st.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    aen = torch.as_tensor(end).detach().cpu().expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    out = np.zeros((B, m, n), dtype=np.float64)
    lib().kmo_dense(
        ctypes.c_int(kt), ctypes.c_int64(B), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(block),
        _f32p(a1), ctypes.c_int64(s1), _f32p(a2), ctypes.c_int64(s2), _f32p(ap), ctypes.c_int64(sp),
        _i32p(ast), _i32p(aen), ctypes.c_int64(R), _f64p(out),
    )
    return torch.from_numpy(out).reshape(*bs, m, n)


def dense_bwd(kernel_type, x1, x2, params, start, end, out_grad, *, block=BLOCK_SIZE, absolute=False):
    kt = KERNEL_TYPES[kernel_type]
    P = NUM_PARAMS[kernel_type]
    bs = _batch_shape((x1, 1), (x2, 1), (params, 1), (start, 1), (end, 1), (out_grad, 2))
    B = int(np.prod(bs)) if bs else 1
    m, n = torch.as_tensor(x1).shape[-1], torch.as_tensor(x2).shape[-1]
    a1, s1 = _flat(x1, bs, 1, torch.float32)
    a2, s2 = _flat(x2, bs, 1, torch.float32)
    ap, sp = _flat(params, bs, 1, torch.float32)
    ag, sg = _flat(out_grad, bs, 2, torch.float32)
    st = torch.as_tensor(start).detach().cpu()
    R = st.shape[-1]
    ast = st.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    aen = torch.as_tensor(end).detach().cpu().expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    out = np.zeros((B, P), dtype=np.float64)
    lib().kmo_dense_bwd(
        ctypes.c_int(kt), ctypes.c_int64(B), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(block),
        _f32p(a1), ctypes.c_int64(s1), _f32p(a2), ctypes.c_int64(s2), _f32p(ap), ctypes.c_int64(sp),
        _i32p(ast), _i32p(aen), ctypes.c_int64(R), _f32p(ag), ctypes.c_int64(sg),
        ctypes.c_int(1 if absolute else 0), _f64p(out),
    )
    return torch.from_numpy(out).reshape(*bs, P)


def _flatten_batch_indices(batch_indices, batch_shape, shape) -> np.ndarray:
    flat = torch.zeros(shape, dtype=torch.int64)
    for idx, size in zip(batch_indices, batch_shape):
        flat = flat * size + torch.as_tensor(idx).cpu().to(torch.int64).expand(shape)
    return np.ascontiguousarray(flat.reshape(-1).numpy())


def index(kernel_type, x1, x2, params, start, end, batch_indices, row_index, col_index, *, block=BLOCK_SIZE):
    kt = KERNEL_TYPES[kernel_type]
    bs = _batch_shape((x1, 1), (x2, 1), (params, 1), (start, 1), (end, 1))
    assert len(batch_indices) == len(bs)
    a1, s1 = _flat(x1, bs, 1, torch.float32)
    a2, s2 = _flat(x2, bs, 1, torch.float32)
    ap, sp = _flat(params, bs, 1, torch.float32)
    st = torch.as_tensor(start).detach().cpu()
    R = st.shape[-1]
    ast = st.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    aen = torch.as_tensor(end).detach().cpu().expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    row = torch.as_tensor(row_index).cpu()
    shape = tuple(row.shape)
    fb = _flatten_batch_indices(batch_indices, bs, shape)
    r = np.ascontiguousarray(row.reshape(-1).to(torch.int32).numpy())
    c = np.ascontiguousarray(torch.as_tensor(col_index).cpu().reshape(-1).to(torch.int32).numpy())
    out = np.zeros(len(r), dtype=np.float64)
    lib().kmo_index(
        ctypes.c_int(kt), ctypes.c_int64(len(r)), ctypes.c_int(block),
        _f32p(a1), ctypes.c_int64(s1), _f32p(a2), ctypes.c_int64(s2), _f32p(ap), ctypes.c_int64(sp),
        _i32p(ast), _i32p(aen), ctypes.c_int64(R), _i64p(fb), _i32p(r), _i32p(c), _f64p(out),
    )
    return torch.from_numpy(out).reshape(shape)


def index_bwd(kernel_type, x1, x2, params, start, end, batch_indices, row_index, col_index, out_grad, *, block=BLOCK_SIZE, absolute=False):
    kt = KERNEL_TYPES[kernel_type]
    P = NUM_PARAMS[kernel_type]
    bs = _batch_shape((x1, 1), (x2, 1), (params, 1), (start, 1), (end, 1))
    B = int(np.prod(bs)) if bs else 1
    a1, s1 = _flat(x1, bs, 1, torch.float32)
    a2, s2 = _flat(x2, bs, 1, torch.float32)
    ap, sp = _flat(params, bs, 1, torch.float32)
    st = torch.as_tensor(start).detach().cpu()
    R = st.shape[-1]
    ast = st.expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    aen = torch.as_tensor(end).detach().cpu().expand(*bs, R).reshape(-1, R).contiguous().to(torch.int32).numpy()
    row = torch.as_tensor(row_index).cpu()
    shape = tuple(row.shape)
    fb = _flatten_batch_indices(batch_indices, bs, shape)
    r = np.ascontiguousarray(row.reshape(-1).to(torch.int32).numpy())
    c = np.ascontiguousarray(torch.as_tensor(col_index).cpu().reshape(-1).to(torch.int32).numpy())
    g = np.ascontiguousarray(torch.as_tensor(out_grad).detach().cpu().expand(shape).reshape(-1).to(torch.float32).numpy())
    out = np.zeros((B, P), dtype=np.float64)
    lib().kmo_index_bwd(
        ctypes.c_int(kt), ctypes.c_int64(B), ctypes.c_int64(len(r)), ctypes.c_int(block),
        _f32p(a1), ctypes.c_int64(s1), _f32p(a2), ctypes.c_int64(s2), _f32p(ap), ctypes.c_int64(sp),
        _i32p(ast), _i32p(aen), ctypes.c_int64(R), _i64p(fb), _i32p(r), _i32p(c), _f32p(g),
        ctypes.c_int(1 if absolute else 0), _f64p(out),
    )
    return torch.from_numpy(out).reshape(*bs, P)


# ------------------------------------------------------------------------------ bands


def _as2d(x) -> tuple[np.ndarray, tuple[int, ...]]:
    t = torch.as_tensor(x).detach().cpu().to(torch.float32)
    bs = tuple(t.shape[:-1])
    return np.ascontiguousarray(t.reshape(-1, t.shape[-1]).contiguous().numpy()), bs


def make_ranges(cutoff, x1, x2=None, *, block_size=BLOCK_SIZE, align=False):
    """Same contract as the reference's ``kernel_matmul.ranges.make_ranges``
    (kernel_matmul/ranges.py:39-89), CPU int32 outputs."""
    a1, bs = _as2d(x1)
    B, m = a1.shape
    R = math.ceil(m / block_size)
    if cutoff is None:
        n = m if x2 is None else torch.as_tensor(x2).shape[-1]
        start = torch.zeros(*bs, R, dtype=torch.int32)
        end = torch.full((*bs, R), n, dtype=torch.int32)
        return start, end
    start = np.zeros((B, R), dtype=np.int32)
    end = np.zeros((B, R), dtype=np.int32)
    if x2 is None:
        lib().kmo_make_ranges_symmetric(
            ctypes.c_int64(B), ctypes.c_int(m), _f32p(a1), ctypes.c_float(cutoff),
            ctypes.c_int(block_size), _i32p(start), _i32p(end),
        )
    else:
        a2, _ = _as2d(x2)
        lib().kmo_make_ranges(
            ctypes.c_int64(B), ctypes.c_int(m), ctypes.c_int(a2.shape[1]), _f32p(a1), _f32p(a2),
            ctypes.c_float(cutoff), ctypes.c_int(block_size), ctypes.c_int(1 if align else 0),
            _i32p(start), _i32p(end),
        )
    return torch.from_numpy(start).reshape(*bs, R), torch.from_numpy(end).reshape(*bs, R)


def transpose_ranges(start, end, x1_size, x2_size, *, block_size=BLOCK_SIZE):
    """kernel_matmul/ranges.py:92-127, including its ValueError for unaligned patterns."""
    st = torch.as_tensor(start).cpu().to(torch.int32)
    en = torch.as_tensor(end).cpu().to(torch.int32)
    if torch.any((st % block_size != 0) & (st != x2_size)) or torch.any(
        (en % block_size != 0) & (en != x2_size)
    ):
        raise ValueError("Ranges must be block-aligned")
    bs = tuple(st.shape[:-1])
    R = st.shape[-1]
    s2 = np.ascontiguousarray(st.reshape(-1, R).contiguous().numpy())
    e2 = np.ascontiguousarray(en.reshape(-1, R).contiguous().numpy())
    B = s2.shape[0]
    C = math.ceil(x2_size / block_size)
    st_t = np.zeros((B, C), dtype=np.int32)
    en_t = np.zeros((B, C), dtype=np.int32)
    lib().kmo_transpose_ranges(
        ctypes.c_int64(B), ctypes.c_int(R), _i32p(s2), _i32p(e2), ctypes.c_int(x1_size),
        ctypes.c_int(x2_size), ctypes.c_int(block_size), _i32p(st_t), _i32p(en_t),
    )
    return torch.from_numpy(st_t).reshape(*bs, C), torch.from_numpy(en_t).reshape(*bs, C)


def count_entries(m, n, start, end, *, block=BLOCK_SIZE) -> int:
    st = torch.as_tensor(start).cpu().to(torch.int32)
    R = st.shape[-1]
    s2 = np.ascontiguousarray(st.reshape(-1, R).contiguous().numpy())
    e2 = np.ascontiguousarray(torch.as_tensor(end).cpu().to(torch.int32).reshape(-1, R).contiguous().numpy())
    return int(
        lib().kmo_count_entries(
            ctypes.c_int64(s2.shape[0]), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(block),
            _i32p(s2), _i32p(e2), ctypes.c_int64(R),
        )
    )
