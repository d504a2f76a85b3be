"""The native ops of the hot path, with the call signatures of the reference's per-op modules.

Each function is what ``load_native(<op>, defines).call`` is in the reference
(``native/<op>/<op>.cpp``), with the kernel type as a runtime argument instead of a
``-DKM_KERNEL_*`` define.  PyTorch is used for device memory and the current stream only;
all arithmetic runs in ``libkm_b200.so`` through its C ABI (``include/km_b200.h``).

Conventions shared with the reference: fp32 CUDA tensors, int32 ranges and indices; arbitrary
leading batch dims shared by all arguments (expanded / stride-0 views are used as they are,
never materialised); gradients are produced for ``params`` only.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch
from torch import Tensor

from . import _lib
from ._lib import KM_MAX_BATCH_DIMS, KERNEL_TYPES, KmBatch, KmView, lib
from ._lib import check as _check

BLOCK_SIZE = 128
NUM_PARAMS = {"rbf": 2, "spectral": 3, "locally_periodic": 4}


def _kernel_id(kernel_type: str) -> int:
    try:
        return KERNEL_TYPES[kernel_type]
    except KeyError:
        raise ValueError(f"Unknown kernel type: {kernel_type}") from None


def _check_cuda(x: Tensor) -> None:
    # native/common/entrypoint.h:3-5
    if not isinstance(x, Tensor) or not x.is_cuda:
        raise RuntimeError("x must be a CUDA tensor")


def _check_f32(x: Tensor) -> None:
    _check_cuda(x)
    if x.dtype != torch.float32:
        raise RuntimeError("x must be float32")


def _check_i32(x: Tensor) -> None:
    # native/common/entrypoint.h:7-14
    _check_cuda(x)
    if x.dtype != torch.int32:
        raise RuntimeError("x must be int32")


def _same_device(*tensors: Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors[1:]:
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
    return dev


def _common_batch(tensors_nb: Sequence[tuple[Tensor, int]]) -> tuple[int, ...]:
    shapes = []
    for t, nb in tensors_nb:
        if t.dim() < nb:
            raise RuntimeError(f"tensor of rank {t.dim()} needs at least {nb} trailing dims")
        shapes.append(t.shape[: t.dim() - nb])
    try:
        return tuple(torch.broadcast_shapes(*shapes))
    except RuntimeError as exc:
        raise RuntimeError(f"batch dimensions do not broadcast: {[tuple(s) for s in shapes]}") from exc


def _expand(t: Tensor, batch: tuple[int, ...], nb: int) -> Tensor:
    core = t.shape[t.dim() - nb :]
    t = t.expand(*batch, *core)
    if len(batch) > KM_MAX_BATCH_DIMS:
        # more batch dims than the ABI carries: flatten them (copies only if not collapsible)
        t = t.reshape(-1, *core)
    return t


def _km_batch(batch: tuple[int, ...]) -> KmBatch:
    if len(batch) > KM_MAX_BATCH_DIMS:
        n = 1
        for s in batch:
            n *= s
        batch = (n,)
    b = KmBatch()
    b.ndim = len(batch)
    for d, s in enumerate(batch):
        b.size[d] = s
    return b


def _view(t: Tensor, nb: int) -> KmView:
    v = KmView()
    v.data = t.data_ptr()
    st = t.stride()
    nbatch = t.dim() - nb
    for d in range(nbatch):
        v.batch_stride[d] = st[d]
    for d in range(nb):
        v.stride[d] = st[nbatch + d]
    return v


def _stream(dev: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _prep(kernel_type: str, x1, x2, params, start, end, extra: Sequence[tuple[Tensor, int]] = ()):
    """Common validation / broadcasting.  Returns (kid, device, batch shape, expanded tensors)."""
    kid = _kernel_id(kernel_type)
    for t in (x1, x2, params):
        _check_f32(t)
    for t in (start, end):
        _check_i32(t)
    for t, _ in extra:
        _check_f32(t)
    dev = _same_device(x1, x2, params, start, end, *(t for t, _ in extra))
    _state(dev).poll(wait=False)  # a tensor-core launch that gave up since the last call raises here
    P = NUM_PARAMS[kernel_type]
    if params.shape[-1] != P:
        raise RuntimeError(f"params must have {P} entries in the last dim for kernel '{kernel_type}', got {params.shape[-1]}")
    m, n = x1.shape[-1], x2.shape[-1]
    R = -(-m // BLOCK_SIZE)
    if start.shape[-1] != R or end.shape[-1] != R:
        raise RuntimeError(f"start/end must have ceil(m/{BLOCK_SIZE}) = {R} entries, got {start.shape[-1]} and {end.shape[-1]}")
    pairs = [(x1, 1), (x2, 1), (params, 1), (start, 1), (end, 1), *extra]
    batch = _common_batch(pairs)
    expanded = [_expand(t, batch, nb) for t, nb in pairs]
    return kid, dev, batch, m, n, expanded


class KernelGaveUpError(RuntimeError):
    """A tensor-core kernel stopped at a hand-off wait that ran out (status word != 0).  The
    results of that launch are invalid (and NaN where the failing CTAs would have written)."""


class _DeviceState:
    """Per device and stream: one cached workspace for the tensor-core kernels and the status
    words of the launches whose outcome has not been looked at yet.

    Every tensor-core launch is followed by an asynchronous 4-byte copy of its status word into
    pinned host memory and an event.  The next op call on the device looks at the copies whose
    events have completed (no synchronisation) and raises ``KernelGaveUpError`` if one is
    non-zero; ``check()`` synchronises first, so that it covers everything launched so far.
    """

    def __init__(self) -> None:
        self.workspaces: dict[int, Tensor] = {}  # stream id -> uint8 workspace
        self.pending: list[tuple[torch.cuda.Event, Tensor, str]] = []
        self.free_words: list[Tensor] = []

    def workspace(self, dev: torch.device, nbytes: int) -> Tensor:
        key = torch.cuda.current_stream(dev).cuda_stream
        ws = self.workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            # grows geometrically; launches that still use the old buffer keep it alive through
            # the stream-ordered allocator
            ws = torch.empty(max(nbytes, 2 * (ws.numel() if ws is not None else 0), 256), device=dev, dtype=torch.uint8)
            self.workspaces[key] = ws
        return ws

    def track(self, ws: Tensor, what: str) -> None:
        word = self.free_words.pop() if self.free_words else torch.zeros(1, dtype=torch.int32).pin_memory()
        word.copy_(ws[:4].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(ws.device))
        self.pending.append((ev, word, what))

    def poll(self, wait: bool) -> None:
        failed = None
        keep = []
        for ev, word, what in self.pending:
            if wait:
                ev.synchronize()
            if wait or ev.query():
                if int(word[0]) != 0 and failed is None:
                    failed = what
                self.free_words.append(word)
            else:
                keep.append((ev, word, what))
        self.pending = keep
        if failed is not None:
            raise KernelGaveUpError(
                f"{failed}: a bounded wait inside the tensor-core kernel gave up (status word != 0); "
                "the results of that call are invalid")


_device_state: dict[int, _DeviceState] = {}


def _state(dev: torch.device) -> _DeviceState:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _device_state.get(idx)
    if st is None:
        st = _device_state[idx] = _DeviceState()
    return st


def check(device: torch.device | int | None = None) -> None:
    """Wait for every tensor-core launch made so far (on ``device``, default: all devices used)
    and raise ``KernelGaveUpError`` if one of them gave up at a hand-off wait.  Op calls do the
    same check, without waiting, for the launches that have already finished."""
    if device is None:
        states = list(_device_state.values())
    else:
        d = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        states = [_state(d)]
    for st in states:
        st.poll(wait=True)


#: rhs widths from which ``matmul`` runs the contraction on the tensor cores (tcgen05; fp16
#: hi/lo operand split, kernel tiles handed over in tensor memory).  The cost of that kernel
#: hardly depends on the width; below 9 columns the FMA pipe is as fast.
TENSOR_CORE_MIN_K = 9
#: The tensor-core kernels run a pre-pass over the rhs (two or three small launches); they are
#: chosen on ``path="auto"`` only for problems with at least this many (batch, row block) items.
TENSOR_CORE_MIN_ITEMS = 256


def _enough_items(batch: tuple[int, ...], m: int) -> bool:
    items = -(-m // BLOCK_SIZE)
    for b in batch:
        items *= b
    return items >= TENSOR_CORE_MIN_ITEMS


def matmul(kernel_type: str, x1: Tensor, x2: Tensor, rhs: Tensor, params: Tensor, start: Tensor, end: Tensor,
           *, path: str = "auto") -> Tensor:
    """``K(x1, x2; params)[masked by ranges] @ rhs`` -> ``(*batch, m, k)``.

    Reference: ``matmul.call(x1, x2, rhs, params, start, end)`` (native/matmul/matmul.cpp:6-17).
    ``path``: ``"fma"`` (FP32 pipe), ``"tc"`` (tensor cores; fp32-level accuracy through operand
    splitting) or ``"auto"`` (tensor cores from ``TENSOR_CORE_MIN_K`` rhs columns, if the problem
    has ``TENSOR_CORE_MIN_ITEMS`` work items).
    """
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee, re) = _prep(kernel_type, x1, x2, params, start, end, [(rhs, 2)])
    if rhs.shape[-2] != n:
        raise RuntimeError(f"rhs must have n = {n} rows, got {rhs.shape[-2]}")
    k = rhs.shape[-1]
    if path not in ("auto", "fma", "tc"):
        raise ValueError(f"unknown path {path!r}")
    out = torch.empty(*batch, m, k, device=dev, dtype=torch.float32)
    oute = out.reshape(-1, m, k) if len(batch) > KM_MAX_BATCH_DIMS else out
    if path == "tc" or (path == "auto" and k >= TENSOR_CORE_MIN_K and _enough_items(batch, m)):
        kb = _km_batch(batch)
        rv = _view(re, 2)
        ws_bytes = lib.km_matmul_tc_workspace_bytes(kb, n, k, rv)
        st = _state(dev)
        ws = st.workspace(dev, ws_bytes)
        with torch.cuda.device(dev):
            _check(lib.km_matmul_tc_f32(
                kid, kb, m, n, k, _view(x1e, 1), _view(x2e, 1), rv, _view(pe, 1), _view(se, 1), _view(ee, 1),
                _view(oute, 2), ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream(dev)))
            st.track(ws, "matmul")
        out._km_tensor_cores = True
        return out
    with torch.cuda.device(dev):
        _check(lib.km_matmul_f32(
            kid, _km_batch(batch), m, n, k, _view(x1e, 1), _view(x2e, 1), _view(re, 2), _view(pe, 1),
            _view(se, 1), _view(ee, 1), _view(oute, 2), _stream(dev)))
    return out


def used_tensor_cores(result: Tensor) -> bool:
    """Whether the op call that returned ``result`` ran its tensor-core kernel."""
    return bool(getattr(result, "_km_tensor_cores", False))


def tc_status(out: Tensor) -> int:
    """1 if a tensor-core launch on ``out``'s device has given up since the last check, else 0
    (synchronises the device's launches; kept for callers that poll instead of catching
    ``KernelGaveUpError`` from ``check``)."""
    try:
        check(out.device)
    except KernelGaveUpError:
        return 1
    return 0


def prepare_sum_phases(kernel_type: str, x1: Tensor, x2: Tensor, params: Tensor, *, rows: tuple[int, int] | None = None,
                       cols: tuple[int, int] | None = None) -> Tensor | None:
    """Phase images for the batch sum of spectral components (``km_sum_phases_prepare_f32``): the
    per-point vectors ``(cos, sin)(2 pi f_b x)`` of all rows and columns, written once per operator
    in the layouts the tensor-core kernel takes them.  Pass the returned workspace to
    ``matmul_rows(..., sum_batches=True, phases=...)``: products with the same ``x1``, ``x2`` and
    ``params`` (frequencies and output scales; one common lengthscale) then copy the vectors instead
    of evaluating them again for every row block.  ``None`` where it does not apply (another kernel
    type, fewer than 2 or more than 1024 components); ``x1`` / ``x2`` of shape ``(m,)`` / ``(n,)``.
    ``rows`` / ``cols``: write only these rows and columns (what the products of one rank of a
    row-sharded solve read: its own rows and the columns of their bands)."""
    if kernel_type != "spectral" or params.dim() < 2:
        return None
    batch = tuple(params.shape[:-1])
    comps = 1
    for b in batch:
        comps *= int(b)
    if comps < 2 or comps > 1024 or len(batch) > KM_MAX_BATCH_DIMS:
        return None
    if x1.dim() != 1 or x2.dim() != 1:
        raise RuntimeError("prepare_sum_phases takes the shared inputs x1 (m,) and x2 (n,)")
    if params.shape[-1] != NUM_PARAMS[kernel_type]:
        raise RuntimeError(f"params must have {NUM_PARAMS[kernel_type]} entries in the last dim")
    for t in (x1, x2, params):
        _check_f32(t)
    dev = _same_device(x1, x2, params)
    m, n = x1.shape[0], x2.shape[0]
    x1e, x2e = x1.expand(*batch, m), x2.expand(*batch, n)
    kb = _km_batch(batch)
    nbytes = int(lib.km_sum_phases_workspace_bytes(kb, m, n))
    raw = torch.empty(max(nbytes, 256) + 256, dtype=torch.uint8, device=dev)
    ws = raw[(-raw.data_ptr()) % 256:][:max(nbytes, 256)]
    with torch.cuda.device(dev):
        r0, r1 = rows if rows is not None else (0, m)
        c0, c1 = cols if cols is not None else (0, n)
        _check(lib.km_sum_phases_prepare_f32(kb, m, n, _view(x1e, 1), _view(x2e, 1), _view(params, 1), r0, r1, c0, c1,
                                             ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream(dev)))
    return ws


def matmul_rows(kernel_type: str, x1: Tensor, x2: Tensor, rhs: Tensor, params: Tensor, start: Tensor, end: Tensor,
                *, row_block_begin: int = 0, row_block_count: int | None = None, sum_batches: bool = False,
                out: Tensor | None = None, path: str = "auto", phases: Tensor | None = None) -> Tensor:
    """``matmul`` restricted to the row blocks ``[row_block_begin, row_block_begin + row_block_count)``
    and, with ``sum_batches``, summed over all batch dims inside the kernel.

    Returns ``(*batch, rows, k)`` or, with ``sum_batches``, ``(rows, k)``, where ``rows`` is the
    number of rows of ``x1`` inside the window.  ``out`` may be passed to receive the result
    (e.g. a rank's slice of an all-gather buffer).  ``path`` as in ``matmul`` (the batch sum runs
    on the FMA pipe).  ``phases``: the workspace of ``prepare_sum_phases`` for this operator (batch
    sum only).
    """
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee, re) = _prep(kernel_type, x1, x2, params, start, end, [(rhs, 2)])
    if rhs.shape[-2] != n:
        raise RuntimeError(f"rhs must have n = {n} rows, got {rhs.shape[-2]}")
    k = rhs.shape[-1]
    R = -(-m // BLOCK_SIZE)
    if row_block_count is None:
        row_block_count = R - row_block_begin
    if row_block_begin < 0 or row_block_count < 0 or row_block_begin + row_block_count > R:
        raise RuntimeError(f"row-block window [{row_block_begin}, {row_block_begin + row_block_count}) outside [0, {R})")
    rows = max(0, min(m, (row_block_begin + row_block_count) * BLOCK_SIZE) - row_block_begin * BLOCK_SIZE)
    shape = (rows, k) if sum_batches else (*batch, rows, k)
    if out is None:
        out = torch.empty(shape, device=dev, dtype=torch.float32)
    elif tuple(out.shape) != shape or out.dtype != torch.float32 or out.device != dev:
        raise RuntimeError(f"out must be a float32 tensor of shape {shape} on {dev}")
    if sum_batches and len(batch) == 0:
        sum_batches = False  # a single kernel: nothing to sum
    oute = out.reshape(-1, rows, k) if (len(batch) > KM_MAX_BATCH_DIMS and not sum_batches) else out
    if path not in ("auto", "fma", "tc"):
        raise ValueError(f"unknown path {path!r}")
    if sum_batches and path == "tc":
        raise RuntimeError("the batch sum runs on the FMA pipe only")
    if not sum_batches and rows > 0 and (path == "tc" or (path == "auto" and k >= TENSOR_CORE_MIN_K and
                                                          _enough_items(batch, row_block_count * BLOCK_SIZE))):
        kb = _km_batch(batch)
        rv = _view(re, 2)
        ws_bytes = lib.km_matmul_tc_workspace_bytes(kb, n, k, rv)
        st = _state(dev)
        ws = st.workspace(dev, ws_bytes)
        with torch.cuda.device(dev):
            _check(lib.km_matmul_tc_rows_f32(
                kid, kb, m, n, k, _view(x1e, 1), _view(x2e, 1), rv, _view(pe, 1), _view(se, 1), _view(ee, 1),
                _view(oute, 2), row_block_begin, row_block_count, ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                _stream(dev)))
            st.track(ws, "matmul_rows")
        out._km_tensor_cores = True
        return out
    with torch.cuda.device(dev):
        if phases is not None and sum_batches:
            _check(lib.km_matmul_rows_phases_f32(
                kid, _km_batch(batch), m, n, k, _view(x1e, 1), _view(x2e, 1), _view(re, 2), _view(pe, 1),
                _view(se, 1), _view(ee, 1), _view(oute, 2), row_block_begin, row_block_count,
                ctypes.c_void_p(phases.data_ptr()), phases.numel(), _stream(dev)))
        else:
            _check(lib.km_matmul_rows_f32(
                kid, _km_batch(batch), m, n, k, _view(x1e, 1), _view(x2e, 1), _view(re, 2), _view(pe, 1),
                _view(se, 1), _view(ee, 1), _view(oute, 2), row_block_begin, row_block_count,
                1 if sum_batches else 0, _stream(dev)))
    return out


class PreparedRowsProduct:
    """``matmul_rows`` with everything but the launch done once: arguments validated and expanded,
    the C structures filled.  For loops that call the same product on the same buffers many times
    (a CG solve: ``rhs`` and ``out`` are fixed buffers whose CONTENTS change) -- a call is then one
    foreign-function call, a few microseconds of host time instead of a few hundred.  Only the
    entry point without a workspace (``km_matmul_rows_f32``: FMA pipe, and the batch sum on either
    pipe) can be prepared; ``prepare_matmul_rows`` returns ``None`` where ``matmul_rows`` would
    take the tensor-core kernel with its workspace."""

    def __init__(self, dev, args, keep, fn=None):
        self._dev, self._args, self._keep = dev, args, keep
        self._fn = fn if fn is not None else lib.km_matmul_rows_f32
        self._state = _state(dev)

    def __call__(self) -> None:
        self._state.poll(wait=False)
        with torch.cuda.device(self._dev):
            _check(self._fn(*self._args, _stream(self._dev)))


def prepare_matmul_rows(kernel_type: str, x1: Tensor, x2: Tensor, rhs: Tensor, params: Tensor, start: Tensor, end: Tensor,
                        *, row_block_begin: int, row_block_count: int, sum_batches: bool, out: Tensor,
                        phases: Tensor | None = None):
    """A ``PreparedRowsProduct`` that computes what ``matmul_rows(..., out=out)`` computes, or ``None``
    (see there).  The tensors must stay alive and in place; their contents may change between calls."""
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee, re) = _prep(kernel_type, x1, x2, params, start, end, [(rhs, 2)])
    if rhs.shape[-2] != n:
        raise RuntimeError(f"rhs must have n = {n} rows, got {rhs.shape[-2]}")
    k = rhs.shape[-1]
    R = -(-m // BLOCK_SIZE)
    if row_block_begin < 0 or row_block_count < 0 or row_block_begin + row_block_count > R:
        raise RuntimeError(f"row-block window [{row_block_begin}, {row_block_begin + row_block_count}) outside [0, {R})")
    rows = max(0, min(m, (row_block_begin + row_block_count) * BLOCK_SIZE) - row_block_begin * BLOCK_SIZE)
    if sum_batches and len(batch) == 0:
        sum_batches = False
    shape = (rows, k) if sum_batches else (*batch, rows, k)
    if tuple(out.shape) != shape or out.dtype != torch.float32 or out.device != dev:
        raise RuntimeError(f"out must be a float32 tensor of shape {shape} on {dev}")
    if len(batch) > KM_MAX_BATCH_DIMS:
        return None
    if not sum_batches and rows > 0 and k >= TENSOR_CORE_MIN_K and _enough_items(batch, row_block_count * BLOCK_SIZE):
        return None  # matmul_rows would run the tensor-core kernel, which needs a workspace per call
    kb = _km_batch(batch)
    views = [_view(x1e, 1), _view(x2e, 1), _view(re, 2), _view(pe, 1), _view(se, 1), _view(ee, 1), _view(out, 2)]
    if phases is not None and sum_batches:
        args = (kid, kb, m, n, k, *views, row_block_begin, row_block_count, ctypes.c_void_p(phases.data_ptr()), phases.numel())
        return PreparedRowsProduct(dev, args, (x1e, x2e, re, pe, se, ee, out, kb, views, phases), lib.km_matmul_rows_phases_f32)
    args = (kid, kb, m, n, k, *views, row_block_begin, row_block_count, 1 if sum_batches else 0)
    return PreparedRowsProduct(dev, args, (x1e, x2e, re, pe, se, ee, out, kb, views))


#: column count from which the gradient ops take the tensor-core kernel on ``path="auto"``
#: (if the problem has ``TENSOR_CORE_MIN_ITEMS`` work items)
GRAD_TENSOR_CORE_MIN_K = 8


def _grad_call(which: str, kernel_type, x1, x2, left, right, params, start, end, path: str) -> Tensor:
    """``which``: "matmul_bwd" (C argument order rhs ... out_grad) or "bilinear_derivative"."""
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee, le, rte) = _prep(
        kernel_type, x1, x2, params, start, end, [(left, 2), (right, 2)])
    if left.shape[-2] != m or right.shape[-2] != n or left.shape[-1] != right.shape[-1]:
        raise RuntimeError(f"left must be (.., {m}, k) and right (.., {n}, k); got {tuple(left.shape)} and {tuple(right.shape)}")
    k = left.shape[-1]
    if path not in ("auto", "fma", "tc"):
        raise ValueError(f"unknown path {path!r}")
    tc = path == "tc" or (path == "auto" and k >= GRAD_TENSOR_CORE_MIN_K and _enough_items(batch, m))
    P = NUM_PARAMS[kernel_type]
    grad = torch.empty(*batch, P, device=dev, dtype=torch.float32)
    grade = grad.reshape(-1, P) if len(batch) > KM_MAX_BATCH_DIMS else grad
    kb = _km_batch(batch)
    lv, rv = _view(le, 2), _view(rte, 2)
    if tc:
        ws_bytes = lib.km_grad_tc_workspace_bytes(kb, m, n, k, rv)
        fn = lib.km_matmul_bwd_tc_f32 if which == "matmul_bwd" else lib.km_bilinear_derivative_tc_f32
    else:
        ws_bytes = lib.km_grad_workspace_bytes(kid, kb, m)
        fn = lib.km_matmul_bwd_f32 if which == "matmul_bwd" else lib.km_bilinear_derivative_f32
    st = _state(dev)
    ws = st.workspace(dev, max(ws_bytes, 16))
    with torch.cuda.device(dev):
        if which == "matmul_bwd":  # argument order: rhs ... out_grad
            _check(fn(kid, kb, m, n, k, _view(x1e, 1), _view(x2e, 1), rv, _view(pe, 1), _view(se, 1), _view(ee, 1),
                      lv, _view(grade, 1), ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream(dev)))
        else:
            _check(fn(kid, kb, m, n, k, _view(x1e, 1), _view(x2e, 1), lv, rv, _view(pe, 1), _view(se, 1), _view(ee, 1),
                      _view(grade, 1), ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream(dev)))
        if tc:
            st.track(ws, which)
    if tc:
        grad._km_tensor_cores = True
    return grad


def matmul_bwd(kernel_type: str, x1, x2, rhs, params, start, end, out_grad, *, path: str = "auto") -> Tensor:
    """Gradient of ``sum(out_grad * matmul(...))`` wrt ``params`` -> ``(*batch, P)``.

    Reference: ``matmul_bwd.call(x1, x2, rhs, params, start, end, out_grad)``
    (native/matmul_bwd/matmul_bwd.cpp:6-19).  ``path`` as in ``matmul``.
    """
    return _grad_call("matmul_bwd", kernel_type, x1, x2, out_grad, rhs, params, start, end, path)


def bilinear_derivative(kernel_type: str, x1, x2, left_vecs, right_vecs, params, start, end, *,
                        path: str = "auto") -> Tensor:
    """Gradient of ``sum_c left[:, c]^T K right[:, c]`` wrt ``params`` -> ``(*batch, P)``.

    Reference: ``bilinear_derivative.call(x1, x2, left_vecs, right_vecs, params, start, end)``
    (native/bilinear_derivative/bilinear_derivative.cpp:6-21).
    """
    return _grad_call("bilinear_derivative", kernel_type, x1, x2, left_vecs, right_vecs, params, start, end, path)


def dense(kernel_type: str, x1, x2, params, start, end) -> Tensor:
    """Masked dense ``K`` -> ``(*batch, m, n)``.  Reference: ``dense.call`` (native/dense/dense.cpp:6-17)."""
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee) = _prep(kernel_type, x1, x2, params, start, end)
    out = torch.empty(*batch, m, n, device=dev, dtype=torch.float32)
    oute = out.reshape(-1, m, n) if len(batch) > KM_MAX_BATCH_DIMS else out
    with torch.cuda.device(dev):
        _check(lib.km_dense_f32(kid, _km_batch(batch), m, n, _view(x1e, 1), _view(x2e, 1), _view(pe, 1),
                               _view(se, 1), _view(ee, 1), _view(oute, 2), _stream(dev)))
    return out


def dense_bwd(kernel_type: str, x1, x2, params, start, end, out_grad) -> Tensor:
    """Gradient of ``sum(out_grad * dense(...))`` wrt ``params``.  Reference: ``dense_bwd.call``
    (native/dense_bwd/dense_bwd.cpp:6-17)."""
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee, ge) = _prep(kernel_type, x1, x2, params, start, end, [(out_grad, 2)])
    if out_grad.shape[-2:] != (m, n):
        raise RuntimeError(f"out_grad must be (.., {m}, {n}), got {tuple(out_grad.shape)}")
    P = NUM_PARAMS[kernel_type]
    grad = torch.empty(*batch, P, device=dev, dtype=torch.float32)
    grade = grad.reshape(-1, P) if len(batch) > KM_MAX_BATCH_DIMS else grad
    kb = _km_batch(batch)
    ws_bytes = lib.km_grad_workspace_bytes(kid, kb, m)
    ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        _check(lib.km_dense_bwd_f32(kid, kb, m, n, _view(x1e, 1), _view(x2e, 1), _view(pe, 1), _view(se, 1),
                                   _view(ee, 1), _view(ge, 2), _view(grade, 1), ctypes.c_void_p(ws.data_ptr()),
                                   ws_bytes, _stream(dev)))
    return grad


def _index_prep(batch: tuple[int, ...], batch_indices, row_index, col_index, dev):
    batch_indices = tuple(batch_indices)
    if len(batch_indices) != len(batch):
        raise RuntimeError(f"expected {len(batch)} batch index tensors, got {len(batch_indices)}")
    for t in (*batch_indices, row_index, col_index):
        _check_i32(t)
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
    shape = tuple(torch.broadcast_shapes(row_index.shape, col_index.shape, *(b.shape for b in batch_indices)))
    flat = [t.expand(shape).contiguous().reshape(-1) for t in (*batch_indices, row_index, col_index)]
    return shape, flat[:-2], flat[-2], flat[-1]


def _bidx_array(bidx: Sequence[Tensor], batch: tuple[int, ...]):
    arr = (ctypes.c_void_p * KM_MAX_BATCH_DIMS)()
    for d, t in enumerate(bidx):
        arr[d] = t.data_ptr()
    return arr


def index(kernel_type: str, x1, x2, params, start, end, batch_indices, row_index, col_index) -> Tensor:
    """``K[batch_indices..., row_index, col_index]`` (0 outside the band) with the shape of the
    index tensors.  Reference: ``index.call`` (native/index/index.cpp:6-24)."""
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee) = _prep(kernel_type, x1, x2, params, start, end)
    if len(batch) > KM_MAX_BATCH_DIMS:
        raise RuntimeError(f"index supports at most {KM_MAX_BATCH_DIMS} batch dims")
    shape, bidx, row, col = _index_prep(batch, batch_indices, row_index, col_index, dev)
    L = row.numel()
    out = torch.empty(L, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        _check(lib.km_index_f32(kid, _km_batch(batch), m, n, L, _view(x1e, 1), _view(x2e, 1), _view(pe, 1),
                               _view(se, 1), _view(ee, 1), _bidx_array(bidx, batch), ctypes.c_void_p(row.data_ptr()),
                               ctypes.c_void_p(col.data_ptr()), ctypes.c_void_p(out.data_ptr()), _stream(dev)))
    return out.reshape(shape)


def index_bwd(kernel_type: str, x1, x2, params, start, end, batch_indices, row_index, col_index, out_grad) -> Tensor:
    """Gradient of ``sum(out_grad * index(...))`` wrt ``params`` -> ``(*batch, P)``.
    Reference: ``index_bwd.call`` (native/index_bwd/index_bwd.cpp:6-27)."""
    kid, dev, batch, m, n, (x1e, x2e, pe, se, ee) = _prep(kernel_type, x1, x2, params, start, end)
    if len(batch) > KM_MAX_BATCH_DIMS:
        raise RuntimeError(f"index_bwd supports at most {KM_MAX_BATCH_DIMS} batch dims")
    shape, bidx, row, col = _index_prep(batch, batch_indices, row_index, col_index, dev)
    _check_f32(out_grad)
    og = out_grad.expand(shape).contiguous().reshape(-1)
    L = row.numel()
    P = NUM_PARAMS[kernel_type]
    grad = torch.empty(*batch, P, device=dev, dtype=torch.float32)
    kb = _km_batch(batch)
    ws_bytes = lib.km_index_bwd_workspace_bytes(kid, kb)
    ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        _check(lib.km_index_bwd_f32(kid, kb, m, n, L, _view(x1e, 1), _view(x2e, 1), _view(pe, 1), _view(se, 1),
                                   _view(ee, 1), _bidx_array(bidx, batch), ctypes.c_void_p(row.data_ptr()),
                                   ctypes.c_void_p(col.data_ptr()), ctypes.c_void_p(og.data_ptr()), _view(grad, 1),
                                   ctypes.c_void_p(ws.data_ptr()), ws_bytes, _stream(dev)))
    return grad


def count_entries(m: int, n: int, start: Tensor, end: Tensor) -> Tensor:
    """Visited kernel entries ``sum rows(r) * (end - start)`` as a 0-dim int64 device tensor."""
    _check_i32(start)
    _check_i32(end)
    dev = _same_device(start, end)
    batch = _common_batch([(start, 1), (end, 1)])
    se, ee = _expand(start, batch, 1), _expand(end, batch, 1)
    out = torch.empty((), device=dev, dtype=torch.int64)
    with torch.cuda.device(dev):
        _check(lib.km_count_entries(_km_batch(batch), m, n, _view(se, 1), _view(ee, 1),
                                   ctypes.c_void_p(out.data_ptr()), _stream(dev)))
    return out


__all__ = [
    "matmul", "matmul_rows", "prepare_matmul_rows", "PreparedRowsProduct", "tc_status", "check", "used_tensor_cores", "KernelGaveUpError", "matmul_bwd", "bilinear_derivative", "dense", "dense_bwd", "index", "index_bwd",
    "count_entries", "BLOCK_SIZE", "NUM_PARAMS",
]
