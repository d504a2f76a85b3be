"""Autograd glue and the operator object of the hot path.

``KernelMatmulOperator`` holds ``(x1, x2, params, start, end, kernel_type)`` and offers the
operations the reference's ``KernelMatmulLinearOperator`` implements
(``kernel_matmul/linear_operator.py:79-289``): ``matmul``, ``to_dense``, ``bilinear_derivative``,
``get_indices``, ``transpose``, ``expand_batch``, ``size``.  It depends on PyTorch only.

When the third-party ``linear_operator`` package is importable, ``KernelMatmulLinearOperator``
is that package's ``LinearOperator`` subclass with the same constructor and private hooks
(``_matmul``, ``_size``, ``_transpose_nonbatch``, ``to_dense``, ``_expand_batch``,
``_bilinear_derivative``, ``_get_indices``, ``to``, ``type``) as the reference; without it the
name is bound to ``KernelMatmulOperator`` so that code using only the operator-level methods
still runs.

The three autograd Functions give a gradient for ``params`` only, as in the reference
(``linear_operator.py:22-76``).  Its index backward unpacks eight saved tensors into seven
names (``:71-72``), which fails as soon as batch indices are present; here the split is
seven / rest.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from . import ranges
from .configurations import (
    BilinearDerivativeConfiguration,
    DenseBwdConfiguration,
    DenseConfiguration,
    IndexBwdConfiguration,
    IndexConfiguration,
    MatmulAutotuneConfiguration,
    MatmulBwdConfiguration,
)
from .native_function import NativeFunction

try:  # optional third-party base class
    from linear_operator import LinearOperator as _LinearOperator
    from linear_operator.utils.generic import _to_helper

    HAVE_LINEAR_OPERATOR = True
except Exception:  # noqa: BLE001 - absent or broken installation: operator-level API only
    _LinearOperator = None
    HAVE_LINEAR_OPERATOR = False


class _MatmulOperator(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, rhs, params, start, end, native_matmul, native_matmul_bwd):
        ctx.save_for_backward(x1, x2, rhs, params, start, end)
        ctx.native_matmul_bwd = native_matmul_bwd
        return native_matmul(x1, x2, rhs, params, start, end)

    @staticmethod
    def backward(ctx, grad_output):
        x1, x2, rhs, params, start, end = ctx.saved_tensors
        grad = ctx.native_matmul_bwd(x1, x2, rhs, params, start, end, grad_output)
        return None, None, None, grad, None, None, None, None


class _DenseOperator(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, params, start, end, native_dense, native_dense_bwd):
        ctx.save_for_backward(x1, x2, params, start, end)
        ctx.native_dense_bwd = native_dense_bwd
        return native_dense(x1, x2, params, start, end)

    @staticmethod
    def backward(ctx, grad_output):
        x1, x2, params, start, end = ctx.saved_tensors
        grad = ctx.native_dense_bwd(x1, x2, params, start, end, grad_output)
        return None, None, grad, None, None, None, None


class _IndexOperator(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x1, x2, params, start, end, native_index, native_index_bwd, row_index, col_index, *batch_indices):
        ctx.save_for_backward(x1, x2, params, start, end, row_index, col_index, *batch_indices)
        ctx.native_index_bwd = native_index_bwd
        return native_index(x1, x2, params, start, end, batch_indices, row_index, col_index)

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        x1, x2, params, start, end, row_index, col_index = saved[:7]
        batch_indices = saved[7:]
        grad = ctx.native_index_bwd(x1, x2, params, start, end, batch_indices, row_index, col_index, grad_output)
        return (None, None, grad, None, None, None, None, None, None, *[None for _ in batch_indices])


class _OperatorCore:
    """State and arithmetic shared by the plain operator and the LinearOperator subclass."""

    def _init_core(self, x1, x2, params, start, end, kernel_type, symmetric, compile_pool) -> None:
        if kernel_type is None:
            raise ValueError("kernel_type must be specified")
        if x1.dim() < 2 or x2.dim() < 2 or x1.size(-1) != 1 or x2.size(-1) != 1:
            raise ValueError("x1 and x2 must have shapes (..., M, 1) and (..., N, 1), respectively")
        if symmetric is None:
            symmetric = x1.shape == x2.shape and torch.equal(x1, x2)
        batch_shape = torch.broadcast_shapes(
            x1.shape[:-2], x2.shape[:-2], params.shape[:-1], start.shape[:-1], end.shape[:-1]
        )
        self._x1 = x1.expand(*batch_shape, *x1.shape[-2:])
        self._x2 = x2.expand(*batch_shape, *x2.shape[-2:])
        self._params = params.expand(*batch_shape, params.shape[-1])
        self._start = start.expand(*batch_shape, start.shape[-1])
        self._end = end.expand(*batch_shape, end.shape[-1])
        self._kernel_type = kernel_type
        self._batch_shape = torch.Size(batch_shape)
        self._symmetric = bool(symmetric)
        self._native_matmul = NativeFunction("matmul", MatmulAutotuneConfiguration(kernel_type), compile_pool=compile_pool)
        self._native_matmul_bwd = NativeFunction("matmul_bwd", MatmulBwdConfiguration(kernel_type))
        self._native_dense = NativeFunction("dense", DenseConfiguration(kernel_type))
        self._native_dense_bwd = NativeFunction("dense_bwd", DenseBwdConfiguration(kernel_type))
        self._native_bilinear_derivative = NativeFunction(
            "bilinear_derivative", BilinearDerivativeConfiguration(kernel_type)
        )
        self._native_index = NativeFunction("index", IndexConfiguration(kernel_type))
        self._native_index_bwd = NativeFunction("index_bwd", IndexBwdConfiguration(kernel_type))

    # -- helpers ---------------------------------------------------------------------------
    def _get_args_for_native(self, batch_shape) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
        def widen(t: Tensor) -> Tensor:
            return t.expand(*batch_shape, t.shape[-1])

        return (
            widen(self._x1.squeeze(-1)),
            widen(self._x2.squeeze(-1)),
            widen(self._params),
            widen(self._start),
            widen(self._end),
        )

    def _core_size(self) -> torch.Size:
        return torch.Size((*self._batch_shape, self._x1.size(-2), self._x2.size(-2)))

    def _core_matmul(self, rhs: Tensor) -> Tensor:
        expected = torch.Size((*self._batch_shape, self._x2.size(-2), rhs.size(-1)))
        full = torch.broadcast_shapes(expected, rhs.shape)
        batch_shape = full[:-2]
        x1, x2, params, start, end = self._get_args_for_native(batch_shape)
        result = _MatmulOperator.apply(
            x1, x2, rhs.expand(*full), params, start, end, self._native_matmul, self._native_matmul_bwd
        )
        return result.reshape(*batch_shape, *result.shape[-2:])

    def _core_to_dense(self) -> Tensor:
        x1, x2, params, start, end = self._get_args_for_native(self._batch_shape)
        return _DenseOperator.apply(x1, x2, params, start, end, self._native_dense, self._native_dense_bwd)

    def _core_bilinear_derivative(self, left_vecs: Tensor, right_vecs: Tensor) -> Tensor:
        batch_shape = torch.broadcast_shapes(left_vecs.shape[:-2], right_vecs.shape[:-2], self._batch_shape)
        left_vecs = left_vecs.expand(*batch_shape, *left_vecs.shape[-2:])
        right_vecs = right_vecs.expand(*batch_shape, *right_vecs.shape[-2:])
        x1, x2, params, start, end = self._get_args_for_native(batch_shape)
        result = self._native_bilinear_derivative(x1, x2, left_vecs, right_vecs, params, start, end)
        return result.reshape(*batch_shape, result.shape[-1])

    def _core_get_indices(self, row_index: Tensor, col_index: Tensor, *batch_indices: Tensor) -> Tensor:
        x1, x2, params, start, end = self._get_args_for_native(self._batch_shape)
        shape = torch.broadcast_shapes(row_index.shape, col_index.shape, *(b.shape for b in batch_indices))

        def prepare(index: Tensor) -> Tensor:
            return index.expand(*shape).to(device=x1.device, dtype=torch.int)

        return _IndexOperator.apply(
            x1, x2, params, start, end, self._native_index, self._native_index_bwd,
            prepare(row_index), prepare(col_index), *(prepare(b) for b in batch_indices),
        )

    def _core_transpose_args(self):
        start_t, end_t = ranges.transpose_ranges(self._start, self._end, self._x1.size(-2), self._x2.size(-2))
        return self._x2, self._x1, self._params, start_t, end_t

    def _core_expand_args(self, batch_shape):
        return (
            self._x1.expand(*batch_shape, *self._x1.shape[-2:]),
            self._x2.expand(*batch_shape, *self._x2.shape[-2:]),
            self._params.expand(*batch_shape, self._params.shape[-1]),
            self._start.expand(*batch_shape, self._start.shape[-1]),
            self._end.expand(*batch_shape, self._end.shape[-1]),
        )


class KernelMatmulOperator(_OperatorCore):
    """The banded kernel matrix ``K(x1, x2; params)`` as an implicit operator (PyTorch only).

    Args:
        x1: ``(..., M, 1)``;  x2: ``(..., N, 1)``;  params: ``(..., P)``;
        start, end: ``(..., ceil(M / 128))`` int32 column ranges per row block;
        kernel_type: ``"rbf"``, ``"spectral"`` or ``"locally_periodic"``;
        symmetric: whether ``K`` is symmetric (computed from ``x1 == x2`` when ``None``).
    """

    def __init__(self, x1, x2, params, start, end, kernel_type: str | None = None,
                 symmetric: bool | None = None, compile_pool: Any = None):
        self._init_core(x1, x2, params, start, end, kernel_type, symmetric, compile_pool)

    @property
    def shape(self) -> torch.Size:
        return self._core_size()

    def size(self, dim: int | None = None):
        s = self._core_size()
        return s if dim is None else s[dim]

    @property
    def batch_shape(self) -> torch.Size:
        return self._batch_shape

    def matmul(self, rhs: Tensor) -> Tensor:
        squeeze = rhs.dim() == 1
        out = self._core_matmul(rhs.unsqueeze(-1) if squeeze else rhs)
        return out.squeeze(-1) if squeeze else out

    __matmul__ = matmul

    def to_dense(self) -> Tensor:
        return self._core_to_dense()

    def bilinear_derivative(self, left_vecs: Tensor, right_vecs: Tensor) -> Tensor:
        """Gradient wrt params of ``sum_c left[:, c]^T K right[:, c]`` -> ``(..., P)``."""
        return self._core_bilinear_derivative(left_vecs, right_vecs)

    def get_indices(self, row_index: Tensor, col_index: Tensor, *batch_indices: Tensor) -> Tensor:
        return self._core_get_indices(row_index, col_index, *batch_indices)

    def transpose(self) -> "KernelMatmulOperator":
        if self._symmetric:
            return self
        x1, x2, params, start, end = self._core_transpose_args()
        return KernelMatmulOperator(x1, x2, params, start, end, kernel_type=self._kernel_type)

    def expand_batch(self, batch_shape) -> "KernelMatmulOperator":
        return KernelMatmulOperator(*self._core_expand_args(batch_shape), kernel_type=self._kernel_type)


if HAVE_LINEAR_OPERATOR:

    class KernelMatmulLinearOperator(_OperatorCore, _LinearOperator):
        """``linear_operator.LinearOperator`` backed by the km_b200 kernels; constructor and
        hooks as in the reference (kernel_matmul/linear_operator.py:79-289)."""

        def __init__(self, x1, x2, params, start, end, kernel_type: str | None = None,
                     symmetric: bool | None = None, compile_pool: Any = None):
            _LinearOperator.__init__(
                self, x1, x2, params, start, end,
                kernel_type=kernel_type, symmetric=symmetric, compile_pool=compile_pool,
            )
            self._init_core(x1, x2, params, start, end, kernel_type, symmetric, compile_pool)

        def _matmul(self, rhs: Tensor) -> Tensor:
            return self._core_matmul(rhs)

        def _size(self) -> torch.Size:
            return self._core_size()

        def _transpose_nonbatch(self):
            if self._symmetric:
                return self
            x1, x2, params, start, end = self._core_transpose_args()
            return KernelMatmulLinearOperator(x1, x2, params, start, end, kernel_type=self._kernel_type)

        def to_dense(self) -> Tensor:
            return self._core_to_dense()

        def _expand_batch(self, batch_shape):
            return KernelMatmulLinearOperator(*self._core_expand_args(batch_shape), kernel_type=self._kernel_type)

        def to(self, *args, **kwargs):
            device, dtype = _to_helper(*args, **kwargs)
            if (device is not None and device.type != "cuda") or (dtype is not None and dtype != torch.float32):
                raise NotImplementedError("KernelMatmulLinearOperator only supports CUDA and float32")
            return super().to(*args, **kwargs)

        def type(self, dtype):
            if dtype != torch.float32:
                raise NotImplementedError("KernelMatmulLinearOperator only supports CUDA and float32")
            return super().type(dtype)

        def _bilinear_derivative(self, left_vecs: Tensor, right_vecs: Tensor):
            return None, None, self._core_bilinear_derivative(left_vecs, right_vecs), None, None

        def _get_indices(self, row_index: Tensor, col_index: Tensor, *batch_indices: Tensor) -> Tensor:
            return self._core_get_indices(row_index, col_index, *batch_indices)

else:
    KernelMatmulLinearOperator = KernelMatmulOperator
