"""The GPyTorch-facing kernels: parameter plumbing around ``KernelMatmulLinearOperator``.

Each kernel owns raw parameters with positivity constraints, stacks the transformed values in
the order the native ops expect, builds the band on the device and returns the operator.
Reference: ``kernel_matmul/gpytorch/base.py:47-84`` (forward), ``rbf.py``, ``spectral.py``,
``locally_periodic.py`` (parameters), ``sum.py`` (batch sum).  One deliberate difference: the
locally periodic kernel passes kernel type ``"locally_periodic"`` to the operator (the
reference passes ``"spectral"``, ``locally_periodic.py:33``, which selects the wrong native
kernel for its four parameters).
"""
from __future__ import annotations

from typing import Any

import torch
from gpytorch.constraints import GreaterThan, Interval
from gpytorch.kernels import Kernel
from gpytorch.priors import Prior
from torch import Size, Tensor, nn

from ..kernels import band_for, same_tensor
from ..linear_operator import KernelMatmulLinearOperator


class KernelMatmulKernel(Kernel):
    """Base class: subclasses declare ``_PARAMS`` (names in native order) and the kernel type."""

    has_lengthscale = False
    _KERNEL_TYPE: str = ""
    _PARAMS: tuple[str, ...] = ()
    _LENGTHSCALES: tuple[str, ...] = ()

    def __init__(
        self,
        cutoff: float | None = None,
        epsilon: float | None = None,
        batch_shape: Size = torch.Size(()),
        compile_pool: Any = None,
        **constraints_and_priors: Any,
    ):
        super().__init__(batch_shape=batch_shape)
        if cutoff is not None and epsilon is not None:
            raise ValueError("Cannot have both a fixed cutoff and an epsilon for dynamic cutoff!")
        self._cutoff = cutoff
        self._epsilon = epsilon
        self._compile_pool = compile_pool
        for name in self._PARAMS:
            constraint: Interval | None = constraints_and_priors.pop(f"{name}_constraint", None)
            prior: Prior | None = constraints_and_priors.pop(f"{name}_prior", None)
            self._add_parameter(name, batch_shape, constraint or GreaterThan(1e-6), prior)
        if constraints_and_priors:
            raise TypeError(f"unexpected arguments: {sorted(constraints_and_priors)}")

    def _add_parameter(self, name: str, batch_shape: Size, constraint: Interval, prior: Prior | None) -> None:
        raw = f"raw_{name}"
        self.register_parameter(raw, nn.Parameter(torch.zeros(batch_shape)))
        self.register_constraint(raw, constraint)
        if prior is not None:
            self.register_prior(
                f"{name}_prior", prior,
                lambda module, n=name: getattr(module, n),
                lambda module, value, n=name: module.initialize(**{n: value}),
            )

    def __getattr__(self, item: str):
        # transformed parameter values: kernel.lengthscale, kernel.outputscale, ...
        if item in type(self)._PARAMS:
            raw = super().__getattr__(f"raw_{item}")
            return super().__getattr__(f"raw_{item}_constraint").transform(raw)
        return super().__getattr__(item)

    def __setattr__(self, key: str, value) -> None:
        if key in type(self)._PARAMS:
            raw = getattr(self, f"raw_{key}")
            value = torch.as_tensor(value, dtype=raw.dtype, device=raw.device).expand(raw.shape)
            constraint = getattr(self, f"raw_{key}_constraint")
            self.initialize(**{f"raw_{key}": constraint.inverse_transform(value)})
        else:
            super().__setattr__(key, value)

    def _get_params(self) -> Tensor:
        return torch.stack([getattr(self, name) for name in self._PARAMS], dim=-1)

    def _get_largest_lengthscale(self) -> float:
        return max(getattr(self, name).max().item() for name in self._LENGTHSCALES)

    def forward(self, x1: Tensor, x2: Tensor, diag: bool = False, last_dim_is_batch: bool = False, **params):
        if last_dim_is_batch:
            raise NotImplementedError("last_dim_is_batch not supported for KernelMatmulKernel")
        # x1 == x2 from the tensors' identity where possible, and the band (fixed cutoff or epsilon
        # rule) built on the device: no host synchronisation on the training path
        # (kernel_matmul/gpytorch/base.py:56-66 compares contents and reads the lengthscale back)
        symmetric = same_tensor(x1, x2) or (x1.shape == x2.shape and torch.equal(x1, x2))
        start, end = band_for(x1, x2, symmetric, self._cutoff, self._epsilon,
                              [getattr(self, name) for name in self._LENGTHSCALES])
        operator = KernelMatmulLinearOperator(
            x1, x2, self._get_params(), start, end,
            kernel_type=self._KERNEL_TYPE, symmetric=symmetric, compile_pool=self._compile_pool,
        )
        return operator.diagonal() if diag else operator


class RBFKernelMatmulKernel(KernelMatmulKernel):
    """``outputscale * exp(-0.5 * (x1 - x2)^2 / lengthscale^2)``"""

    _KERNEL_TYPE = "rbf"
    _PARAMS = ("lengthscale", "outputscale")
    _LENGTHSCALES = ("lengthscale",)


class SpectralKernelMatmulKernel(KernelMatmulKernel):
    """``outputscale * exp(-0.5 * (x1 - x2)^2 / lengthscale^2) * cos(2 pi frequency (x1 - x2))``"""

    _KERNEL_TYPE = "spectral"
    _PARAMS = ("lengthscale", "frequency", "outputscale")
    _LENGTHSCALES = ("lengthscale",)


class LocallyPeriodicKernelMatmulKernel(KernelMatmulKernel):
    """``outputscale * exp(-0.5 tau^2 / l_rbf^2) * exp(-2 sin^2(pi tau / period) / l_periodic)``"""

    _KERNEL_TYPE = "locally_periodic"
    _PARAMS = ("lengthscale_rbf", "lengthscale_periodic", "period_length", "outputscale")
    _LENGTHSCALES = ("lengthscale_rbf",)


class SumKernel(Kernel):
    """Sum of a batched kernel over one of its batch dimensions (mixture of components)."""

    has_lengthscale = False

    def __init__(self, base_kernel: Kernel, dim: int = -1):
        super().__init__()
        self.base_kernel = base_kernel
        self.dim = dim

    def forward(self, x1, x2, diag: bool = False, **params):
        base = self.base_kernel.forward(x1, x2, diag=diag, **params)
        if self.dim >= 0:
            dim = self.dim
        else:
            dim = self.dim - (1 if diag else 2)  # skip the matrix dims of the operator
        return base.sum(dim=dim)

    @property
    def batch_shape(self) -> Size:
        shape = list(self.base_kernel.batch_shape)
        del shape[self.dim]
        return Size(shape)
