"""Kernel modules on plain PyTorch: learnable hyper-parameters -> band -> ``KernelMatmulOperator``.

What the reference's GPyTorch kernels do in ``forward`` (kernel_matmul/gpytorch/base.py:47-84:
stack the parameters in native order, pick the cutoff, build the band, return the operator),
without the GPyTorch dependency, so that the whole training step -- parameters, band, product,
gradients back to the raw parameters -- runs and is tested wherever PyTorch and a B200 are.
``kernel_matmul_b200.gpytorch`` wraps the same logic into ``gpytorch.kernels.Kernel`` subclasses
when GPyTorch is installed.

Differences from the reference that matter on a GPU:
* the band is built on the device (``ranges.make_ranges*``), and with ``epsilon`` the cutoff
  ``sqrt(2) erfinv(1 - epsilon) * max lengthscale`` stays a device tensor: no ``.item()`` per
  forward (base.py:59-64 reads the lengthscale back on every call);
* ``x1 == x2`` is recognised from the tensors' identity (same storage, shape and strides) without
  comparing their contents on the device and waiting for the answer (base.py:56 calls
  ``torch.equal``); tensors that merely hold equal values take the comparison, as before.
With both, ``forward`` + product + backward issue no host synchronisation.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor, nn

from .linear_operator import KernelMatmulOperator
from .ranges import make_ranges, make_ranges_symmetric_cutoffs


def same_tensor(a: Tensor, b: Tensor) -> bool:
    """True when ``a`` and ``b`` are views of the same memory with the same layout (then their
    contents are equal, and nothing has to be read to know it)."""
    return a is b or (a.device == b.device and a.dtype == b.dtype and a.shape == b.shape
                      and a.stride() == b.stride() and a.data_ptr() == b.data_ptr())


def dynamic_cutoff(epsilon: float, lengthscales: list[Tensor]) -> Tensor:
    """``sqrt(2) erfinv(1 - epsilon) * max lengthscale`` as a 0-dim fp32 tensor on the lengthscales'
    device (double product, rounded once: the value the reference computes on the host)."""
    z = math.sqrt(2.0) * torch.special.erfinv(torch.tensor(1.0 - epsilon, dtype=torch.float64)).item()
    largest = torch.stack([ls.detach().max() for ls in lengthscales]).max()
    return (largest.double() * z).float()


def band_for(x1: Tensor, x2: Tensor, symmetric: bool, cutoff: float | None, epsilon: float | None,
             lengthscales: list[Tensor]) -> tuple[Tensor, Tensor]:
    """start / end for inputs ``(..., n, 1)``: fixed cutoff, or the epsilon rule."""
    xs = x1.squeeze(-1)
    if epsilon is not None:
        if symmetric and xs.is_cuda and xs.dim() == 1:
            start, end = make_ranges_symmetric_cutoffs(dynamic_cutoff(epsilon, lengthscales).reshape(1), xs)
            return start[0], end[0]
        cutoff = float(dynamic_cutoff(epsilon, lengthscales))  # batched or rectangular inputs: host value
    if symmetric:
        return make_ranges(cutoff, xs, align=True)
    return make_ranges(cutoff, xs, x2.squeeze(-1), align=True)


class KernelMatmulModule(nn.Module):
    """Base class: subclasses declare the kernel type, the parameter names in native order and
    which of them are lengthscales.  Parameters are stored raw and mapped to positive values by
    ``lower_bound + softplus(raw)`` (what GPyTorch's ``GreaterThan(1e-6)`` constraint does)."""

    _KERNEL_TYPE: str = ""
    _PARAMS: tuple[str, ...] = ()
    _LENGTHSCALES: tuple[str, ...] = ()
    LOWER_BOUND = 1e-6

    def __init__(self, cutoff: float | None = None, epsilon: float | None = None, batch_shape=torch.Size(())):
        super().__init__()
        if cutoff is not None and epsilon is not None:
            raise ValueError("Cannot have both a fixed cutoff and an epsilon for dynamic cutoff!")
        self._cutoff, self._epsilon = cutoff, epsilon
        self.batch_shape = torch.Size(batch_shape)
        for name in self._PARAMS:
            self.register_parameter(f"raw_{name}", nn.Parameter(torch.zeros(self.batch_shape)))

    def value(self, name: str) -> Tensor:
        return self.LOWER_BOUND + nn.functional.softplus(getattr(self, f"raw_{name}"))

    def initialize(self, **values) -> "KernelMatmulModule":
        """Set parameters by their (positive) values: ``initialize(lengthscale=1.5, outputscale=2.0)``."""
        with torch.no_grad():
            for name, v in values.items():
                raw = getattr(self, f"raw_{name}")
                v = torch.as_tensor(v, dtype=raw.dtype, device=raw.device).expand(raw.shape) - self.LOWER_BOUND
                raw.copy_(v + torch.log(-torch.expm1(-v)))  # inverse softplus
        return self

    def params(self) -> Tensor:
        """``(*batch_shape, P)`` in the order the native ops expect."""
        return torch.stack([self.value(name) for name in self._PARAMS], dim=-1)

    def forward(self, x1: Tensor, x2: Tensor | None = None) -> KernelMatmulOperator:
        if x2 is None:
            x2 = x1
        symmetric = same_tensor(x1, x2) or (x1.shape == x2.shape and torch.equal(x1, x2))
        start, end = band_for(x1, x2, symmetric, self._cutoff, self._epsilon, [self.value(n) for n in self._LENGTHSCALES])
        return KernelMatmulOperator(x1, x2, self.params(), start, end, kernel_type=self._KERNEL_TYPE, symmetric=symmetric)


class RBFKernelMatmulModule(KernelMatmulModule):
    """``outputscale * exp(-0.5 * (x1 - x2)^2 / lengthscale^2)``  (kernel_matmul/gpytorch/rbf.py)"""

    _KERNEL_TYPE = "rbf"
    _PARAMS = ("lengthscale", "outputscale")
    _LENGTHSCALES = ("lengthscale",)


class SpectralKernelMatmulModule(KernelMatmulModule):
    """``outputscale * exp(-0.5 tau^2 / lengthscale^2) * cos(2 pi frequency tau)``  (spectral.py)"""

    _KERNEL_TYPE = "spectral"
    _PARAMS = ("lengthscale", "frequency", "outputscale")
    _LENGTHSCALES = ("lengthscale",)


class LocallyPeriodicKernelMatmulModule(KernelMatmulModule):
    """``outputscale * exp(-0.5 tau^2 / l_rbf^2) * exp(-2 sin^2(pi tau / period) / l_periodic)``
    (locally_periodic.py; the reference passes kernel type "spectral" to its operator there,
    locally_periodic.py:33, which selects the wrong native kernel for these four parameters)."""

    _KERNEL_TYPE = "locally_periodic"
    _PARAMS = ("lengthscale_rbf", "lengthscale_periodic", "period_length", "outputscale")
    _LENGTHSCALES = ("lengthscale_rbf",)
