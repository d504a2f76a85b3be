"""GPyTorch kernels backed by the km_b200 operator (needs ``gpytorch`` and ``linear_operator``).

Same class names, constructor arguments and parameter order as the reference package
(``kernel_matmul/gpytorch/``).  Importing this sub-package without GPyTorch raises
``ImportError``; the rest of ``kernel_matmul_b200`` does not depend on it.
"""
try:
    import gpytorch as _gpytorch  # noqa: F401
    import linear_operator as _linear_operator  # noqa: F401
except ImportError as exc:  # pragma: no cover - depends on the environment
    raise ImportError(
        "kernel_matmul_b200.gpytorch needs the third-party packages 'gpytorch' and "
        "'linear_operator'; use kernel_matmul_b200.linear_operator.KernelMatmulOperator "
        "or kernel_matmul_b200.ops without them"
    ) from exc

from .kernels import (  # noqa: E402
    KernelMatmulKernel,
    LocallyPeriodicKernelMatmulKernel,
    RBFKernelMatmulKernel,
    SpectralKernelMatmulKernel,
    SumKernel,
)

__all__ = [
    "KernelMatmulKernel",
    "RBFKernelMatmulKernel",
    "SpectralKernelMatmulKernel",
    "LocallyPeriodicKernelMatmulKernel",
    "SumKernel",
]
