"""Configuration objects of the reference's autotuner, kept as thin shims.

In the reference a ``Configuration`` turns call arguments into ``-DKM_*`` define sets and a
cache key (``kernel_matmul/configurations.py:11-234``).  Here launch parameters are fixed at
build time, so every configuration yields exactly one define set whose only meaningful entry
is the ``KERNEL_*`` flag; the tuning keys of the reference are still present (with the values
this build effectively uses) because callers read and overwrite them.
"""
from __future__ import annotations

import abc

from torch import Tensor

from . import _BLOCK_SIZE
from .compile import Defines

_KERNEL_FLAG = {
    "rbf": "KERNEL_RBF",
    "spectral": "KERNEL_SPECTRAL",
    "locally_periodic": "KERNEL_LOCALLY_PERIODIC",
}


def get_kernel_type_defines(kernel_type: str, params: Tensor | None = None) -> Defines:
    if kernel_type == "compact":
        raise NotImplementedError("the 'compact' kernel is not part of this build")
    return {_KERNEL_FLAG[kernel_type]: None}


class Configuration(abc.ABC):
    """Maps call arguments to define sets (always one here) and to a cache key."""

    #: tuning keys of the reference for this op, with the fixed values of this build
    _fixed: Defines = {}
    #: index of the tensor whose rank gives BATCH_DIM
    _x1_index = 0

    def __init__(self, kernel_type: str):
        self.kernel_type = kernel_type

    def make_config(self, args: tuple) -> Defines:
        x1 = args[self._x1_index]
        return {
            "BLOCK_SIZE": _BLOCK_SIZE,
            "BATCH_DIM": x1.dim() - 1,
            **self._extra(args),
            **get_kernel_type_defines(self.kernel_type),
        }

    def _extra(self, args: tuple) -> Defines:
        return dict(self._fixed)

    def make_candidates(self, args: tuple) -> list[Defines]:
        return [self.make_config(args)]

    def cache_key(self, args: tuple) -> str:
        return f"{args[self._x1_index].dim() - 1}"


class SingleConfiguration(Configuration):
    pass


class MatmulSingleConfiguration(SingleConfiguration):
    def _extra(self, args: tuple) -> Defines:
        rhs = args[2]
        return {
            "MATMUL_K_BLOCK_SIZE": min(rhs.shape[-1], 32),
            "MATMUL_THREADS": 128,
            "MATMUL_PER_THREAD": 4,
            "MATMUL_COL_BLOCKS": 1,
            "MATMUL_USE_SHM": 1,
        }

    def cache_key(self, args: tuple) -> str:
        return f"{args[0].dim() - 1}_{args[2].shape[-1]}"


class MatmulAutotuneConfiguration(MatmulSingleConfiguration):
    """The reference times 12-36 candidates here; this build has one kernel per rhs width."""


class MatmulBwdConfiguration(SingleConfiguration):
    _fixed = {"MATMUL_BWD_THREAD_DIM": 16, "MATMUL_BWD_PER_THREAD": 8}


class BilinearDerivativeConfiguration(SingleConfiguration):
    _fixed = {"BILINEAR_DERIVATIVE_THREAD_DIM": 16, "BILINEAR_DERIVATIVE_PER_THREAD": 8}


class DenseConfiguration(SingleConfiguration):
    _fixed = {"DENSE_THREAD_DIM": 16}


class DenseBwdConfiguration(SingleConfiguration):
    _fixed = {"DENSE_BWD_THREAD_DIM": 16}


class IndexConfiguration(SingleConfiguration):
    def _extra(self, args: tuple) -> Defines:
        return {"INDEX_THREAD_DIM": 64, "INDEX_BATCH_DIM": args[6].dim() - 1}

    def cache_key(self, args: tuple) -> str:
        return f"{args[0].dim() - 1}_{args[6].dim() - 1}"


class IndexBwdConfiguration(SingleConfiguration):
    def _extra(self, args: tuple) -> Defines:
        return {"INDEX_BWD_THREAD_DIM": 64, "INDEX_BWD_BATCH_DIM": args[6].dim() - 1}

    def cache_key(self, args: tuple) -> str:
        return f"{args[0].dim() - 1}_{args[6].dim() - 1}"
