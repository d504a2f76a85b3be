"""B200-native drop-in for the hot path of Turakar/kernel-matmul.

Same Python surface as the reference package ``kernel_matmul`` for that path:
``ranges.make_ranges / transpose_ranges / RangesCache``, ``compile.load_native(name, defines).call``,
``native_function.NativeFunction``, the ``*Configuration`` classes,
``linear_operator.KernelMatmulLinearOperator`` and the GPyTorch kernels in ``gpytorch``.
All arithmetic runs in hand-written sm_100a CUDA kernels behind the C ABI of
``libkm_b200.so`` (``include/km_b200.h``); importing the package without that library fails.
"""
_BLOCK_SIZE = 128
"""Rows per row block of the sparsity pattern (kernel_matmul/__init__.py:1 in the reference)."""

from . import _lib  # noqa: E402,F401  (raises ImportError when libkm_b200.so is missing)
from . import ops  # noqa: E402,F401
