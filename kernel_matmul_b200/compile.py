"""Stand-ins for the reference's JIT layer (``kernel_matmul/compile.py``).

The reference compiles one extension per (op, ``-DKM_*`` define set) at run time and times
candidates to pick launch parameters.  This build has one ahead-of-time sm_100a library, so
nothing is compiled or tuned here; the functions keep their names and call conventions so that
code written against the reference keeps working:

* ``load_native(name, defines).call(*args)`` resolves the ``KERNEL_*`` define to the runtime
  kernel type and calls the matching op of ``libkm_b200.so``; tuning defines are accepted and
  ignored.
* ``find_best`` returns the first candidate (all candidates run the same kernel).
* ``compile_pool`` is a context manager that does nothing.
* ``cuda_time`` times a callable with CUDA events.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Callable

import torch

from . import ops

Defines = dict[str, Any]

_KERNEL_DEFINES = {
    "KERNEL_RBF": "rbf",
    "KERNEL_SPECTRAL": "spectral",
    "KERNEL_LOCALLY_PERIODIC": "locally_periodic",
}

_OPS = {
    "matmul": ops.matmul,
    "matmul_bwd": ops.matmul_bwd,
    "bilinear_derivative": ops.bilinear_derivative,
    "dense": ops.dense,
    "dense_bwd": ops.dense_bwd,
    "index": ops.index,
    "index_bwd": ops.index_bwd,
}


def kernel_type_from_defines(defines: Defines | None) -> str:
    found = [kt for key, kt in _KERNEL_DEFINES.items() if defines and key in defines]
    if defines and "KERNEL_COMPACT" in defines:
        raise NotImplementedError(
            "the 'compact' kernel is not part of this build (its gradient is unfinished in the "
            "reference, native/common/kernel_function.cuh:184)"
        )
    if len(found) != 1:
        raise ValueError("defines must contain exactly one of " + ", ".join(_KERNEL_DEFINES))
    return found[0]


class NativeModule:
    """What ``load_native`` returns: an object with a ``call`` method, like the reference's
    per-op pybind11 modules (e.g. native/matmul/matmul.cpp:17)."""

    def __init__(self, name: str, kernel_type: str, defines: Defines):
        self.name = name
        self.kernel_type = kernel_type
        self.defines = dict(defines)
        self._op = _OPS[name]

    def call(self, *args):
        return self._op(self.kernel_type, *args)

    def __repr__(self) -> str:
        return f"NativeModule({self.name!r}, kernel_type={self.kernel_type!r})"


def load_native(name: str, defines: Defines | None = None) -> NativeModule:
    """Return the native op ``name`` bound to the kernel type named in ``defines``."""
    if name == "ranges":
        raise ValueError("use kernel_matmul_b200.ranges for the band construction functions")
    if name not in _OPS:
        raise ValueError(f"Unknown native module: {name}")
    return NativeModule(name, kernel_type_from_defines(defines), defines or {})


@contextmanager
def compile_pool(processes: int):
    """Kept for source compatibility; there is nothing to compile at run time."""
    yield


def find_best(
    name: str,
    args: list[Any],
    candidates: list[Defines],
    return_timings: bool = False,
    num_measurements: int = 1,
    compile_pool: Any = None,
):
    """All candidates map to the same fixed kernel; the first one is returned.  With
    ``return_timings`` every candidate reports the same measured time."""
    best = candidates[0]
    if not return_timings:
        return best
    module = load_native(name, best)
    t = cuda_time(lambda: module.call(*args), num_measurements=num_measurements)
    mean = sum(t) / len(t)
    return best, [mean for _ in candidates]


def cuda_time(fn: Callable, num_measurements: int | None = None) -> float | list[float]:
    """Milliseconds of ``fn()`` measured with CUDA events on the current stream."""
    single = num_measurements is None
    reps = 1 if single else num_measurements
    timings = []
    for _ in range(reps):
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        timings.append(start.elapsed_time(end))
    return timings[0] if single else timings
