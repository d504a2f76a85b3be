"""``NativeFunction``: a callable bound to one native op and one kernel type.

The reference's class of the same name autotunes and JIT-compiles on first call and caches the
chosen module per argument signature (``kernel_matmul/native_function.py:12-86``).  With a fixed
ahead-of-time build there is nothing to choose: the call goes straight to the op.  The
constructor arguments, ``__call__`` and the ``defines`` property are kept.
"""
from __future__ import annotations

from typing import Any

from .compile import Defines, load_native
from .configurations import Configuration


class NativeFunction:
    def __init__(
        self,
        name: str,
        config: Configuration,
        num_measurements: int = 1,
        verbose: bool = False,
        compile_pool: Any = None,
    ):
        self.name = name
        self.config = config
        self.num_measurements = num_measurements
        self.verbose = verbose
        self.compile_pool = compile_pool
        self._defines: Defines | None = None
        self._module = None

    def __call__(self, *args: Any) -> Any:
        if self._module is None:
            self._defines = self.config.make_candidates(args)[0]
            self._module = load_native(self.name, self._defines)
            if self.verbose:
                print(f"{self.name}: fixed sm_100a build, nothing to tune ({self._module})")
        return self._module.call(*args)

    @property
    def defines(self) -> Defines | None:
        """Defines of the first call's configuration (``None`` before the first call)."""
        return self._defines
