"""B200 (sm_100a) backend for kapy-lang's matmul / elementwise / reduce path.

The directory name carries a hyphen, so the package is registered under the
importable name ``kapy_lang_b200`` by ``__graft_entry__.load_package()``.
Nothing here computes on the CPU: every op is a CUDA kernel reached through the
C ABI in ``include/kapyb.h``.
"""
from . import _abi as abi  # noqa: F401
from . import dist  # noqa: F401
from . import executor  # noqa: F401
from . import ir  # noqa: F401
from . import mlir_text  # noqa: F401
from . import programs  # noqa: F401
from . import runtime  # noqa: F401
from .build import build  # noqa: F401
from .runtime import (Handle, KapybError, KapybTimeout, matmul_plan, shard_range, tensor2d,  # noqa: F401
                      tune_matmul, tuning_clear, tuning_load)

__all__ = ["abi", "dist", "executor", "ir", "mlir_text", "programs", "runtime", "build", "Handle", "KapybError", "KapybTimeout", "matmul_plan", "shard_range", "tune_matmul",
           "tuning_clear", "tuning_load",
           "tensor2d"]
