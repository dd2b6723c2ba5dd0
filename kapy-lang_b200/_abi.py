"""ctypes view of ``include/kapyb.h``: structures, enums and prototypes.

Loading fails loudly when ``libkapyb.so`` is missing: there is no Python or CPU
stand-in for the kernels.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libkapyb.so")

# kapyb_status
OK, INVALID_ARG, UNSUPPORTED, CUDA_ERROR, _UNUSED_4, TIMEOUT = range(6)
# kapyb_dtype
F16, BF16, F32, F8E4M3, F8E5M2, I1 = 0, 1, 2, 3, 4, 5
# kapyb_padding (Enums.td:52-61)
PAD_ZERO, PAD_QNAN, PAD_PINF, PAD_NINF = 0, 1, 2, 3
# kapyb_cache_modifier / kapyb_evict_priority (Enums.td:63-88)
CACHE_NONE, CACHE_CA, CACHE_CG, CACHE_CS, CACHE_WB, CACHE_WT, CACHE_LU, CACHE_CV = range(8)
EVICT_NORMAL, EVICT_FIRST, EVICT_LAST, EVICT_UNCHANGED, NO_ALLOCATE = range(5)


def cache_hints(modifier: int = 0, priority: int = 0, is_volatile: bool = False) -> int:
    """KAPYB_CACHE_HINTS: the `cache` field of a tensor descriptor."""
    return int(modifier) | (int(priority) << 8) | ((1 << 16) if is_volatile else 0)


# kapyb_rounding (Enums.td:102-109)
RZ, RN = 0, 1
# kapyb_activation
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3
# kapyb_combiner
RED_ADD, RED_MUL, RED_MAX, RED_MIN = 0, 1, 2, 3
# kapyb_matmul_impl_way (Enums.td:90-100)
MMA_ANY, MMA_M16N8K8_F16, MMA_M16N8K16_F16, MMA_M16N8K8_TF32, MMA_M16N8K16_F8 = 0, 1, 2, 3, 4

# kapyb_opcode
(OP_LOAD, OP_CONST, OP_CVT, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_FMA, OP_MAXIMUM, OP_MINIMUM,
 OP_MAXNUM, OP_MINNUM, OP_CLAMP, OP_ABS, OP_NEG, OP_EXP, OP_EXP2, OP_LOG, OP_LOG2, OP_SQRT,
 OP_RSQRT, OP_ERF, OP_SIN, OP_COS, OP_FLOOR, OP_CEIL, OP_TANH, OP_STORE, OP_CMP, OP_SELECT,
 OP_AND, OP_OR, OP_XOR) = range(33)
# kapyb_cmp_predicate (arith.cmpf as ir.cc:941-1000 binds it)
CMP_PREDICATES = ["olt", "ogt", "ole", "oge", "oeq", "one", "ult", "ugt", "ule", "uge", "ueq", "une"]

MAX_REGS, MAX_INSTS, MAX_INPUTS = 16, 64, 4


class Tensor2d(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("offset_elems", C.c_int64),
                ("size0", C.c_int32), ("size1", C.c_int32),
                ("stride0", C.c_int32), ("stride1", C.c_int32),
                ("dtype", C.c_int32), ("padding", C.c_int32),
                ("cache", C.c_int32), ("reserved_", C.c_int32)]


class Epilogue(C.Structure):
    _fields_ = [("alpha", C.c_float), ("bias", C.c_void_p),
                ("bias_dtype", C.c_int32), ("bias_axis", C.c_int32),
                ("activation", C.c_int32), ("rounding", C.c_int32)]


class ShardCtx(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32),
                ("peer_lhs", C.POINTER(C.c_void_p)), ("peer_flags", C.POINTER(C.c_void_p)),
                ("seq", C.c_uint32), ("wait_limit_ms", C.c_uint32)]


class Inst(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("dst", C.c_int32),
                ("a", C.c_int32), ("b", C.c_int32), ("c", C.c_int32),
                ("imm", C.c_float), ("flags", C.c_int32)]


# name -> (restype, argtypes); every symbol include/kapyb.h declares.
PROTOTYPES = {
    "kapyb_version": (C.c_int, []),
    "kapyb_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int]),
    "kapyb_destroy": (C.c_int, [C.c_void_p]),
    "kapyb_last_error_string": (C.c_char_p, [C.c_void_p]),
    "kapyb_check": (C.c_int, [C.c_void_p, C.c_void_p]),
    "kapyb_reserve_workspace": (C.c_int, [C.c_void_p, C.c_size_t]),
    "kapyb_matmul": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                               C.POINTER(Tensor2d), C.POINTER(Tensor2d), C.POINTER(Epilogue),
                               C.c_int32, C.c_void_p]),
    "kapyb_matmul_reduce": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                      C.POINTER(Tensor2d), C.POINTER(Tensor2d), C.c_int32,
                                      C.c_int32, C.POINTER(Epilogue), C.c_int32, C.c_void_p]),
    "kapyb_matmul_batched": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                       C.POINTER(Tensor2d), C.c_int32, C.c_int64, C.c_int64,
                                       C.c_int64, C.POINTER(Epilogue), C.c_int32, C.c_void_p]),
    "kapyb_matmul_host": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                    C.POINTER(Tensor2d), C.POINTER(Epilogue), C.c_int32,
                                    C.c_void_p]),
    "kapyb_matmul_push": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                    C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32,
                                    C.c_int32, C.c_int32, C.POINTER(Epilogue), C.c_int32,
                                    C.c_void_p]),
    "kapyb_gather_signal": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                      C.c_uint32, C.c_void_p]),
    "kapyb_gather_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint32, C.c_uint32,
                                    C.c_void_p]),
    "kapyb_matmul_host_sharded": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.c_int32, C.c_int32,
                                            C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                            C.POINTER(Epilogue), C.POINTER(ShardCtx), C.c_int32,
                                            C.c_void_p]),
    "kapyb_matmul_decode_static": (C.c_int, [C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                             C.POINTER(Tensor2d), C.POINTER(Epilogue), C.c_int32,
                                             C.c_void_p]),
    "kapyb_elementwise": (C.c_int, [C.c_void_p, C.POINTER(Inst), C.c_int32, C.POINTER(Tensor2d),
                                    C.c_int32, C.POINTER(Tensor2d), C.c_void_p]),
    "kapyb_reduce": (C.c_int, [C.c_void_p, C.POINTER(Tensor2d), C.POINTER(Tensor2d), C.c_int32,
                               C.c_int32, C.c_void_p]),
    "kapyb_shard_range": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.c_int64,
                                    C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "kapyb_last_kernel": (C.c_char_p, [C.c_void_p]),
    "kapyb_launch_count": (C.c_int64, [C.c_void_p]),
    "kapyb_tuning_load": (C.c_int, [C.c_char_p, C.POINTER(C.c_int32)]),
    "kapyb_tuning_clear": (C.c_int, []),
    "kapyb_matmul_plan": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                    C.POINTER(Tensor2d), C.c_int32, C.c_char_p, C.c_size_t]),
    "kapyb_probe_read": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32), C.c_int32]),
    "kapyb_set_matmul_path": (C.c_int, [C.c_void_p, C.c_char_p]),
}

_lib = None


def load():
    """dlopen the library and attach prototypes; raises if it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python kapy-lang_b200/build.py` "
                "(there is no fallback implementation)")
        lib = C.CDLL(SO_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
