"""CPU checker for the kapy matmul / elementwise / reduce path (ctypes front of
``kapy_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Imported by ``tests/``, by the smoke check and by the
CPU-baseline / reference arm of the benchmark; never by the product package.

PARITY UNPINNED: the reference has no golden vectors for this path and cannot be
built in this environment, so the restatement is pinned by closed-form cases
only (see the header of ``kapy_oracle.c``).

Arrays are numpy; bf16 and f16 tensors are carried as ``uint16`` bit patterns
(``dtype`` says which), f32 as ``float32``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libkapy_oracle.so")

F16, BF16, F32, F8E4M3, F8E5M2, I1 = 0, 1, 2, 3, 4, 5
RZ, RN = 0, 1
PAD_ZERO, PAD_QNAN, PAD_PINF, PAD_NINF = 0, 1, 2, 3
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_SILU = 0, 1, 2, 3
RED_ADD, RED_MUL, RED_MAX, RED_MIN = 0, 1, 2, 3


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


class Inst(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("dst", C.c_int32),
                ("a", C.c_int32), ("b", C.c_int32), ("c", C.c_int32),
                ("imm", C.c_float), ("flags", C.c_int32)]


def build(force: bool = False) -> str:
    """Compiles the C restatement with the Makefile beside it."""
    src = os.path.join(_HERE, "kapy_oracle.c")
    hdr = os.path.join(_HERE, "..", "include", "kapyb.h")
    stale = (not os.path.exists(_SO)
             or os.path.getmtime(_SO) < os.path.getmtime(src)
             or (os.path.exists(hdr) and os.path.getmtime(_SO) < os.path.getmtime(hdr)))
    if force or stale:
        env = dict(os.environ)
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()     # compiles only when the source is newer than the library
        L = C.CDLL(_SO)
        L.ko_bf16_to_f32.restype = C.c_float
        L.ko_bf16_to_f32.argtypes = [C.c_uint16]
        L.ko_f16_to_f32.restype = C.c_float
        L.ko_f16_to_f32.argtypes = [C.c_uint16]
        L.ko_f32_to_bf16.restype = C.c_uint16
        L.ko_f32_to_bf16.argtypes = [C.c_float, C.c_int]
        L.ko_f32_to_f16.restype = C.c_uint16
        L.ko_f32_to_f16.argtypes = [C.c_float, C.c_int]
        L.ko_f32_to_f8.restype = C.c_uint8
        L.ko_f32_to_f8.argtypes = [C.c_float, C.c_int, C.c_int]
        L.ko_eltwise.restype = C.c_int
        L.ko_eltwise.argtypes = [C.POINTER(Inst), C.c_int, C.POINTER(Tensor2d), C.c_int,
                                 C.POINTER(Tensor2d)]
        L.ko_affine_gelu_bf16.restype = None
        L.ko_affine_gelu_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_float,
                                          C.c_int]
        L.ko_reduce_f64.restype = C.c_int
        L.ko_reduce_f64.argtypes = [C.POINTER(Tensor2d), C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.ko_rowsum_bf16_f32.restype = None
        L.ko_rowsum_bf16_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
        L.ko_matmul_f64.restype = C.c_int
        L.ko_matmul_f64.argtypes = [C.POINTER(Tensor2d), C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                    C.POINTER(Epilogue), C.c_void_p, C.c_int32, C.c_void_p,
                                    C.c_int32, C.c_void_p]
        L.ko_matmul_f32acc.restype = C.c_int
        L.ko_matmul_f32acc.argtypes = [C.POINTER(Tensor2d), C.POINTER(Tensor2d),
                                       C.POINTER(Tensor2d), C.POINTER(Epilogue), C.c_int32,
                                       C.c_int32]
        L.ko_max_rel_err.restype = C.c_double
        L.ko_max_rel_err.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(C.c_double)]
        L.ko_num_threads.restype = C.c_int
        L.ko_set_num_threads.restype = C.c_int
        L.ko_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


# --------------------------------------------------------------- numpy helpers

def np_dtype(dtype: int):
    if dtype in (F8E4M3, F8E5M2):
        return np.uint8
    return np.float32 if dtype == F32 else np.uint16


def f8_table(dtype: int) -> np.ndarray:
    """The 256 values of an 8-bit float type, indexed by bit pattern (f64;
    decoded by the C oracle, one descriptor element at a time)."""
    bits = np.arange(256, dtype=np.uint8).reshape(1, 256)
    ident = np.ones((1, 1), dtype=np.float32)
    # 1x1 . 1x256 product: exact, one term per output.
    return matmul_f64(ident, F32, bits, dtype)[0]


def to_bits(x: np.ndarray, dtype: int, rounding: int = RN) -> np.ndarray:
    """float32/float64 array -> storage array of `dtype` (RN-even or RZ)."""
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == F32:
        return x32
    if dtype in (F8E4M3, F8E5M2):
        f = np.vectorize(lambda v: lib().ko_f32_to_f8(float(v), dtype, rounding), otypes=[np.uint8])
        return f(x32)
    if dtype == F16:
        if rounding == RN:
            return x32.astype(np.float16).view(np.uint16)
        f = np.vectorize(lambda v: lib().ko_f32_to_f16(float(v), 0), otypes=[np.uint16])
        return f(x32)
    u = x32.view(np.uint32)
    if rounding == RN:
        r = ((u >> 16) & 1) + np.uint32(0x7FFF)
        out = ((u + r) >> 16).astype(np.uint16)
    else:
        out = (u >> 16).astype(np.uint16)
    out = np.where(np.isnan(x32), np.uint16(0x7FFF), out)
    return out.astype(np.uint16)


def from_bits(a: np.ndarray, dtype: int) -> np.ndarray:
    """storage array -> float64 values (exact)."""
    if dtype == F32:
        return a.astype(np.float64)
    if dtype == F16:
        return a.view(np.float16).astype(np.float64)
    if dtype in (F8E4M3, F8E5M2):
        return f8_table(dtype)[a]
    return (a.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def tensor2d(a: np.ndarray, dtype: int, padding: int = PAD_ZERO, shape=None, strides=None,
             offset: int = 0) -> Tensor2d:
    """Descriptor over a numpy storage array (kept alive by the caller)."""
    assert a.dtype == np_dtype(dtype), (a.dtype, dtype)
    if shape is None:
        assert a.ndim == 2
        shape = a.shape
        strides = (a.strides[0] // a.itemsize, a.strides[1] // a.itemsize)
    return Tensor2d(a.ctypes.data, offset, int(shape[0]), int(shape[1]), int(strides[0]),
                    int(strides[1]), dtype, padding)


def epilogue(alpha=1.0, bias: np.ndarray | None = None, bias_dtype=F32, bias_axis=1,
             activation=ACT_NONE, rounding=RN) -> Epilogue:
    return Epilogue(float(alpha), bias.ctypes.data if bias is not None else None, bias_dtype,
                    bias_axis, activation, rounding)


# ------------------------------------------------------------------- wrappers

def matmul_f64(A, a_dtype, B, b_dtype, *, alpha=1.0, bias=None, bias_dtype=F32, bias_axis=1,
               activation=ACT_NONE, acc=None, acc_dtype=F32, rows=None, cols=None) -> np.ndarray:
    """f64 reference of out = act(alpha * A.B + bias (+ acc)) at the requested
    rows/cols (all when None).  A: [M,K] storage array (any strides), B: [K,N]."""
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    ta, tb = tensor2d(A, a_dtype), tensor2d(B, b_dtype)
    tacc = tensor2d(acc, acc_dtype) if acc is not None else None
    ep = epilogue(alpha, bias, bias_dtype, bias_axis, activation)
    r = np.ascontiguousarray(rows, dtype=np.int32) if rows is not None else None
    c = np.ascontiguousarray(cols, dtype=np.int32) if cols is not None else None
    nr = len(r) if r is not None else M
    nc = len(c) if c is not None else N
    ref = np.empty((nr, nc), dtype=np.float64)
    st = lib().ko_matmul_f64(C.byref(ta), C.byref(tb), C.byref(tacc) if tacc else None,
                             C.byref(ep), r.ctypes.data if r is not None else None, nr,
                             c.ctypes.data if c is not None else None, nc, ref.ctypes.data)
    assert st == 0, st
    return ref


def matmul_f32acc(A, a_dtype, B, b_dtype, out_dtype, *, alpha=1.0, bias=None, bias_dtype=F32,
                  bias_axis=1, activation=ACT_NONE, rounding=RN, row_begin=0, row_end=None):
    """fp32-accumulate CPU matmul with the reference's rounding points; returns
    the [M,N] storage array (only rows [row_begin,row_end) are computed)."""
    M, K = A.shape
    N = B.shape[1]
    out = np.zeros((M, N), dtype=np_dtype(out_dtype))
    ta, tb, to = tensor2d(A, a_dtype), tensor2d(B, b_dtype), tensor2d(out, out_dtype)
    ep = epilogue(alpha, bias, bias_dtype, bias_axis, activation, rounding)
    st = lib().ko_matmul_f32acc(C.byref(ta), C.byref(tb), C.byref(to), C.byref(ep), row_begin,
                                M if row_end is None else row_end)
    assert st == 0, st
    return out


def max_rel_err(c64: np.ndarray, ref64: np.ndarray):
    """(max_i |c-ref| / max(|ref|, tau), tau) with tau = 2^-6 rms(ref)."""
    c64 = np.ascontiguousarray(c64, dtype=np.float64)
    ref64 = np.ascontiguousarray(ref64, dtype=np.float64)
    assert c64.shape == ref64.shape
    tau = C.c_double(0)
    e = lib().ko_max_rel_err(c64.ctypes.data, ref64.ctypes.data, c64.size, C.byref(tau))
    return float(e), float(tau.value)


def make_prog(insts) -> "C.Array":
    arr = (Inst * len(insts))()
    for i, t in enumerate(insts):
        arr[i] = Inst(*t)
    return arr


def eltwise(insts, inputs, in_dtypes, out_shape, out_dtype, paddings=None) -> np.ndarray:
    """Runs a program [(op,dtype,dst,a,b,c,imm,flags), ...] over numpy inputs."""
    prog = make_prog(insts)
    tin = (Tensor2d * max(1, len(inputs)))()
    for i, (a, dt) in enumerate(zip(inputs, in_dtypes)):
        tin[i] = tensor2d(a, dt, paddings[i] if paddings else PAD_ZERO)
    out = np.zeros(out_shape, dtype=np_dtype(out_dtype))
    tout = tensor2d(out, out_dtype)
    st = lib().ko_eltwise(prog, len(insts), tin, len(inputs), C.byref(tout))
    assert st == 0, st
    return out


def affine_gelu_bf16(x_bits: np.ndarray, s: float, b: float, linear_only=False) -> np.ndarray:
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    y = np.empty_like(x_bits)
    lib().ko_affine_gelu_bf16(x_bits.ctypes.data, y.ctypes.data, x_bits.size, s, b,
                              1 if linear_only else 0)
    return y


def reduce_f64(src: np.ndarray, dtype: int, axis: int, combiner: int = RED_ADD):
    """(f64 result, sum|x|) along `axis` of a 2-D storage array."""
    t = tensor2d(src, dtype)
    n = src.shape[0] if axis == 1 else src.shape[1]
    out = np.empty(n, dtype=np.float64)
    ab = np.empty(n, dtype=np.float64)
    st = lib().ko_reduce_f64(C.byref(t), axis, combiner, out.ctypes.data, ab.ctypes.data)
    assert st == 0, st
    return out, ab


def rowsum_bf16_f32(x_bits: np.ndarray) -> np.ndarray:
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    out = np.empty(x_bits.shape[0], dtype=np.float32)
    lib().ko_rowsum_bf16_f32(x_bits.ctypes.data, out.ctypes.data, x_bits.shape[0], x_bits.shape[1])
    return out


def num_threads() -> int:
    return int(lib().ko_num_threads())


def set_num_threads(n: int = 0) -> int:
    """Threads the OpenMP loops use from now on (0: every processor this process
    may run on, whatever OMP_NUM_THREADS a launcher exported)."""
    return int(lib().ko_set_num_threads(int(n)))


def ulp_diff(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two uint16 float patterns
    (bf16 or f16: both are sign-magnitude, so the mapping is the same)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a_bits) - key(b_bits))
