"""Canonical elementwise op lists (the graphs the fused kernels recognise),
written as the instruction tuples ``Handle.elementwise`` takes.  The same tuples
are what the Builder shim records for the equivalent ``create_*`` sequence."""
from __future__ import annotations

from . import _abi as abi

GELU_C0 = 0.7978845608
GELU_C1 = 0.044715


def affine(dtype: int, s: float, b: float, rounding: int = abi.RN):
    """y = truncf(fma(extf(x), s, b))"""
    F = abi.F32
    return [
        (abi.OP_LOAD, dtype, 0, -1, -1, -1, 0.0, 0),
        (abi.OP_CVT, F, 1, 0, -1, -1, 0.0, abi.RN),
        (abi.OP_CONST, F, 2, -1, -1, -1, s, 0),
        (abi.OP_CONST, F, 3, -1, -1, -1, b, 0),
        (abi.OP_FMA, F, 4, 1, 2, 3, 0.0, 0),
        (abi.OP_CVT, dtype, 5, 4, -1, -1, 0.0, rounding),
        (abi.OP_STORE, dtype, -1, 5, -1, -1, 0.0, 0),
    ]


def affine_gelu_tanh(dtype: int, s: float, b: float, rounding: int = abi.RN):
    """y = truncf(u / (1 + exp(-2k))), u = fma(extf(x), s, b),
    k = c0 * fma(c1*u*u, u, u): gelu_tanh without the 1+tanh cancellation."""
    F = abi.F32
    return [
        (abi.OP_LOAD, dtype, 0, -1, -1, -1, 0.0, 0),
        (abi.OP_CVT, F, 1, 0, -1, -1, 0.0, abi.RN),
        (abi.OP_CONST, F, 2, -1, -1, -1, s, 0),
        (abi.OP_CONST, F, 3, -1, -1, -1, b, 0),
        (abi.OP_FMA, F, 4, 1, 2, 3, 0.0, 0),          # u
        (abi.OP_CONST, F, 5, -1, -1, -1, GELU_C1, 0),
        (abi.OP_MUL, F, 6, 5, 4, -1, 0.0, 0),         # c1*u
        (abi.OP_MUL, F, 7, 6, 4, -1, 0.0, 0),         # c1*u*u
        (abi.OP_FMA, F, 8, 7, 4, 4, 0.0, 0),          # c1*u^3 + u
        (abi.OP_CONST, F, 9, -1, -1, -1, GELU_C0, 0),
        (abi.OP_MUL, F, 10, 9, 8, -1, 0.0, 0),        # k
        (abi.OP_CONST, F, 11, -1, -1, -1, -2.0, 0),
        (abi.OP_MUL, F, 12, 11, 10, -1, 0.0, 0),      # -2k
        (abi.OP_EXP, F, 13, 12, -1, -1, 0.0, 0),
        (abi.OP_CONST, F, 14, -1, -1, -1, 1.0, 0),
        (abi.OP_ADD, F, 15, 14, 13, -1, 0.0, 0),      # 1 + exp(-2k)
        (abi.OP_DIV, F, 6, 4, 15, -1, 0.0, 0),        # u / (...)
        (abi.OP_CVT, dtype, 7, 6, -1, -1, 0.0, rounding),
        (abi.OP_STORE, dtype, -1, 7, -1, -1, 0.0, 0),
    ]


def binary(op: int, dtype: int):
    """z = a (op) b at one element type (elementwise_add.mlir:17-23)."""
    return [
        (abi.OP_LOAD, dtype, 0, -1, -1, -1, 0.0, 0),
        (abi.OP_LOAD, dtype, 1, -1, -1, -1, 0.0, 1),
        (op, dtype, 2, 0, 1, -1, 0.0, 0),
        (abi.OP_STORE, dtype, -1, 2, -1, -1, 0.0, 0),
    ]
