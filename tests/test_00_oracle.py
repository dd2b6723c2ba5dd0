"""The CPU checker against the committed known-answer vectors and closed forms.

The reference holds no golden vectors for this path, so the vectors under
tests/golden/ were generated independently of the checker (exact rational
arithmetic, exact integer products) by tests/golden/make_golden.py.
"""
import os

import numpy as np
import pytest
import torch

from util import bits

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_cvt_known_answers(ko):
    cvt = np.load(os.path.join(GOLD, "kat_rounding.npz"))["cvt"]
    L = ko.lib()
    for f32b, h_rn, h_rz, b_rn, b_rz in cvt:
        x = np.uint32(f32b).view(np.float32).item()
        assert L.ko_f32_to_f16(x, 1) == h_rn
        assert L.ko_f32_to_f16(x, 0) == h_rz
        assert L.ko_f32_to_bf16(x, 1) == b_rn
        assert L.ko_f32_to_bf16(x, 0) == b_rz


def test_fma_known_answers(ko):
    """Single-rounding fma at f16 / bf16 (ElementwiseOpToLLVM.cpp:771-892)."""
    fma = np.load(os.path.join(GOLD, "kat_rounding.npz"))["fma"]
    for fmt in (ko.F16, ko.BF16):
        rows = fma[fma[:, 0] == fmt]
        a = rows[:, 1].astype(np.uint16).reshape(1, -1)
        b = rows[:, 2].astype(np.uint16).reshape(1, -1)
        c = rows[:, 3].astype(np.uint16).reshape(1, -1)
        prog = [(0, fmt, 0, -1, -1, -1, 0.0, 0), (0, fmt, 1, -1, -1, -1, 0.0, 1),
                (0, fmt, 2, -1, -1, -1, 0.0, 2), (7, fmt, 3, 0, 1, 2, 0.0, 0),
                (27, fmt, -1, 3, -1, -1, 0.0, 0)]
        got = ko.eltwise(prog, [a, b, c], [fmt] * 3, a.shape, fmt)
        want = rows[:, 4].astype(np.uint16).reshape(1, -1)
        assert np.array_equal(got, want), np.flatnonzero(got != want)[:8]


def test_widening_matches_numpy_and_torch(ko):
    L = ko.lib()
    allb = np.arange(65536, dtype=np.uint16)
    f16 = allb.view(np.float16).astype(np.float32)
    bf = torch.from_numpy(allb.view(np.int16)).view(torch.bfloat16).float().numpy()
    for i in range(0, 65536, 97):
        a, b = L.ko_f16_to_f32(int(allb[i])), L.ko_bf16_to_f32(int(allb[i]))
        assert (np.isnan(a) and np.isnan(f16[i])) or a == f16[i]
        assert (np.isnan(b) and np.isnan(bf[i])) or b == bf[i]


def test_to_bits_matches_torch(ko):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1 << 16, generator=g) * torch.exp(torch.rand(1 << 16, generator=g) * 40 - 20)
    assert np.array_equal(ko.to_bits(x.numpy(), ko.BF16), bits(x.to(torch.bfloat16)))
    assert np.array_equal(ko.to_bits(x.numpy(), ko.F16), bits(x.to(torch.float16)))


@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("dtype", [0, 1])
def test_matmul_integer_exact(ko, name, dtype):
    """Ops.td:416-439: result = lhs . rhs + acc; bias as accumulator init
    (Combine.td:38-88).  With small integers everything is exact."""
    z = np.load(os.path.join(GOLD, "kat_matmul_int.npz"))
    A = ko.to_bits(z[f"A_{name}"].astype(np.float32), dtype)
    B = ko.to_bits(z[f"B_{name}"].astype(np.float32), dtype)
    bias = ko.to_bits(z[f"bias_{name}"].astype(np.float32), dtype)
    C = z[f"C_{name}"].astype(np.float64)
    ref = ko.matmul_f64(A, dtype, B, dtype, bias=bias, bias_dtype=dtype)
    assert np.array_equal(ref, C)
    out = ko.matmul_f32acc(A, dtype, B, dtype, ko.F32, bias=bias, bias_dtype=dtype)
    assert np.array_equal(out.astype(np.float64), C)
    # column-major B (config 1 layout) gives the same answer
    Bt = np.ascontiguousarray(B.T).T
    assert np.array_equal(ko.matmul_f64(A, dtype, Bt, dtype, bias=bias, bias_dtype=dtype), C)


def test_matmul_f64_vs_numpy(ko):
    rng = np.random.default_rng(5)
    A = ko.to_bits(rng.uniform(-1, 1, (130, 200)).astype(np.float32), ko.F16)
    B = ko.to_bits(rng.uniform(-1, 1, (200, 70)).astype(np.float32), ko.F16)
    ref = ko.matmul_f64(A, ko.F16, B, ko.F16, alpha=0.25)
    want = 0.25 * (ko.from_bits(A, ko.F16) @ ko.from_bits(B, ko.F16))
    assert np.allclose(ref, want, rtol=1e-13, atol=1e-13)
    rows, cols = [0, 5, 129], [1, 69]
    sub = ko.matmul_f64(A, ko.F16, B, ko.F16, alpha=0.25, rows=rows, cols=cols)
    assert np.allclose(sub, want[np.ix_(rows, cols)], rtol=1e-13, atol=1e-13)
    # fp32-accumulate port stays inside the parity tolerance of the f64 result
    o = ko.matmul_f32acc(A, ko.F16, B, ko.F16, ko.F16, alpha=0.25)
    err, _ = ko.max_rel_err(ko.from_bits(o, ko.F16), ref)
    assert err < 1e-2


def test_padding_and_broadcast(ko):
    """ld_global pads out-of-bounds lanes (Enums.td:52-61); size-1 axes broadcast."""
    x = ko.to_bits(np.arange(6, dtype=np.float32).reshape(2, 3), ko.F32)
    prog = [(0, ko.F32, 0, -1, -1, -1, 0.0, 0), (27, ko.F32, -1, 0, -1, -1, 0.0, 0)]
    for pad, val in ((ko.PAD_ZERO, 0.0), (ko.PAD_PINF, np.inf), (ko.PAD_NINF, -np.inf)):
        out = ko.eltwise(prog, [x], [ko.F32], (3, 4), ko.F32, paddings=[pad])
        assert np.array_equal(out[:2, :3], x)
        assert np.all(out[2, :] == val) and np.all(out[:, 3] == val)
    out = ko.eltwise(prog, [x], [ko.F32], (3, 4), ko.F32, paddings=[ko.PAD_QNAN])
    assert np.isnan(out[2, :]).all() and np.isnan(out[:, 3]).all()
    row = ko.to_bits(np.array([[1.0, 2.0, 3.0]], dtype=np.float32), ko.F32)
    out = ko.eltwise(prog, [row], [ko.F32], (4, 3), ko.F32)
    assert np.array_equal(out, np.repeat(row, 4, axis=0))


def test_clamp_nan_rules(ko):
    """ClampFOpConversion (ElementwiseOpToLLVM.cpp:699-728)."""
    x = np.array([[np.nan, -5.0, 0.5, 9.0]], dtype=np.float32)
    lo = np.full_like(x, -1.0)
    hi = np.full_like(x, 1.0)
    for flag in (0, 1):
        prog = [(0, ko.F32, 0, -1, -1, -1, 0.0, 0), (0, ko.F32, 1, -1, -1, -1, 0.0, 1),
                (0, ko.F32, 2, -1, -1, -1, 0.0, 2), (12, ko.F32, 3, 0, 1, 2, 0.0, flag),
                (27, ko.F32, -1, 3, -1, -1, 0.0, 0)]
        out = ko.eltwise(prog, [x, lo, hi], [ko.F32] * 3, x.shape, ko.F32)
        assert np.array_equal(out[0, 1:], [-1.0, 0.5, 1.0])
        assert np.isnan(out[0, 0]) if flag else out[0, 0] == -1.0


def test_gelu_graph_fast_port_matches_interpreter(ko, pkg):
    """The timed CPU baseline loop agrees with the op-by-op interpreter to 2 ulp
    (expf vs an exactly rounded exp) and is bit-exact without the exp."""
    x = ko.to_bits(np.random.default_rng(9).standard_normal((1, 20000)).astype(np.float32), ko.BF16)
    lin = ko.eltwise(pkg.programs.affine(ko.BF16, 0.5, 0.1), [x], [ko.BF16], x.shape, ko.BF16)
    assert np.array_equal(lin, ko.affine_gelu_bf16(x, 0.5, 0.1, linear_only=True))
    gel = ko.eltwise(pkg.programs.affine_gelu_tanh(ko.BF16, 0.5, 0.1), [x], [ko.BF16], x.shape,
                     ko.BF16)
    assert ko.ulp_diff(gel, ko.affine_gelu_bf16(x, 0.5, 0.1)).max() <= 2
    # and the composite is gelu_tanh: compare with torch's definition in f64
    u = ko.from_bits(x, ko.BF16) * 0.5 + np.float64(np.float32(0.1))
    want = torch.nn.functional.gelu(torch.from_numpy(u), approximate="tanh").numpy()
    assert np.allclose(ko.from_bits(gel, ko.BF16), want, rtol=2 ** -7, atol=1e-6)


def test_reduce(ko):
    rng = np.random.default_rng(2)
    X = ko.to_bits(rng.standard_normal((37, 300)).astype(np.float32), ko.BF16)
    v = ko.from_bits(X, ko.BF16)
    s, ab = ko.reduce_f64(X, ko.BF16, 1)
    assert np.allclose(s, v.sum(axis=1), rtol=1e-12) and np.allclose(ab, np.abs(v).sum(axis=1))
    s0, _ = ko.reduce_f64(X, ko.BF16, 0)
    assert np.allclose(s0, v.sum(axis=0), rtol=1e-12)
    mx, _ = ko.reduce_f64(X, ko.BF16, 1, ko.RED_MAX)
    assert np.array_equal(mx, v.max(axis=1))
    fast = ko.rowsum_bf16_f32(X)
    assert np.all(np.abs(fast - s) <= 4 * 2.0 ** -24 * ab)


def test_cmpf_select_truth_table(ko):
    """arith.cmpf predicates (ir.cc:941-1000) and arith.select (ir.cc:1162) in the
    checker's interpreter against a table written out by hand: ordered
    predicates are false and unordered ones true as soon as an operand is NaN."""
    nan = np.float32(np.nan)
    a = np.array([[1.0, 2.0, 2.0, nan, 1.0, nan, 0.0]], dtype=np.float32)
    b = np.array([[2.0, 1.0, 2.0, 1.0, nan, nan, -0.0]], dtype=np.float32)
    #            a<b   a>b  a==b  NaN?  NaN?  NaN?  +0 == -0
    table = {"olt": [1, 0, 0, 0, 0, 0, 0], "ogt": [0, 1, 0, 0, 0, 0, 0],
             "ole": [1, 0, 1, 0, 0, 0, 1], "oge": [0, 1, 1, 0, 0, 0, 1],
             "oeq": [0, 0, 1, 0, 0, 0, 1], "one": [1, 1, 0, 0, 0, 0, 0],
             "ult": [1, 0, 0, 1, 1, 1, 0], "ugt": [0, 1, 0, 1, 1, 1, 0],
             "ule": [1, 0, 1, 1, 1, 1, 1], "uge": [0, 1, 1, 1, 1, 1, 1],
             "ueq": [0, 0, 1, 1, 1, 1, 1], "une": [1, 1, 0, 1, 1, 1, 0]}
    names = ["olt", "ogt", "ole", "oge", "oeq", "one", "ult", "ugt", "ule", "uge", "ueq", "une"]
    F, I1 = ko.F32, ko.I1
    for pred, name in enumerate(names):
        # out = select(a <pred> b, 10, 20)
        prog = [(0, F, 0, -1, -1, -1, 0.0, 0), (0, F, 1, -1, -1, -1, 0.0, 1),
                (28, I1, 2, 0, 1, -1, 0.0, pred),
                (1, F, 3, -1, -1, -1, 10.0, 0), (1, F, 4, -1, -1, -1, 20.0, 0),
                (29, F, 5, 2, 3, 4, 0.0, 0), (27, F, -1, 5, -1, -1, 0.0, 0)]
        got = ko.eltwise(prog, [a, b], [F, F], a.shape, F)
        want = np.where(np.array(table[name]) == 1, 10.0, 20.0).astype(np.float32).reshape(1, -1)
        assert np.array_equal(got, want), name
    # and / or / xor on conditions
    for op, fn in ((30, np.logical_and), (31, np.logical_or), (32, np.logical_xor)):
        prog = [(0, F, 0, -1, -1, -1, 0.0, 0), (0, F, 1, -1, -1, -1, 0.0, 1),
                (28, I1, 2, 0, 1, -1, 0.0, 0), (28, I1, 3, 0, 1, -1, 0.0, 4),
                (op, I1, 4, 2, 3, -1, 0.0, 0), (1, F, 5, -1, -1, -1, 1.0, 0),
                (1, F, 6, -1, -1, -1, 0.0, 0), (29, F, 7, 4, 5, 6, 0.0, 0),
                (27, F, -1, 7, -1, -1, 0.0, 0)]
        got = ko.eltwise(prog, [a, b], [F, F], a.shape, F)
        want = fn(np.array(table["olt"]) == 1, np.array(table["oeq"]) == 1).astype(np.float32)
        assert np.array_equal(got.ravel(), want), op


def test_thread_count_can_be_set(ko):
    """The timed CPU baseline must not inherit a launcher's OMP_NUM_THREADS=1."""
    import os
    before = ko.num_threads()
    assert ko.set_num_threads(1) == 1 and ko.num_threads() == 1
    n = ko.set_num_threads(0)
    assert n == ko.num_threads() and 1 <= n <= (os.cpu_count() or 1)
    ko.set_num_threads(before)


def test_f8_decode_tables(ko):
    """The checker's f8E4M3 / f8E5M2 decoders against torch's conversions, all
    256 bit patterns each (an independent implementation of the two formats)."""
    for code, td in ((ko.F8E4M3, torch.float8_e4m3fn), (ko.F8E5M2, torch.float8_e5m2)):
        table = ko.f8_table(code)
        ref = torch.arange(256, dtype=torch.uint8).view(td).to(torch.float64).numpy()
        assert np.array_equal(np.isnan(table), np.isnan(ref))
        assert np.array_equal(table[~np.isnan(ref)], ref[~np.isnan(ref)])


def test_f8_downcasts(ko):
    """cvt.rn.satfinite to f8E4M3 / f8E5M2 over every f16 value: equal to torch's
    conversion wherever the value is within the format's finite range (an
    independent implementation), the largest finite value beyond it (torch gives
    NaN / Inf there, the reference saturates), NaN for NaN.  rz to f8E5M2 is the
    high byte of the f16 pattern."""
    h = np.arange(65536, dtype=np.uint16)
    x = h.view(np.float16).astype(np.float32)
    for code, td, maxv in ((ko.F8E4M3, torch.float8_e4m3fn, 448.0), (ko.F8E5M2, torch.float8_e5m2, 57344.0)):
        got = ko.to_bits(x, code, ko.RN)
        ref = torch.from_numpy(x).to(td).view(torch.uint8).numpy()
        inr = np.isfinite(x) & (np.abs(x) <= maxv)
        assert np.array_equal(got[inr], ref[inr])
        big = ~np.isnan(x) & (np.abs(x) > maxv)
        assert np.array_equal(ko.from_bits(got[big], code), np.sign(x[big]) * maxv)
        assert np.isnan(ko.from_bits(got[np.isnan(x)], code)).all()
    rz = ko.to_bits(x, ko.F8E5M2, ko.RZ)
    ok = ~np.isnan(x)
    assert np.array_equal(rz[ok], (h >> 8).astype(np.uint8)[ok])
