"""Elementwise kernels against the CPU checker, through the C ABI.
Bit-exact for pure arithmetic; <= 2 ulp of the output type once a
transcendental or a division is involved."""
import numpy as np
import pytest
import torch

from util import bits, code, gen, normal

pytestmark = pytest.mark.gpu


def run_both(handle, ko, prog, inputs, out_shape, out_dtype, paddings=None):
    dev = [t.cuda() for t in inputs]
    out = torch.empty(out_shape, dtype=out_dtype, device="cuda")
    handle.elementwise(prog, dev, out, paddings=paddings)
    handle.check()
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
    want = ko.eltwise(prog, [bits(t) for t in inputs], [code[t.dtype] for t in inputs], out_shape,
                      code[out_dtype], paddings=paddings)
    return bits(out.cpu()), want


@pytest.mark.parametrize("n", [1 << 16, 8 * 1000 + 3, 5, 0])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_affine_bit_exact(handle, ko, pkg, n, dt):
    x = normal((1, n), 1003, dtype=dt)
    prog = pkg.programs.affine(pkg.runtime.dtype_code(dt), 0.5, 0.1)
    got, want = run_both(handle, ko, prog, [x], (1, n), dt)
    if n:
        assert handle.last_kernel == "elt_affine"
    assert np.array_equal(got, want)


@pytest.mark.parametrize("n", [1 << 18, 4099])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_affine_gelu_within_2ulp(handle, ko, pkg, n, dt):
    x = normal((1, n), 1003, dtype=dt) * 2
    prog = pkg.programs.affine_gelu_tanh(pkg.runtime.dtype_code(dt), 0.5, 0.1)
    got, want = run_both(handle, ko, prog, [x], (1, n), dt)
    assert handle.last_kernel == "elt_affine_gelu"
    d = ko.ulp_diff(got, want)
    assert d.max() <= 2, (d.max(), np.flatnonzero(d > 2)[:5])
    assert (d == 0).mean() > 0.95


def test_fused_equals_interpreter(handle, ko, pkg):
    """A misaligned view forces the generic interpreter; it must give the same
    bits as the fused kernel."""
    x = normal((1, 4096 + 1), 11)
    xd = x.cuda()
    prog = pkg.programs.affine_gelu_tanh(pkg.abi.BF16, 0.5, 0.1)
    y_fused = torch.empty((1, 4096), dtype=torch.bfloat16, device="cuda")
    handle.elementwise(prog, [xd[:, :4096]], y_fused)
    assert handle.last_kernel == "elt_affine_gelu"
    y_interp = torch.empty((1, 4096), dtype=torch.bfloat16, device="cuda")
    src = torch.empty((1, 4097), dtype=torch.bfloat16, device="cuda")
    src[:, 1:] = xd[:, :4096]
    handle.elementwise(prog, [src[:, 1:]], y_interp)
    assert handle.last_kernel == "elt_interp"
    handle.check()
    assert torch.equal(y_fused, y_interp)


@pytest.mark.parametrize("op", ["ADD", "SUB", "MUL", "DIV", "MAXIMUM", "MINIMUM", "MAXNUM", "MINNUM"])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_binary_bit_exact(handle, ko, pkg, op, dt):
    """elementwise_add.mlir:17-23 at whole-tensor scope: [1,n] f16 add, and its
    siblings; bf16 ops are single-rounding fma (ElementwiseOpToLLVM.cpp:771-892)."""
    n = 512 * 37 + 5
    a, b = normal((1, n), 21, dtype=dt), normal((1, n), 22, dtype=dt) * 3
    prog = pkg.programs.binary(getattr(pkg.abi, "OP_" + op), pkg.runtime.dtype_code(dt))
    got, want = run_both(handle, ko, prog, [a, b], (1, n), dt)
    assert handle.last_kernel == "elt_binary"
    if dt == torch.float32 and op == "DIV":
        # div.full.f32 (ElementwiseOpToLLVM.cpp:730-769) is good to 2 ulp, not correctly rounded
        g, w = got.view(np.uint32).astype(np.int64), want.view(np.uint32).astype(np.int64)
        assert np.abs(g - w).max() <= 2
    elif dt == torch.float32:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    else:
        assert np.array_equal(got, want)


def test_interpreter_all_bf16_graph(handle, ko, pkg):
    """An all-bf16 chain rounds after every op: ((x*s)+b) clamp, abs, max."""
    A = pkg.abi
    x = normal((48, 200), 31)
    y = normal((48, 1), 32)      # broadcast along axis 1
    B = A.BF16
    prog = [
        (A.OP_LOAD, B, 0, -1, -1, -1, 0.0, 0), (A.OP_LOAD, B, 1, -1, -1, -1, 0.0, 1),
        (A.OP_CONST, B, 2, -1, -1, -1, 0.3, 0), (A.OP_MUL, B, 3, 0, 2, -1, 0.0, 0),
        (A.OP_ADD, B, 4, 3, 1, -1, 0.0, 0), (A.OP_FMA, B, 5, 4, 0, 1, 0.0, 0),
        (A.OP_CONST, B, 6, -1, -1, -1, -0.75, 0), (A.OP_CONST, B, 7, -1, -1, -1, 0.75, 0),
        (A.OP_CLAMP, B, 8, 5, 6, 7, 0.0, 0), (A.OP_ABS, B, 9, 8, -1, -1, 0.0, 0),
        (A.OP_SUB, B, 10, 9, 1, -1, 0.0, 0), (A.OP_MAXIMUM, B, 11, 10, 3, -1, 0.0, 0),
        (A.OP_STORE, B, -1, 11, -1, -1, 0.0, 0),
    ]
    got, want = run_both(handle, ko, prog, [x, y], (48, 200), torch.bfloat16)
    assert handle.last_kernel == "elt_interp"
    assert np.array_equal(got, want)


def test_interpreter_transcendentals_f32(handle, ko, pkg):
    A = pkg.abi
    x = normal((4, 1000), 41, dtype=torch.float32).abs() + 0.01
    F = A.F32
    for op in (A.OP_EXP, A.OP_EXP2, A.OP_LOG, A.OP_LOG2, A.OP_SQRT, A.OP_RSQRT, A.OP_ERF,
               A.OP_SIN, A.OP_COS, A.OP_TANH):
        prog = [(A.OP_LOAD, F, 0, -1, -1, -1, 0.0, 0), (op, F, 1, 0, -1, -1, 0.0, 0),
                (A.OP_STORE, F, -1, 1, -1, -1, 0.0, 0)]
        got, want = run_both(handle, ko, prog, [x], (4, 1000), torch.float32)
        ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
        # ex2.approx / lg2-based paths: a few f32 ulp; after a bf16 downcast
        # these are far inside 2 ulp of the output type
        assert ulp.max() <= 64, (op, ulp.max())
        prog16 = prog[:2] + [(A.OP_CVT, A.BF16, 2, 1, -1, -1, 0.0, A.RN),
                             (A.OP_STORE, A.BF16, -1, 2, -1, -1, 0.0, 0)]
        g16, w16 = run_both(handle, ko, prog16, [x], (4, 1000), torch.bfloat16)
        assert ko.ulp_diff(g16, w16).max() <= 2, op


def test_padding_broadcast_and_strides(handle, ko, pkg):
    A = pkg.abi
    x = normal((20, 30), 51, dtype=torch.float32)
    prog = [(A.OP_LOAD, A.F32, 0, -1, -1, -1, 0.0, 0), (A.OP_NEG, A.F32, 1, 0, -1, -1, 0.0, 0),
            (A.OP_STORE, A.F32, -1, 1, -1, -1, 0.0, 0)]
    for pad in (A.PAD_ZERO, A.PAD_PINF, A.PAD_NINF):
        got, want = run_both(handle, ko, prog, [x], (24, 32), torch.float32, paddings=[pad])
        assert np.array_equal(got, want)
    # transposed (column-major) input view and output
    xt = x.t()
    out = torch.empty((20, 30), dtype=torch.float32, device="cuda").t()
    handle.elementwise(prog, [xt.cuda()], out)
    handle.check()
    assert torch.equal(out.cpu(), -xt)


def test_cvt_rounding_modes(handle, ko, pkg):
    A = pkg.abi
    x = normal((1, 5000), 61, dtype=torch.float32) * 100
    for dt, tdt in ((A.BF16, torch.bfloat16), (A.F16, torch.float16)):
        for rnd in (A.RN, A.RZ):
            prog = [(A.OP_LOAD, A.F32, 0, -1, -1, -1, 0.0, 0),
                    (A.OP_CVT, dt, 1, 0, -1, -1, 0.0, rnd), (A.OP_STORE, dt, -1, 1, -1, -1, 0.0, 0)]
            got, want = run_both(handle, ko, prog, [x], (1, 5000), tdt)
            assert np.array_equal(got, want)


def test_verifier_rejections(handle, pkg):
    A = pkg.abi
    x = torch.zeros((1, 8), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((1, 8), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="undefined value"):
        handle.elementwise([(A.OP_ADD, A.BF16, 0, 1, 2, -1, 0.0, 0),
                            (A.OP_STORE, A.BF16, -1, 0, -1, -1, 0.0, 0)], [x], y)
    with pytest.raises(ValueError, match="same element type"):
        handle.elementwise([(A.OP_LOAD, A.BF16, 0, -1, -1, -1, 0.0, 0),
                            (A.OP_CONST, A.F32, 1, -1, -1, -1, 1.0, 0),
                            (A.OP_ADD, A.F32, 2, 0, 1, -1, 0.0, 0),
                            (A.OP_CVT, A.BF16, 3, 2, -1, -1, 0.0, 1),
                            (A.OP_STORE, A.BF16, -1, 3, -1, -1, 0.0, 0)], [x], y)
    with pytest.raises(ValueError, match="rounding mode must be set"):
        handle.elementwise([(A.OP_LOAD, A.BF16, 0, -1, -1, -1, 0.0, 0),
                            (A.OP_CVT, A.F32, 1, 0, -1, -1, 0.0, 1),
                            (A.OP_CVT, A.BF16, 2, 1, -1, -1, 0.0, 7),
                            (A.OP_STORE, A.BF16, -1, 2, -1, -1, 0.0, 0)], [x], y)
    with pytest.raises(ValueError, match="stores exactly once"):
        handle.elementwise([(A.OP_LOAD, A.BF16, 0, -1, -1, -1, 0.0, 0)], [x], y)


# ------------------------------------------------------------ cmpf / select

@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_cmpf_select_every_predicate(handle, ko, pkg, dt):
    """arith.cmpf with each predicate Builder.create_cmpf_* offers (ir.cc:941-1000)
    feeding arith.select (ir.cc:1162): bit-exact, NaN operands included (ordered
    predicates false, unordered true), equal values and signed zeros too."""
    A = pkg.abi
    D = pkg.runtime.dtype_code(dt)
    a = normal((6, 300), 71, dtype=dt)
    b = normal((6, 300), 72, dtype=dt)
    b[:, ::7] = a[:, ::7]                      # equal pairs
    a[0, 5], b[1, 9] = float("nan"), float("nan")
    a[2, 11], b[2, 11] = float("nan"), float("nan")
    a[3, 1], b[3, 1] = 0.0, -0.0
    for pred in range(len(A.CMP_PREDICATES)):
        prog = [(A.OP_LOAD, D, 0, -1, -1, -1, 0.0, 0), (A.OP_LOAD, D, 1, -1, -1, -1, 0.0, 1),
                (A.OP_CMP, A.I1, 2, 0, 1, -1, 0.0, pred),
                (A.OP_SELECT, D, 3, 2, 0, 1, 0.0, 0), (A.OP_STORE, D, -1, 3, -1, -1, 0.0, 0)]
        got, want = run_both(handle, ko, prog, [a, b], (6, 300), dt)
        assert handle.last_kernel == "elt_interp"
        same = (got.view(np.uint32) == want.view(np.uint32)) if dt == torch.float32 else got == want
        assert same.all(), (A.CMP_PREDICATES[pred], int((~same).sum()))


def test_select_graph_with_condition_logic(handle, ko, pkg):
    """y = (x > lo and not (x >= hi)) ? x * 2 : -1, conditions combined with
    andi / xori on i1 values."""
    A = pkg.abi
    F = A.F32
    x = normal((5, 777), 73, dtype=torch.float32)
    prog = [(A.OP_LOAD, F, 0, -1, -1, -1, 0.0, 0),
            (A.OP_CONST, F, 1, -1, -1, -1, -0.5, 0), (A.OP_CONST, F, 2, -1, -1, -1, 0.75, 0),
            (A.OP_CMP, A.I1, 3, 0, 1, -1, 0.0, A.CMP_PREDICATES.index("ogt")),
            (A.OP_CMP, A.I1, 4, 0, 2, -1, 0.0, A.CMP_PREDICATES.index("oge")),
            (A.OP_XOR, A.I1, 5, 3, 4, -1, 0.0, 0),      # in (lo, hi): exactly one holds
            (A.OP_AND, A.I1, 6, 5, 3, -1, 0.0, 0),
            (A.OP_CONST, F, 7, -1, -1, -1, 2.0, 0), (A.OP_MUL, F, 8, 0, 7, -1, 0.0, 0),
            (A.OP_CONST, F, 9, -1, -1, -1, -1.0, 0),
            (A.OP_SELECT, F, 10, 6, 8, 9, 0.0, 0), (A.OP_STORE, F, -1, 10, -1, -1, 0.0, 0)]
    got, want = run_both(handle, ko, prog, [x], (5, 777), torch.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ref = torch.where((x > -0.5) & ~(x >= 0.75), x * 2, torch.full_like(x, -1.0))
    assert np.array_equal(got, ref.numpy())


def test_cmpf_select_rules(handle, pkg):
    A = pkg.abi
    x = torch.zeros((1, 8), dtype=torch.float32, device="cuda")
    y = torch.zeros((1, 8), dtype=torch.float32, device="cuda")
    ld = [(A.OP_LOAD, A.F32, 0, -1, -1, -1, 0.0, 0)]
    with pytest.raises(ValueError, match="i1 condition"):
        handle.elementwise(ld + [(A.OP_SELECT, A.F32, 1, 0, 0, 0, 0.0, 0),
                                 (A.OP_STORE, A.F32, -1, 1, -1, -1, 0.0, 0)], [x], y)
    with pytest.raises(ValueError, match="unknown cmpf predicate"):
        handle.elementwise(ld + [(A.OP_CMP, A.I1, 1, 0, 0, -1, 0.0, 12),
                                 (A.OP_SELECT, A.F32, 2, 1, 0, 0, 0.0, 0),
                                 (A.OP_STORE, A.F32, -1, 2, -1, -1, 0.0, 0)], [x], y)
    with pytest.raises(ValueError, match="st_global source is"):
        handle.elementwise(ld + [(A.OP_CMP, A.I1, 1, 0, 0, -1, 0.0, 0),
                                 (A.OP_STORE, A.F32, -1, 1, -1, -1, 0.0, 0)], [x], y)
    with pytest.raises(ValueError, match="same element type"):    # arithmetic on a condition
        handle.elementwise(ld + [(A.OP_CMP, A.I1, 1, 0, 0, -1, 0.0, 0),
                                 (A.OP_ADD, A.F32, 2, 0, 1, -1, 0.0, 0),
                                 (A.OP_STORE, A.F32, -1, 2, -1, -1, 0.0, 0)], [x], y)


# ---------------------------------------------------------------- cache hints

def test_cache_hints_never_change_a_result(handle, ko, pkg):
    """Every cache operator, eviction priority and the volatile flag of ld_global /
    st_global (Enums.td:63-88) on the general kernel: the ld / st forms differ,
    the bits do not.  All three element widths are loaded and stored."""
    A = pkg.abi
    x32 = normal((7, 333), 91, dtype=torch.float32)
    y16 = normal((7, 333), 92)
    # z = select(x > y, x, y) in f32, stored as bf16: loads of 4 and 2 bytes, store of 2
    prog = [(A.OP_LOAD, A.F32, 0, -1, -1, -1, 0.0, 0), (A.OP_LOAD, A.BF16, 1, -1, -1, -1, 0.0, 1),
            (A.OP_CVT, A.F32, 2, 1, -1, -1, 0.0, A.RN), (A.OP_CMP, A.I1, 3, 0, 2, -1, 0.0, 1),
            (A.OP_SELECT, A.F32, 4, 3, 0, 2, 0.0, 0), (A.OP_CVT, A.BF16, 5, 4, -1, -1, 0.0, A.RN),
            (A.OP_STORE, A.BF16, -1, 5, -1, -1, 0.0, 0)]
    xd, yd = x32.cuda(), y16.cuda()
    base = torch.empty((7, 333), dtype=torch.bfloat16, device="cuda")
    handle.elementwise(prog, [xd, yd], base)
    assert handle.last_kernel == "elt_interp"
    want = ko.eltwise(prog, [bits(x32), bits(y16)], [2, 1], (7, 333), 1)
    assert np.array_equal(bits(base.cpu()), want)
    hints = [A.cache_hints(m, 0, False) for m in range(8)] + \
            [A.cache_hints(0, p, False) for p in range(5)] + \
            [A.cache_hints(0, 0, True), A.cache_hints(A.CACHE_CG, A.EVICT_LAST, False)]
    for hint in hints:
        out = torch.zeros_like(base)
        handle.elementwise(prog, [xd, yd], out, caches=[hint, hint], out_cache=hint)
        handle.check()
        assert torch.equal(out, base), hex(hint)
    # one-byte elements: an f8 cast through the general kernel (column-major output)
    f8 = torch.arange(256, dtype=torch.uint8).repeat(4, 1).view(torch.float8_e5m2).cuda()
    up = [(0, 4, 0, -1, -1, -1, 0.0, 0), (2, A.F16, 1, 0, -1, -1, 0.0, 1), (27, A.F16, -1, 1, -1, -1, 0.0, 0)]
    o0 = torch.empty((256, 4), dtype=torch.float16, device="cuda").t()
    handle.elementwise(up, [f8], o0)
    o1 = torch.empty((256, 4), dtype=torch.float16, device="cuda").t()
    handle.elementwise(up, [f8], o1, caches=[A.cache_hints(A.CACHE_CS)], out_cache=A.cache_hints(A.CACHE_WT))
    handle.check()
    assert handle.last_kernel == "elt_interp"
    assert torch.equal(o0.view(torch.int16), o1.view(torch.int16))
    with pytest.raises(ValueError, match="cache operator or eviction priority"):
        handle.elementwise(prog, [xd, yd], base, caches=[A.cache_hints(9), 0])
    with pytest.raises(ValueError, match="cache operator or eviction priority"):
        handle.elementwise(prog, [xd, yd], base, out_cache=A.cache_hints(0, 5))


# ------------------------------------------------------ output against inputs

def test_in_place_and_overlap(handle, ko, pkg):
    """An input that is exactly the output runs in place (on the interpreter: the
    streaming kernels read through the read-only path) and gives the same bits
    as the out-of-place call; a partial overlap is refused."""
    A = pkg.abi
    x = normal((1, 1 << 15), 81)
    prog = pkg.programs.affine_gelu_tanh(A.BF16, 0.5, 0.1)
    xd = x.cuda()
    y = torch.empty_like(xd)
    handle.elementwise(prog, [xd], y)
    assert handle.last_kernel == "elt_affine_gelu"
    handle.elementwise(prog, [xd], xd)
    assert handle.last_kernel == "elt_interp"
    handle.check()
    assert torch.equal(xd, y)
    # binary op accumulating into its first operand
    a, b = normal((1, 4096), 82), normal((1, 4096), 83)
    ad, bd = a.cuda(), b.cuda()
    handle.elementwise(pkg.programs.binary(A.OP_ADD, A.BF16), [ad, bd], ad)
    assert handle.last_kernel == "elt_interp"
    handle.check()
    want = ko.eltwise(pkg.programs.binary(A.OP_ADD, A.BF16), [bits(a), bits(b)], [1, 1], (1, 4096), 1)
    assert np.array_equal(bits(ad.cpu()), want)
    # shifted by one element: every output element is some other thread's input
    buf = torch.zeros((1, 4097), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="overlaps input 0"):
        handle.elementwise(pkg.programs.affine(A.BF16, 0.5, 0.1), [buf[:, 1:]], buf[:, :4096])
    # disjoint halves of one allocation are fine
    handle.elementwise(pkg.programs.affine(A.BF16, 0.5, 0.1), [buf[:, :2048]], buf[:, 2048:4096])
    handle.check()


# ------------------------------------------------------------------ f8 casts

F8_TORCH = {3: torch.float8_e4m3fn, 4: torch.float8_e5m2}


def _cast_prog(src, dst, rounding):
    return [(0, src, 0, -1, -1, -1, 0.0, 0), (2, dst, 1, 0, -1, -1, 0.0, rounding),
            (27, dst, -1, 1, -1, -1, 0.0, 0)]


def _same_f8(got: np.ndarray, want: np.ndarray, code: int, ko):
    """Equal bit patterns, NaN patterns compared as NaN (payload and sign free)."""
    g, w = ko.from_bits(got, code), ko.from_bits(want, code)
    nan = np.isnan(w)
    assert np.array_equal(np.isnan(g), nan)
    assert np.array_equal(got[~nan], want[~nan])


@pytest.mark.parametrize("dst", [3, 4])
@pytest.mark.parametrize("src_dt", [torch.float16, torch.bfloat16, torch.float32])
def test_downcast_to_f8_rn_every_pattern(handle, ko, dst, src_dt):
    """FPToFPOp to f8 with rn (cvt.rn.satfinite, ElementwiseOpToLLVM.cpp:83-289):
    every f16 / bf16 bit pattern, and f32 values around every f8 rounding
    boundary; bit-exact against the checker, saturation and NaN included."""
    if src_dt == torch.float32:
        base = ko.f8_table(dst)
        base = base[np.isfinite(base)]
        mids = (base[:, None] * np.array([1.0, 1.0 + 2.0 ** -4, 1.0 + 2.0 ** -3, 1.5, 1.0625])).ravel()
        x = np.concatenate([mids, -mids, np.nextafter(mids.astype(np.float32), np.float32(np.inf)),
                            np.array([np.inf, -np.inf, np.nan, 1e30, -1e30, 1e-30, 0.0, -0.0])])
        src = torch.from_numpy(x.astype(np.float32)).view(1, -1)
    else:
        src = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(src_dt).view(256, 256)
    scode = code(src_dt)
    want = ko.eltwise(_cast_prog(scode, dst, 1), [bits(src)], [scode], tuple(src.shape), dst)
    # contiguous: the fused cast kernel; a column-major output: the interpreter
    out = torch.empty(src.shape, dtype=torch.uint8, device="cuda").view(F8_TORCH[dst])
    handle.elementwise(_cast_prog(scode, dst, 1), [src.cuda()], out)
    handle.check()
    assert handle.last_kernel == "elt_cast_f8"
    _same_f8(out.view(torch.uint8).cpu().numpy(), want, dst, ko)
    out_t = torch.empty(src.shape[::-1], dtype=torch.uint8, device="cuda").view(F8_TORCH[dst]).t()
    handle.elementwise(_cast_prog(scode, dst, 1), [src.cuda()], out_t)
    handle.check()
    assert handle.last_kernel == ("elt_interp" if min(src.shape) > 1 else "elt_cast_f8")
    _same_f8(out_t.contiguous().view(torch.uint8).cpu().numpy(), want, dst, ko)


@pytest.mark.parametrize("src_dt", [torch.float16, torch.float32])
def test_downcast_to_f8e5m2_rz(handle, ko, src_dt):
    """rz to f8E5M2 is the high byte of the f16 pattern (:104-112); f32 goes
    through f16 toward zero first (:583-600)."""
    if src_dt == torch.float16:
        src = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(src_dt).view(256, 256)
    else:
        src = (torch.randn(64, 1024, generator=gen(5)) * torch.logspace(-8, 5, 1024)).float()
    scode = code(src_dt)
    out = torch.empty(src.shape, dtype=torch.uint8, device="cuda").view(torch.float8_e5m2)
    handle.elementwise(_cast_prog(scode, 4, 0), [src.cuda()], out)
    handle.check()
    want = ko.eltwise(_cast_prog(scode, 4, 0), [bits(src)], [scode], tuple(src.shape), 4)
    got = out.view(torch.uint8).cpu().numpy()
    _same_f8(got, want, 4, ko)
    if src_dt == torch.float16:
        pat = np.arange(65536, dtype=np.uint16).reshape(256, 256)
        finite = np.isfinite(pat.view(np.float16))
        assert np.array_equal(got[finite], (pat >> 8).astype(np.uint8)[finite])


@pytest.mark.parametrize("src", [3, 4])
@pytest.mark.parametrize("dst_dt", [torch.float16, torch.bfloat16, torch.float32])
def test_upcast_from_f8_is_exact(handle, ko, src, dst_dt):
    pat = torch.arange(256, dtype=torch.uint8).repeat(4, 1)
    out = torch.empty(pat.shape, dtype=dst_dt, device="cuda")
    dcode = code(dst_dt)
    handle.elementwise(_cast_prog(src, dcode, 1), [pat.view(F8_TORCH[src]).cuda()], out)
    handle.check()
    table = ko.f8_table(src)
    got = out.cpu().double().numpy()
    assert np.array_equal(np.isnan(got[0]), np.isnan(table))
    ok = ~np.isnan(table)
    assert np.array_equal(got[:, ok], np.broadcast_to(table[ok], (4, ok.sum())))


def test_f8_cast_rules(handle):
    """FPToFPOp::verify (Kapy.cpp:272-287) and the gaps of the conversion table."""
    z = lambda dt: torch.zeros(4, 8, device="cuda").to(dt)
    f8a, f8b = z(torch.float8_e4m3fn), z(torch.float8_e5m2)
    with pytest.raises(ValueError, match="convert f8 to f8 is not supported"):
        handle.elementwise(_cast_prog(3, 4, 1), [f8a], f8b)
    with pytest.raises(ValueError, match="unsupported rounding mode when convert bf16 to f8"):
        handle.elementwise(_cast_prog(1, 4, 0), [z(torch.bfloat16)], f8b)
    with pytest.raises(ValueError, match="rounding mode must be set for down cast"):
        handle.elementwise(_cast_prog(0, 3, -1), [z(torch.float16)], f8a)
    with pytest.raises(pkg_error(handle), match="no toward-zero conversion to f8E4M3"):
        handle.elementwise(_cast_prog(0, 3, 0), [z(torch.float16)], f8a)
    with pytest.raises(ValueError, match="cannot compute in an f8 element type"):
        handle.elementwise([(0, 3, 0, -1, -1, -1, 0.0, 0), (3, 3, 1, 0, 0, -1, 0.0, 0),
                            (27, 3, -1, 1, -1, -1, 0.0, 0)], [f8a], f8a)


def pkg_error(handle):
    import sys
    return sys.modules[type(handle).__module__].KapybError
