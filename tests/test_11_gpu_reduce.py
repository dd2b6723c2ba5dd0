"""kapy.reduce against the f64 checker.  The reference fixes no combination
order (ReduceOpToLLVM.cpp:76-119), so f32 sums are held to 4*eps_f32*sum|x|;
a sum whose lambda runs at a 16-bit type (source and result f16 or bf16) rounds
at every step, which any order keeps within n*u*sum|x| (u the type's unit
roundoff); max/min are exact."""
import numpy as np
import pytest
import torch

from util import bits, code, normal

pytestmark = pytest.mark.gpu
EPS32 = 2.0 ** -24


def check_sum(ko, got64, X, dt, axis, out_dtype):
    ref, ab = ko.reduce_f64(bits(X), code(dt), axis)
    tol = 4 * EPS32 * ab + 1e-30
    if out_dtype != torch.float32:
        # a rounding to the 16-bit type per combination, in whatever order
        n = X.shape[axis]
        tol = n * (2.0 ** -8 if out_dtype == torch.bfloat16 else 2.0 ** -11) * ab + 1e-30
    assert np.all(np.abs(got64 - ref) <= tol), np.abs(got64 - ref).max()


@pytest.mark.parametrize("shape", [(64, 4096), (37, 300), (5, 8), (3, 1), (1000, 2056)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_row_sum_f32(handle, ko, shape, dt):
    X = normal(shape, 1004, dtype=dt)
    out = handle.reduce(X.cuda(), axis=1, out_dtype=torch.float32)
    handle.check()
    assert out.shape == (shape[0], 1)
    assert handle.last_kernel == "reduce_rows"
    check_sum(ko, out.cpu().numpy().ravel().astype(np.float64), X, dt, 1, torch.float32)


def test_reduce_sum_mlir_shape(handle, ko):
    """reduce_sum.mlir:10-25: [n, 256] f16 -> [n, 1] f16 with an addf lambda."""
    X = normal((128, 256), 5, dtype=torch.float16)
    out = handle.reduce(X.cuda(), axis=1)
    handle.check()
    assert out.dtype == torch.float16 and out.shape == (128, 1)
    check_sum(ko, out.cpu().double().numpy().ravel(), X, torch.float16, 1, torch.float16)


def _add_at(ko, a, b, dt):
    """Elementwise a + b with one rounding at the 16-bit type `dt` (the checker's add)."""
    prog = [(0, dt, 0, -1, -1, -1, 0.0, 0), (0, dt, 1, -1, -1, -1, 0.0, 1),
            (3, dt, 2, 0, 1, -1, 0.0, 0), (27, dt, -1, 2, -1, -1, 0.0, 0)]
    return ko.eltwise(prog, [np.ascontiguousarray(a), np.ascontiguousarray(b)], [dt, dt], a.shape, dt)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_sixteen_bit_sum_rounds_at_every_step(handle, ko, dt):
    """The lambda of reduce_sum.mlir:10-25 adds at the tensor's 16-bit type.  For
    a [n, 256] tensor whose rows start on 32-byte boundaries the kernel's order
    is: lanes 0..15 each add 16 consecutive elements in ascending order, then
    meet in a butterfly over lane distances 8, 4, 2, 1.  Restated with the
    checker's single-rounding add, that order must give the same bits."""
    X = normal((128, 256), 5, dtype=dt)
    out = handle.reduce(X.cuda(), axis=1)
    handle.check()
    assert out.dtype == dt
    xb = bits(X)
    code_dt = code(dt)
    lanes = []
    for lane in range(16):
        acc = xb[:, 16 * lane:16 * lane + 1].copy()
        for e in range(1, 16):
            acc = _add_at(ko, acc, xb[:, 16 * lane + e:16 * lane + e + 1], code_dt)
        lanes.append(acc)
    v = np.concatenate(lanes, axis=1)                      # [128, 16]
    for off in (8, 4, 2, 1):
        v = _add_at(ko, v, v[:, np.arange(16) ^ off], code_dt)
    want = v[:, 0]
    got = bits(out.cpu()).ravel()
    assert np.array_equal(got, want), int((got != want).sum())
    # and it differs from the sum formed in f32 and rounded once, in some rows at least
    once = handle.reduce(X.cuda(), axis=1, out_dtype=torch.float32).cpu().ravel().to(dt)
    assert (bits(once).ravel() != got).any()


@pytest.mark.parametrize("shape", [(300, 37), (4096, 64), (7, 1)])
def test_axis0_and_strided(handle, ko, shape):
    X = normal(shape, 77)
    out = handle.reduce(X.cuda(), axis=0, out_dtype=torch.float32)
    handle.check()
    assert out.shape == (1, shape[1])
    assert handle.last_kernel == ("reduce_rows" if shape[1] == 1 else
                                  "reduce_cols_slabs" if shape == (4096, 64) else "reduce_cols")
    check_sum(ko, out.cpu().numpy().ravel().astype(np.float64), X, torch.bfloat16, 0,
              torch.float32)
    # a column-major view reduced along axis 1 is the same computation
    Xt = X.t()
    out2 = handle.reduce(Xt.cuda(), axis=1, out_dtype=torch.float32)
    handle.check()
    assert torch.equal(out2.cpu().ravel(), out.cpu().ravel())
    # misaligned rows fall off the 128-bit path but give a valid sum
    Y = normal((shape[0], shape[1] + 1), 78)[:, 1:]
    o3 = handle.reduce(Y.cuda(), axis=1, out_dtype=torch.float32)
    handle.check()
    check_sum(ko, o3.cpu().numpy().ravel().astype(np.float64), Y, torch.bfloat16, 1,
              torch.float32)


@pytest.mark.parametrize("comb", ["MAX", "MIN", "MUL"])
def test_other_combiners(handle, ko, pkg, comb):
    X = normal((33, 129), 9, dtype=torch.float32)
    if comb == "MUL":
        X = X * 0.1 + 1.0
    c = getattr(pkg.abi, "RED_" + comb)
    out = handle.reduce(X.cuda(), axis=1, combiner=c)
    handle.check()
    ref, _ = ko.reduce_f64(bits(X), 2, 1, c)
    got = out.cpu().numpy().ravel().astype(np.float64)
    if comb == "MUL":
        assert np.allclose(got, ref, rtol=129 * 2 * EPS32)
    else:
        assert np.array_equal(got, ref)
    Xn = X.clone()
    Xn[3, 5] = float("nan")
    if comb != "MUL":
        o = handle.reduce(Xn.cuda(), axis=1, combiner=c).cpu().ravel()
        assert torch.isnan(o[3]) and not torch.isnan(o[2])   # maximumf propagates NaN


def test_shape_rules(handle, pkg):
    X = torch.zeros((4, 8), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="result shape"):
        handle.reduce(X, axis=1, out=torch.zeros((4, 2), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError, match="axis"):
        handle.reduce(X, axis=2)
    with pytest.raises(ValueError, match="element type"):
        handle.reduce(X, axis=1, out=torch.zeros((4, 1), dtype=torch.float16, device="cuda"))
    e = handle.reduce(torch.zeros((0, 8), dtype=torch.bfloat16, device="cuda"), axis=1)
    assert e.shape == (0, 1)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("comb", ["ADD", "MAX", "MIN"])
def test_column_reduction_in_slabs(handle, ko, pkg, dt, comb):
    """Results on the unit-stride axis of a tall source: the reduced axis is cut into
    slabs (first pass) that a second pass combines.  f32 results and, for 16-bit
    sources, results at the source's type (a rounding per combination)."""
    shape = (3000, 520)
    X = normal(shape, 91, dtype=dt)
    c = getattr(pkg.abi, "RED_" + comb)
    for od in ([torch.float32] if dt == torch.float32 else [torch.float32, dt]):
        out = handle.reduce(X.cuda(), axis=0, combiner=c, out_dtype=od)
        handle.check()
        assert handle.last_kernel == "reduce_cols_slabs" and out.shape == (1, shape[1])
        got = out.cpu().double().numpy().ravel()
        if comb == "ADD":
            check_sum(ko, got, X, dt, 0, od)
        else:
            ref, _ = ko.reduce_f64(bits(X), code(dt), 0, c)
            assert np.array_equal(got, ref)
    # a NaN reaches its column's result whatever slab it sits in
    if comb != "ADD":
        Xn = X.clone()
        Xn[2999, 7] = float("nan")
        o = handle.reduce(Xn.cuda(), axis=0, combiner=c, out_dtype=torch.float32).cpu().ravel()
        assert torch.isnan(o[7]) and not torch.isnan(o[8])
