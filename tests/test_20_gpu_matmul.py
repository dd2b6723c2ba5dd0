"""Matmul kernels through the C ABI against the f64 checker.

Tolerance (stated by the path's contract): max_i |c_i - ref_i| / max(|ref_i|, tau)
<= 1e-2 with tau = 2^-6 * rms(ref); f16/bf16 operands, fp32 accumulation.
Integer-valued cases must be bit-exact."""
import os

import numpy as np
import pytest
import torch

from util import bits, code, normal, uniform

pytestmark = pytest.mark.gpu
TOL = 1e-2
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def check(ko, out, A, B, *, alpha=1.0, bias=None, bias_axis=1, activation=0, acc=None,
          rows=None, cols=None, tol=TOL):
    ref = ko.matmul_f64(bits(A), code(A.dtype), bits(B), code(B.dtype), alpha=alpha,
                        bias=bits(bias) if bias is not None else None,
                        bias_dtype=code(bias.dtype) if bias is not None else 2,
                        bias_axis=bias_axis, activation=activation,
                        acc=bits(acc) if acc is not None else None,
                        acc_dtype=code(acc.dtype) if acc is not None else 2, rows=rows, cols=cols)
    o = out.cpu().double().numpy()
    if rows is not None:
        o = o[np.ix_(rows, cols)]
    err, tau = ko.max_rel_err(o, ref)
    assert err <= tol, f"max rel err {err:.3e} (tau {tau:.3e})"
    return err


PATHS = ["1cta:64", "1cta:128", "1cta:256", "simt"]


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_integer_exact(handle, ko, path, dt):
    """Golden: small-integer operands, exact products and sums -> exact output."""
    z = np.load(os.path.join(GOLD, "kat_matmul_int.npz"))
    handle.set_matmul_path(path)
    try:
        for name in "ab":
            A = torch.from_numpy(z[f"A_{name}"].astype(np.float32)).to(dt)
            B = torch.from_numpy(z[f"B_{name}"].astype(np.float32)).to(dt)
            bias = torch.from_numpy(z[f"bias_{name}"].astype(np.float32)).to(dt)
            out = handle.matmul(A.cuda(), B.cuda(), bias=bias.cuda(), out_dtype=torch.float32)
            handle.check()
            assert np.array_equal(out.cpu().numpy().astype(np.int64), z[f"C_{name}"])
    finally:
        handle.set_matmul_path("auto")


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 320), (200, 264, 136), (8, 16, 8),
                                   (384, 72, 1024)])
def test_row_major_bf16(handle, ko, path, shape):
    M, N, K = shape
    handle.set_matmul_path(path)
    try:
        A, B = normal((M, K), 1, K ** -0.5), normal((K, N), 2)
        out = handle.matmul(A.cuda(), B.cuda())
        handle.check()
        assert handle.last_kernel.startswith("simt" if path == "simt" else "tcgen05_1cta")
        check(ko, out, A, B)
    finally:
        handle.set_matmul_path("auto")


@pytest.mark.parametrize("path", ["1cta:128", "1cta:256", "simt"])
@pytest.mark.parametrize("layout", ["nt", "tn", "tt"])
def test_operand_layouts(handle, ko, path, layout):
    """lhs/rhs row- or column-major (one unit stride, CoalesceAccess.cpp:32-40).
    'nt' is config 1's layout: A row-major, B column-major."""
    M, N, K = 256, 320, 192
    handle.set_matmul_path(path)
    try:
        A = uniform((M, K), 3)
        B = uniform((K, N), 4)
        Ad = A.cuda() if layout[0] == "n" else A.t().contiguous().cuda().t()
        Bd = B.cuda() if layout[1] == "n" else B.t().contiguous().cuda().t()
        out = handle.matmul(Ad, Bd)
        handle.check()
        check(ko, out, A, B)
        # column-major output: the transposed problem
        out_t = torch.empty((N, M), dtype=torch.float16, device="cuda").t()
        handle.matmul(Ad, Bd, out=out_t)
        handle.check()
        assert torch.equal(out_t.contiguous(), out)
    finally:
        handle.set_matmul_path("auto")


@pytest.mark.parametrize("path", ["1cta:128", "simt"])
def test_epilogue_variants(handle, ko, pkg, path):
    A_ = pkg.abi
    M, N, K = 192, 200, 256
    A, B = normal((M, K), 5, K ** -0.5), normal((K, N), 6)
    bias_c = uniform((N,), 7, -0.1, 0.1, torch.bfloat16)
    bias_r = uniform((M,), 8, -0.1, 0.1, torch.float32)
    acc = normal((M, N), 9, dtype=torch.float32)
    handle.set_matmul_path(path)
    try:
        Ad, Bd = A.cuda(), B.cuda()
        for od in (torch.bfloat16, torch.float32):
            out = handle.matmul(Ad, Bd, bias=bias_c.cuda(), alpha=0.5, out_dtype=od)
            check(ko, out, A, B, alpha=0.5, bias=bias_c)
            out = handle.matmul(Ad, Bd, bias=bias_r.cuda(), bias_axis=0, out_dtype=od)
            check(ko, out, A, B, bias=bias_r, bias_axis=0)
            out = handle.matmul(Ad, Bd, acc=acc.cuda(), out_dtype=od)
            check(ko, out, A, B, acc=acc)
        for act in (A_.ACT_RELU, A_.ACT_GELU_TANH, A_.ACT_SILU):
            out = handle.matmul(Ad, Bd, bias=bias_c.cuda(), activation=act)
            check(ko, out, A, B, bias=bias_c, activation=act, tol=2e-2)
        # RZ downcast never rounds away from zero: |rz| <= |rn| elementwise
        rn = handle.matmul(Ad, Bd, out_dtype=torch.bfloat16).float()
        rz = handle.matmul(Ad, Bd, out_dtype=torch.bfloat16, rounding=A_.RZ).float()
        f32 = handle.matmul(Ad, Bd, out_dtype=torch.float32)
        handle.check()
        assert torch.all(rz.abs() <= f32.abs()) and torch.all((rz - rn).abs() <= (f32.abs() * 2 ** -7))
        assert torch.equal(rn, f32.to(torch.bfloat16).float())
    finally:
        handle.set_matmul_path("auto")


def test_unaligned_operands_take_simt(handle, ko):
    """Odd leading dimensions / offsets cannot be described to TMA."""
    M, N, K = 45, 37, 51
    A, B = normal((M, K + 1), 10)[:, 1:], normal((K, N), 11)
    out = handle.matmul(A.cuda(), B.cuda())
    handle.check()
    assert handle.last_kernel == "simt"
    check(ko, out, A, B)


def test_config1_fp16_1024(handle, ko):
    """fp16 1024^3, A row-major, B column-major, fp32 accumulate, fp16 output;
    entries uniform[-1,1] from seed 1001."""
    A = uniform((1024, 1024), 1001)
    B = uniform((1024, 1024), 2001).t()          # column-major [K,N]
    out = handle.matmul(A.cuda(), B.cuda(), impl_way=1)
    handle.check()
    assert handle.last_kernel.startswith("tcgen05")
    check(ko, out, A, B)


def test_verifier_rejections(handle):
    """MatmulOp::verify (Kapy.cpp:459-487) diagnostics."""
    z = lambda s, d: torch.zeros(s, dtype=d, device="cuda")
    with pytest.raises(ValueError, match="columns of lhs"):
        handle.matmul(z((8, 16), torch.bfloat16), z((8, 8), torch.bfloat16))
    with pytest.raises(ValueError, match="same element type"):
        handle.matmul(z((8, 16), torch.bfloat16), z((16, 8), torch.float16))
    with pytest.raises(ValueError, match="f32 element type when operands are bf16"):
        handle.matmul(z((8, 16), torch.bfloat16), z((16, 8), torch.bfloat16),
                      acc=z((8, 8), torch.float16))
    with pytest.raises(ValueError, match="mma_m16n8k8_tf32"):
        handle.matmul(z((8, 16), torch.bfloat16), z((16, 8), torch.bfloat16), impl_way=3)
    with pytest.raises(ValueError, match="rows of acc"):
        handle.matmul(z((8, 16), torch.bfloat16), z((16, 8), torch.bfloat16),
                      out=z((4, 8), torch.bfloat16))
    e = handle.matmul(z((0, 16), torch.bfloat16), z((16, 8), torch.bfloat16))
    assert e.shape == (0, 8)


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("shape", [(512, 384, 256), (200, 264, 136), (1000, 72, 64)])
def test_reduce_fused_into_the_epilogue(handle, ko, pkg, axis, shape):
    """kapy.reduce with an addf lambda on the accumulator tile, after scale, bias
    and relu: the f32 values are summed along `axis` by the epilogue itself.
    Checked against the f64 matmul summed in f64 (the order of the f32 atomic adds
    is unspecified: bound = 1e-5 * sum|c| per result), and `out` against the same
    tolerance as any matmul; ragged tiles must not leak their padding into the sums."""
    M, N, K = shape
    A, B = normal((M, K), 61, K ** -0.5), normal((K, N), 62)
    bias = uniform((N,), 63, -0.5, 0.5, torch.bfloat16)
    ep = dict(alpha=0.75, bias=bias.cuda(), activation=pkg.abi.ACT_RELU)
    out, red = handle.matmul_reduce(A.cuda(), B.cuda(), axis, **ep)
    handle.check()
    assert handle.last_kernel.startswith("tcgen05_1cta")
    assert red.shape == ((1, N) if axis == 0 else (M, 1)) and red.dtype == torch.float32
    ref = ko.matmul_f64(bits(A), 1, bits(B), 1, alpha=0.75, bias=bits(bias), bias_dtype=1,
                        activation=pkg.abi.ACT_RELU)
    err, _ = ko.max_rel_err(out.cpu().double().numpy(), ref)
    assert err <= TOL
    want, scale = ref.sum(axis=axis), np.abs(ref).sum(axis=axis)
    got = red.cpu().double().numpy().ravel()
    assert np.all(np.abs(got - want) <= 1e-5 * scale + 1e-12), np.abs(got - want).max()
    # the unfused pair of calls gives the same sums to the same bound
    plain = handle.matmul(A.cuda(), B.cuda(), out_dtype=torch.float32, **ep)
    two_pass = handle.reduce(plain, axis=axis).cpu().double().numpy().ravel()
    assert np.all(np.abs(got - two_pass) <= 1e-5 * scale + 1e-12)
    # a second call starts from zero again (the sums are cleared, not accumulated)
    out2, red2 = handle.matmul_reduce(A.cuda(), B.cuda(), axis, out=out, reduced=red, **ep)
    handle.check()
    assert np.all(np.abs(red2.cpu().double().numpy().ravel() - want) <= 1e-5 * scale + 1e-12)


def test_reduce_epilogue_rules(handle, pkg):
    z = lambda s, d=torch.bfloat16: torch.zeros(s, dtype=d, device="cuda")
    with pytest.raises(ValueError, match="result shape"):
        handle.matmul_reduce(z((64, 64)), z((64, 128)), 1, reduced=z((1, 128), torch.float32))
    with pytest.raises(pkg.KapybError, match="only the addf lambda"):
        handle.matmul_reduce(z((64, 64)), z((64, 128)), 1, combiner=pkg.abi.RED_MAX)
    with pytest.raises(pkg.KapybError, match="dense f32 vector"):
        handle.matmul_reduce(z((64, 64)), z((64, 128)), 1, reduced=z((64, 1)))
    o, r = handle.matmul_reduce(z((0, 64)), z((64, 128)), 0)
    assert o.shape == (0, 128) and r.shape == (1, 128)


def test_operand_padding_is_zero_only(handle, pkg):
    """ld_global's QNAN / +-INF padding (Enums.td:52-61) has no whole-problem
    meaning for a matmul operand (it would poison every output whose K range is
    ragged against a tile size the caller cannot see): refused, not ignored."""
    import ctypes as C
    a = torch.zeros((64, 72), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((72, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    lib = pkg.abi.load()
    ep = pkg.abi.Epilogue(1.0, None, pkg.abi.F32, 1, 0, pkg.abi.RN)
    for pad_l, pad_r in ((pkg.abi.PAD_QNAN, 0), (0, pkg.abi.PAD_PINF), (pkg.abi.PAD_NINF, pkg.abi.PAD_NINF)):
        tl, tr, to = pkg.tensor2d(a, pad_l), pkg.tensor2d(b, pad_r), pkg.tensor2d(c)
        st = lib.kapyb_matmul(handle._h, C.byref(tl), C.byref(tr), None, C.byref(to), C.byref(ep), 0,
                              handle._stream())
        assert st == pkg.abi.UNSUPPORTED
        assert "padded with zeros only" in lib.kapyb_last_error_string(handle._h).decode()
    tl, tr, to = pkg.tensor2d(a), pkg.tensor2d(b), pkg.tensor2d(c)
    assert lib.kapyb_matmul(handle._h, C.byref(tl), C.byref(tr), None, C.byref(to), C.byref(ep), 0,
                            handle._stream()) == pkg.abi.OK
    handle.check()


def test_host_buffers(handle, ko):
    """kapyb_matmul_host: host tensors in, host tensor out."""
    M, N, K = 256, 384, 512
    A, B = normal((M, K), 12, K ** -0.5), normal((K, N), 13)
    bias = uniform((N,), 14, -0.1, 0.1, torch.bfloat16)
    out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    handle.matmul_host(A.pin_memory(), B.pin_memory(), out, bias=bias)
    check(ko, out, A, B, bias=bias)
    dev = handle.matmul(A.cuda(), B.cuda(), bias=bias.cuda())
    handle.check()
    assert torch.equal(dev.cpu(), out)
    # large row-major problems go through the chunked upload / compute / download
    # pipeline (ragged last chunk, per-row bias offset per chunk)
    M, N, K = 2304 + 40, 512, 2048
    A, B = normal((M, K), 15, K ** -0.5), normal((K, N), 16)
    bias_r = uniform((M,), 17, -0.1, 0.1, torch.float32)
    out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        out.zero_()
        handle.matmul_host(A.pin_memory(), B.pin_memory(), out, bias=bias_r, bias_axis=0)
        dev = handle.matmul(A.cuda(), B.cuda(), bias=bias_r.cuda(), bias_axis=0)
        handle.check()
        assert torch.equal(dev.cpu(), out)
    check(ko, out, A, B, bias=bias_r, bias_axis=0)


@pytest.mark.parametrize("n", [8192])
def test_config2_bf16_8192_bias(handle, ko, n):
    """bf16 8192^3, row-major A/B, per-column bias, bf16 out (seed 1002).  The
    f64 checker evaluates 64 rows x all columns... too slow in full, so: 48 full
    rows, 48 full columns and 4096 scattered entries; plus linearity in alpha as
    a size-independent property on the whole output."""
    M = N = K = n
    A = normal((M, K), 1002, K ** -0.5)
    B = normal((K, N), 3002, K ** -0.5)
    bias = uniform((N,), 4002, -0.1, 0.1, torch.bfloat16)
    Ad, Bd, bd = A.cuda(), B.cuda(), bias.cuda()
    out = handle.matmul(Ad, Bd, bias=bd)
    handle.check()
    assert handle.last_kernel.startswith("tcgen05")
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(M, 48, replace=False)).astype(np.int32)
    cols = np.sort(rng.choice(N, 48, replace=False)).astype(np.int32)
    all_c = np.arange(N, dtype=np.int32)
    all_r = np.arange(M, dtype=np.int32)
    check(ko, out, A, B, bias=bias, rows=rows, cols=all_c)
    check(ko, out, A, B, bias=bias, rows=all_r, cols=cols)
    # first/last tiles explicitly
    edge = np.array([0, 1, 127, 128, 255, 256, n - 129, n - 128, n - 1], dtype=np.int32)
    check(ko, out, A, B, bias=bias, rows=edge, cols=edge)
    # property: out(alpha=2, no bias) == 2 * out(alpha=1, no bias) exactly in f32
    o1 = handle.matmul(Ad, Bd, out_dtype=torch.float32)
    o2 = handle.matmul(Ad, Bd, alpha=2.0, out_dtype=torch.float32)
    handle.check()
    assert torch.equal(o2, o1 * 2)
    # property: against torch's own fp32-accumulate matmul on the whole matrix
    ref = torch.matmul(Ad, Bd).float() + bd.float()[None, :]
    d = (out.float() - ref).abs().max().item()
    assert d <= 2 ** -6, d
