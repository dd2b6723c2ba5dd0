"""tf32 and f8 operand kinds of the matmul (verifier rules Kapy.cpp:469-564:
same bit width; same element type unless both are f8; mma_m16n8k8_tf32 takes
f32 operands, mma_m16n8k16_f8 takes f8E4M3 / f8E5M2 in any mix).

f32 operands are multiplied as tf32: the 13 low mantissa bits do not take part.
Inputs already representable in tf32 (and every f8 input) have exact products,
so those cases hold to the f16/bf16 tolerance of 1e-2 against the f64 checker
with fp32 accumulation; small-integer cases are bit-exact."""
import numpy as np
import pytest
import torch

from util import bits, code, gen, normal

pytestmark = pytest.mark.gpu
TOL = 1e-2
F8 = [torch.float8_e4m3fn, torch.float8_e5m2]
PATHS = ["1cta:64", "1cta:128", "1cta:256", "2cta:256", "2cta:512", "simt"]


def tf32_trunc(t: torch.Tensor) -> torch.Tensor:
    return (t.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)


def check(ko, out, A, B, tol=TOL, **kw):
    ref = ko.matmul_f64(bits(A), code(A.dtype), bits(B), code(B.dtype), **kw)
    err, tau = ko.max_rel_err(out.cpu().double().numpy(), ref)
    assert err <= tol, f"max rel err {err:.3e} (tau {tau:.3e})"


def layouts(A, B, layout):
    """Device copies with the requested majors ('n' row-major, 't' column-major)."""
    a = A.cuda() if layout[0] == "n" else A.t().contiguous().cuda().t()
    b = B.cuda() if layout[1] == "n" else B.t().contiguous().cuda().t()
    return a, b


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
def test_tf32_integer_exact(handle, path, layout):
    M, N, K = 256, 512, 160
    A = torch.randint(-8, 9, (M, K), generator=gen(1)).float()
    B = torch.randint(-8, 9, (K, N), generator=gen(2)).float()
    a, b = layouts(A, B, layout)
    handle.set_matmul_path(path)
    try:
        out = handle.matmul(a, b, out_dtype=torch.float32)
        handle.check()
    finally:
        handle.set_matmul_path("auto")
    assert torch.equal(out.cpu(), A @ B)


@pytest.mark.parametrize("path", ["auto", "1cta:128", "2cta:256", "simt"])
@pytest.mark.parametrize("shape", [(128, 128, 32), (200, 264, 136), (512, 1024, 1000), (16, 8, 8)])
def test_tf32_random(handle, ko, path, shape):
    M, N, K = shape
    A = tf32_trunc(normal((M, K), 3, K ** -0.5, torch.float32))
    B = tf32_trunc(normal((K, N), 4, 1.0, torch.float32))
    bias = normal((N,), 5, 1.0, torch.float32)
    handle.set_matmul_path(path)
    try:
        out = handle.matmul(A.cuda(), B.cuda(), bias=bias.cuda(), out_dtype=torch.float32,
                            impl_way=3)
        handle.check()
    finally:
        handle.set_matmul_path("auto")
    check(ko, out, A, B, bias=bits(bias), bias_dtype=2)


def test_tf32_drops_low_mantissa_bits(handle, ko):
    """Operands with all 23 mantissa bits in use: the tensor core reads the upper
    19 bits, so the result is that of the truncated operands (to the usual
    tolerance), on the tcgen05 path and on the CUDA-core path alike.  Against the
    product of the untruncated operands the dropped bits show: each term is off
    by up to 2^-9 relative, about 6e-2 in the metric whose floor is rms / 64."""
    M, N, K = 128, 128, 256
    A = normal((M, K), 6, K ** -0.5, torch.float32)
    B = normal((K, N), 7, 1.0, torch.float32)
    out = handle.matmul(A.cuda(), B.cuda(), out_dtype=torch.float32)
    handle.check()
    assert handle.last_kernel.startswith("tcgen05")
    check(ko, out, tf32_trunc(A), tf32_trunc(B))
    check(ko, out, A, B, tol=2e-1)
    handle.set_matmul_path("simt")
    try:
        ref = handle.matmul(A.cuda(), B.cuda(), out_dtype=torch.float32)
        handle.check()
    finally:
        handle.set_matmul_path("auto")
    check(ko, ref, tf32_trunc(A), tf32_trunc(B))


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
def test_f8_integer_exact(handle, path, layout):
    M, N, K = 256, 512, 320
    A = torch.randint(-4, 5, (M, K), generator=gen(8)).float()
    B = torch.randint(-4, 5, (K, N), generator=gen(9)).float()
    a, b = layouts(A.to(F8[0]), B.to(F8[1]), layout)
    handle.set_matmul_path(path)
    try:
        out = handle.matmul(a, b, out_dtype=torch.float32)
        handle.check()
    finally:
        handle.set_matmul_path("auto")
    assert torch.equal(out.cpu(), A @ B)


@pytest.mark.parametrize("ta", F8)
@pytest.mark.parametrize("tb", F8)
@pytest.mark.parametrize("path", ["auto", "1cta:128", "2cta:256", "simt"])
def test_f8_mixed_types(handle, ko, ta, tb, path):
    M, N, K = 384, 640, 1000 if path == "simt" else 1024
    A = normal((M, K), 10, 1.0, torch.float32).to(ta)
    B = normal((K, N), 11, 1.0, torch.float32).to(tb)
    bias = normal((N,), 12, 1.0, torch.bfloat16)
    handle.set_matmul_path(path)
    try:
        out = handle.matmul(A.cuda(), B.cuda(), alpha=K ** -0.5, bias=bias.cuda(), activation=2,
                            out_dtype=torch.bfloat16, impl_way=4)
        handle.check()
    finally:
        handle.set_matmul_path("auto")
    check(ko, out, A, B, alpha=K ** -0.5, bias=bits(bias), bias_dtype=1, activation=2)


def test_f8_every_value(handle, ko):
    """All 256 bit patterns of each f8 type against an identity: the product is
    the decoded value itself (NaN patterns stay NaN)."""
    for dt in F8:
        V = torch.arange(256, dtype=torch.uint8).repeat(128, 1).view(dt)      # [128, 256]
        # keep NaN/Inf out of the sums: one value per output through a diagonal
        eye = torch.eye(128).to(dt)
        out = handle.matmul(eye.cuda(), V.cuda(), out_dtype=torch.float32)
        handle.check()
        table = ko.f8_table(code(dt))
        got = out.cpu().double().numpy()
        finite = np.isfinite(table)
        # 0 * Inf and 0 * NaN poison a column's sum: only finite columns are comparable
        assert np.array_equal(got[:, finite], np.broadcast_to(table[finite], (128, finite.sum())))
        assert np.isnan(got[:, ~finite]).all()


def test_kind_diagnostics(handle):
    A32 = torch.zeros(64, 64, device="cuda")
    A16 = torch.zeros(64, 64, device="cuda", dtype=torch.float16)
    A8 = torch.zeros(64, 64, device="cuda").to(F8[0])
    with pytest.raises(ValueError, match="same element bit width"):
        handle.matmul(A32, A16, out_dtype=torch.float32)
    with pytest.raises(ValueError, match="mma_m16n8k8_tf32 operands must have f32"):
        handle.matmul(A16, A16, out_dtype=torch.float32, impl_way=3)
    with pytest.raises(ValueError, match="mma_m16n8k16_f8 operands must have f8E4M3 or f8E5M2"):
        handle.matmul(A16, A16, out_dtype=torch.float32, impl_way=4)
    with pytest.raises(ValueError, match="mma_m16n8k16_f16 operands must have f16 or bf16"):
        handle.matmul(A8, A8, out_dtype=torch.float32, impl_way=2)
    with pytest.raises(ValueError, match="same element type unless"):
        handle.matmul(A16, A16.to(torch.bfloat16), out_dtype=torch.float32)


@pytest.mark.parametrize("dt", [torch.float32, torch.float8_e4m3fn])
def test_kinds_through_host_buffers(handle, ko, dt):
    """kapyb_matmul_host with f32 (tf32) and f8 operands: the chunked upload /
    compute / download pipeline moves 4- and 1-byte elements as well."""
    M, N, K = 2304 + 40, 512, 2048
    A = normal((M, K), 21, K ** -0.5, torch.float32)
    B = normal((K, N), 22, 1.0, torch.float32)
    if dt == torch.float32:
        A, B = tf32_trunc(A), tf32_trunc(B)
    else:
        A, B = (A * 16).to(dt), B.to(dt)
    out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    handle.matmul_host(A.pin_memory(), B.pin_memory(), out)
    dev = handle.matmul(A.cuda(), B.cuda(), out_dtype=torch.bfloat16)
    handle.check()
    assert torch.equal(dev.cpu(), out)
    check(ko, out, A, B)
