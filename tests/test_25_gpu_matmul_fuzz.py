"""Seeded sweep over shapes, operand layouts, element types, kernel families and
epilogues: every combination the dispatcher can reach, checked against an fp32
torch product of the same (exactly widened) operands.  The checker-based parity
tests are in test_20 .. test_23; this one is about coverage of the corners
(ragged tiles, one-row problems, forced tile widths on shapes that do not suit
them, batches)."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

M_CHOICES = [1, 7, 16, 64, 65, 128, 200, 256, 384, 512, 1000, 1024, 2048, 3000]
N_CHOICES = [8, 64, 72, 128, 264, 512, 520, 1024, 1536, 2048, 4104]
K_CHOICES = [8, 64, 72, 128, 192, 256, 264, 512, 1000, 1024, 2048]
PATHS = ["auto", "auto", "auto", "1cta:64", "1cta:128", "1cta:256", "2cta:128", "2cta:256", "2cta:512"]
DTYPES = [torch.bfloat16, torch.float16, torch.float32, torch.float8_e4m3fn]


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_sweep(handle, seed):
    rng = random.Random(seed)
    torch.manual_seed(seed)
    kernels = set()
    for case in range(80):
        batch = rng.choice([1, 1, 1, 3])
        M, N, K = rng.choice(M_CHOICES), rng.choice(N_CHOICES), rng.choice(K_CHOICES)
        dt = rng.choice(DTYPES)
        if dt == torch.float8_e4m3fn:  # keep 16-byte leading dimensions for 1-byte elements
            K, N = (K + 15) // 16 * 16, (N + 15) // 16 * 16
            if rng.random() < 0.5:
                M = (M + 15) // 16 * 16
        la, lb = rng.choice("nt"), rng.choice("nt")
        path = rng.choice(PATHS)
        out_dt = rng.choice([torch.float16, torch.float32]) if dt == torch.float16 else \
            rng.choice([torch.bfloat16, torch.float32])
        A32 = torch.randn(*((batch, M, K) if batch > 1 else (M, K)), device="cuda") * K ** -0.5
        B32 = torch.randn(*((batch, K, N) if batch > 1 else (K, N)), device="cuda")
        if dt == torch.float32:  # tf32 reads 19 bits: make the operands exact in it
            A32 = (A32.view(torch.int32) & ~0x1FFF).view(torch.float32)
            B32 = (B32.view(torch.int32) & ~0x1FFF).view(torch.float32)
        A, B = A32.to(dt), B32.to(dt)
        if batch == 1:
            if la == "t":
                A = A.t().contiguous().t()
            if lb == "t":
                B = B.t().contiguous().t()
        bias = None
        if batch == 1 and rng.random() < 0.5:
            bias = (torch.rand(N, device="cuda") * 0.2 - 0.1).to(
                torch.float16 if dt == torch.float16 else torch.bfloat16)
        alpha = rng.choice([1.0, 0.37])
        what = f"case {case}: {(M, N, K)} x{batch} {dt} {la}{lb} {path} -> {out_dt}"
        try:
            handle.set_matmul_path(path)
            out = handle.matmul(A, B, alpha=alpha, bias=bias, out_dtype=out_dt)
            handle.check()
            kernels.add(handle.last_kernel)
        except Exception as ex:  # a forced tcgen05 path on operands TMA cannot describe
            assert "TMA-describable" in str(ex) and path != "auto", f"{what}: {ex}"
            continue
        finally:
            handle.set_matmul_path("auto")
        ref = alpha * torch.matmul(A.float(), B.float())
        if bias is not None:
            ref = ref + bias.float()
        err = (out.float() - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1e-3)
        tol = (2 ** -7 if out_dt != torch.float32 else 2 ** -10) * scale + 1e-3
        assert err <= tol, f"{what}: err {err:.3e} > {tol:.3e} ({handle.last_kernel})"
    assert {"tcgen05_1cta", "tcgen05_2cta"} <= kernels
