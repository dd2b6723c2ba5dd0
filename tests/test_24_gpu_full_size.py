"""The configurations' full sizes, checked through properties that do not need
the CPU checker to walk the whole problem:

  * elementwise (2^28 bf16): the op is position-free, so an input made of 16
    copies of one 2^24 block must give 16 identical output blocks, and block 0
    must equal the checker's output for that block;
  * row sum ([65536, 4096] bf16): permuting rows permutes the sums bit for bit
    (each row is reduced in the same fixed order), a sample of rows agrees
    with the f64 checker, and the sum of the sums agrees with an f64 total;
  * batched matmul (64 x [2048,128].[128,2048], scale 1/sqrt(128)): batches are
    independent, so 8 distinct batches repeated 8 times give 8 repeated output
    groups bit for bit, and batch 0 agrees with the f64 checker.
(Config 2 and config 4 at full size are in test_20 / test_21.)"""
import numpy as np
import pytest
import torch

from util import bits, code, gen, normal

pytestmark = pytest.mark.gpu


def test_config3a_gelu_full_size(handle, ko, pkg):
    block = normal((1, 1 << 24), 1003, dtype=torch.bfloat16)
    x = block.cuda().repeat(1, 16)
    assert x.shape == (1, 1 << 28)
    for prog, linear in ((pkg.programs.affine_gelu_tanh(pkg.abi.BF16, 0.5, 0.1), False),
                         (pkg.programs.affine(pkg.abi.BF16, 0.5, 0.1), True)):
        y = torch.empty_like(x)
        handle.elementwise(prog, [x], y)
        handle.check()
        blocks = y.view(16, 1 << 24).view(torch.int16)
        assert torch.equal(blocks, blocks[0:1].expand(16, -1)), "output depends on position"
        want = ko.affine_gelu_bf16(bits(block).ravel(), 0.5, 0.1, linear_only=linear)
        got = blocks[0].cpu().numpy().view(np.uint16)
        if linear:
            assert np.array_equal(got, want)  # pure arithmetic: bit-exact
        else:
            ulp = ko.ulp_diff(got, want)
            assert ulp.max() <= 2, f"{ulp.max()} ulp"  # exp / div inside: <= 2 ulp of bf16


def test_config3b_row_sum_full_size(handle, ko):
    rows, cols = 65536, 4096
    X = normal((rows, cols), 1004, dtype=torch.bfloat16)
    Xd = X.cuda()
    s = handle.reduce(Xd, axis=1, out_dtype=torch.float32)
    handle.check()
    perm = torch.randperm(rows, generator=gen(7))
    s_perm = handle.reduce(Xd[perm.cuda()].contiguous(), axis=1, out_dtype=torch.float32)
    handle.check()
    assert torch.equal(s_perm.cpu(), s.cpu()[perm]), "a row's sum depends on where the row sits"
    sample = np.sort(np.random.default_rng(3).choice(rows, 256, replace=False))
    ref, ab = ko.reduce_f64(bits(X[sample]), code(torch.bfloat16), 1)
    got = s.cpu().numpy().ravel().astype(np.float64)
    assert np.all(np.abs(got[sample] - ref) <= 4 * 2.0 ** -24 * ab + 1e-30)
    total = X.double().sum().item()
    abs_total = X.double().abs().sum().item()
    assert abs(got.sum() - total) <= 4 * 2.0 ** -24 * abs_total


def test_config5_batched_full_size(handle, ko):
    Q8 = normal((8, 2048, 128), 1006, dtype=torch.bfloat16)
    K8 = normal((8, 128, 2048), 2006, dtype=torch.bfloat16)
    Q, Kt = Q8.cuda().repeat(8, 1, 1), K8.cuda().repeat(8, 1, 1)
    S = handle.matmul(Q, Kt, alpha=128 ** -0.5)
    handle.check()
    assert S.shape == (64, 2048, 2048) and S.dtype == torch.bfloat16
    groups = S.view(8, 8, 2048, 2048).view(torch.int16)
    assert torch.equal(groups, groups[0:1].expand(8, -1, -1, -1)), "a batch's result depends on its index"
    # every one of the eight distinct batch entries against the f64 checker
    for e in range(8):
        ref = ko.matmul_f64(bits(Q8[e]), code(torch.bfloat16), bits(K8[e]), code(torch.bfloat16),
                            alpha=128 ** -0.5)
        err, tau = ko.max_rel_err(S[e].cpu().double().numpy(), ref)
        assert err <= 1e-2, f"batch entry {e}: max rel err {err:.3e} (tau {tau:.3e})"
