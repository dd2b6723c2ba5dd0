"""The last, partly filled wave of a tcgen05 launch, split on request (":x1"): its
tiles' K blocks are dealt out as one span per CTA (pair), partial accumulators travel through a
scratch buffer and are added in CTA order.  Checked against the f64 checker
(max relative error 1e-2 over a floor of 2^-6 rms, the matmul tolerance), for
bit-stability across runs, and against the same kernel with whole tiles
(different summation order: equal within fp32 rounding of the accumulators,
i.e. at most one unit in the last place of the 16-bit output apart from ties)."""
import numpy as np
import pytest
import torch

from util import normal, uniform
from test_20_gpu_matmul import check

pytestmark = pytest.mark.gpu


def run(handle, path, A, B, **kw):
    handle.set_matmul_path(path)
    try:
        out = handle.matmul(A, B, **kw)
        handle.check()
        return out, handle.last_kernel
    finally:
        handle.set_matmul_path("auto")


# (path, M, N, K): leftover tiles < CTAs (pairs), spans crossing tile boundaries;
# several whole waves first; ragged edges; spans shorter than a tile's half; a
# tile shared by three and more CTAs
CASES = [
    ("2cta:512", 2048, 4096, 2048),    # 64 tiles on 74 pairs: every tile split
    ("2cta:512", 2560, 8192 + 264, 1024),  # 170 tiles: two whole waves, 22 split (ragged last column block)
    ("2cta:512", 1024, 2048, 4096),    # 16 tiles on 74 pairs: a tile shared by 5-6 pairs
    ("2cta:256", 2048, 3072, 1536),    # 96 tiles of 256 x 256: one wave + 22
    ("2cta:128", 1024, 1536 + 72, 2048),  # 52 tiles of 256 x 128
    ("1cta:256", 1280, 2560 + 40, 1024),  # 110 tiles on 148 CTAs
    ("1cta:256:e8", 2304, 4096, 512),  # 288 tiles: one wave + 140 (more than 90 %: whole unless forced)
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[0]}-{c[1]}x{c[2]}x{c[3]}")
def test_split_last_wave(handle, ko, case):
    path, M, N, K = case
    A, B = normal((M, K), 61, K ** -0.5), normal((K, N), 62)
    bias = uniform((N,), 63, -0.1, 0.1, torch.bfloat16)
    Ad, Bd, bd = A.cuda(), B.cuda(), bias.cuda()
    whole, k0 = run(handle, path + ":x0", Ad, Bd, bias=bd)
    split, k1 = run(handle, path + ":x1", Ad, Bd, bias=bd)
    assert not k0.endswith("_split") and k1.endswith("_split"), (k0, k1)
    again, _ = run(handle, path + ":x1", Ad, Bd, bias=bd)
    assert torch.equal(split, again), "split tiles are summed in a fixed order"
    rows = np.unique(np.concatenate([np.arange(0, M, 97), [127, 128, 255, 256, M - 1]])).astype(np.int32)
    check(ko, split, A, B, bias=bias, rows=rows[rows < M], cols=np.arange(N, dtype=np.int32))
    d = (split.float() - whole.float()).abs()
    scale = whole.float().abs().clamp_min(1.0)
    assert (d / scale).max().item() <= 2 ** -7, "more than a rounding step from the whole-tile result"


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
def test_split_epilogues(handle, ko, out_dtype):
    """f32 output (chunked epilogue) and an f16 problem with alpha, a per-row bias
    and an activation, on split 256 x 512 tiles."""
    M, N, K = 1536, 2048, 1024
    dt = torch.float16 if out_dtype == torch.float16 else torch.bfloat16
    A, B = normal((M, K), 71, K ** -0.5, dt), normal((K, N), 72, 1.0, dt)
    kw, okw = {}, {}
    if out_dtype == torch.float16:
        rb = uniform((M,), 73, -0.5, 0.5, torch.float32)
        kw = dict(bias=rb.cuda(), bias_axis=0, activation=1, alpha=0.6)
        okw = dict(bias=rb, bias_axis=0, activation=1, alpha=0.6)
    out, kern = run(handle, "2cta:512:x1", A.cuda(), B.cuda(), out_dtype=out_dtype, **kw)
    assert kern == "tcgen05_2cta_split"
    check(ko, out, A, B, **okw)


def test_split_is_on_request_only(handle, ko, pkg):
    """8192 x 1024 x 8192 (the column shard of the 8192^3 problem on eight GPUs) is
    64 tiles of 256 x 512 on 74 CTA pairs.  Whole tiles by default (the split was
    measured slower); with ":x1" the plan names the split and the result holds."""
    M, N, K = 8192, 1024, 8192
    A, B = normal((M, K), 81, K ** -0.5).cuda(), normal((K, N), 82).cuda()
    out = handle.matmul(A, B)
    handle.check()
    assert handle.last_kernel == "tcgen05_2cta"
    assert "last wave" not in pkg.matmul_plan(M, N, K, handle=handle)
    handle.set_matmul_path("auto:x1")
    try:
        split = handle.matmul(A, B)
        handle.check()
        assert handle.last_kernel == "tcgen05_2cta_split"
        assert "last wave: 64 tile(s) x 128 k-blocks split between the 74 CTA pairs" in \
            pkg.matmul_plan(M, N, K, handle=handle)
    finally:
        handle.set_matmul_path("auto")
    rows = np.array([0, 255, 256, 4095, 8191], dtype=np.int32)
    for o in (out, split):
        check(ko, o, A.cpu(), B.cpu(), rows=rows, cols=np.arange(N, dtype=np.int32))


def test_split_time_out_is_bounded(handle, pkg):
    """The producer stays silent (debug bit 4): every wait, the one for the other
    CTAs' partial sums included, runs out after the limit; the context stays
    usable and the next launch gives the right bits."""
    A, B = normal((1024, 2048), 91, 2048 ** -0.5).cuda(), normal((2048, 2048), 92).cuda()
    want, _ = run(handle, "2cta:512:x1", A, B)
    handle.set_matmul_path("2cta:512:x1:d16:w50")
    try:
        handle.matmul(A, B)
        with pytest.raises(pkg.KapybTimeout):
            handle.check()
    finally:
        handle.set_matmul_path("auto")
    got, _ = run(handle, "2cta:512:x1", A, B)
    assert torch.equal(got, want)
