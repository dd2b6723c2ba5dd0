"""The shape-specialised matmul paths: decode-shape (skinny) weight streaming,
batched, and the CTA-pair kernel."""
import numpy as np
import pytest
import torch

from util import bits, code, normal, uniform
from test_20_gpu_matmul import check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(16, 512, 256), (1, 384, 8192), (16, 3584, 2048), (5, 200, 136),
                                   (33, 1000, 520), (64, 256, 64)])
@pytest.mark.parametrize("wl", ["n", "t"])
def test_skinny(handle, ko, shape, wl):
    M, N, K = shape
    X = normal((M, K), 1005)
    W = normal((K, N), 2005, 0.02)
    Wd = W.cuda() if wl == "n" else W.t().contiguous().cuda().t()
    bias = uniform((N,), 15, -0.1, 0.1, torch.bfloat16)
    out = handle.matmul(X.cuda(), Wd, bias=bias.cuda())
    handle.check()
    assert handle.last_kernel == "tcgen05_skinny"
    check(ko, out, X, W, bias=bias)
    # a second launch reuses the (self-cleaned) scratch and must agree
    out2 = handle.matmul(X.cuda(), Wd, bias=bias.cuda(), out_dtype=torch.float32)
    handle.check()
    check(ko, out2, X, W, bias=bias)


def test_config4_decode_shape(handle, ko):
    """M=16, N=28672, K=8192 bf16; activations N(0,1), weights N(0,0.02)."""
    X = normal((16, 8192), 1005)
    W = normal((8192, 28672), 2005, 0.02)
    out = handle.matmul(X.cuda(), W.cuda())
    handle.check()
    assert handle.last_kernel == "tcgen05_skinny"
    cols = np.sort(np.random.default_rng(1).choice(28672, 512, replace=False)).astype(np.int32)
    cols[:4] = [0, 127, 128, 28671]
    cols = np.unique(cols).astype(np.int32)
    check(ko, out, X, W, rows=np.arange(16, dtype=np.int32), cols=cols)
    # whole output against the big-tile kernel (different summation order)
    handle.set_matmul_path("1cta:128")
    try:
        ref = handle.matmul(X.cuda(), W.cuda(), out_dtype=torch.float32)
    finally:
        handle.set_matmul_path("auto")
    handle.check()
    assert (out.float() - ref).abs().max().item() <= 2 ** -5 * ref.abs().max().item()


@pytest.mark.parametrize("batch,M,N,K", [(3, 128, 256, 64), (4, 200, 136, 128), (64, 256, 256, 128)])
def test_batched(handle, ko, batch, M, N, K):
    Q = normal((batch, M, K), 1006)
    Kt = normal((batch, K, N), 2006)
    alpha = K ** -0.5
    out = handle.matmul(Q.cuda(), Kt.cuda(), alpha=alpha)
    handle.check()
    assert out.shape == (batch, M, N) and handle.last_kernel.startswith("tcgen05")
    for b in {0, batch // 2, batch - 1}:
        check(ko, out[b], Q[b], Kt[b], alpha=alpha)


def test_config5_attention_scores(handle, ko):
    """batch 64 x (2048 x 2048 x 128) bf16 with the fused 1/sqrt(128) scale."""
    Q = normal((64, 2048, 128), 1006)
    Kt = normal((64, 128, 2048), 2006)
    alpha = 128 ** -0.5
    out = handle.matmul(Q.cuda(), Kt.cuda(), alpha=alpha)
    handle.check()
    rows = np.array([0, 1, 127, 128, 1000, 2047], dtype=np.int32)
    for b in (0, 31, 63):
        check(ko, out[b], Q[b], Kt[b], alpha=alpha, rows=rows, cols=np.arange(2048, dtype=np.int32))
    ref = torch.bmm(Q.cuda(), Kt.cuda()).float() * alpha
    assert (out.float() - ref).abs().max().item() <= 2 ** -4


@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 320), (300, 264, 136), (1024, 1024, 1024)])
@pytest.mark.parametrize("bn", [128, 256, 512])
@pytest.mark.parametrize("layout", ["nn", "nt"])
def test_cta_pair_kernel(handle, ko, shape, bn, layout):
    """tcgen05.mma.cta_group::2: two CTAs share one 256-row tile."""
    M, N, K = shape
    A, B = normal((M, K), 16, K ** -0.5), normal((K, N), 17)
    Bd = B.cuda() if layout[1] == "n" else B.t().contiguous().cuda().t()
    bias = uniform((N,), 18, -0.1, 0.1, torch.bfloat16)
    handle.set_matmul_path(f"2cta:{bn}")
    try:
        out = handle.matmul(A.cuda(), Bd, bias=bias.cuda())
        handle.check()
        assert handle.last_kernel in ("tcgen05_2cta", "tcgen05_2cta_split")
    finally:
        handle.set_matmul_path("auto")
    check(ko, out, A, B, bias=bias)


@pytest.mark.parametrize("K", [64, 192, 256, 320, 1024])
def test_wide_pair_tile_many_tiles_per_pair(handle, ko, K):
    """256 x 512 tiles, several per CTA pair, K loops shorter and longer than the
    skew between the halves at tile boundaries (1, 3, 4, 5 and 16 K blocks)."""
    M, N = 2048, 8192 + 264          # 8 x 17 tiles on 74 pairs, ragged last column block
    A, B = normal((M, K), 31, K ** -0.5), normal((K, N), 32)
    bias = uniform((N,), 33, -0.1, 0.1, torch.bfloat16)
    handle.set_matmul_path("2cta:512")
    try:
        out = handle.matmul(A.cuda(), B.cuda(), bias=bias.cuda())
        handle.check()
    finally:
        handle.set_matmul_path("auto")
    rows = np.array([0, 127, 128, 255, 256, 1000, 2047], dtype=np.int32)
    cols = np.concatenate([np.arange(0, 1024), np.arange(4000, 4700), np.arange(8100, N)]).astype(np.int32)
    check(ko, out, A, B, bias=bias, rows=rows, cols=cols)
    ref = torch.addmm(bias.cuda().float(), A.cuda().float(), B.cuda().float())
    assert (out.float() - ref).abs().max().item() <= 2 ** -5 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("variant", ["f16_out", "f32_out", "alpha", "bias_f32", "row_bias", "relu", "addend", "rz"])
def test_wide_pair_tile_epilogues(handle, ko, variant):
    """Every epilogue flavour on the 256 x 512 tile: the register-drain path
    (16-bit out, scale, optional 16-bit column bias) and the chunked one."""
    M, N, K = 512, 1280, 384
    dt = torch.float16 if variant == "f16_out" else torch.bfloat16
    A, B = normal((M, K), 41, K ** -0.5, dt), normal((K, N), 42, 1.0, dt)
    kw, okw = {}, {}
    out_dtype = torch.float32 if variant in ("f32_out", "addend") else dt
    if variant == "alpha":
        kw["alpha"] = okw["alpha"] = 0.37
        bias = uniform((N,), 43, -0.1, 0.1, dt)
        kw["bias"], okw["bias"] = bias.cuda(), bias
    if variant == "bias_f32":
        bias = uniform((N,), 43, -0.1, 0.1, torch.float32)
        kw["bias"], okw["bias"] = bias.cuda(), bias
    if variant == "row_bias":
        bias = uniform((M,), 43, -0.1, 0.1, dt)
        kw["bias"], okw["bias"] = bias.cuda(), bias
        kw["bias_axis"] = okw["bias_axis"] = 0
    if variant == "relu":
        kw["activation"] = okw["activation"] = 1
    if variant == "rz":
        kw["rounding"] = 0
    acc = None
    if variant == "addend":
        acc = normal((M, N), 44, 1.0, torch.float32)
        kw["acc"], okw["acc"] = acc.cuda(), acc
    handle.set_matmul_path("2cta:512")
    try:
        out = handle.matmul(A.cuda(), B.cuda(), out_dtype=out_dtype, **kw)
        handle.check()
        assert handle.last_kernel in ("tcgen05_2cta", "tcgen05_2cta_split")
    finally:
        handle.set_matmul_path("auto")
    check(ko, out, A, B, **okw)


def test_tune_then_dispatch_from_the_table(handle, ko, pkg, tmp_path):
    """tune_matmul times the kernel families on a problem and records the winner;
    once loaded, kapyb_matmul takes that choice for exactly that problem."""
    M, N, K = 1024, 1536, 512
    A, B = normal((M, K), 51, K ** -0.5).cuda(), normal((K, N), 52).cuda()
    f = tmp_path / "tuned.txt"
    best, times = pkg.tune_matmul(handle, A, B, file=str(f), iters=5,
                                  candidates=["auto", "1cta:128", "2cta:256", "1cta:64"])
    assert best in times and len(times) == 4
    # whatever won, force a distinctive entry and see it honoured
    f.write_text(f"{M} {N} {K} 1 bf16 k mn 1cta:64\n")
    pkg.tuning_clear()
    try:
        assert pkg.tuning_load(str(f)) == 1
        assert "tile: 128 x 64" in pkg.matmul_plan(M, N, K, handle=handle)
        out = handle.matmul(A, B)
        handle.check()
        assert handle.last_kernel in ("tcgen05_1cta", "tcgen05_1cta_split")
        check(ko, out, A.cpu(), B.cpu())
        ref = handle.matmul(A, B[:, :1024].contiguous())   # another problem: heuristics again
        handle.check()
        assert ref.shape == (M, 1024)
    finally:
        pkg.tuning_clear()


@pytest.mark.parametrize("path", ["1cta:128", "2cta:256", "2cta:512", "skinny"])
def test_eviction_priorities_become_l2_policies(handle, pkg, path):
    """EvictPriority on a matmul operand or on the output (Enums.td:78-88) turns
    into an L2 policy of the tile loads / stores: same bits with any of them."""
    A_ = pkg.abi
    M, N, K = (48, 1024, 1024) if path == "skinny" else (512, 1024, 1024)
    X, W = normal((M, K), 71, K ** -0.5).cuda(), normal((K, N), 72).cuda()
    handle.set_matmul_path(path)
    try:
        want = handle.matmul(X, W)
        for a, b, c in ((A_.EVICT_LAST, A_.EVICT_FIRST, A_.EVICT_FIRST),
                        (A_.EVICT_FIRST, A_.EVICT_LAST, A_.NO_ALLOCATE),
                        (A_.EVICT_UNCHANGED, A_.EVICT_NORMAL, A_.EVICT_LAST)):
            got = handle.matmul(X, W, cache=(A_.cache_hints(0, a), A_.cache_hints(0, b),
                                             A_.cache_hints(0, c)))
            handle.check()
            assert torch.equal(got, want), (a, b, c)
    finally:
        handle.set_matmul_path("auto")
    with pytest.raises(ValueError, match="cache operator or eviction priority"):
        handle.matmul(X, W, cache=(A_.cache_hints(0, 7), 0, 0))


@pytest.mark.parametrize("path", ["2cta:512", "2cta:256", "2cta:128", "1cta:256", "1cta:256:e8", "1cta:64"])
def test_addend_fetched_by_tiles(handle, ko, path):
    """kapy.matmul's third operand.  An addend of the output's type with a layout
    TMA can describe comes into the epilogue tile by tile; any other (here: unit
    stride on the rows) element by element.  Same arithmetic, same bits; ragged
    edges, f16 and f32."""
    M, N, K = 600, 1096, 320
    for dt, odt in ((torch.float16, torch.float16), (torch.bfloat16, torch.float32)):
        A, B = normal((M, K), 71, K ** -0.5, dt), normal((K, N), 72, 1.0, dt)
        acc = normal((M, N), 73, 1.0, odt)
        bias = uniform((N,), 74, -0.1, 0.1, dt)
        handle.set_matmul_path(path)
        try:
            fast = handle.matmul(A.cuda(), B.cuda(), acc=acc.cuda(), bias=bias.cuda(), alpha=0.75,
                                 activation=1, out_dtype=odt)
            by_element = handle.matmul(A.cuda(), B.cuda(), acc=acc.t().contiguous().cuda().t(),
                                       bias=bias.cuda(), alpha=0.75, activation=1, out_dtype=odt)
            handle.check()
        finally:
            handle.set_matmul_path("auto")
        check(ko, fast, A, B, acc=acc, bias=bias, alpha=0.75, activation=1)
        assert torch.equal(fast, by_element)
        # in place (C = act(alpha * A.B + bias + C)): every tile is read before it is written
        handle.set_matmul_path(path)
        try:
            inplace = acc.cuda()
            handle.matmul(A.cuda(), B.cuda(), acc=inplace, out=inplace, bias=bias.cuda(), alpha=0.75,
                          activation=1)
            handle.check()
        finally:
            handle.set_matmul_path("auto")
        assert torch.equal(inplace, fast)

