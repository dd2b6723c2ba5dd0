"""kapyb_matmul_plan: the dispatch decisions of the matmul, checked on the host
(no GPU: only shapes, strides, dtypes and address alignment are looked at).
The benchmark configurations must land on the kernels the design names."""
import pytest


def plan(pkg, *a, **k):
    return pkg.matmul_plan(*a, **k)


def test_config2_takes_the_512_wide_pair_tile(pkg):
    text = plan(pkg, 8192, 8192, 8192)
    assert "tcgen05_2cta" in text and "tile: 256 x 512" in text and "epilogue warps 8" in text
    assert "32 x 16 x 1 = 512 tile(s) on 74 CTA pairs: 7 wave(s)" in text
    assert "A K contiguous" in text and "B N contiguous" in text


@pytest.mark.parametrize("n_gpus,n_local", [(2, 4096), (4, 2048), (8, 1024)])
def test_config2_shards_keep_the_pair_tile(pkg, n_gpus, n_local):
    text = plan(pkg, 8192, n_local, 8192, rhs_strides=(n_local, 1), out_strides=(n_local, 1))
    assert "tile: 256 x 512" in text


def test_config1_small_fp16_colmajor_b(pkg):
    text = plan(pkg, 1024, 1024, 1024, dtype=pkg.abi.F16, rhs_strides=(1, 1024))
    assert "tcgen05_1cta" in text and "B K contiguous" in text


def test_config4_decode_streams_weights(pkg):
    text = plan(pkg, 16, 28672, 8192)
    assert "tcgen05_skinny" in text
    assert "224 weight tiles x 128 k-blocks on 148 CTAs" in text
    assert "76 split tile(s) first, in spans of 66 k-block(s); then 1 whole tile(s) per CTA" in text


def test_config5_short_k_gets_eight_epilogue_warps(pkg):
    text = plan(pkg, 2048, 2048, 128, batch=64)
    assert "tcgen05_1cta" in text and "tile: 128 x 256" in text and "epilogue warps 8" in text
    assert "x 64 = 8192 tile(s)" in text


def test_one_wave_problem_avoids_the_wide_tile(pkg):
    # 2048^3: 8 x 4 tiles of 256 x 512 would fill 32 of 74 pairs; 256-wide tiles fill 64
    assert "tile: 256 x 256" in plan(pkg, 2048, 2048, 2048)


def test_fallbacks_and_transposition(pkg):
    # leading dimension of 1001 bf16 elements: not a multiple of 16 bytes -> CUDA cores
    assert "path: simt" in plan(pkg, 512, 512, 1001)
    # base address off 16 bytes
    assert "path: simt" in plan(pkg, 512, 512, 512, align=8)
    # column-major output: the transposed problem runs
    text = plan(pkg, 512, 1024, 512, out_strides=(1, 512))
    assert "the transposed problem is computed" in text
    # f8 with an N-contiguous B needs 128 columns per CTA and half: narrow N leaves the pair path
    text = plan(pkg, 512, 384, 1024, dtype=pkg.abi.F8E4M3, out_dtype=pkg.abi.BF16)
    assert "tcgen05_1cta" in text


def test_verifier_applies(pkg):
    with pytest.raises(ValueError, match="same element bit width"):
        plan(pkg, 64, 64, 64, dtype=pkg.abi.F32, rhs_dtype=pkg.abi.F16, out_dtype=pkg.abi.F32)
    assert "path: none" in plan(pkg, 0, 64, 64)


def test_tuning_table(pkg, tmp_path):
    """Tuned choices override the heuristics for exactly the listed problem, are
    ignored where they cannot apply, and bad files are refused with the line."""
    f = tmp_path / "tuned.txt"
    f.write_text("# M N K batch dtype lhs rhs path\n"
                 "2048 2048 2048 1 bf16 k mn 1cta:256:e8   # one-wave problem\n"
                 "\n"
                 "512 512 1001 1 bf16 k mn 2cta:256\n")
    pkg.tuning_clear()
    try:
        assert "tile: 256 x 256" in plan(pkg, 2048, 2048, 2048)
        assert pkg.tuning_load(str(f)) == 2
        text = plan(pkg, 2048, 2048, 2048)
        assert "tcgen05_1cta" in text and "tile: 128 x 256" in text and "epilogue warps 8" in text
        assert "from the tuning table" in text
        # another problem, another operand type or another major: untouched
        assert "from the tuning table" not in plan(pkg, 2048, 2048, 1024)
        assert "from the tuning table" not in plan(pkg, 2048, 2048, 2048, dtype=pkg.abi.F16)
        assert "from the tuning table" not in plan(pkg, 2048, 2048, 2048, rhs_strides=(1, 2048))
        # a tuned tcgen05 path for operands TMA cannot describe is ignored
        assert "path: simt" in plan(pkg, 512, 512, 1001)
        pkg.tuning_clear()
        assert "tile: 256 x 256" in plan(pkg, 2048, 2048, 2048)
        bad = tmp_path / "bad.txt"
        bad.write_text("128 128 128 1 bf16 k mn 2cta:256\n128 128 128 1 int8 k mn auto\n")
        with pytest.raises(ValueError, match="line 2"):
            pkg.tuning_load(str(bad))
    finally:
        pkg.tuning_clear()


def test_few_row_problems_spread_over_the_sms(pkg):
    """One wave of tiles either way: the narrower tile fills more SMs."""
    assert "tile: 128 x 64" in plan(pkg, 128, 8192, 8192)        # 128 tiles instead of 32
    assert "tile: 256 x 128" in plan(pkg, 256, 8192, 8192)       # 64 pair tiles instead of 32
    assert "tile: 256 x 256" in plan(pkg, 8192, 8192, 512)       # K loop too short for the wide tile
    assert "tile: 128 x 256" in plan(pkg, 8192, 8192, 64)        # many waves: the widest single-CTA tile


def test_partly_filled_last_wave_stays_whole_unless_asked(pkg):
    """The column shards of the 8192^3 problem on 2, 4 and 8 GPUs leave 34, 54 and
    64 tiles of 256 x 512 for 74 CTA pairs in their last wave.  Splitting those
    tiles' K blocks between all pairs was measured slower on a power-capped part,
    so the plan keeps whole tiles; the split is there on request."""
    for n in (1024, 2048, 4096, 8192):
        assert "last wave" not in plan(pkg, 8192, n, 8192)
