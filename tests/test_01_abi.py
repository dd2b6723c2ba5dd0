"""The C-ABI library: loads without a GPU, exports every symbol the header
declares, and refuses to pretend it can compute without a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "kapyb.h")).read()
    return sorted(set(re.findall(r"KAPYB_API[^;(]*?\b(kapyb_[a-z0-9_]+)\s*\(", text, flags=re.S)))


def test_header_symbols_exported(pkg):
    lib = pkg.abi.load()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/kapyb.h but not exported"
        assert n in pkg.abi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert lib.kapyb_version() >= 100


def test_struct_layout_matches_header(pkg):
    abi = pkg.abi
    assert C.sizeof(abi.Tensor2d) == 48
    assert C.sizeof(abi.Epilogue) == 32
    assert C.sizeof(abi.Inst) == 32


def test_shard_range(pkg):
    # N = 8192 over 8 ranks in 128-column blocks: equal contiguous blocks
    spans = [pkg.shard_range(8192, 8, r, 128) for r in range(8)]
    assert spans == [(1024 * r, 1024 * (r + 1)) for r in range(8)]
    # ragged: 28672 columns over 8 ranks, 3584 each (28 blocks of 128)
    spans = [pkg.shard_range(28672, 8, r, 128) for r in range(8)]
    assert spans[0] == (0, 3584) and spans[-1] == (25088, 28672)
    # cover-exactly-once property on awkward sizes, including empty shards
    for total, parts, align in [(1000, 3, 128), (5, 8, 1), (0, 4, 16), (64, 4, 64), (130, 4, 8)]:
        spans = [pkg.shard_range(total, parts, r, align) for r in range(parts)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
            assert e0 == b1 and b0 <= e0
        assert all(b % align == 0 or b == total for b, _ in spans)
    with pytest.raises(ValueError):
        pkg.shard_range(10, 0, 0, 1)
    with pytest.raises(ValueError):
        pkg.shard_range(10, 2, 2, 1)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_create_fails_loudly_without_gpu(pkg):
    with pytest.raises(pkg.KapybError) as ei:
        pkg.Handle(0)
    assert "no CPU path" in str(ei.value) or "CUDA" in str(ei.value)


def test_product_does_not_import_oracle():
    """The checker is test infrastructure: nothing in the package may reach it."""
    pkg_dir = os.path.join(ROOT, "kapy-lang_b200")
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
                assert "kapy_oracle" not in src, f
