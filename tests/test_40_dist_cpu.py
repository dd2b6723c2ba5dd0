"""Host logic of the sharded paths with two gloo ranks on CPU: shard ranges,
ragged column all-gather and the batch split.  The per-shard product is a CPU
stand-in injected by the test (the library itself has no CPU compute)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    pkg = entry.load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        M, K, N = 24, 40, 1000            # 1000 columns in 256-blocks over 2 ranks: 512 + 488
        A = torch.randn(M, K, generator=g)
        B = torch.randn(K, N, generator=g)
        bias = torch.randn(N, generator=g)
        spans = pkg.dist.column_shards(N, world, 256)
        b, e = spans[rank]
        cpu_mm = lambda a, bb, bs: a @ bb + bs
        full = pkg.dist.sharded_matmul(None, A, B[:, b:e].contiguous(), spans,
                                       bias_shard=bias[b:e], gather="nccl", compute=cpu_mm)
        ok1 = torch.allclose(full, A @ B + bias, atol=1e-5)
        local = pkg.dist.sharded_matmul(None, A, B[:, b:e].contiguous(), spans,
                                        bias_shard=bias[b:e], gather="none", compute=cpu_mm)
        ok2 = local.shape == (M, e - b)
        # an empty shard (more ranks' worth of blocks than columns)
        spans3 = [(0, 256), (256, 256)] if world == 2 else None
        small = torch.randn(4, 256, generator=g)
        sh = small if rank == 0 else small[:, :0]
        got = pkg.dist.all_gather_columns(sh, spans3)
        ok3 = torch.equal(got, small)
        q.put((rank, ok1, ok2, ok3, spans))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_gather():
    world, port = 2, 29000 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok1, ok2, ok3, spans in res:
        assert ok1 and ok2 and ok3, (rank, ok1, ok2, ok3)
        assert spans == [(0, 512), (512, 1000)]


def test_shard_helpers(pkg):
    assert pkg.dist.column_shards(8192, 8) == [(1024 * r, 1024 * (r + 1)) for r in range(8)]
    assert pkg.dist.column_shards(28672, 8, 128)[3] == (10752, 14336)
    assert pkg.dist.batch_shards(64, 8) == [(8 * r, 8 * r + 8) for r in range(8)]
    assert pkg.dist.batch_shards(3, 4) == [(0, 1), (1, 2), (2, 3), (3, 3)]
