"""N-sharded matmul on two GPUs: local shards, the NCCL gather and the fused
push epilogue agree with the single-GPU result.  Skipped on a one-GPU box."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KAPYB_ROOT"])
import __graft_entry__ as entry
pkg = entry.load_package()
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
h = pkg.Handle(rank)
g = torch.Generator().manual_seed(3)
M, K, N = 512, 1024, 1536
A = (torch.randn(M, K, generator=g) * K ** -0.5).bfloat16().cuda()
B = torch.randn(K, N, generator=g).bfloat16().cuda()
bias = (torch.rand(N, generator=g) * 0.2 - 0.1).bfloat16().cuda()
ref = h.matmul(A, B, bias=bias)
spans = pkg.dist.column_shards(N, world, 256)
b, e = spans[rank]
Bs, bs = B[:, b:e].contiguous(), bias[b:e].contiguous()
local = pkg.dist.sharded_matmul(h, A, Bs, spans, bias_shard=bs)
assert torch.equal(local, ref[:, b:e]), "local shard differs"
full = pkg.dist.sharded_matmul(h, A, Bs, spans, bias_shard=bs, gather="nccl")
assert torch.equal(full, ref), "nccl gather differs"
pg = pkg.dist.PushGather(M, N, torch.bfloat16, torch.device("cuda", rank))
pg.full.zero_()
dist.barrier()
for _ in range(2):
    pg.matmul(h, A, Bs, b, bias_shard=bs)
    out = pg.wait()
h.check()
torch.cuda.synchronize()
assert torch.equal(out, ref), "push gather differs"
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_matmul(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, KAPYB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("ok") == 2
