"""Sharded paths on two GPUs (skipped on a one-GPU box): the column-sharded
GEMM with its two ways of assembling the full output, the decode-shape GEMM
sharded by weight columns, the batched GEMM sharded by batch, the end-to-end
host-buffer call whose upload of lhs is sharded by rows, and the bounded wait
when a peer stays silent.  NVLS is off and the library's own flags use plain
peer stores."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KAPYB_ROOT"])
import __graft_entry__ as entry
import oracle as ko
pkg = entry.load_package()
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
h = pkg.Handle(rank)
dev = torch.device("cuda", rank)
bits = lambda t: t.contiguous().cpu().view(torch.int16).numpy().view(np.uint16)

# ---- column-sharded GEMM: local shard, NCCL gather, fused push gather
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
pg = pkg.dist.PushGather(M, N, torch.bfloat16, dev)
pg.full.zero_()
torch.cuda.synchronize()
dist.barrier()
for _ in range(3):
    pg.matmul(h, A, Bs, b, bias_shard=bs)
    out = pg.wait(limit_ms=5000)
h.check()
torch.cuda.synchronize()
assert torch.equal(out, ref), "push gather differs (local or remote block)"
dist.barrier()

# ---- decode shape sharded by weight columns: 3584 columns per rank (28 tiles,
# all of them split between SMs), against the checker and the one-GPU result
g = torch.Generator().manual_seed(5)
Md, Kd, Nd = 16, 2048, 3584 * world
X = torch.randn(Md, Kd, generator=g).bfloat16()
W = (torch.randn(Kd, Nd, generator=g) * 0.02).bfloat16()
spans = pkg.dist.column_shards(Nd, world, 128)
b, e = spans[rank]
assert e - b == 3584
Xd, Wd = X.cuda(), W[:, b:e].contiguous().cuda()
mine = h.matmul(Xd, Wd)
h.check()
assert h.last_kernel == "tcgen05_skinny"
want = ko.matmul_f64(bits(X), ko.BF16, bits(W[:, b:e]), ko.BF16)
err, _ = ko.max_rel_err(ko.from_bits(bits(mine), ko.BF16), want)
assert err <= 1e-2, f"decode shard: max rel err {err}"
# (a shard and the whole problem split their tiles between SMs at different k
# blocks, so they agree to the tolerance, not bit for bit)
gathered = pkg.dist.all_gather_columns(mine, spans)
assert torch.equal(gathered[:, b:e], mine), "decode gather moved this rank's block"
want_all = ko.matmul_f64(bits(X), ko.BF16, bits(W), ko.BF16)
err, _ = ko.max_rel_err(ko.from_bits(bits(gathered), ko.BF16), want_all)
assert err <= 1e-2, f"decode gather: max rel err {err}"

# ---- batched shape sharded by batch
g = torch.Generator().manual_seed(6)
Bt = 4 * world
Q = torch.randn(Bt, 512, 128, generator=g).bfloat16().cuda()
Kt = torch.randn(Bt, 128, 768, generator=g).bfloat16().cuda()
b0, b1 = pkg.dist.batch_shards(Bt, world)[rank]
part = h.matmul(Q[b0:b1].contiguous(), Kt[b0:b1].contiguous(), alpha=128 ** -0.5)
h.check()
assert part.shape == (b1 - b0, 512, 768)
for i in range(b1 - b0):
    want = ko.matmul_f64(bits(Q[b0 + i]), ko.BF16, bits(Kt[b0 + i]), ko.BF16, alpha=128 ** -0.5)
    err, _ = ko.max_rel_err(ko.from_bits(bits(part[i]), ko.BF16), want)
    assert err <= 1e-2, f"batch entry {b0 + i}: max rel err {err}"

# ---- end to end from host buffers, upload of lhs sharded by rows
g = torch.Generator().manual_seed(7)
Mh, Kh, Nh = 2048, 1024, 1536
Ah = (torch.randn(Mh, Kh, generator=g) * Kh ** -0.5).bfloat16()
Bh = torch.randn(Kh, Nh, generator=g).bfloat16()
biash = (torch.rand(Nh, generator=g) * 0.2 - 0.1).bfloat16()
spans = pkg.dist.column_shards(Nh, world, 256)
b, e = spans[rank]
devref = h.matmul(Ah.cuda(), Bh[:, b:e].contiguous().cuda(), bias=biash[b:e].contiguous().cuda())
shm = pkg.dist.ShardedHostMatmul(Mh, Kh, torch.bfloat16, dev)
r0, r1 = shm.rows
A_rows = Ah[r0:r1].contiguous().pin_memory()
B_shard, b_shard = Bh[:, b:e].contiguous().pin_memory(), biash[b:e].contiguous().pin_memory()
out = torch.empty((Mh, e - b), dtype=torch.bfloat16).pin_memory()
for it in range(3):       # three calls: both staging copies are used and reused
    out.zero_()
    shm(h, A_rows, B_shard, out, bias=b_shard, wait_limit_ms=5000)
    assert torch.equal(out, devref.cpu()), f"sharded host call {it} differs from the device path"
dist.barrier()

# ---- a silent peer: rank 1 does not signal; rank 0's wait runs out and says so
flags = pkg.dist.RankFlags(dev)
seq = flags.next()
if rank == 0:
    h.gather_signal(flags.ptrs, rank, seq)
    h.gather_wait(flags.ptrs[rank], world, seq, limit_ms=100)
    try:
        h.check()
        raise AssertionError("the wait should have timed out")
    except pkg.KapybTimeout:
        pass
torch.cuda.synchronize()
dist.barrier()
if rank != 0:
    h.gather_signal(flags.ptrs, rank, seq)      # the late signal
h.gather_wait(flags.ptrs[rank], world, seq, limit_ms=5000) if rank == 0 else None
h.check()
torch.cuda.synchronize()
dist.barrier()
assert torch.equal(h.matmul(A, B, bias=bias), ref), "context not usable after the time-out"
h.check()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_paths(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, KAPYB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("ok") == 2
