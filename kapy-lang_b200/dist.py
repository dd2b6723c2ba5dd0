"""Multi-GPU plumbing for the sharded matmul paths (one process per GPU,
``torch.distributed`` for rendezvous and collectives).

The reference has no multi-GPU code; the partitioning follows the shapes it is
asked to run: large GEMMs shard by columns of B and of the output, batched
GEMMs by batch.  Outputs stay sharded unless the caller asks for the full
matrix, in which case there are two ways to assemble it:

  * ``all_gather_columns``: NCCL all-gather of the column blocks into a staging
    buffer followed by a strided copy (column blocks of a row-major matrix are
    not contiguous, so the gather cannot land in place);
  * ``PushGather``: every rank's GEMM epilogue stores its finished tiles
    straight into all peers' full-size outputs through peer-mapped pointers
    (``kapyb_matmul_push``), so the transfer overlaps the main loop tile by
    tile and no staging copy exists.  Only stores cross NVLink.

Ranks meet through flag words the library's own kernels write and poll with a
time limit (``RankFlags``), so a missing peer becomes ``KapybTimeout``.
``ShardedHostMatmul`` is the end-to-end form for host tensors.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

from . import runtime


def column_shards(n_total: int, world: int, align: int = 256) -> List[Tuple[int, int]]:
    """[begin, end) of output columns per rank, in blocks of `align` columns."""
    return [runtime.shard_range(n_total, world, r, align) for r in range(world)]


def batch_shards(batch: int, world: int) -> List[Tuple[int, int]]:
    return [runtime.shard_range(batch, world, r, 1) for r in range(world)]


def all_gather_columns(shard, spans: Sequence[Tuple[int, int]], group=None, out=None):
    """Assembles [M, N] from per-rank column blocks [M, end-begin] (ragged or
    empty blocks allowed).  Works on any backend (NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    assert len(spans) == world
    M = shard.shape[0]
    width = max(e - b for b, e in spans)
    n_total = spans[-1][1]
    rank = dist.get_rank(group)
    if shard.shape[1] != spans[rank][1] - spans[rank][0]:
        raise ValueError("shard width does not match this rank's span")
    staging = torch.empty((world, M, width), dtype=shard.dtype, device=shard.device)
    mine = shard
    if shard.shape[1] != width:
        mine = torch.zeros((M, width), dtype=shard.dtype, device=shard.device)
        mine[:, : shard.shape[1]] = shard
    dist.all_gather_into_tensor(staging.view(world * M, width), mine.contiguous(), group=group)
    if out is None:
        out = torch.empty((M, n_total), dtype=shard.dtype, device=shard.device)
    for r, (b, e) in enumerate(spans):
        if e > b:
            out[:, b:e] = staging[r, :, : e - b]
    return out


def sharded_matmul(handle, lhs, rhs_shard, spans, *, bias_shard=None, gather: str = "none",
                   group=None, compute: Optional[Callable] = None, **epilogue):
    """N-sharded matmul: this rank multiplies by its column block of B.  `gather`
    is "none" (return the local [M, n_local] block) or "nccl" (return [M, N])."""
    compute = compute or (lambda a, b, bias: handle.matmul(a, b, bias=bias, **epilogue))
    local = compute(lhs, rhs_shard, bias_shard)
    if gather == "none":
        return local
    if gather == "nccl":
        return all_gather_columns(local, spans, group=group)
    raise ValueError("gather must be 'none' or 'nccl' (use PushGather for the fused variant)")


class RankFlags:
    """One flag word per rank in every rank's symmetric memory, and the sequence
    number the ranks count together (kapyb_gather_signal / kapyb_gather_wait)."""

    def __init__(self, device, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        # 64 words: the array the library's kernels index by rank
        self.words = symm.empty((64,), dtype=torch.int32, device=device)
        self.words.zero_()
        self.hdl = symm.rendezvous(self.words, group=self.group)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(self.group)      # nobody signals before every array is zero
        self.seq = 0

    def next(self) -> int:
        self.seq += 1
        return self.seq

    def signal_and_wait(self, handle, limit_ms: int = 0, stream=None) -> int:
        """Announces this rank's work so far on the stream to every rank, then
        waits (bounded, on the stream) for the same announcement from all."""
        seq = self.next()
        handle.gather_signal(self.ptrs, self.rank, seq, stream=stream)
        handle.gather_wait(self.ptrs[self.rank], self.world, seq, limit_ms, stream=stream)
        return seq


class PushGather:
    """Full-size outputs in symmetric memory plus the fused push epilogue."""

    def __init__(self, M: int, n_total: int, dtype, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group or dist.group.WORLD
        self.full = symm.empty((M, n_total), dtype=dtype, device=device)
        self.hdl = symm.rendezvous(self.full, group=self.group)
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        # Each rank walks the destinations starting after itself (its own copy
        # last), so that at any moment the ranks push to different peers instead
        # of all converging on rank 0's NVLink port, then rank 1's, ...
        r = dist.get_rank(self.group)
        self.peer_ptrs = [ptrs[(r + 1 + i) % len(ptrs)] for i in range(len(ptrs))]
        self.M, self.n_total, self.dtype = M, n_total, dtype
        self.flags = RankFlags(device, self.group)
        self._handle = None

    def matmul(self, handle, lhs, rhs_shard, col_begin: int, *, bias_shard=None, **epilogue):
        """Runs this rank's shard and stores it into every rank's `full`."""
        self._handle = handle
        handle.matmul_push(lhs, rhs_shard, self.peer_ptrs, out_dtype=self.dtype,
                           out_stride0=self.n_total, col_begin=col_begin, n_total=self.n_total,
                           bias=bias_shard, **epilogue)

    def wait(self, limit_ms: int = 0):
        """Stream-ordered and bounded: after it, every peer's stores into this
        rank's `full` have landed.  The ranks meet through the library's flag
        words; a peer that never arrives surfaces as KapybTimeout in
        handle.check(), not as a hang."""
        if self._handle is None:
            raise RuntimeError("PushGather.wait() before matmul()")
        self.flags.signal_and_wait(self._handle, limit_ms)
        return self.full


class ShardedHostMatmul:
    """End-to-end matmul on host tensors across the ranks of one box.  The
    output is sharded by columns; the UPLOAD of lhs is sharded by rows (each rank
    sends its rows over PCIe once and forwards them to its peers over NVLink),
    so the host-side traffic per step does not grow with the number of GPUs."""

    def __init__(self, m_total: int, k: int, dtype, device, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.m_total, self.k = m_total, k
        esz = torch.empty((), dtype=dtype).element_size()
        half = (m_total * k * esz + 255) // 256 * 256
        # two staging copies of lhs, used in turn (see kapyb_shard_ctx)
        self.staging = symm.empty((2 * half,), dtype=torch.uint8, device=device)
        self.hdl = symm.rendezvous(self.staging, group=self.group)
        self.lhs_ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.flags = RankFlags(device, self.group)
        self.rows = runtime.shard_range(m_total, self.world, self.rank, 256)

    def __call__(self, handle, lhs_rows, rhs_shard, out, *, wait_limit_ms: int = 0, **epilogue):
        """lhs_rows: host rows [self.rows[0], self.rows[1]) of lhs; rhs_shard: this
        rank's host column block of B; out: host [m_total, n_local]."""
        return handle.matmul_host_sharded(
            lhs_rows, self.m_total, self.rows[0], rhs_shard, out, peer_lhs_ptrs=self.lhs_ptrs,
            peer_flag_ptrs=self.flags.ptrs, rank=self.rank, seq=self.flags.next(),
            wait_limit_ms=wait_limit_ms, **epilogue)
