// Cross-GPU completion flags for the sharded paths: one 32-bit word per rank in
// memory every rank can reach (peer-mapped device memory, or pinned host memory).
// Rank r announces "everything I issued on this stream before now has landed"
// by storing a sequence number into word r of EVERY rank's flag array; a rank
// that needs its peers' data waits until each word of its OWN array has reached
// that number.  Only stores cross the link, never a load of remote memory.
//
// The wait is bounded by wall-clock time: when it runs out the kernel records
// kStatusTimeout in the handle's status word and returns, so the context stays
// usable and the host reads KAPYB_TIMEOUT from kapyb_check().
#pragma once

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace kapyb {

constexpr int kMaxGatherRanks = 64;

struct GatherFlagPtrs {
  uint32_t *p[kMaxGatherRanks];
};

// One thread per destination rank: flags_of_rank[dst][my_rank] = seq, ordered
// after every write this GPU made before the kernel (system-scope release).
__global__ void gather_signal_kernel(const GatherFlagPtrs flags, int n_ranks, int my_rank,
                                     uint32_t seq) {
  const int dst = threadIdx.x;
  if (dst >= n_ranks) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[dst] + my_rank), "r"(seq)
               : "memory");
}

// One thread per source rank polls its word until it is at or past `seq`
// (sequence numbers wrap: the comparison is on the signed difference).  Gives up
// after limit_ns and reports through *status.
__global__ void gather_wait_kernel(const uint32_t *my_flags, int n_ranks, uint32_t seq,
                                   unsigned long long limit_ns, uint32_t *status) {
  const int src = threadIdx.x;
  if (src >= n_ranks) return;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_flags + src) : "memory");
    if (static_cast<int32_t>(v - seq) >= 0) break;
    if ((it & 15u) == 15u && ptx::globaltimer_ns() - t0 > limit_ns) {
      atomicExch(status, kStatusTimeout);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

// Forwards `n16` 16-byte words from this GPU's memory to the same offset of up to
// kMaxGatherRanks - 1 peers: read once, stored once per peer (plain stores through
// peer-mapped pointers; nothing is loaded from a peer).  The copy engines, which
// could do the same, are busy with the host traffic of the call this serves: seven
// engine copies of 4 MB each took 0.42 ms per piece there, this kernel's NVLink
// time is a tenth of that.
struct ForwardPeers {
  uint4 *dst[kMaxGatherRanks];
  int n;
};

__global__ void __launch_bounds__(256) forward_to_peers_kernel(const uint4 *__restrict__ src,
                                                               size_t n16, const ForwardPeers peers) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // four independent loads in flight per thread
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(src + i + u * stride);
    for (int p = 0; p < peers.n; ++p) {
#pragma unroll
      for (int u = 0; u < 4; ++u) peers.dst[p][i + u * stride] = v[u];
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = __ldcs(src + i);
    for (int p = 0; p < peers.n; ++p) peers.dst[p][i] = v;
  }
}

}  // namespace kapyb
