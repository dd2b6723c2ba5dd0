// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier,
// TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05 (TMEM
// allocation, MMA, commit, load) and cluster addressing.  Every wait is
// bounded: it polls mbarrier.try_wait and gives up after a wall-clock limit so a
// broken pipeline returns an error status instead of hanging the GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kapyb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Programmatic dependent launch.  griddep_launch: the next kernel in the stream
// (if it was launched with programmatic stream serialization) may start being
// scheduled now instead of when this grid has drained; griddep_wait: blocks until
// every grid this one depends on has completed and its writes are visible.  A
// kernel launched without the attribute sees both as no-ops.
__device__ __forceinline__ void griddep_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that may live in another CTA of the cluster
// (`bar` is a shared::cluster address, e.g. from mapa()).  Used to hand a TMEM
// slot back to the pair's MMA thread: what has to be ordered are the tcgen05.ld
// reads (tcgen05.wait::ld and tcgen05.fence::before_thread_sync ahead of the
// arrival do that), not this thread's ordinary memory traffic, so the arrival
// carries the default semantics; asking for a release at cluster scope made each
// hand-over cost about 1200 clocks.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait with a suspend-time hint: the thread may sleep in hardware for up to
// `ns` and is woken as soon as the phase completes, instead of re-issuing the
// probe every few hundred nanoseconds (waiting roles then cost no issue slots).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}

// Wall-clock budget of one wait.  A healthy pipeline waits microseconds; two
// seconds means something upstream will never arrive.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait.  Returns false when the limit ran out or another role already
// raised *abort_flag (a word in shared memory); the caller then leaves its
// loop and the kernel tears down in an orderly way.  abort_flag[1], when not
// zero, is the limit in microseconds (tests shorten it).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_hint(bar, parity, 100000u)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag != 0u) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      const uint32_t lim_us = abort_flag[1];
      if (now - t0 > (lim_us ? static_cast<uint64_t>(lim_us) * 1000ull : kWaitLimitNs)) {
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// global -> shared tile load, completion reported on `bar` (same CTA).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *tmap, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Same, for a CTA pair: `bar` may be the leader CTA's barrier (shared::cluster
// address) while `dst` is this CTA's own shared memory.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void *tmap, uint32_t bar,
                                                 int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// L2 eviction policy for TMA traffic (createpolicy): 1 = evict_first (data read
// or written once), 2 = evict_last (data other CTAs will come back for).
// (0 = evict_normal, for the tensor without a hint when another one has one.)
__device__ __forceinline__ uint64_t make_l2_policy(int kind) {
  uint64_t pol;
  if (kind == 2)
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  else if (kind == 1)
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  else
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// The loads above with an L2 cache hint.
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const void *tmap, uint32_t bar,
                                                 int x, int y, int z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z),
        "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair_hint(uint32_t dst, const void *tmap, uint32_t bar,
                                                      int x, int y, int z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z),
        "l"(policy)
      : "memory");
}

// shared -> global tile store (bulk async-group completion); clips at the
// tensor's bounds.
__device__ __forceinline__ void tma_store_3d(const void *tmap, uint32_t src, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_store_3d_hint(const void *tmap, uint32_t src, int x, int y,
                                                  int z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;"
      :
      : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Waits until at most N committed store groups still READ their shared-memory
// source (the hardware bounds this wait: stores always drain).
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// --------------------------------------------------------------- cluster

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cta address of this CTA -> shared::cluster address of the same
// offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// --------------------------------------------------------------- tcgen05

template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result),
                 "r"(ncols)
                 : "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] . B[smem desc] with an f32 accumulator.  KIND 0:
// kind::f16 (f16 / bf16 operands), 1: kind::tf32 (f32 operands, upper 19 bits),
// 2: kind::f8f6f4 (fp8 operands).  Issued by ONE thread.
#define KAPYB_UMMA_ASM(GROUP, KINDSTR)                                                     \
  asm volatile(                                                                            \
      "{\n\t"                                                                              \
      ".reg .pred p;\n\t"                                                                  \
      "setp.ne.b32 p, %4, 0;\n\t"                                                          \
      "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], %1, %2, %3, p;\n\t"        \
      "}\n"                                                                                 \
      :                                                                                    \
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)                 \
      : "memory")

template <int CTAS>
__device__ __forceinline__ void umma(int kind, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                     uint32_t idesc, uint32_t accumulate) {
  if constexpr (CTAS == 1) {
    if (kind == 0)
      KAPYB_UMMA_ASM("1", "f16");
    else if (kind == 1)
      KAPYB_UMMA_ASM("1", "tf32");
    else
      KAPYB_UMMA_ASM("1", "f8f6f4");
  } else {
    if (kind == 0)
      KAPYB_UMMA_ASM("2", "f16");
    else if (kind == 1)
      KAPYB_UMMA_ASM("2", "tf32");
    else
      KAPYB_UMMA_ASM("2", "f8f6f4");
  }
}

// Same with the kind fixed at compile time (the main loop's form).
template <int CTAS, int KIND>
__device__ __forceinline__ void umma_k(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  if constexpr (CTAS == 1) {
    if constexpr (KIND == 0)
      KAPYB_UMMA_ASM("1", "f16");
    else if constexpr (KIND == 1)
      KAPYB_UMMA_ASM("1", "tf32");
    else
      KAPYB_UMMA_ASM("1", "f8f6f4");
  } else {
    if constexpr (KIND == 0)
      KAPYB_UMMA_ASM("2", "f16");
    else if constexpr (KIND == 1)
      KAPYB_UMMA_ASM("2", "tf32");
    else
      KAPYB_UMMA_ASM("2", "f8f6f4");
  }
}

template <int CTAS>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  umma<CTAS>(0, d_tmem, a_desc, b_desc, idesc, accumulate);
}

// Makes `bar` (a shared::cluster address; a plain shared::cta address names
// this CTA's own barrier) complete once every MMA this thread issued so far
// has finished.  Implies tcgen05.fence::before_thread_sync.
template <int CTAS>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                     "r"(bar)
                 : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                     "r"(bar)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row
// (lane base + i), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
        "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The reverse of tmem_ld_32x32: thread i of the warp writes row (lane base + i),
// columns [col, col+32).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
        "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
        "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Flag words in global memory that one CTA sets and another polls.
__device__ __forceinline__ void st_release_gpu(uint32_t *p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ----------------------------------------------------------- descriptors

// Shared-memory matrix descriptor (tcgen05), SWIZZLE_128B:
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1
//   bits [61,64) layout type: 2 = 128-byte swizzle in 16-byte units, 1 = 128-byte
//   swizzle in 32-byte units (the only layout an MN-major 32-bit operand may use)
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes,
                                                         uint32_t layout_type = 2) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(layout_type) << 61;
  return d;
}

// Instruction descriptor with an f32 accumulator:
//   [4,6) D format (1 = f32)  [7,10) A format  [10,13) B format
//   [15] A major (0 = K, 1 = MN)  [16] B major  [17,23) N >> 3  [24,29) M >> 4
// Operand format codes: kind::f16 0 = f16, 1 = bf16; kind::tf32 2 = tf32;
// kind::f8f6f4 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t make_idesc(int a_fmt, int b_fmt, int a_mn_major,
                                                  int b_mn_major, int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
         (static_cast<uint32_t>(a_mn_major ? 1 : 0) << 15) |
         (static_cast<uint32_t>(b_mn_major ? 1 : 0) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__host__ __device__ constexpr uint32_t make_idesc_f16(int bf16, int a_mn_major, int b_mn_major,
                                                      int m, int n) {
  return make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, a_mn_major, b_mn_major, m, n);
}

}  // namespace ptx
}  // namespace kapyb
