// Decode-shape matmul (few rows of activations against a large weight matrix):
// HBM-bound weight streaming.  The operands are swapped so the weights fill the
// 128-row side of tcgen05.mma and the activations its narrow side:
//   D[n, m] = sum_k W[k, n] * X[m, k]      (instruction shape 128 x M_pad x 16)
// Whole weight tiles go round-robin to the CTAs while they fill the GPU evenly;
// the (tile, k block) units of the leftover tiles are dealt out as equal
// contiguous spans ("stream-K"), so all SMs stream the same number of bytes
// whatever the tile count.  A tile that is split between CTAs goes through
// scratch memory without a counter, a fence or an atomic: every contributor but
// the first writes its partial sums as (value, launch number) pairs, one 8-byte
// store each, into its own slot; the FIRST contributor of the tile (whose span
// ends with the tile, so it is among the last to finish) reads the others'
// pairs until each carries this launch's number, adds them to its own
// accumulator IN CTA ORDER, applies the epilogue and writes the output.  A pair
// is written in one piece, so a reader sees either an older launch's pair and
// tries again, or the value.  The critical path after the last MMA is one L2
// round trip and the output stores (the counter scheme it replaces needed
// four round trips, 5-6 us of a 17 us launch when every tile is split).
// Nothing in the scratch has to be zero or reset between launches: launch
// numbers only grow.
//
// Same arithmetic contract as the big-tile kernel (fp32 accumulation of exact
// products, fused epilogue).  Because a split tile's slots are added in CTA
// order, not arrival order, the result is the same bits from run to run.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace kapyb {

#ifdef KAPYB_DEBUG_SWITCHES
constexpr int kSkinnyDebugMask = 0xff;
#else
constexpr int kSkinnyDebugMask = 128;
#endif
template <int BITS>
__device__ __forceinline__ bool skinny_debug_on(int debug) {
  if constexpr ((kSkinnyDebugMask & BITS) == 0)
    return false;
  else
    return (debug & (kSkinnyDebugMask & BITS)) != 0;
}

constexpr int kSkinnyMaxM = 64;
constexpr int kSkinnyThreads = 192;
constexpr int kSkinnyMaxStages = 12;   // barrier slots; see kSkinnyStages for the depth used
// Pipeline depth actually used.  Measured on the decode shape (M = 16, N = 28672,
// K = 8192): 12 stages stream 5.89 TB/s, 8 stages 6.28 TB/s, 6 stages 6.16 TB/s;
// the same optimum at M = 1 .. 64 and for narrower shards.  More bytes in flight
// than the memory system needs only scatter its accesses.
constexpr int kSkinnyStages = 8;
constexpr size_t kSkinnyScratchBytes = 16u << 20;

struct SkinnyParams {
  int M, N, K;
  int m_pad;      // M rounded up to 16: the MMA's N extent
  int num_kb;     // ceil(K / 64)
  int n_tiles;    // ceil(N / 128)
  int span;       // k-block units of the split region per CTA
  int sk_tiles;   // the first sk_tiles weight tiles are split between CTAs ...
  int dp_per_cta; // ... the rest are whole tiles, up to this many per CTA (tile = sk_tiles + cta +
                  // i * grid while that is < n_tiles: the last round may be ragged)
  int stages;
  int w_mn_major;  // weights N-contiguous ([K,N] row-major)
  int x_mn_major;  // activations M-contiguous
  int x_bytes;     // shared-memory bytes of one activation stage
  int tmem_cols;
  int out_dtype;
  long long c_s0, c_s1;
  void *c;
  uint2 *scratch;      // [grid][m_pad][128] (fp32 partial sum, launch number): one slot per CTA
  uint32_t epoch;      // this launch's number: never 0, different from any number still in scratch
  uint32_t idesc;
  uint32_t *status;
  uint32_t wait_limit_us;  // 0: the default limit of a bounded wait
  int debug;               // bit7: record the timeline probes in status[2..8] (results stay
                           // right).  Only in a build with -DKAPYB_DEBUG_SWITCHES, for
                           // profiling (results are wrong): bit1 skip the MMAs, bit2 skip the epilogue body,
                           // bit3 skip the publish/count/owner pass, bit4 skip whole-tile
                           // stores, bit5 skip the partial-sum stores
  EpilogueArgs ep;
  int w_l2, x_l2;  // L2 policy of the weight / activation tile loads: 0 default, 1 evict_first, 2 evict_last
};

// The work of one CTA, as a list of per-tile segments.  The first `sk_tiles`
// weight tiles form the split region: their (tile, k-block) units are dealt out
// as equal contiguous spans, so a CTA's share is up to two partial tiles (and
// whole ones between them when spans are long).  The remaining tiles are whole
// and go round-robin, `dp_per_cta` to each CTA.  The split region comes FIRST:
// its publish / count / owner round trips then hide under the whole tiles' main
// loops instead of forming the kernel's tail.
struct SkinnyWork {
  int first_tile, n_split_segs, head_kb, tail_kb, num_kb;
  int dp_first, dp_stride, dp_count;
  __device__ SkinnyWork(long long g_begin, long long g_end, int num_kb_, int sk_tiles, int dp_per_cta,
                        int n_tiles)
      : num_kb(num_kb_) {
    first_tile = static_cast<int>(g_begin / num_kb);
    const int last_tile = g_end > g_begin ? static_cast<int>((g_end - 1) / num_kb) : first_tile;
    n_split_segs = g_end > g_begin ? last_tile - first_tile + 1 : 0;
    head_kb = static_cast<int>(g_begin - static_cast<long long>(first_tile) * num_kb);
    tail_kb = static_cast<int>(g_end - static_cast<long long>(last_tile) * num_kb);
    dp_first = sk_tiles + static_cast<int>(blockIdx.x);
    dp_stride = static_cast<int>(gridDim.x);
    dp_count = 0;
    for (int i = 0; i < dp_per_cta; ++i)
      if (dp_first + i * dp_stride < n_tiles) dp_count = i + 1;
  }
  __device__ int count() const { return n_split_segs + dp_count; }
  // j-th segment in processing order
  __device__ void get(int j, int &tile, int &kb_begin, int &kb_end) const {
    if (j < n_split_segs) {
      tile = first_tile + j;
      kb_begin = j == 0 ? head_kb : 0;
      kb_end = j == n_split_segs - 1 ? tail_kb : num_kb;
    } else {
      tile = dp_first + (j - n_split_segs) * dp_stride;
      kb_begin = 0;
      kb_end = num_kb;
    }
  }
};

// Sixteen finished rows of one output column, the common epilogue (scale and an
// optional per-column bias, 16-bit output rounded to nearest): a multiply-add, a
// conversion and a store per element.  One warp per scheduler runs this, so every
// instruction saved comes off the kernel's tail.
template <int DT, int ACT = KAPYB_ACT_NONE>
__device__ __forceinline__ void skinny_store16(uint16_t *col, long long row_stride, int rows,
                                               const float (&v)[16], float alpha, float bias_n) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (i < rows) {
      const float r = apply_activation_t<ACT>(fmaf(v[i], alpha, bias_n));
      col[i * row_stride] = static_cast<uint16_t>(cvt_pack2_t<DT, 1>(r, 0.0f) & 0xffffu);
    }
  }
}

// The same with the activation picked once per 16 values.
template <int DT>
__device__ __forceinline__ void skinny_store16_act(int act, uint16_t *col, long long row_stride,
                                                   int rows, const float (&v)[16], float alpha,
                                                   float bias_n) {
  switch (act) {
  case KAPYB_ACT_RELU: skinny_store16<DT, KAPYB_ACT_RELU>(col, row_stride, rows, v, alpha, bias_n); break;
  case KAPYB_ACT_GELU_TANH: skinny_store16<DT, KAPYB_ACT_GELU_TANH>(col, row_stride, rows, v, alpha, bias_n); break;
  case KAPYB_ACT_SILU: skinny_store16<DT, KAPYB_ACT_SILU>(col, row_stride, rows, v, alpha, bias_n); break;
  default: skinny_store16<DT>(col, row_stride, rows, v, alpha, bias_n); break;
  }
}

// Epilogue of one output element.  `bias_n` is the per-column bias of column n,
// fetched once per tile by the caller (0 when the bias runs along rows or is absent).
__device__ __forceinline__ void skinny_finish(const SkinnyParams &p, int n, int m, float v,
                                              float bias_n) {
  v = v * p.ep.alpha + bias_n;
  if (p.ep.bias != nullptr && p.ep.bias_axis != 1) v += load_as_f32(p.ep.bias, p.ep.bias_dtype, m);
  if (p.ep.acc != nullptr)
    v += load_as_f32(p.ep.acc, p.ep.acc_dtype, m * p.ep.acc_stride0 + n * p.ep.acc_stride1);
  v = apply_activation(p.ep.activation, v);
  store_from_f32(p.c, p.out_dtype, m * p.c_s0 + n * p.c_s1, v, p.ep.rounding);
}

__global__ void __launch_bounds__(kSkinnyThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr int W_BYTES = 128 * 64 * 2;
  uint8_t *sW = smem;
  uint8_t *sX = sW + p.stages * W_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sX + p.stages * p.x_bytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + kSkinnyMaxStages;
  uint64_t *tfull_bar = bars + 2 * kSkinnyMaxStages;
  uint64_t *tempty_bar = tfull_bar + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty_bar + 2);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  // the shuffle makes the warp index provably uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const bool probe = skinny_debug_on<128>(p.debug);
  if (probe && threadIdx.x == 0) {
    const uint32_t t = static_cast<uint32_t>(ptx::globaltimer_ns());
    atomicMax(p.status + 4, ~t);  // earliest start, kept as the largest complement
    atomicMax(p.status + 5, t);   // latest start
  }
  const long long total = static_cast<long long>(p.sk_tiles) * p.num_kb;  // units of the split region
  const long long g_begin = min(total, static_cast<long long>(blockIdx.x) * p.span);
  const long long g_end = min(total, g_begin + p.span);
  const SkinnyWork work(g_begin, g_end, p.num_kb, p.sk_tiles, p.dp_per_cta, p.n_tiles);
  constexpr uint32_t kWBytes = 128 * 64 * 2;

  // One stage's loads: a 128-column x 64-k weight tile and the activations of the same
  // k block (plain form, or with the tensors' L2 policies when HINTED).
  auto issue_stage = [&](auto hinted, int st, int tile, int kb, uint64_t pol_w, uint64_t pol_x) {
    constexpr bool HINTED = decltype(hinted)::value;
    (void)pol_w;
    (void)pol_x;
#define KAPYB_LOAD1(POL, DST, TM, BAR, X, Y)                       \
  do {                                                             \
    if constexpr (HINTED)                                          \
      ptx::tma_load_3d_hint(DST, &TM, BAR, X, Y, 0, POL);          \
    else                                                           \
      ptx::tma_load_3d(DST, &TM, BAR, X, Y, 0);                    \
  } while (0)
    const uint32_t fb = ptx::smem_u32(&full_bar[st]);
    ptx::mbar_arrive_expect_tx(fb, kWBytes + p.x_bytes);
    const int k0 = kb * 64, n0 = tile * 128;
    const uint32_t w_dst = ptx::smem_u32(sW + st * kWBytes);
    const uint32_t x_dst = ptx::smem_u32(sX + st * p.x_bytes);
    if (p.w_mn_major) {
      KAPYB_LOAD1(pol_w, w_dst, tmW, fb, n0, k0);
      KAPYB_LOAD1(pol_w, w_dst + 8192, tmW, fb, n0 + 64, k0);
    } else {
      KAPYB_LOAD1(pol_w, w_dst, tmW, fb, k0, n0);
    }
    if (p.x_mn_major)
      KAPYB_LOAD1(pol_x, x_dst, tmX, fb, 0, k0);
    else
      KAPYB_LOAD1(pol_x, x_dst, tmX, fb, k0, 0);
#undef KAPYB_LOAD1
  };

  // Thread 0 sets the barriers up and, without waiting for the rest of the CTA
  // (TMEM allocation, the CTA-wide barrier), already fills the pipeline: the first
  // bytes are then on their way a microsecond earlier, which is most of what a
  // short launch has to lose.  The producer loop below carries on after them.
  int prefilled = 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&tfull_bar[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&tempty_bar[a]), 4);
    }
    abort_flag[0] = 0u;
    abort_flag[1] = p.wait_limit_us;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmW);
    ptx::prefetch_tensormap(&tmX);
    // nothing above touched global memory; the loads below do
    ptx::griddep_wait();
    const bool hinted = (p.w_l2 | p.x_l2) != 0;
    const uint64_t pol_w = hinted ? ptx::make_l2_policy(p.w_l2) : 0ull;
    const uint64_t pol_x = hinted ? ptx::make_l2_policy(p.x_l2) : 0ull;
    for (int j = 0; j < work.count() && prefilled < p.stages; ++j) {
      int tile, kb_begin, kb_end;
      work.get(j, tile, kb_begin, kb_end);
      for (int kb = kb_begin; kb < kb_end && prefilled < p.stages; ++kb, ++prefilled) {
        if (hinted)
          issue_stage(std::true_type{}, prefilled, tile, kb, pol_w, pol_x);
        else
          issue_stage(std::false_type{}, prefilled, tile, kb, 0ull, 0ull);
      }
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(ptx::smem_u32(tmem_slot), p.tmem_cols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // let the next kernel of the stream start its own set-up; every thread that reads
  // global memory first waits for the kernels ahead (see gemm_tcgen05_kernel)
  ptx::griddep_launch();
  ptx::griddep_wait();

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    // Two copies of the loop, plain loads and loads with an L2 policy per tensor: see
    // the producer of gemm_tcgen05_kernel.  The first `prefilled` k blocks are
    // already in flight.
    int stage = prefilled == p.stages ? 0 : prefilled;
    uint32_t phase = prefilled == p.stages ? 1u : 0u;
    bool ok = true;
    auto produce = [&](auto hinted) {
      constexpr bool HINTED = decltype(hinted)::value;
      const uint64_t pol_w = HINTED ? ptx::make_l2_policy(p.w_l2) : 0ull;
      const uint64_t pol_x = HINTED ? ptx::make_l2_policy(p.x_l2) : 0ull;
      int skip = prefilled;
      for (int j = 0; j < work.count() && ok; ++j) {
        int tile, kb_begin, kb_end;
        work.get(j, tile, kb_begin, kb_end);
        if (skip > 0) {
          const int d = min(skip, kb_end - kb_begin);
          kb_begin += d;
          skip -= d;
        }
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          issue_stage(hinted, stage, tile, kb, pol_w, pol_x);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    };
    if (p.w_l2 | p.x_l2)
      produce(std::true_type{});
    else
      produce(std::false_type{});
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // The whole warp walks the loops in step and one elected lane issues (uniform
    // control flow keeps the descriptor arithmetic in uniform registers); every
    // wait ends in a vote, so the lanes never part ways, not even on a time-out.
    auto wait_all = [&](uint32_t bar, uint32_t parity) {
      const bool mine = ptx::mbar_wait(bar, parity, abort_flag);
      return __all_sync(0xffffffffu, mine) != 0;
    };
    // Descriptor constants folded up front; a K step is one add on the low word
    // (the issuing thread must keep pace with a 16 KB stage every few hundred ns).
    const uint32_t w_lbo = p.w_mn_major ? 8192u : 16u, w_kstep = (p.w_mn_major ? 2048u : 32u) >> 4;
    const uint32_t x_lbo = p.x_mn_major ? 8192u : 16u, x_kstep = (p.x_mn_major ? 2048u : 32u) >> 4;
    const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version 1, 128B swizzle
    const uint32_t w_lo0 = ((w_lbo >> 4) << 16) | (ptx::smem_u32(sW) >> 4);
    const uint32_t x_lo0 = ((x_lbo >> 4) << 16) | (ptx::smem_u32(sX) >> 4);
    const uint32_t x_stage_step = static_cast<uint32_t>(p.x_bytes) >> 4;
    const uint32_t idesc = p.idesc;
    bool seen_first = false;
    const long long probe_c0 = clock64();
    const uint64_t probe_t0 = ptx::globaltimer_ns();
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int j = 0; j < work.count() && ok; ++j) {
      int tile, kb_begin, kb_end;
      work.get(j, tile, kb_begin, kb_end);
      (void)tile;
      if (!wait_all(ptx::smem_u32(&tempty_bar[acc]), acc_phase ^ 1u)) break;
      ptx::tc_fence_after();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.m_pad);
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!wait_all(ptx::smem_u32(&full_bar[stage]), phase)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        if (probe && !seen_first) {
          seen_first = true;
          if (lane == 0) atomicMax(p.status + 6, static_cast<uint32_t>(ptx::globaltimer_ns()));
        }
        const uint32_t w_lo = w_lo0 + static_cast<uint32_t>(stage) * (W_BYTES >> 4);
        const uint32_t x_lo = x_lo0 + static_cast<uint32_t>(stage) * x_stage_step;
        const uint32_t first = kb > kb_begin ? 1u : 0u;
        if (ptx::elect_one()) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (skinny_debug_on<2>(p.debug)) break;  // (debug builds) stream without multiplying
            const uint64_t wdesc = (static_cast<uint64_t>(desc_hi) << 32) | (w_lo + k * w_kstep);
            const uint64_t xdesc = (static_cast<uint64_t>(desc_hi) << 32) | (x_lo + k * x_kstep);
            ptx::umma_k<1, 0>(d_tmem, wdesc, xdesc, idesc, k == 0 ? first : 1u);
          }
          ptx::umma_commit<1>(ptx::smem_u32(&empty_bar[stage]));
        }
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      if (ptx::elect_one()) ptx::umma_commit<1>(ptx::smem_u32(&tfull_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (probe && lane == 0) {
      atomicMax(p.status + 7, static_cast<uint32_t>(ptx::globaltimer_ns()));
      if (blockIdx.x == 0) {
        p.status[2] = static_cast<uint32_t>(clock64() - probe_c0);
        p.status[3] = static_cast<uint32_t>(ptx::globaltimer_ns() - probe_t0);
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    // scale, optional per-column bias and activation into a 16-bit output, rounded to nearest
    const bool fast16 = p.ep.acc == nullptr &&
                        (p.ep.bias == nullptr || p.ep.bias_axis == 1) &&
                        p.out_dtype != KAPYB_F32 && p.ep.rounding == KAPYB_RN;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    for (int j = 0; j < work.count() && alive; ++j) {
      int tile, kb_begin, kb_end;
      work.get(j, tile, kb_begin, kb_end);
      // warp vote after the wait: the lanes leave together or not at all (what
      // follows is warp-collective)
      if (!__all_sync(0xffffffffu,
                      ptx::mbar_wait(ptx::smem_u32(&tfull_bar[acc]), acc_phase, abort_flag)))
        break;
      ptx::tc_fence_after();
      const bool whole = kb_begin == 0 && kb_end == p.num_kb;
      // A split tile is finished by its first contributor (the segment that starts
      // the tile); every other contributor publishes its partial sums.
      const bool owner = !whole && kb_begin == 0;
      const int n = tile * 128 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * p.m_pad);
      const long long t0 = static_cast<long long>(tile) * p.num_kb;
      // contributors of a split tile: CTAs first .. last, this one included
      const int first = whole ? 0 : static_cast<int>(t0 / p.span);
      const int last = whole ? 0 : static_cast<int>((t0 + p.num_kb - 1) / p.span);
      auto slot_of = [&](int c) {
        return p.scratch + (static_cast<long long>(c) * p.m_pad) * 128 + q * 32 + lane;
      };
      float bias_n = 0.0f;
      if (p.ep.bias != nullptr && p.ep.bias_axis == 1 && n < p.N)
        bias_n = load_as_f32(p.ep.bias, p.ep.bias_dtype, n);
      uint16_t *col16 = static_cast<uint16_t *>(p.c) + n * p.c_s1;
      for (int mc = 0; mc < p.m_pad && alive && !skinny_debug_on<4>(p.debug); mc += 16) {
        uint32_t v[16];
        ptx::tmem_ld_32x16(t_row + static_cast<uint32_t>(mc), v);
        ptx::tmem_ld_wait();
        if (!whole && !owner) {
          // publish: one 8-byte store per element, the value and this launch's number
          if (!skinny_debug_on<32>(p.debug)) {
            uint2 *scr = slot_of(static_cast<int>(blockIdx.x));
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (mc + i < p.M) __stcg(scr + (mc + i) * 128, make_uint2(v[i], p.epoch));
          }
          continue;
        }
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(v[i]);
        if (owner && !skinny_debug_on<8>(p.debug)) {
          // Add the other contributors' rows mc .. mc+15, two slots per batch: all 32
          // loads of a batch are issued before anything looks at them (one L2 round
          // trip per batch), then every pair must carry this launch's number, else
          // the batch is read again.  CTA order: own sums first, then first+1, ...
          constexpr int CB = 2;
          for (int c = first + 1; c <= last && alive; c += CB) {
            uint2 part[CB][16];
            uint64_t spin_t0 = 0;
            for (uint32_t it = 1;; ++it) {
              // every round reads memory afresh (other CTAs are writing it)
              asm volatile("" ::: "memory");
#pragma unroll
              for (int bb = 0; bb < CB; ++bb) {
                const bool have = c + bb <= last;
                const uint2 *src = slot_of(have ? c + bb : c);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  part[bb][i] = (have && mc + i < p.M) ? __ldcg(src + (mc + i) * 128)   // L2, never L1
                                                       : make_uint2(0u, p.epoch);
              }
              bool good = true;
#pragma unroll
              for (int bb = 0; bb < CB; ++bb)
#pragma unroll
                for (int i = 0; i < 16; ++i) good = good && part[bb][i].y == p.epoch;
              if (__all_sync(0xffffffffu, good)) break;
              // bounded: give up like any other wait of this kernel
              bool give_up = false;
              if ((it & 15u) == 0u) {
                if (*abort_flag != 0u) {
                  give_up = true;
                } else {
                  const uint64_t now = ptx::globaltimer_ns();
                  if (spin_t0 == 0) spin_t0 = now;
                  const uint32_t lim_us = abort_flag[1];
                  if (now - spin_t0 > (lim_us ? static_cast<uint64_t>(lim_us) * 1000ull : ptx::kWaitLimitNs)) {
                    *abort_flag = 1u;
                    give_up = true;
                  }
                }
              }
              if (__any_sync(0xffffffffu, give_up)) {
                alive = false;
                break;
              }
              __nanosleep(100);
            }
            if (!alive) break;
#pragma unroll
            for (int bb = 0; bb < CB; ++bb)
#pragma unroll
              for (int i = 0; i < 16; ++i) f[i] += __uint_as_float(part[bb][i].x);
          }
          if (!alive) break;
        }
        if (n < p.N && !skinny_debug_on<16>(p.debug)) {
          if (fast16) {
            if (p.out_dtype == KAPYB_BF16)
              skinny_store16_act<KAPYB_BF16>(p.ep.activation, col16 + mc * p.c_s0, p.c_s0, p.M - mc, f,
                                             p.ep.alpha, bias_n);
            else
              skinny_store16_act<KAPYB_F16>(p.ep.activation, col16 + mc * p.c_s0, p.c_s0, p.M - mc, f,
                                            p.ep.alpha, bias_n);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (mc + i < p.M) skinny_finish(p, n, mc + i, f[i], bias_n);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (probe && lane == 0) atomicMax(p.status + 8, static_cast<uint32_t>(ptx::globaltimer_ns()));
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusTimeout);
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, p.tmem_cols);
  }
}

}  // namespace kapyb
