// Decode-shape matmul (few rows of activations against a large weight matrix):
// HBM-bound weight streaming.  The operands are swapped so the weights fill the
// 128-row side of tcgen05.mma and the activations its narrow side:
//   D[n, m] = sum_k W[k, n] * X[m, k]      (instruction shape 128 x M_pad x 16)
// The (weight tile, k block) units are dealt to the CTAs as equal contiguous
// spans ("stream-K"), so all SMs stream the same number of bytes whatever the
// tile count.  A tile that is split between CTAs is accumulated with fp32
// atomics in scratch memory; the last contributor applies the epilogue, writes
// the output and leaves the scratch zeroed for the next launch.
//
// Same arithmetic contract as the big-tile kernel (fp32 accumulation of exact
// products, fused epilogue), but a split tile sums its spans in arrival order.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace kapyb {

constexpr int kSkinnyMaxM = 64;
constexpr int kSkinnyThreads = 192;
constexpr int kSkinnyMaxStages = 12;
constexpr int kSkinnyCounterBytes = 64 * 1024;  // 4 counters per weight tile
constexpr size_t kSkinnyScratchBytes = 16u << 20;

struct SkinnyParams {
  int M, N, K;
  int m_pad;      // M rounded up to 16: the MMA's N extent
  int num_kb;     // ceil(K / 64)
  int n_tiles;    // ceil(N / 128)
  int span;       // k-block units per CTA
  int stages;
  int w_mn_major;  // weights N-contiguous ([K,N] row-major)
  int x_mn_major;  // activations M-contiguous
  int x_bytes;     // shared-memory bytes of one activation stage
  int tmem_cols;
  int out_dtype;
  long long c_s0, c_s1;
  void *c;
  float *scratch;      // [n_tiles][m_pad][128] fp32, zero between launches
  uint32_t *counters;  // [n_tiles][4], zero between launches
  uint32_t idesc;
  uint32_t *status;
  uint32_t wait_limit_us;  // 0: the default limit of a bounded wait
  EpilogueArgs ep;
};

__device__ __forceinline__ void skinny_finish(const SkinnyParams &p, int n, int m, float v) {
  v *= p.ep.alpha;
  if (p.ep.bias != nullptr) v += load_as_f32(p.ep.bias, p.ep.bias_dtype, p.ep.bias_axis == 1 ? n : m);
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmW);
    ptx::prefetch_tensormap(&tmX);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(ptx::smem_u32(tmem_slot), p.tmem_cols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const long long total = static_cast<long long>(p.n_tiles) * p.num_kb;
  const long long g_begin = static_cast<long long>(blockIdx.x) * p.span;
  const long long g_end = min(total, g_begin + p.span);

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    const uint32_t stage_bytes = W_BYTES + p.x_bytes;
    for (long long g = g_begin; g < g_end; ++g) {
      const int tile = static_cast<int>(g / p.num_kb);
      const int kb = static_cast<int>(g - static_cast<long long>(tile) * p.num_kb);
      if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) break;
      const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
      ptx::mbar_arrive_expect_tx(fb, stage_bytes);
      const int k0 = kb * 64, n0 = tile * 128;
      const uint32_t w_dst = ptx::smem_u32(sW + stage * W_BYTES);
      const uint32_t x_dst = ptx::smem_u32(sX + stage * p.x_bytes);
      if (p.w_mn_major) {
        ptx::tma_load_3d(w_dst, &tmW, fb, n0, k0, 0);
        ptx::tma_load_3d(w_dst + 8192, &tmW, fb, n0 + 64, k0, 0);
      } else {
        ptx::tma_load_3d(w_dst, &tmW, fb, k0, n0, 0);
      }
      if (p.x_mn_major)
        ptx::tma_load_3d(x_dst, &tmX, fb, 0, k0, 0);
      else
        ptx::tma_load_3d(x_dst, &tmX, fb, k0, 0, 0);
      if (++stage == p.stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------- MMA issuer
    const uint32_t w_lbo = p.w_mn_major ? 8192u : 16u, w_kadv = p.w_mn_major ? 2048u : 32u;
    const uint32_t x_lbo = p.x_mn_major ? 8192u : 16u, x_kadv = p.x_mn_major ? 2048u : 32u;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    long long g = g_begin;
    while (g < g_end && ok) {
      const int tile = static_cast<int>(g / p.num_kb);
      const int kb_begin = static_cast<int>(g - static_cast<long long>(tile) * p.num_kb);
      const int kb_end = static_cast<int>(min(static_cast<long long>(p.num_kb), kb_begin + (g_end - g)));
      if (!ptx::mbar_wait(ptx::smem_u32(&tempty_bar[acc]), acc_phase ^ 1u, abort_flag)) break;
      ptx::tc_fence_after();
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.m_pad);
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t w_base = ptx::smem_u32(sW + stage * W_BYTES);
        const uint32_t x_base = ptx::smem_u32(sX + stage * p.x_bytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t wdesc = ptx::make_smem_desc_sw128(w_base + k * w_kadv, w_lbo, 1024u);
          const uint64_t xdesc = ptx::make_smem_desc_sw128(x_base + k * x_kadv, x_lbo, 1024u);
          ptx::umma_f16<1>(d_tmem, wdesc, xdesc, p.idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
        }
        ptx::umma_commit<1>(ptx::smem_u32(&empty_bar[stage]));
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      ptx::umma_commit<1>(ptx::smem_u32(&tfull_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
      g += kb_end - kb_begin;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    long long g = g_begin;
    while (g < g_end) {
      const int tile = static_cast<int>(g / p.num_kb);
      const int kb_begin = static_cast<int>(g - static_cast<long long>(tile) * p.num_kb);
      const int kb_end = static_cast<int>(min(static_cast<long long>(p.num_kb), kb_begin + (g_end - g)));
      if (!ptx::mbar_wait(ptx::smem_u32(&tfull_bar[acc]), acc_phase, abort_flag)) break;
      ptx::tc_fence_after();
      const bool whole = kb_begin == 0 && kb_end == p.num_kb;
      const int n = tile * 128 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(acc * p.m_pad);
      float *scr = p.scratch + (static_cast<long long>(tile) * p.m_pad) * 128 + q * 32 + lane;
      for (int mc = 0; mc < p.m_pad; mc += 16) {
        uint32_t v[16];
        ptx::tmem_ld_32x16(t_row + static_cast<uint32_t>(mc), v);
        ptx::tmem_ld_wait();
        if (whole) {
          if (n < p.N) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (mc + i < p.M) skinny_finish(p, n, mc + i, __uint_as_float(v[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (mc + i < p.M) atomicAdd(scr + (mc + i) * 128, __uint_as_float(v[i]));
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tempty_bar[acc]));
      if (!whole) {
        // Publish this span's partial sums, then count it.  The contributor that
        // completes the count owns the tile quarter: it reads the total, applies
        // the epilogue and restores the zeros.
        const long long t0 = static_cast<long long>(tile) * p.num_kb;
        const int first = static_cast<int>(t0 / p.span);
        const int last = static_cast<int>((t0 + p.num_kb - 1) / p.span);
        const uint32_t expected = static_cast<uint32_t>(last - first + 1);
        __threadfence();
        __syncwarp();
        uint32_t seen = 0;
        if (lane == 0) seen = atomicAdd(p.counters + tile * 4 + q, 1u);
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (seen == expected - 1) {
          __threadfence();
          for (int m = 0; m < p.M; ++m) {
            const float s = __ldcg(scr + m * 128);
            __stcg(scr + m * 128, 0.0f);
            if (n < p.N) skinny_finish(p, n, m, s);
          }
          __syncwarp();
          if (lane == 0) atomicExch(p.counters + tile * 4 + q, 0u);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
      g += kb_end - kb_begin;
    }
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
