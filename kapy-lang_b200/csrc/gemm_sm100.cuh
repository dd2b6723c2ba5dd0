// Persistent warp-specialised GEMM for sm_100a:
//   TMA (cp.async.bulk.tensor, per-CTA loads only) -> 128-byte-swizzled shared
//   memory ring -> tcgen05.mma with fp32 accumulators in TMEM (two accumulator
//   slots, so the epilogue of tile i overlaps the main loop of tile i+1) ->
//   tcgen05.ld -> fused epilogue (alpha, bias, addend, activation, downcast)
//   -> swizzled staging -> TMA store.
//
// Replaces the schedule the reference spells out by hand in
// test/Conversion/KapyToKgpu/matmul.mlir:46-128 (2-stage cp.async ring, ldmatrix,
// mma.sync m16n8k8 chain, MatmulOpToLLVM.cpp:58-266) at whole-problem scope.
//
// Warp roles: warp 0 = TMA producer (one lane), warp 1 = TMEM allocator + MMA
// issuer (one lane), warps 2 .. 2+EPI-1 = epilogue (warp w may touch TMEM lanes
// 32*(w%4) .. +31; with EPI = 8 two warps share a lane quarter and alternate
// column chunks, for problems whose K loop is too short to hide the epilogue).
//
// CTAS == 2 pairs two CTAs of a cluster on one 256-row tile
// (tcgen05.mma.cta_group::2): each CTA loads its own 128 rows of A and its own
// half of the B columns; only the leader CTA (cluster rank 0) issues MMAs.  The
// pair shares no loads, so no multicast is involved.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace kapyb {

constexpr int kMaxOutputs = 8;  // own output + up to 7 peers for the push epilogue

struct TmapArray {
  CUtensorMap m[kMaxOutputs];
};

struct GemmParams {
  int M, N, K, batch;
  int tiles_m, tiles_n;  // tile grid of one batch entry
  int num_tiles;         // tiles_m * tiles_n * batch
  int num_kb;            // ceil(K / 64)
  int group_m;           // rasterisation: tiles_m are walked in groups of this many
  int a_mn_major;        // 1: lhs is column-major (M contiguous)
  int b_mn_major;        // 1: rhs is row-major [K,N] (N contiguous)
  int out_dtype;
  int n_out;             // number of output tensor maps (1, or n_peers for push)
  int out_col_offset;    // column offset of this shard inside each output
  uint32_t idesc;
  uint32_t *status;
  int debug;  // profiling aid (results are garbage): bit0 skip loads, bit1 skip MMAs,
              // bit2 skip the epilogue body, bit3 skip only the TMA stores
  EpilogueArgs ep;
};

template <int BN, int CTAS, int EPI = 4>
struct GemmCfg {
  static constexpr int BM = 128;  // rows per CTA (TMEM lanes)
  static constexpr int BK = 64;   // 128 bytes of a 16-bit type: one swizzle span
  static constexpr int TILE_M = BM * CTAS;
  static constexpr int BN_CTA = BN / CTAS;  // B columns this CTA loads
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN_CTA * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // 32-row x 128-byte staging buffers per epilogue warp: two, except where eight
  // warps and 48 KB stages leave room for one only
  static constexpr int C_BUFS = (BN == 512 && EPI == 8) ? 1 : 2;
  static constexpr int C_WARP_BYTES = C_BUFS * 4096;
  static constexpr int C_BYTES = EPI * C_WARP_BYTES;
  static constexpr int THREADS = 64 + 32 * EPI;  // producer warp, MMA warp, EPI epilogue warps
  static constexpr int CTRL_BYTES = 1024;
  static constexpr int SMEM_LIMIT = 232448;  // 227 KB opt-in maximum
  static constexpr int STAGES_RAW = (SMEM_LIMIT - 1024 - CTRL_BYTES - C_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + C_BYTES + CTRL_BYTES;
  // BN = 512 (CTA pairs only): the tile is two 256-column halves that share the A
  // stage, each with its own accumulator; together they fill TMEM, so the two
  // slots hold the halves of ONE tile instead of two tiles in flight.  That cuts
  // the operand bytes pulled from L2 per flop by a quarter.
  static constexpr int HALVES = BN == 512 ? 2 : 1;
  static constexpr int MMA_N = BN / HALVES;
  static constexpr int TMEM_COLS = HALVES == 2 ? 512 : (2 * BN < 32 ? 32 : 2 * BN);
  static_assert(BN % 64 == 0 && (BN <= 256 || (BN == 512 && CTAS == 2)),
                "BN must be 64, 128, 256, or 512 for CTA pairs");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");
  static_assert(STAGES >= 2, "pipeline too shallow");
  static_assert(EPI == 4 || EPI == 8, "4 or 8 epilogue warps");
};

// Linear tile index -> (batch, m block, n block); m blocks are walked in groups
// so that concurrently running CTAs share A rows and B columns in L2.
__device__ __forceinline__ void decode_tile(const GemmParams &p, int tile, int &b, int &mb,
                                            int &nb) {
  const int per_batch = p.tiles_m * p.tiles_n;
  b = tile / per_batch;
  const int r = tile - b * per_batch;
  const int in_group = p.group_m * p.tiles_n;
  const int g = r / in_group;
  const int first_m = g * p.group_m;
  const int gsize = min(p.group_m, p.tiles_m - first_m);
  const int rr = r - g * in_group;
  mb = first_m + rr % gsize;
  nb = rr / gsize;
}

// 32 finished columns of one row -> the row's slot in the swizzled staging tile.
__device__ __forceinline__ void stage_half_f32(uint8_t *srow, const float (&f)[32], int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 w = make_uint4(__float_as_uint(f[4 * j]), __float_as_uint(f[4 * j + 1]),
                               __float_as_uint(f[4 * j + 2]), __float_as_uint(f[4 * j + 3]));
    *reinterpret_cast<uint4 *>(srow + ((j ^ (lane & 7)) << 4)) = w;
  }
}

template <int DT, int RN>
__device__ __forceinline__ void stage_half_16(uint8_t *srow, const float (&f)[32], int lane,
                                              int h) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 w;
    w.x = cvt_pack2_t<DT, RN>(f[8 * j], f[8 * j + 1]);
    w.y = cvt_pack2_t<DT, RN>(f[8 * j + 2], f[8 * j + 3]);
    w.z = cvt_pack2_t<DT, RN>(f[8 * j + 4], f[8 * j + 5]);
    w.w = cvt_pack2_t<DT, RN>(f[8 * j + 6], f[8 * j + 7]);
    const int jj = h * 4 + j;
    *reinterpret_cast<uint4 *>(srow + ((jj ^ (lane & 7)) << 4)) = w;
  }
}

// f[0..32) += 32 consecutive 16-bit bias values read with uniform 128-bit loads.
template <int DT>
__device__ __forceinline__ void add_bias32(float (&f)[32], const uint4 *bp) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 w = __ldg(bp + j);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float lo, hi;
      unpack2_16<DT>(ws[t], lo, hi);
      f[8 * j + 2 * t] += lo;
      f[8 * j + 2 * t + 1] += hi;
    }
  }
}

// What one epilogue warp needs to drain its share of one accumulator tile.
struct EpiTile {
  int b, m0, n0, row, lane, cpart;
  int col_begin, col_end;  // tile columns to drain in this call (one accumulator slot)
  uint32_t tempty_addr;    // barrier that returns the slot to the MMA thread
  bool remote_arrive;      // the barrier lives in the pair's leader CTA
  uint32_t t_row;   // TMEM address of this warp's lanes at tile column 0
  uint8_t *stg;     // this warp's two 4 KB staging buffers
  bool bias_col, bias_fast;
  float bias_row;
};

// OUTK: 0 f32, 1/2 bf16 rn/rz, 3/4 f16 rn/rz.  PLAIN: the epilogue is only the
// scale (no bias, addend or activation), so none of those are even tested.
// Returns whether the slot was handed back (false when this warp had no chunk).
template <int BN, int EPI, int OUTK, bool PLAIN>
__device__ __forceinline__ bool epilogue_tile(const GemmParams &p, const TmapArray &tmC,
                                              const EpiTile &t, int &buf) {
  constexpr bool OUT32 = OUTK == 0;
  constexpr int CW = OUT32 ? 32 : 64;  // output columns per 128-byte staging row
  constexpr int NH = CW / 32;
  constexpr int CSTEP = EPI / 4;
  constexpr int C_BUFS = (BN == 512 && EPI == 8) ? 1 : 2;
  const int lane = t.lane;
  bool handed_back = false;
  for (int c = t.col_begin / CW + t.cpart; c < t.col_end / CW; c += CSTEP) {
    const int nc = t.n0 + c * CW;
    if (nc >= p.N) break;
    uint8_t *sbuf = t.stg + (C_BUFS == 2 ? buf : 0) * 4096;
    // All loads of the chunk are in flight before the one wait.
    uint32_t v[NH][32];
#pragma unroll
    for (int h = 0; h < NH; ++h)
      ptx::tmem_ld_32x32(t.t_row + static_cast<uint32_t>(c * CW + h * 32), v[h]);
    // The store that last read this buffer (two chunks ago, or the previous one
    // with a single buffer) must have finished reading it.
    if (lane == 0) ptx::tma_store_wait_read<C_BUFS - 1>();
    __syncwarp();
    ptx::tmem_ld_wait();
    if (c + CSTEP >= t.col_end / CW || t.n0 + (c + CSTEP) * CW >= p.N) {
      // That was this warp's last read of the slot: hand it back now, so the next
      // tile's MMAs do not wait for the arithmetic and the stores below.
      handed_back = true;
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (t.remote_arrive)
          ptx::mbar_arrive_cluster(t.tempty_addr);
        else
          ptx::mbar_arrive(t.tempty_addr);
      }
    }
    uint8_t *srow = sbuf + lane * 128;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      const int col0 = nc + h * 32;
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[h][i]);
      if (p.ep.alpha != 1.0f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] *= p.ep.alpha;
      }
      if constexpr (!PLAIN) {
        if (t.bias_col) {
          if (t.bias_fast && col0 + 32 <= p.N) {
            const uint4 *bp =
                reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.ep.bias) + col0);
            if (p.ep.bias_dtype == KAPYB_BF16)
              add_bias32<KAPYB_BF16>(f, bp);
            else
              add_bias32<KAPYB_F16>(f, bp);
          } else {
            float bias_lane = 0.0f;
            if (col0 + lane < p.N) bias_lane = load_as_f32(p.ep.bias, p.ep.bias_dtype, col0 + lane);
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] += __shfl_sync(0xffffffffu, bias_lane, i);
          }
        } else if (p.ep.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] += t.bias_row;
        }
        if (p.ep.acc != nullptr && t.row < p.M) {
          const long long base = static_cast<long long>(t.b) * p.ep.acc_batch_stride +
                                 static_cast<long long>(t.row) * p.ep.acc_stride0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N)
              f[i] += load_as_f32(p.ep.acc, p.ep.acc_dtype,
                                  base + static_cast<long long>(col0 + i) * p.ep.acc_stride1);
        }
        if (p.ep.activation != KAPYB_ACT_NONE) {
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = apply_activation(p.ep.activation, f[i]);
        }
      }
      // Row `lane` of the staging tile, 128-byte swizzle: 16-byte chunk j of row
      // r lives at chunk position j ^ (r & 7).
      if constexpr (OUTK == 0) stage_half_f32(srow, f, lane);
      if constexpr (OUTK == 1) stage_half_16<KAPYB_BF16, 1>(srow, f, lane, h);
      if constexpr (OUTK == 2) stage_half_16<KAPYB_BF16, 0>(srow, f, lane, h);
      if constexpr (OUTK == 3) stage_half_16<KAPYB_F16, 1>(srow, f, lane, h);
      if constexpr (OUTK == 4) stage_half_16<KAPYB_F16, 0>(srow, f, lane, h);
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && !(p.debug & 8)) {
      for (int o = 0; o < p.n_out; ++o)
        ptx::tma_store_3d(&tmC.m[o], ptx::smem_u32(sbuf), p.out_col_offset + nc, t.m0, t.b);
      ptx::tma_store_commit();
    }
    buf ^= 1;
  }
  return handed_back;
}

template <int BN, int CTAS, int EPI>
__global__ void __launch_bounds__(64 + 32 * EPI, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ TmapArray tmC, const GemmParams p) {
  using Cfg = GemmCfg<BN, CTAS, EPI>;
  constexpr int STAGES = Cfg::STAGES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t *sA = smem;
  uint8_t *sB = sA + STAGES * Cfg::A_BYTES;
  uint8_t *sC = sB + STAGES * Cfg::B_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(sC + Cfg::C_BYTES);
  uint64_t *full_bar = bars;                 // [STAGES]
  uint64_t *empty_bar = bars + STAGES;       // [STAGES]
  uint64_t *tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t *tempty_bar = tfull_bar + 2;      // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty_bar + 2);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;
  const int unit = CTAS == 2 ? (blockIdx.x >> 1) : blockIdx.x;      // CTA (pair) index
  const int unit_step = CTAS == 2 ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);     // the (leader's) expect_tx arrival
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);    // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&tfull_bar[a]), 1);          // one tcgen05.commit
      ptx::mbar_init(ptx::smem_u32(&tempty_bar[a]), EPI * CTAS);  // one arrival per epilogue warp
    }
    *abort_flag = 0u;
    ptx::fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    ptx::prefetch_tensormap(&tmC.m[0]);
  }
  if (warp == 1) {
    ptx::tmem_alloc<CTAS>(ptx::smem_u32(tmem_slot), Cfg::TMEM_COLS);
    ptx::tmem_relinquish<CTAS>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = unit; tile < p.num_tiles && ok; tile += unit_step) {
      int b, mb, nb;
      decode_tile(p, tile, b, mb, nb);
      const int m0 = mb * Cfg::TILE_M + static_cast<int>(rank) * Cfg::BM;
      // first B column this CTA loads; with two halves its columns are two groups
      // of MMA_N / CTAS, one per half
      const int nB0 = nb * BN + static_cast<int>(rank) * (Cfg::MMA_N / CTAS);
      constexpr int kGroupCols = Cfg::MMA_N / CTAS;   // columns per half this CTA owns
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const int k0 = kb * Cfg::BK;
        const uint32_t a_dst = ptx::smem_u32(sA + stage * Cfg::A_BYTES);
        const uint32_t b_dst = ptx::smem_u32(sB + stage * Cfg::B_BYTES);
        if (p.debug & 1) {
          if (rank == 0) ptx::mbar_arrive(ptx::smem_u32(&full_bar[stage]));
        } else if constexpr (CTAS == 1) {
          const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
          ptx::mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
          if (!p.a_mn_major) {
            ptx::tma_load_3d(a_dst, &tmA, fb, k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::BM / 64; ++j)
              ptx::tma_load_3d(a_dst + j * 8192, &tmA, fb, m0 + 64 * j, k0, b);
          }
          if (!p.b_mn_major) {
            ptx::tma_load_3d(b_dst, &tmB, fb, k0, nB0, b);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::BN_CTA / 64; ++j)
              ptx::tma_load_3d(b_dst + j * 8192, &tmB, fb, nB0 + 64 * j, k0, b);
          }
          (void)kGroupCols;
        } else {
          // Both CTAs' loads report their bytes to the leader's barrier; the
          // leader alone posts the arrival, expecting the bytes of both.  (A
          // remote arrive.expect_tx from the peer instead halves the throughput.)
          const uint32_t fb = ptx::mapa(ptx::smem_u32(&full_bar[stage]), 0);
          if (rank == 0)
            ptx::mbar_arrive_expect_tx(ptx::smem_u32(&full_bar[stage]), 2 * Cfg::STAGE_BYTES);
          if (!p.a_mn_major) {
            ptx::tma_load_3d_pair(a_dst, &tmA, fb, k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::BM / 64; ++j)
              ptx::tma_load_3d_pair(a_dst + j * 8192, &tmA, fb, m0 + 64 * j, k0, b);
          }
          if (!p.b_mn_major) {
            // one box of kGroupCols rows per half
#pragma unroll
            for (int hh = 0; hh < Cfg::HALVES; ++hh)
              ptx::tma_load_3d_pair(b_dst + hh * (kGroupCols * 128), &tmB, fb, k0,
                                    nB0 + hh * Cfg::MMA_N, b);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::BN_CTA / 64; ++j) {
              const int hh = (j * 64) / kGroupCols, within = (j * 64) % kGroupCols;
              ptx::tma_load_3d_pair(b_dst + j * 8192, &tmB, fb, nB0 + hh * Cfg::MMA_N + within,
                                    k0, b);
            }
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------------------------------------------------- MMA issuer
    // K-major operand: rows are 128 bytes, 8-row groups 1024 bytes apart; one
    // UMMA K step (16 elements) is 32 bytes along the row.
    // MN-major operand: 64-element (128-byte) MN chunks 8192 bytes apart, K
    // rows 128 bytes apart in groups of 8 (1024 bytes); one K step is 16 rows.
    const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, a_sbo = 1024u;
    const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u, b_sbo = 1024u;
    const uint32_t a_kadv = p.a_mn_major ? 2048u : 32u;
    const uint32_t b_kadv = p.b_mn_major ? 2048u : 32u;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = unit; tile < p.num_tiles && ok; tile += unit_step) {
      if constexpr (Cfg::HALVES == 2) {
        // both halves of the previous tile must have been drained
        if (!ptx::mbar_wait(ptx::smem_u32(&tempty_bar[0]), acc_phase ^ 1u, abort_flag)) break;
        if (!ptx::mbar_wait(ptx::smem_u32(&tempty_bar[1]), acc_phase ^ 1u, abort_flag)) break;
      } else {
        if (!ptx::mbar_wait(ptx::smem_u32(&tempty_bar[acc]), acc_phase ^ 1u, abort_flag)) break;
      }
      ptx::tc_fence_after();
      const uint32_t d_tmem =
          tmem_base + (Cfg::HALVES == 2 ? 0u : static_cast<uint32_t>(acc * BN));
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t a_base = ptx::smem_u32(sA + stage * Cfg::A_BYTES);
        const uint32_t b_base = ptx::smem_u32(sB + stage * Cfg::B_BYTES);
        if (!(p.debug & 2)) {
#pragma unroll
          for (int k = 0; k < Cfg::BK / 16; ++k) {
            const uint64_t adesc = ptx::make_smem_desc_sw128(a_base + k * a_kadv, a_lbo, a_sbo);
#pragma unroll
            for (int hh = 0; hh < Cfg::HALVES; ++hh) {
              // this CTA's B bytes of half hh start (MMA_N / CTAS) rows of 128 bytes
              // after those of half hh-1, in either layout
              const uint32_t b_half = b_base + hh * (Cfg::MMA_N / CTAS) * 128;
              const uint64_t bdesc = ptx::make_smem_desc_sw128(b_half + k * b_kadv, b_lbo, b_sbo);
              ptx::umma_f16<CTAS>(d_tmem + hh * Cfg::MMA_N, adesc, bdesc, p.idesc,
                                  (kb | k) != 0 ? 1u : 0u);
            }
          }
        }
        // Free the stage in every CTA that filled it.
        ptx::umma_commit<CTAS>(ptx::smem_u32(&empty_bar[stage]));
        if constexpr (CTAS == 2)
          ptx::umma_commit<CTAS>(ptx::mapa(ptx::smem_u32(&empty_bar[stage]), 1));
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      if constexpr (Cfg::HALVES == 2) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          ptx::umma_commit<CTAS>(ptx::smem_u32(&tfull_bar[hh]));
          ptx::umma_commit<CTAS>(ptx::mapa(ptx::smem_u32(&tfull_bar[hh]), 1));
        }
        acc_phase ^= 1u;
      } else {
        ptx::umma_commit<CTAS>(ptx::smem_u32(&tfull_bar[acc]));
        if constexpr (CTAS == 2)
          ptx::umma_commit<CTAS>(ptx::mapa(ptx::smem_u32(&tfull_bar[acc]), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ epilogue
    const int e = warp - 2;          // epilogue warp index, 0 .. EPI-1
    const int q = warp & 3;          // TMEM lane quarter this warp may touch
    const int cpart = e >> 2;        // with 8 epilogue warps two warps share a quarter
                                     //   and take alternate column chunks
    uint8_t *stg = sC + e * Cfg::C_WARP_BYTES;
    const bool out32 = p.out_dtype == KAPYB_F32;
    // 0: f32; 1/2: bf16 rn/rz; 3/4: f16 rn/rz -- picked once, outside the loops
    const int out_kind = out32 ? 0
                         : (p.out_dtype == KAPYB_BF16 ? (p.ep.rounding ? 1 : 2)
                                                      : (p.ep.rounding ? 3 : 4));
    const uint32_t tempty_leader = CTAS == 2 ? ptx::mapa(ptx::smem_u32(&tempty_bar[0]), 0)
                                             : ptx::smem_u32(&tempty_bar[0]);
    const bool bias_col = p.ep.bias != nullptr && p.ep.bias_axis == 1;
    // 16-bit bias vectors that start on a 16-byte boundary are read with uniform
    // 128-bit loads; anything else goes through one load per lane and shuffles.
    const bool bias_fast = bias_col && p.ep.bias_dtype != KAPYB_F32 &&
                           (reinterpret_cast<uintptr_t>(p.ep.bias) & 15u) == 0;
    // "plain": nothing but the scale between the accumulator and the downcast
    const bool plain = p.ep.bias == nullptr && p.ep.acc == nullptr &&
                       p.ep.activation == KAPYB_ACT_NONE;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    for (int tile = unit; tile < p.num_tiles; tile += unit_step) {
      int b, mb, nb;
      decode_tile(p, tile, b, mb, nb);
      const int m0 = mb * Cfg::TILE_M + static_cast<int>(rank) * Cfg::BM + q * 32;
      const int n0 = nb * BN;
      const int row = m0 + lane;
      bool alive = true;
#pragma unroll 1
      for (int hh = 0; hh < Cfg::HALVES; ++hh) {
        // slot: with two halves, half hh of this tile; otherwise the tile's slot
        const int slot = Cfg::HALVES == 2 ? hh : acc;
        if (!ptx::mbar_wait(ptx::smem_u32(&tfull_bar[slot]), acc_phase, abort_flag)) {
          alive = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                               (Cfg::HALVES == 2 ? 0u : static_cast<uint32_t>(acc * BN));
        bool handed_back = false;
        const uint32_t slot_bar = tempty_leader + static_cast<uint32_t>(slot * 8);
        if (m0 < p.M && !(p.debug & 4)) {
          EpiTile et;
          et.tempty_addr = slot_bar;
          et.remote_arrive = CTAS == 2;
          et.b = b;
          et.m0 = m0;
          et.n0 = n0;
          et.row = row;
          et.lane = lane;
          et.t_row = t_row;
          et.cpart = cpart;
          et.col_begin = hh * Cfg::MMA_N;
          et.col_end = (hh + 1) * Cfg::MMA_N;
          et.stg = stg;
          et.bias_col = bias_col;
          et.bias_fast = bias_fast;
          et.bias_row = 0.0f;
          if (p.ep.bias != nullptr && p.ep.bias_axis == 0 && row < p.M)
            et.bias_row = load_as_f32(p.ep.bias, p.ep.bias_dtype, row);
          // One specialised copy of the chunk loop per (output kind, plain/full
          // epilogue): the switch runs once per slot, the loops inside are tight.
          switch (out_kind * 2 + (plain ? 1 : 0)) {
          case 0: handed_back = epilogue_tile<BN, EPI, 0, false>(p, tmC, et, buf); break;
          case 1: handed_back = epilogue_tile<BN, EPI, 0, true>(p, tmC, et, buf); break;
          case 2: handed_back = epilogue_tile<BN, EPI, 1, false>(p, tmC, et, buf); break;
          case 3: handed_back = epilogue_tile<BN, EPI, 1, true>(p, tmC, et, buf); break;
          case 4: handed_back = epilogue_tile<BN, EPI, 2, false>(p, tmC, et, buf); break;
          case 5: handed_back = epilogue_tile<BN, EPI, 2, true>(p, tmC, et, buf); break;
          case 6: handed_back = epilogue_tile<BN, EPI, 3, false>(p, tmC, et, buf); break;
          case 7: handed_back = epilogue_tile<BN, EPI, 3, true>(p, tmC, et, buf); break;
          case 8: handed_back = epilogue_tile<BN, EPI, 4, false>(p, tmC, et, buf); break;
          default: handed_back = epilogue_tile<BN, EPI, 4, true>(p, tmC, et, buf); break;
          }
        }
        if (!handed_back) {
          // nothing was read (rows or columns outside the problem): return the slot
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTAS == 2)
              ptx::mbar_arrive_cluster(slot_bar);
            else
              ptx::mbar_arrive(slot_bar);
          }
        }
      }
      if (!alive) break;
      if constexpr (Cfg::HALVES == 2) {
        acc_phase ^= 1u;
      } else {
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    if (lane == 0) ptx::tma_store_wait_all<0>();
    __syncwarp();
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusTimeout);
    // Give loads that are still in flight time to land before the shared
    // memory they target is released.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if constexpr (CTAS == 2) {
    // The peer may still address this CTA's barriers / shared memory.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace kapyb
