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
// issuer (the whole warp walks the loops in step, one elected lane issues, so the
// descriptor arithmetic stays in uniform registers), warps 2 .. 2+EPI-1 =
// epilogue (warp w may touch TMEM lanes 32*(w%4) .. +31; with EPI = 8 two warps
// share a lane quarter and alternate column chunks, for problems whose K loop is
// too short to hide the epilogue).
//
// Operand kinds: kind::f16 (f16 / bf16), kind::tf32 (f32 operands) and
// kind::f8f6f4 (f8E4M3 / f8E5M2) share the kernel: a shared-memory row is always
// 128 bytes and a K step 32 bytes, whatever the element width.
//
// 512-wide tiles (pairs only) hold two 256-column halves that fill TMEM; the MMA
// role skews the halves at tile boundaries and the epilogue drains them through
// registers (see epilogue_two_halves and the MMA role below).  The drain is
// instruction-bound, so it is compiled per output type (the kernel's DRAIN
// parameter), and a CTA's last tile stages its stores through the operand ring.
//
// CTAS == 2 pairs two CTAs of a cluster on one 256-row tile
// (tcgen05.mma.cta_group::2): each CTA loads its own 128 rows of A and its own
// half of the B columns; only the leader CTA (cluster rank 0) issues MMAs.  The
// pair shares no loads, so no multicast is involved.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace kapyb {

constexpr int kMaxOutputs = 8;  // own output + up to 7 peers for the push epilogue

// Debug switches (GemmParams::debug).  Bits 0-3 and 5 make a kernel skip part of
// its work, so its results are garbage: they exist for profiling only and are
// compiled in only with -DKAPYB_DEBUG_SWITCHES, together with the per-phase
// clock probes of the epilogue warps.  A normal build keeps bit 4 (the producer
// stays silent, so that every other role's bounded wait runs out: the test of the
// time-out path) and bit 7 (timeline and clock probes of the MMA warp; results
// stay right), and neither costs the epilogue warps a register.
#ifdef KAPYB_DEBUG_SWITCHES
constexpr int kDebugMask = 0xff;
constexpr bool kEpilogueProbes = true;
#else
constexpr int kDebugMask = 16 | 128;
constexpr bool kEpilogueProbes = false;
#endif
template <int BITS>
__device__ __forceinline__ bool debug_on(int debug) {
  if constexpr ((kDebugMask & BITS) == 0)
    return false;
  else
    return (debug & (kDebugMask & BITS)) != 0;
}

struct TmapArray {
  CUtensorMap m[kMaxOutputs];
};

// Division by a launch-time constant as a multiply-high and a shift (exact for
// dividends below 2^31): mul = ceil(2^(31 + ceil(log2 d)) / d), shr = ceil(log2 d) - 1.
struct FastDiv {
  uint32_t mul, shr, d;
  static FastDiv make(uint32_t d) {  // host side
    FastDiv f{0u, 0u, d};
    if (d > 1) {
      uint32_t l = 0;
      while ((1ull << l) < d) ++l;
      const uint32_t p = 31 + l;
      f.mul = static_cast<uint32_t>(((1ull << p) + d - 1) / d);
      f.shr = p - 32;
    }
    return f;
  }
  __device__ __forceinline__ int div(int n) const {
    return d == 1 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shr);
  }
};

struct GemmParams {
  int M, N, K, batch;
  int tiles_m, tiles_n;  // tile grid of one batch entry
  int num_tiles;         // tiles_m * tiles_n * batch
  int num_kb;            // ceil(K / 64)
  int group_m;           // rasterisation: tiles_m are walked in groups of this many
  FastDiv div_per_batch, div_in_group, div_group_m, div_last_group;  // decode_tile's divisors:
                         // tiles_m * tiles_n, group_m * tiles_n, group_m, max(1, tiles_m % group_m)
  int a_mn_major;        // 1: lhs is column-major (M contiguous)
  int b_mn_major;        // 1: rhs is row-major [K,N] (N contiguous)
  int out_dtype;
  int n_out;             // number of output tensor maps (1, or n_peers for push)
  int out_col_offset;    // column offset of this shard inside each output
  uint32_t idesc;
  // Operand element width: a shared-memory row is always 128 bytes, so the K
  // extent of a stage and of a 128-byte MN chunk is 128 / size elements.
  int kind;            // tcgen05.mma kind: 0 f16/bf16, 1 tf32, 2 fp8
  int bk_elems;        // K elements per stage: 64 (16-bit), 32 (f32), 128 (fp8)
  uint32_t mn_lbo;     // bytes of one MN-major chunk: bk_elems rows x 128 bytes
  uint32_t mn_kadv;    // bytes one MMA K step (32 bytes of K) advances in an MN-major tile
  uint32_t mn_sbo;     // bytes between K-row groups of an MN-major tile: 8 rows (1024), or
                       // 4 rows (512) in the 32-byte-unit swizzle 32-bit operands need
  uint32_t mn_layout;  // descriptor layout type of an MN-major tile: 2, or 1 for 32-bit operands
  uint32_t *status;
  uint32_t wait_limit_us;  // 0: the default limit of a bounded wait
  int debug;  // profiling aid (results are garbage): bit0 skip loads, bit1 skip MMAs,
              // bit2 skip the epilogue body, bit3 skip only the TMA stores,
              // bit4 the producer never loads nor signals (every other role's wait
              // then runs out: the test of the time-out path),
              // bit5 free-running MMAs over whatever shared memory holds (no producer,
              // no stage barriers): an issue-rate probe,
              // bit7 the first CTA's MMA thread records cycles and nanoseconds of its
              // tile loop in status[2], status[3]; status[4..8] collect over all CTAs
              // (timer low words): complement of the earliest start, latest start,
              // latest first stage, latest last MMA issue, latest epilogue end; status[9..13]:
              // clocks the first CTA's first epilogue warp spent, summed over its chunks,
              // waiting for its staging buffer, for the accumulator loads, in arithmetic +
              // staging, issuing the store, and (per tile) waiting for the accumulator;
              // status[14], [15]: clocks the first CTA's MMA warp waited for operand stages
              // and for accumulator slots
  EpilogueArgs ep;
  // kapy.reduce fused after the epilogue (REDUCE instantiations only): the f32
  // values the epilogue produces, before the downcast, are also summed along
  // red_axis (1: over the columns, one sum per row; 0: over the rows, one per
  // column) into the zero-initialised vector `red` with fp32 atomics.
  float *red;
  int red_axis;
  // L2 policy of the TMA traffic per tensor (from the descriptors' eviction
  // priority): 0 default, 1 evict_first, 2 evict_last
  int a_l2, b_l2, c_l2;
  // 1: the addend (ep.acc) has the output's type and a TMA-describable layout; its
  // tensor map sits in the last slot of the output maps and the epilogue fetches it
  // tile by tile into the staging buffer.  0: element by element (any type, any strides).
  int acc_tma;
  // SPLIT instantiations only.  Tiles below sk_first_tile are dealt to the CTAs
  // (pairs) whole, round-robin; the K blocks of the tiles from there on, sk_total in
  // all, are dealt out as one contiguous span per CTA (pair), so a last wave that
  // would fill only part of the GPU keeps all of it busy.  A CTA whose span starts
  // inside a tile leaves its fp32 partial accumulator in its slot of sk_scratch
  // ([CTA][128 x BN] floats) and sets its warps' words of sk_flags to sk_epoch, the
  // number of this launch; the CTA that did the tile's first K blocks adds the
  // partial sums to its own in CTA order (the same bits on every run) and runs the
  // epilogue.
  int sk_first_tile, sk_total;
  float *sk_scratch;
  uint32_t *sk_flags;
  uint32_t sk_epoch;
};

// First K block (in the numbering that runs through all split tiles) of CTA (pair)
// `unit` of `units`.
__device__ __forceinline__ int sk_span_begin(const GemmParams &p, int unit, int units) {
  return static_cast<int>(static_cast<long long>(unit) * p.sk_total / units);
}

// The work of one CTA (pair), item by item: tile `tile`, K blocks [kb0, kb1).
template <bool SK>
struct WorkIter {
  int tile, kb0, kb1;
  int next_tile, step, lin, lin_end;
  __device__ __forceinline__ WorkIter(const GemmParams &p, int unit, int units)
      : tile(0), kb0(0), kb1(p.num_kb), next_tile(unit), step(units), lin(0), lin_end(0) {
    if constexpr (SK) {
      lin = sk_span_begin(p, unit, units);
      lin_end = sk_span_begin(p, unit + 1, units);
    }
  }
  // after next() returned true: whether that item is this CTA's last
  __device__ __forceinline__ bool last(const GemmParams &p) const {
    if constexpr (!SK)
      return next_tile >= p.num_tiles;
    else
      return next_tile >= p.sk_first_tile && lin >= lin_end;
  }
  __device__ __forceinline__ bool next(const GemmParams &p) {
    if constexpr (!SK) {
      tile = next_tile;
      next_tile += step;
      return tile < p.num_tiles;
    } else {
      if (next_tile < p.sk_first_tile) {
        tile = next_tile;
        next_tile += step;
        kb0 = 0;
        kb1 = p.num_kb;
        return true;
      }
      if (lin >= lin_end) return false;
      const int t = lin / p.num_kb;
      kb0 = lin - t * p.num_kb;
      kb1 = min(p.num_kb, kb0 + (lin_end - lin));
      tile = p.sk_first_tile + t;
      lin += kb1 - kb0;
      return true;
    }
  }
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
  // warps and 48 KB stages leave room for one only (the 512-wide pair tile), or
  // where one buffer buys a fourth stage (256-wide single-CTA tiles with eight
  // epilogue warps: the short-K shapes, whose main loop is load latency)
  static constexpr int C_BUFS = ((BN == 512 || (BN == 256 && CTAS == 1)) && EPI == 8) ? 1 : 2;
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
  static constexpr int SLOT_COLS = BN / HALVES;  // accumulator columns behind one tfull/tempty pair
  // Column groups a K step is issued in, one MMA each (the two halves of a 512-wide
  // tile; splitting 256-wide tiles into 2 x 128 was measured slower: 54 % of the
  // pipe's peak against 76 % for one 256-wide MMA per step).
  static constexpr int SPLIT = BN == 512 ? 2 : 1;
  static constexpr int MMA_N = BN / SPLIT;
  static constexpr int TMEM_COLS = HALVES == 2 ? 512 : (2 * BN < 32 ? 32 : 2 * BN);
  static_assert(BN % 64 == 0 && (BN <= 256 || (BN == 512 && CTAS == 2)),
                "BN must be 64, 128, 256, or 512 for CTA pairs");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");
  static_assert(STAGES >= 2, "pipeline too shallow");
  static_assert(EPI == 4 || EPI == 8, "4 or 8 epilogue warps");
};

// Linear tile index -> (batch, m block, n block); m blocks are walked in groups
// so that concurrently running CTAs share A rows and B columns in L2.  Every
// role of every CTA runs this once per tile, so its divisions are FastDivs.
__device__ __forceinline__ void decode_tile(const GemmParams &p, int tile, int &b, int &mb,
                                            int &nb) {
  b = p.div_per_batch.div(tile);
  const int r = tile - b * static_cast<int>(p.div_per_batch.d);
  const int g = p.div_in_group.div(r);
  const int first_m = g * p.group_m;
  const int rr = r - g * static_cast<int>(p.div_in_group.d);
  // every group has group_m row blocks but the last, which has the remainder
  const bool last = first_m + p.group_m > p.tiles_m;
  nb = last ? p.div_last_group.div(rr) : p.div_group_m.div(rr);
  mb = first_m + rr - nb * (last ? static_cast<int>(p.div_last_group.d) : p.group_m);
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
  // A 16-bit column bias fetched before the accumulator was awaited (so its latency
  // hides behind the main loop): lane l holds the eight values of tile columns
  // 8 l .. 8 l + 7; the pieces pick theirs up by shuffle.  Kernels with four epilogue
  // warps and one accumulator per tile (a warp then drains up to 256 adjacent columns).
  bool bias_lanes;
  uint4 bias8;      // eight 16-bit values, or the first four of eight f32 values
  uint4 bias8_hi;   // f32 bias: the other four
  volatile uint32_t *abort_flag;
  uint32_t *prof;   // profiling (debug bit 7, one warp of the first CTA): shared words that
                    // collect clocks spent per phase of the chunk loop; else nullptr
};

// The fused arithmetic on 32 consecutive accumulator columns of one row
// (columns col0 .. col0+31 of row t.row): scale, bias, addend, activation.
// LEVEL 0: scale only; 1: scale and bias; 2: scale, bias, addend, activation.
// `acc_srow` (ACCK >= 0): this lane's row of the addend tile in the staging buffer
// (128-byte swizzle), piece `acc_h` of it; ACCK 0 f32, 1 bf16, 2 f16.
template <int LEVEL, bool REDUCE = false, int ACCK = -1>
__device__ __forceinline__ void finish32(const GemmParams &p, const EpiTile &t, float (&f)[32],
                                         int col0, const uint8_t *acc_srow = nullptr, int acc_h = 0) {
  const int lane = t.lane;
  if (p.ep.alpha != 1.0f) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] *= p.ep.alpha;
  }
  if constexpr (LEVEL >= 1) {
    if (t.bias_col) {
      if (t.bias_lanes && p.ep.bias_dtype == KAPYB_F32) {
        const int src0 = (col0 - t.n0) >> 3;  // the lane that holds the piece's first eight values
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          f[8 * jj + 0] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8.x, src0 + jj));
          f[8 * jj + 1] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8.y, src0 + jj));
          f[8 * jj + 2] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8.z, src0 + jj));
          f[8 * jj + 3] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8.w, src0 + jj));
          f[8 * jj + 4] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8_hi.x, src0 + jj));
          f[8 * jj + 5] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8_hi.y, src0 + jj));
          f[8 * jj + 6] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8_hi.z, src0 + jj));
          f[8 * jj + 7] += __uint_as_float(__shfl_sync(0xffffffffu, t.bias8_hi.w, src0 + jj));
        }
      } else if (t.bias_lanes) {
        const int src0 = (col0 - t.n0) >> 3;  // the lane that holds the piece's first eight values
        const bool bf16 = p.ep.bias_dtype == KAPYB_BF16;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const uint32_t ws[4] = {__shfl_sync(0xffffffffu, t.bias8.x, src0 + jj),
                                  __shfl_sync(0xffffffffu, t.bias8.y, src0 + jj),
                                  __shfl_sync(0xffffffffu, t.bias8.z, src0 + jj),
                                  __shfl_sync(0xffffffffu, t.bias8.w, src0 + jj)};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float lo, hi;
            if (bf16)
              unpack2_16<KAPYB_BF16>(ws[e], lo, hi);
            else
              unpack2_16<KAPYB_F16>(ws[e], lo, hi);
            f[8 * jj + 2 * e] += lo;
            f[8 * jj + 2 * e + 1] += hi;
          }
        }
      } else if (t.bias_fast && col0 + 32 <= p.N) {
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
  }
  if constexpr (LEVEL >= 2) {
    if (ACCK >= 0 && acc_srow != nullptr) {
      if constexpr (ACCK == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 q = *reinterpret_cast<const uint4 *>(acc_srow + ((j ^ (lane & 7)) << 4));
          f[4 * j] += __uint_as_float(q.x);
          f[4 * j + 1] += __uint_as_float(q.y);
          f[4 * j + 2] += __uint_as_float(q.z);
          f[4 * j + 3] += __uint_as_float(q.w);
        }
      } else if constexpr (ACCK > 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 q = *reinterpret_cast<const uint4 *>(acc_srow + (((acc_h * 4 + j) ^ (lane & 7)) << 4));
          const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float lo, hi;
            unpack2_16<ACCK == 1 ? KAPYB_BF16 : KAPYB_F16>(ws[e], lo, hi);
            f[8 * j + 2 * e] += lo;
            f[8 * j + 2 * e + 1] += hi;
          }
        }
      }
    } else if (p.ep.acc != nullptr && t.row < p.M) {
      const long long base = static_cast<long long>(t.b) * p.ep.acc_batch_stride +
                             static_cast<long long>(t.row) * p.ep.acc_stride0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N)
          f[i] += load_as_f32(p.ep.acc, p.ep.acc_dtype,
                              base + static_cast<long long>(col0 + i) * p.ep.acc_stride1);
    }
    // one branch per 32 values: with the choice inside the unrolled loop a fused
    // relu made a 4096 x 4096 x 1024 product three times slower
    switch (p.ep.activation) {
    case KAPYB_ACT_RELU:
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = apply_activation_t<KAPYB_ACT_RELU>(f[i]);
      break;
    case KAPYB_ACT_GELU_TANH:
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = apply_activation_t<KAPYB_ACT_GELU_TANH>(f[i]);
      break;
    case KAPYB_ACT_SILU:
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = apply_activation_t<KAPYB_ACT_SILU>(f[i]);
      break;
    default:
      break;
    }
  }
  if constexpr (REDUCE) {
    // Lane l holds row t.row, columns col0 .. col0+31.  Rows and columns outside
    // the problem hold the products of TMA's zero fill plus bias: leave them out.
    const bool row_ok = t.row < p.M;
    if (p.red_axis == 1) {
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) s += f[i];
      if (row_ok) atomicAdd(p.red + t.row, s);
    } else {
      float mine = 0.0f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float v = row_ok ? f[i] : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == i) mine = v;
      }
      if (col0 + lane < p.N) atomicAdd(p.red + col0 + lane, mine);
    }
  }
}

// 32 finished columns -> 16 packed bf16 or f16 pairs, rounded to nearest.
__device__ __forceinline__ void pack32_rn(const float (&f)[32], uint32_t (&w)[16], bool bf16) {
#pragma unroll
  for (int i = 0; i < 16; ++i)
    w[i] = bf16 ? cvt_pack2_t<KAPYB_BF16, 1>(f[2 * i], f[2 * i + 1])
                : cvt_pack2_t<KAPYB_F16, 1>(f[2 * i], f[2 * i + 1]);
}

// 16 packed pairs (32 columns, half h of a 64-column chunk) -> the row's slot in
// the swizzled staging tile.
__device__ __forceinline__ void stage_packed16(uint8_t *srow, const uint32_t (&w)[16], int lane,
                                               int h) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 q = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    const int jj = h * 4 + j;
    *reinterpret_cast<uint4 *>(srow + ((jj ^ (lane & 7)) << 4)) = q;
  }
}

// OUTK: 0 f32, 1/2 bf16 rn/rz, 3/4 f16 rn/rz.  PLAIN: the epilogue is only the
// scale (no bias, addend or activation), so none of those are even tested.
// Returns whether the slot was handed back (false when this warp had no chunk).
template <int BN, int EPI, int OUTK, bool PLAIN, bool REDUCE = false>
__device__ __forceinline__ bool epilogue_tile(const GemmParams &p, const TmapArray &tmC,
                                              const EpiTile &t, int &buf, uint32_t acc_bar,
                                              uint32_t &acc_parity) {
  constexpr bool OUT32 = OUTK == 0;
  constexpr int ACCK = PLAIN ? -1 : (OUTK == 0 ? 0 : (OUTK <= 2 ? 1 : 2));
  const bool acc_tma = !PLAIN && p.acc_tma != 0;
  constexpr int CW = OUT32 ? 32 : 64;  // output columns per 128-byte staging row
  constexpr int NH = CW / 32;
  constexpr int CSTEP = EPI / 4;
  constexpr int C_BUFS = ((BN == 512 || BN == 256) && EPI == 8) ? 1 : 2;
  const int lane = t.lane;
  bool handed_back = false;
  for (int c = t.col_begin / CW + t.cpart; c < t.col_end / CW; c += CSTEP) {
    const int nc = t.n0 + c * CW;
    if (nc >= p.N) break;
    uint8_t *sbuf = t.stg + (C_BUFS == 2 ? buf : 0) * 4096;
    // All loads of the chunk are in flight before the one wait.
    uint32_t v[NH][32];
    const bool probing = kEpilogueProbes && t.prof != nullptr;
    const uint32_t c0 = probing ? static_cast<uint32_t>(clock()) : 0u;
#pragma unroll
    for (int h = 0; h < NH; ++h)
      ptx::tmem_ld_32x32(t.t_row + static_cast<uint32_t>(c * CW + h * 32), v[h]);
    // The store that last read this buffer (two chunks ago, or the previous one
    // with a single buffer) must have finished reading it.
    if (lane == 0) {
      ptx::tma_store_wait_read<C_BUFS - 1>();
      if (acc_tma) {
        // the addend's tile of this chunk comes into the buffer the result will leave
        // from (each lane then reads and rewrites its own row)
        ptx::mbar_arrive_expect_tx(acc_bar, 4096u);
        ptx::tma_load_3d(ptx::smem_u32(sbuf), &tmC.m[kMaxOutputs - 1], acc_bar, nc, t.m0, t.b);
      }
    }
    __syncwarp();
    const uint32_t c1 = probing ? static_cast<uint32_t>(clock()) : 0u;
    ptx::tmem_ld_wait();
    const uint32_t c2 = probing ? static_cast<uint32_t>(clock()) : 0u;
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
    bool acc_here = false;
    if (acc_tma) {
      // (a wait that runs out has raised the abort flag: the kernel is on its way out
      // and the status word will say so; the sums below then go without the addend)
      acc_here = __all_sync(0xffffffffu, ptx::mbar_wait(acc_bar, acc_parity, t.abort_flag)) != 0;
      acc_parity ^= 1u;
    }
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      const int col0 = nc + h * 32;
      float f[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[h][i]);
      finish32<PLAIN ? 0 : 2, REDUCE, ACCK>(p, t, f, col0, acc_here ? srow : nullptr, h);
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
    const uint32_t c3 = probing ? static_cast<uint32_t>(clock()) : 0u;
    if (lane == 0 && !debug_on<8>(p.debug)) {
      if (p.c_l2) {
        const uint64_t pol = ptx::make_l2_policy(p.c_l2);
        for (int o = 0; o < p.n_out; ++o)
          ptx::tma_store_3d_hint(&tmC.m[o], ptx::smem_u32(sbuf), p.out_col_offset + nc, t.m0, t.b, pol);
      } else {
        for (int o = 0; o < p.n_out; ++o)
          ptx::tma_store_3d(&tmC.m[o], ptx::smem_u32(sbuf), p.out_col_offset + nc, t.m0, t.b);
      }
      ptx::tma_store_commit();
    }
    if (probing && lane == 0) {
      atomicAdd(t.prof + 0, c2 - c0);  // staging buffer free again, accumulator loads landed
      (void)c1;
      atomicAdd(t.prof + 2, c3 - c2);  // arithmetic, staging, fence
      atomicAdd(t.prof + 3, static_cast<uint32_t>(clock()) - c3);  // store issued
    }
    buf ^= 1;
  }
  return handed_back;
}

// Two-half tiles (BN = 512) with a 16-bit output: the accumulator fills TMEM, so
// the next tile's MMAs wait for the drain.  Staging chunk by chunk through the
// one 4 KB buffer would keep TMEM busy for the whole store sequence; instead the
// warp pulls its four 64-column chunks (two per half) into packed registers,
// hands each half back as soon as its last load has landed, and stores from the
// registers afterwards, under the next tile's main loop.  Covers the epilogues
// that are a scale and an optional bias, rounded to nearest; anything more goes
// chunk by chunk.  `spare`: 12 KB of the operand ring when this is the CTA's last
// tile (its three register-held chunks are then staged there and stored together),
// else nullptr.  Returns false when a wait ran out.
// MODE 1 / 2: the output is bf16 / f16, known at compile time, and a column bias
// kept in registers is of the same type (one type throughout, the usual case).
// The drain is bound by the instructions these warps issue, and choosing the
// conversions per element at run time tripled them; two specialised copies
// inlined into one kernel made the register allocator spill, so the kernel
// itself is instantiated per MODE (its DRAIN parameter).
template <int EPI, int MODE>
__device__ __forceinline__ bool epilogue_two_halves(const GemmParams &p, const TmapArray &tmC,
                                                 EpiTile &t, uint32_t tfull0, uint32_t parity,
                                                 volatile uint32_t *abort_flag, bool active,
                                                 uint8_t *spare) {
  static_assert(EPI == 8, "register drain: eight epilogue warps");
  static_assert(MODE == 1 || MODE == 2, "bf16 or f16");
  constexpr bool bf16 = MODE == 1;
  const int lane = t.lane;
  uint8_t *srow = t.stg + lane * 128;
  // Chunk i = hh*2 + j covers tile columns (hh*4 + cpart + 2*j) * 64 ..  Chunk 0
  // goes straight through the (idle) staging buffer; 1..3 wait in registers.
  uint32_t pk[3][2][16];
  // lane 0, after the staged bytes were fenced towards the async proxy
  auto issue_store = [&](const uint8_t *src, int nc) {
    if (debug_on<8>(p.debug)) return;
    if (p.c_l2) {
      const uint64_t pol = ptx::make_l2_policy(p.c_l2);
      for (int o = 0; o < p.n_out; ++o)
        ptx::tma_store_3d_hint(&tmC.m[o], ptx::smem_u32(src), p.out_col_offset + nc, t.m0, t.b, pol);
    } else {
      for (int o = 0; o < p.n_out; ++o)
        ptx::tma_store_3d(&tmC.m[o], ptx::smem_u32(src), p.out_col_offset + nc, t.m0, t.b);
    }
    ptx::tma_store_commit();
  };
  auto store_chunk = [&](int nc) {
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) issue_store(t.stg, nc);
  };
  // A 16-bit column bias is fetched before the accumulator is awaited, so its
  // latency hides behind the main loop: lane l keeps the eight values of columns
  // (l & 7) * 8 .. +7 of chunk l >> 3; the pieces below pick them up by shuffle.
  constexpr bool bias_bf16 = MODE == 1;
  const bool bias_regs = t.bias_col && t.bias_fast &&
                         p.ep.bias_dtype == (MODE == 1 ? KAPYB_BF16 : KAPYB_F16);
  // an f32 column bias (the usual companion of 16-bit operands) the same way, eight
  // values per lane in two words
  const bool bias_regs32 = t.bias_col && p.ep.bias_dtype == KAPYB_F32;
  const float alpha = p.ep.alpha;
  uint4 bv = make_uint4(0u, 0u, 0u, 0u), bv_hi = make_uint4(0u, 0u, 0u, 0u);
  if (bias_regs32) {
    const int ci = lane >> 3;
    const int col = t.n0 + ((ci >> 1) * 4 + t.cpart + 2 * (ci & 1)) * 64 + (lane & 7) * 8;
    const float *bp = static_cast<const float *>(p.ep.bias);
    uint32_t w[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = col + e < p.N ? __float_as_uint(__ldg(bp + col + e)) : 0u;
    bv = make_uint4(w[0], w[1], w[2], w[3]);
    bv_hi = make_uint4(w[4], w[5], w[6], w[7]);
  } else if (bias_regs) {
    const int ci = lane >> 3;
    const int col = t.n0 + ((ci >> 1) * 4 + t.cpart + 2 * (ci & 1)) * 64 + (lane & 7) * 8;
    const uint16_t *bp = static_cast<const uint16_t *>(p.ep.bias);
    if (col + 8 <= p.N) {
      bv = __ldg(reinterpret_cast<const uint4 *>(bp + col));
    } else {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col + e < p.N) w[e >> 1] |= static_cast<uint32_t>(__ldg(bp + col + e)) << (16 * (e & 1));
      bv = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  bool alive = true;  // false once a wait has run out: nothing more is read or stored
  uint32_t ld_clocks = 0, drain_c0 = 0;
  // debug builds, timeline on: when the first CTA's first epilogue warp saw half 0
  // published, handed it back, saw half 1 published, handed it back, issued its last
  // store (of the CTA's last tile) -> status[9..13]
  auto stamp = [&](int word) {
    if constexpr (kEpilogueProbes) {
      if (t.prof != nullptr && lane == 0)
        t.prof[word] = static_cast<uint32_t>(ptx::globaltimer_ns());
    }
  };
  uint32_t hb_clocks = 0, st_clocks = 0;
  auto hand_back = [&](int hh) {
    const uint32_t k0 = (kEpilogueProbes && t.prof) ? static_cast<uint32_t>(clock()) : 0u;
    ptx::tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (t.remote_arrive)
        ptx::mbar_arrive_cluster(t.tempty_addr + hh * 8);
      else
        ptx::mbar_arrive(t.tempty_addr + hh * 8);
    }
    if (kEpilogueProbes && t.prof) hb_clocks += static_cast<uint32_t>(clock()) - k0;
  };
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int hh = i >> 1, j = i & 1;
    if (j == 0) {
      // every lane polls, then the warp votes: a time-out must take all lanes or none,
      // since the loads, shuffles and __syncwarp below are warp-collective
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(tfull0 + hh * 8, parity, abort_flag))) alive = false;
      ptx::tc_fence_after();
      if (hh == 0) {
        stamp(0);
        drain_c0 = static_cast<uint32_t>(clock());
      }
    }
    const int c = hh * 4 + t.cpart + 2 * j;
    const int nc = t.n0 + c * 64;
    const bool valid = alive && active && nc < p.N;
    // 32 columns at a time: the registers hold three packed chunks already
    uint32_t v[32];
    if (valid) {
      if (i == 0) {
        // the previous tile's last store has long finished reading the buffer
        if (lane == 0) ptx::tma_store_wait_read<0>();
        __syncwarp();
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t k0 = (kEpilogueProbes && t.prof) ? static_cast<uint32_t>(clock()) : 0u;
        ptx::tmem_ld_32x32(t.t_row + static_cast<uint32_t>(c * 64 + h * 32), v);
        ptx::tmem_ld_wait();
        if (kEpilogueProbes && t.prof) ld_clocks += static_cast<uint32_t>(clock()) - k0;
        if (j == 1 && h == 1) {
          hand_back(hh);  // this warp's last read of half hh
          if (kEpilogueProbes && t.prof && hh == 1 && lane == 0) {
            t.prof[3] = hb_clocks;
            t.prof[4] = st_clocks;
            t.prof[1] = ld_clocks;                                   // clocks in tcgen05.ld + wait::ld, 8 pieces
            t.prof[2] = static_cast<uint32_t>(clock()) - drain_c0;   // clocks from half 0 seen to half 1 handed back
          }
        }
        float f[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) f[k] = __uint_as_float(v[k]);
        if (bias_regs) {
          // the piece's 32 bias values sit in lanes i*8 + h*4 .. +3, eight per lane;
          // scale and bias are one fused multiply-add per element
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int src = i * 8 + h * 4 + jj;
            const uint32_t ws[4] = {__shfl_sync(0xffffffffu, bv.x, src),
                                    __shfl_sync(0xffffffffu, bv.y, src),
                                    __shfl_sync(0xffffffffu, bv.z, src),
                                    __shfl_sync(0xffffffffu, bv.w, src)};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              if (bias_bf16)
                unpack2_16<KAPYB_BF16>(ws[e], lo, hi);
              else
                unpack2_16<KAPYB_F16>(ws[e], lo, hi);
              f[8 * jj + 2 * e] = fmaf(f[8 * jj + 2 * e], alpha, lo);
              f[8 * jj + 2 * e + 1] = fmaf(f[8 * jj + 2 * e + 1], alpha, hi);
            }
          }
        } else if (bias_regs32) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int src = i * 8 + h * 4 + jj;
            f[8 * jj + 0] = fmaf(f[8 * jj + 0], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv.x, src)));
            f[8 * jj + 1] = fmaf(f[8 * jj + 1], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv.y, src)));
            f[8 * jj + 2] = fmaf(f[8 * jj + 2], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv.z, src)));
            f[8 * jj + 3] = fmaf(f[8 * jj + 3], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv.w, src)));
            f[8 * jj + 4] = fmaf(f[8 * jj + 4], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv_hi.x, src)));
            f[8 * jj + 5] = fmaf(f[8 * jj + 5], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv_hi.y, src)));
            f[8 * jj + 6] = fmaf(f[8 * jj + 6], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv_hi.z, src)));
            f[8 * jj + 7] = fmaf(f[8 * jj + 7], alpha, __uint_as_float(__shfl_sync(0xffffffffu, bv_hi.w, src)));
          }
        } else {
          finish32<1>(p, t, f, nc + h * 32);
        }
        if (i == 0) {
          uint32_t w[16];
          pack32_rn(f, w, bf16);
          stage_packed16(srow, w, lane, h);
        } else {
          pack32_rn(f, pk[i == 0 ? 0 : i - 1][h], bf16);
        }
      }
    } else if (j == 1) {
      hand_back(hh);
    }
    if (i == 1 && alive && active && t.n0 + t.cpart * 64 < p.N) {
      // chunk 0 sits in the staging buffer: its store goes out now that half 0 is
      // back with the MMA thread (the fence and the store's issue cost that thread
      // several hundred clocks when they came first)
      const uint32_t k0 = (kEpilogueProbes && t.prof) ? static_cast<uint32_t>(clock()) : 0u;
      store_chunk(t.n0 + t.cpart * 64);
      if (kEpilogueProbes && t.prof) st_clocks += static_cast<uint32_t>(clock()) - k0;
    }
  }
  if (spare != nullptr) {
    // The CTA's last tile: every MMA has read its operands (half 1 was published
    // after the last of them), so the operand ring is free.  The three chunks go
    // through 4 KB of it each and leave together instead of taking turns in the one
    // staging buffer, each waiting for the store before it to have read that.
    if (alive && active) {
#pragma unroll
      for (int i = 1; i < 4; ++i) {
        uint8_t *row = spare + (i - 1) * 4096 + lane * 128;
        stage_packed16(row, pk[i - 1][0], lane, 0);
        stage_packed16(row, pk[i - 1][1], lane, 1);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int i = 1; i < 4; ++i) {
          const int nc = t.n0 + ((i >> 1) * 4 + t.cpart + 2 * (i & 1)) * 64;
          if (nc < p.N) issue_store(spare + (i - 1) * 4096, nc);
        }
      }
    }
    return alive;
  }
#pragma unroll
  for (int i = 1; i < 4; ++i) {
    const int c = (i >> 1) * 4 + t.cpart + 2 * (i & 1);
    const int nc = t.n0 + c * 64;
    if (alive && active && nc < p.N) {
      if (lane == 0) ptx::tma_store_wait_read<0>();
      __syncwarp();
      stage_packed16(srow, pk[i - 1][0], lane, 0);
      stage_packed16(srow, pk[i - 1][1], lane, 1);
      store_chunk(nc);
    }
  }
  return alive;
}

// The MMAs of one K block (four K steps of 32 bytes; with a split tile, both
// column halves per step, sharing the A descriptor).  Descriptors arrive as
// (low word of K step 0, constant high word, low-word increment per K step);
// `half_mask` picks the column halves to issue (bit hh), all of them = 3;
// this CTA's B bytes of half hh start (MMA_N / CTAS) rows of 128 bytes after
// those of half hh-1, in either layout and for any element width.
template <int CTAS, int SPLIT, int MMA_N, int KIND>
__device__ __forceinline__ void issue_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                             uint32_t a_kstep, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t b_kstep, uint32_t idesc, uint32_t first,
                                             uint32_t half_mask) {
  constexpr uint32_t kHalfStep = (MMA_N / CTAS) * 128 / 16;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint64_t adesc = (static_cast<uint64_t>(a_hi) << 32) | (a_lo + k * a_kstep);
#pragma unroll
    for (int hh = 0; hh < SPLIT; ++hh) {
      if (SPLIT > 1 && !(half_mask & (1u << hh))) continue;
      const uint64_t bdesc =
          (static_cast<uint64_t>(b_hi) << 32) | (b_lo + k * b_kstep + hh * kHalfStep);
      ptx::umma_k<CTAS, KIND>(d_tmem + hh * MMA_N, adesc, bdesc, idesc, k == 0 ? first : 1u);
    }
  }
}

// BN: tile width; CTAS: CTAs per tile (2 = a pair on a 256-row tile); EPI: epilogue
// warps; REDUCE: kapy.reduce fused after the epilogue; SK: the K blocks of the last
// wave's tiles are dealt out as spans (GemmParams::sk_*); DRAIN: the 16-bit output
// type the register drain of the 512-wide tile is compiled for (1 bf16, 2 f16).
template <int BN, int CTAS, int EPI, bool REDUCE = false, bool SK = false, int DRAIN = 1>
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
  uint32_t *prof_words = tmem_slot + 8;  // [5] clocks per epilogue phase (debug bit 7)
  uint64_t *acc_bars = bars + 64;        // [EPI] one per epilogue warp: its addend tile has landed

  // the shuffle makes the warp index provably uniform for the compiler
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;
  const bool timeline = debug_on<128>(p.debug);  // probes: see GemmParams::debug
  if (timeline && threadIdx.x == 0) {
    const uint32_t t = static_cast<uint32_t>(ptx::globaltimer_ns());
    atomicMax(p.status + 4, ~t);  // earliest CTA start, kept as the largest complement
    atomicMax(p.status + 5, t);   // latest CTA start
  }
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
    for (int w = 0; w < EPI; ++w) ptx::mbar_init(ptx::smem_u32(&acc_bars[w]), 1);  // one TMA load of an addend tile
    abort_flag[0] = 0u;
    abort_flag[1] = p.wait_limit_us;
    for (int i = 0; i < 5; ++i) prof_words[i] = 0u;
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
  // Everything above touched only shared and tensor memory: let the next kernel of
  // the stream start its own set-up while this grid runs, and do not touch global
  // memory before the kernels ahead of this one are done.
  ptx::griddep_launch();
  ptx::griddep_wait();

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // The tile loop exists twice: with plain loads, and with loads that carry an L2
    // policy per tensor (from the descriptors' eviction priority).  Choosing the
    // form per load inside one loop cost the benchmark kernel 6 % although the
    // choice never changed: this thread's issue rate is on the critical path.
    // (The loads are macros, not helpers taking the map's address: the maps are
    // __grid_constant__ parameters, named where the TMA instruction is issued.)
#define KAPYB_LOAD1(POL, DST, TM, BAR, X, Y, Z)                    \
  do {                                                             \
    if constexpr (HINTED)                                          \
      ptx::tma_load_3d_hint(DST, &TM, BAR, X, Y, Z, POL);          \
    else                                                           \
      ptx::tma_load_3d(DST, &TM, BAR, X, Y, Z);                    \
  } while (0)
#define KAPYB_LOAD2(POL, DST, TM, BAR, X, Y, Z)                    \
  do {                                                             \
    if constexpr (HINTED)                                          \
      ptx::tma_load_3d_pair_hint(DST, &TM, BAR, X, Y, Z, POL);     \
    else                                                           \
      ptx::tma_load_3d_pair(DST, &TM, BAR, X, Y, Z);               \
  } while (0)
    auto produce = [&](auto hinted, auto chunk_elems) {
    constexpr bool HINTED = decltype(hinted)::value;
    // elements per 128-byte row of shared memory (64 / 32 / 128 for 2- / 4- / 1-byte
    // operands) as a constant, so that the chunk loops below unroll
    constexpr int ce = decltype(chunk_elems)::value;
    const uint64_t pol_a = HINTED ? ptx::make_l2_policy(p.a_l2) : 0ull;
    const uint64_t pol_b = HINTED ? ptx::make_l2_policy(p.b_l2) : 0ull;
    (void)pol_a;
    (void)pol_b;
    for (WorkIter<SK> w(p, unit, unit_step); ok && !debug_on<16 | 32>(p.debug) && w.next(p);) {
      int b, mb, nb;
      decode_tile(p, w.tile, b, mb, nb);
      const int m0 = mb * Cfg::TILE_M + static_cast<int>(rank) * Cfg::BM;
      // first B column this CTA loads; with a split tile its columns are two groups
      // of MMA_N / CTAS, one per column half, so that accumulator column c of the
      // pair's MMA is tile column c
      const int nB0 = nb * BN + static_cast<int>(rank) * (Cfg::MMA_N / CTAS);
      constexpr int kGroupCols = Cfg::MMA_N / CTAS;   // columns per half this CTA owns
      for (int kb = w.kb0; kb < w.kb1; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const int k0 = kb * ce;
        constexpr int a_chunks = Cfg::BM / ce;
        constexpr int b_chunks = Cfg::BN_CTA / ce;
        const uint32_t a_dst = ptx::smem_u32(sA + stage * Cfg::A_BYTES);
        const uint32_t b_dst = ptx::smem_u32(sB + stage * Cfg::B_BYTES);
        if (debug_on<1>(p.debug)) {
          if (rank == 0) ptx::mbar_arrive(ptx::smem_u32(&full_bar[stage]));
        } else if constexpr (CTAS == 1) {
          const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
          ptx::mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
          if (!p.a_mn_major) {
            KAPYB_LOAD1(pol_a, a_dst, tmA, fb, k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < a_chunks; ++j)
              KAPYB_LOAD1(pol_a, a_dst + j * p.mn_lbo, tmA, fb, m0 + ce * j, k0, b);
          }
          if (!p.b_mn_major) {
            // one box of kGroupCols rows per column half
#pragma unroll
            for (int hh = 0; hh < Cfg::SPLIT; ++hh)
              KAPYB_LOAD1(pol_b, b_dst + hh * (kGroupCols * 128), tmB, fb, k0, nB0 + hh * Cfg::MMA_N, b);
          } else {
#pragma unroll
            for (int j = 0; j < b_chunks; ++j)
              KAPYB_LOAD1(pol_b, b_dst + j * p.mn_lbo, tmB, fb, nB0 + ce * j, k0, b);
          }
        } else {
          // Both CTAs' loads report their bytes to the leader's barrier; the
          // leader alone posts the arrival, expecting the bytes of both.  (A
          // remote arrive.expect_tx from the peer instead halves the throughput.)
          const uint32_t fb = ptx::mapa(ptx::smem_u32(&full_bar[stage]), 0);
          if (rank == 0)
            ptx::mbar_arrive_expect_tx(ptx::smem_u32(&full_bar[stage]), 2 * Cfg::STAGE_BYTES);
          if (!p.a_mn_major) {
            KAPYB_LOAD2(pol_a, a_dst, tmA, fb, k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < a_chunks; ++j)
              KAPYB_LOAD2(pol_a, a_dst + j * p.mn_lbo, tmA, fb, m0 + ce * j, k0, b);
          }
          if (!p.b_mn_major) {
            // one box of kGroupCols rows per half
#pragma unroll
            for (int hh = 0; hh < Cfg::SPLIT; ++hh)
              KAPYB_LOAD2(pol_b, b_dst + hh * (kGroupCols * 128), tmB, fb, k0, nB0 + hh * Cfg::MMA_N, b);
          } else {
#pragma unroll
            for (int j = 0; j < b_chunks; ++j) {
              constexpr int per_group = kGroupCols >= ce ? kGroupCols / ce : 1;  // chunks per column half
              const int hh = j / per_group, within = (j % per_group) * ce;
              KAPYB_LOAD2(pol_b, b_dst + j * p.mn_lbo, tmB, fb, nB0 + hh * Cfg::MMA_N + within, k0, b);
            }
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    };  // produce
    const bool hinted = (p.a_l2 | p.b_l2) != 0;
    if (p.bk_elems == 64) {
      if (hinted)
        produce(std::true_type{}, std::integral_constant<int, 64>{});
      else
        produce(std::false_type{}, std::integral_constant<int, 64>{});
    } else if (p.bk_elems == 32) {
      if (hinted)
        produce(std::true_type{}, std::integral_constant<int, 32>{});
      else
        produce(std::false_type{}, std::integral_constant<int, 32>{});
    } else {
      if (hinted)
        produce(std::true_type{}, std::integral_constant<int, 128>{});
      else
        produce(std::false_type{}, std::integral_constant<int, 128>{});
    }
#undef KAPYB_LOAD1
#undef KAPYB_LOAD2
  } else if (warp == 1 && rank == 0) {
    // ---------------------------------------------------------- MMA issuer
    // The whole warp walks the loops in step and one elected lane issues: with
    // warp-uniform control flow the descriptor arithmetic and the MMA operands
    // stay in uniform registers.  Every wait ends in a vote, so the lanes can
    // never part ways (elect.sync needs all of them), not even on a time-out.
    auto wait_all = [&](uint32_t bar, uint32_t parity) {
      const bool mine = ptx::mbar_wait(bar, parity, abort_flag);
      return __all_sync(0xffffffffu, mine) != 0;
    };
    // K-major operand: rows are 128 bytes, 8-row groups 1024 bytes apart; one
    // UMMA K step is 32 bytes along the row (16 / 8 / 32 elements of 2 / 4 / 1
    // bytes).  MN-major operand: 128-byte MN chunks mn_lbo bytes apart (8192 for
    // 16-bit types), K rows 128 bytes apart in groups of 8 (1024 bytes); one K
    // step is mn_kadv bytes (16 rows = 2048 for 16-bit types).
    //
    // This one thread has to issue an MMA every ~128 clocks, so the loop below
    // does as little as it can per instruction: everything in a descriptor but
    // the start address is folded into two constants per operand up front, and
    // each K step is one 32-bit add on the descriptor's low word.
    const uint32_t a_lbo = p.a_mn_major ? p.mn_lbo : 16u, a_sbo = p.a_mn_major ? p.mn_sbo : 1024u;
    const uint32_t b_lbo = p.b_mn_major ? p.mn_lbo : 16u, b_sbo = p.b_mn_major ? p.mn_sbo : 1024u;
    const uint32_t a_lay = p.a_mn_major ? p.mn_layout : 2u;
    const uint32_t b_lay = p.b_mn_major ? p.mn_layout : 2u;
    // low word: start address >> 4 | LBO >> 4 << 16; high word: SBO >> 4, version 1
    // (bit 46), layout type (bits 61..63)
    const uint32_t a_lo_c = ((a_lbo >> 4) & 0x3FFFu) << 16;
    const uint32_t b_lo_c = ((b_lbo >> 4) & 0x3FFFu) << 16;
    const uint32_t a_hi = ((a_sbo >> 4) & 0x3FFFu) | (1u << 14) | (a_lay << 29);
    const uint32_t b_hi = ((b_sbo >> 4) & 0x3FFFu) | (1u << 14) | (b_lay << 29);
    const uint32_t a_kstep = (p.a_mn_major ? p.mn_kadv : 32u) >> 4;   // descriptor units per K step
    const uint32_t b_kstep = (p.b_mn_major ? p.mn_kadv : 32u) >> 4;
    const uint32_t a_lo0 = a_lo_c | (ptx::smem_u32(sA) >> 4);
    const uint32_t b_lo0 = b_lo_c | (ptx::smem_u32(sB) >> 4);
    const uint32_t idesc = p.idesc;
    const int kind = p.kind;
    const bool skip_mma = debug_on<2>(p.debug), free_run = debug_on<32>(p.debug);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    bool seen_first = false;
    const bool probe = timeline && blockIdx.x == 0;
    const long long probe_c0 = probe ? clock64() : 0;
    const uint64_t probe_t0 = probe ? ptx::globaltimer_ns() : 0;
    uint32_t stall_full = 0, stall_drain = 0;  // probe: clocks this thread waited for operands / for TMEM
    for (WorkIter<SK> w(p, unit, unit_step); ok && w.next(p);) {
      // ---- helpers (every lane runs them; one elected lane issues)
      // waits for the next operand stage; returns its index, or -1 when the wait ran out
      auto wait_stage = [&]() -> int {
        const uint32_t f0 = probe ? static_cast<uint32_t>(clock()) : 0u;
        if (!free_run && !wait_all(ptx::smem_u32(&full_bar[stage]), phase)) return -1;
        if (probe) stall_full += static_cast<uint32_t>(clock()) - f0;
        ptx::tc_fence_after();
        if (timeline && !seen_first) {
          seen_first = true;
          if (lane == 0) atomicMax(p.status + 6, static_cast<uint32_t>(ptx::globaltimer_ns()));
        }
        const int st = stage;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        return st;
      };
      // the MMAs of stage `st` into the accumulator(s) at d_tmem; `first` = 0 overwrites
      auto issue = [&](int st, uint32_t d_tmem, uint32_t first, uint32_t half_mask) {
        if (skip_mma || !ptx::elect_one()) return;
        const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(st) * (Cfg::A_BYTES >> 4);
        const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(st) * (Cfg::B_BYTES >> 4);
        if (kind == 0)
          issue_kblock<CTAS, Cfg::SPLIT, Cfg::MMA_N, 0>(d_tmem, a_lo, a_hi, a_kstep, b_lo, b_hi,
                                                         b_kstep, idesc, first, half_mask);
        else if (kind == 1)
          issue_kblock<CTAS, Cfg::SPLIT, Cfg::MMA_N, 1>(d_tmem, a_lo, a_hi, a_kstep, b_lo, b_hi,
                                                         b_kstep, idesc, first, half_mask);
        else
          issue_kblock<CTAS, Cfg::SPLIT, Cfg::MMA_N, 2>(d_tmem, a_lo, a_hi, a_kstep, b_lo, b_hi,
                                                         b_kstep, idesc, first, half_mask);
      };
      // frees stage `st` in every CTA that filled it, once the MMAs issued so far are done
      auto release = [&](int st) {
        if (free_run || !ptx::elect_one()) return;
        ptx::umma_commit<CTAS>(ptx::smem_u32(&empty_bar[st]));
        if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(ptx::smem_u32(&empty_bar[st]), 1));
      };
      // publishes accumulator slot `slot` to the epilogue warps of every CTA
      auto publish = [&](int slot) {
        if (!ptx::elect_one()) return;
        ptx::umma_commit<CTAS>(ptx::smem_u32(&tfull_bar[slot]));
        if constexpr (CTAS == 2) ptx::umma_commit<CTAS>(ptx::mapa(ptx::smem_u32(&tfull_bar[slot]), 1));
      };
      auto wait_drained = [&](int slot) {
        const uint32_t d0 = probe ? static_cast<uint32_t>(clock()) : 0u;
        const bool got = wait_all(ptx::smem_u32(&tempty_bar[slot]), acc_phase ^ 1u);
        if (probe) stall_drain += static_cast<uint32_t>(clock()) - d0;
        ptx::tc_fence_after();
        return got;
      };

      if constexpr (Cfg::HALVES == 2) {
        // The two halves fill TMEM, so a tile's MMAs cannot start before the
        // previous tile has been drained.  To keep the tensor pipe fed across
        // that hand-over the halves are skewed by kSkew K blocks at the tile
        // boundaries only: the tile ENDS with half 0's last blocks, then half
        // 1's (half 0 drains under those), and STARTS with half 0's first
        // blocks (half 1 still draining), then half 1's.  In between both halves
        // of a K block are issued together and share its A stage.
        constexpr int kSkew = 2;
        static_assert(kSkew < STAGES, "the skewed blocks stay resident until both halves used them");
        const uint32_t d_tmem = tmem_base;
        const int n = w.kb1 - w.kb0;
        const int skew = n >= 2 * kSkew ? kSkew : 0;
        int held[kSkew];
        if (!wait_drained(0)) break;
        for (int i = 0; i < skew && ok; ++i) {
          held[i] = wait_stage();
          if (held[i] < 0) ok = false;
          else issue(held[i], d_tmem, i != 0 ? 1u : 0u, 1u);
        }
        if (!ok) break;
        if (!wait_drained(1)) break;
        for (int i = 0; i < skew; ++i) {
          issue(held[i], d_tmem, i != 0 ? 1u : 0u, 2u);
          release(held[i]);
        }
        for (int kb = skew; kb < n - skew; ++kb) {
          const int st = wait_stage();
          if (st < 0) {
            ok = false;
            break;
          }
          issue(st, d_tmem, kb != 0 ? 1u : 0u, 3u);
          release(st);
        }
        if (!ok) break;
        for (int i = 0; i < skew && ok; ++i) {
          held[i] = wait_stage();
          if (held[i] < 0) ok = false;
          else issue(held[i], d_tmem, 1u, 1u);
        }
        if (!ok) break;
        publish(0);
        for (int i = 0; i < skew; ++i) {
          issue(held[i], d_tmem, 1u, 2u);
          release(held[i]);
        }
        publish(1);
        acc_phase ^= 1u;
      } else {
        if (!wait_drained(acc)) break;
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        const int n = w.kb1 - w.kb0;
        for (int kb = 0; kb < n; ++kb) {
          const int st = wait_stage();
          if (st < 0) {
            ok = false;
            break;
          }
          issue(st, d_tmem, kb != 0 ? 1u : 0u, 3u);
          release(st);
        }
        if (!ok) break;
        publish(acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    if (timeline && lane == 0) atomicMax(p.status + 7, static_cast<uint32_t>(ptx::globaltimer_ns()));
    if (probe && lane == 0) {
      p.status[14] = stall_full;
      p.status[15] = stall_drain;
      p.status[2] = static_cast<uint32_t>(clock64() - probe_c0);
      p.status[3] = static_cast<uint32_t>(ptx::globaltimer_ns() - probe_t0);
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
    const bool plain = !REDUCE && p.ep.bias == nullptr && p.ep.acc == nullptr &&
                       p.ep.activation == KAPYB_ACT_NONE;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    const uint32_t acc_bar = ptx::smem_u32(&acc_bars[e]);
    uint32_t acc_parity = 0;
    uint32_t *prof = (kEpilogueProbes && timeline && blockIdx.x == 0 && e == 0) ? prof_words : nullptr;
    for (WorkIter<SK> w(p, unit, unit_step); w.next(p);) {
      const uint32_t s0 = prof ? static_cast<uint32_t>(clock()) : 0u;
      int b, mb, nb;
      decode_tile(p, w.tile, b, mb, nb);
      if (prof && lane == 0) atomicAdd(prof + 1, static_cast<uint32_t>(clock()) - s0);  // tile decode
      const int m0 = mb * Cfg::TILE_M + static_cast<int>(rank) * Cfg::BM + q * 32;
      const int n0 = nb * BN;
      const int row = m0 + lane;
      bool alive = true;
      if constexpr (SK) {
        // A tile whose K blocks are shared between CTAs (pairs).  Its pieces: 32 rows
        // (this warp's TMEM lanes) x 32 columns, 4 KB each, piece (c32, q) of CTA
        // `rank` of pair `u` at sk_scratch + ((u * CTAS + rank) * BN / 32 * 4 + c32 * 4 + q) KB * 4,
        // lane l holding row l as eight float4 at [j * 32 + l].
        // With eight epilogue warps two warps share a lane quarter: each takes the
        // columns it will drain in the epilogue proper (alternate chunks of 64
        // columns, of 32 for a 32-bit output), so the sums a warp writes back to TMEM
        // are read by that warp only.
        constexpr int CSTEP = EPI / 4;
        constexpr int kSlotPieces = Cfg::SLOT_COLS / 32;
        const int pw = out32 ? 1 : 2;  // pieces per chunk
        auto mine_piece = [&](int c32) { return CSTEP == 1 || ((c32 / pw) & 1) == cpart; };
        const uint32_t t_row0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        auto pieces_of = [&](int u) {
          return p.sk_scratch + (static_cast<size_t>(u) * CTAS + rank) * (128 * BN);
        };
        if (w.kb0 != 0) {
          // Not the tile's first K blocks: leave the accumulator for the CTA that did those.
          float *mine = pieces_of(unit);
#pragma unroll 1
          for (int hh = 0; hh < Cfg::HALVES; ++hh) {
            const int slot = Cfg::HALVES == 2 ? hh : acc;
            if (!__all_sync(0xffffffffu,
                            ptx::mbar_wait(ptx::smem_u32(&tfull_bar[slot]), acc_phase, abort_flag))) {
              alive = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t t_row = t_row0 + (Cfg::HALVES == 2 ? 0u : static_cast<uint32_t>(acc * BN));
            if (m0 < p.M) {
              for (int c32 = hh * kSlotPieces; c32 < (hh + 1) * kSlotPieces; ++c32) {
                if (n0 + c32 * 32 >= p.N) break;
                if (!mine_piece(c32)) continue;
                uint32_t v[32];
                ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(c32 * 32), v);
                ptx::tmem_ld_wait();
                float4 *dst = reinterpret_cast<float4 *>(mine + (c32 * 4 + q) * 1024) + lane;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  __stcg(dst + j * 32, make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                   __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
              }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              const uint32_t slot_bar = tempty_leader + static_cast<uint32_t>(slot * 8);
              if constexpr (CTAS == 2)
                ptx::mbar_arrive_cluster(slot_bar);
              else
                ptx::mbar_arrive(slot_bar);
            }
          }
          if (!alive) break;
          // every lane's stores, then the warp's word: release by one lane after the
          // warp barrier covers them all
          __syncwarp();
          if (lane == 0) {
            __threadfence();
            ptx::st_release_gpu(p.sk_flags + (static_cast<size_t>(unit) * CTAS + rank) * 8 + e, p.sk_epoch);
          }
          if constexpr (Cfg::HALVES == 2) {
            acc_phase ^= 1u;
          } else {
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
          }
          continue;
        }
        if (w.kb1 != p.num_kb) {
          // The tile's first K blocks, the rest done elsewhere: add the other CTAs'
          // partial sums into the accumulator (in CTA order), then carry on as usual.
#pragma unroll 1
          for (int hh = 0; hh < Cfg::HALVES && alive; ++hh) {
            const int slot = Cfg::HALVES == 2 ? hh : acc;
            if (!__all_sync(0xffffffffu,
                            ptx::mbar_wait(ptx::smem_u32(&tfull_bar[slot]), acc_phase, abort_flag)))
              alive = false;
          }
          if (!alive) break;
          ptx::tc_fence_after();
          const uint32_t t_row = t_row0 + (Cfg::HALVES == 2 ? 0u : static_cast<uint32_t>(acc * BN));
          const int tile_end = (w.tile - p.sk_first_tile + 1) * p.num_kb;
#pragma unroll 1
          for (int u = unit + 1; u < unit_step && sk_span_begin(p, u, unit_step) < tile_end; ++u) {
            const uint32_t *flag = p.sk_flags + (static_cast<size_t>(u) * CTAS + rank) * 8 + e;
            bool here = ptx::ld_acquire_gpu(flag) == p.sk_epoch;
            uint64_t t0 = 0;
            for (uint32_t it = 1; !here; ++it) {
              __nanosleep(64);
              here = ptx::ld_acquire_gpu(flag) == p.sk_epoch;
              if (!here && (it & 63u) == 0u) {
                if (*abort_flag != 0u) break;
                const uint64_t now = ptx::globaltimer_ns();
                if (t0 == 0) t0 = now;
                const uint32_t lim_us = abort_flag[1];
                if (now - t0 > (lim_us ? static_cast<uint64_t>(lim_us) * 1000ull : ptx::kWaitLimitNs)) {
                  *abort_flag = 1u;
                  break;
                }
              }
            }
            if (!__all_sync(0xffffffffu, here)) {
              alive = false;
              break;
            }
            if (m0 >= p.M) continue;
            const float *theirs = pieces_of(u);
            for (int c32 = 0; c32 < BN / 32; ++c32) {
              if (n0 + c32 * 32 >= p.N) break;
              if (!mine_piece(c32)) continue;
              const float4 *src = reinterpret_cast<const float4 *>(theirs + (c32 * 4 + q) * 1024) + lane;
              float4 add[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) add[j] = __ldcg(src + j * 32);
              uint32_t v[32];
              ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>(c32 * 32), v);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + add[j].x);
                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + add[j].y);
                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + add[j].z);
                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + add[j].w);
              }
              ptx::tmem_st_32x32(t_row + static_cast<uint32_t>(c32 * 32), v);
            }
            ptx::tmem_st_wait();
          }
          if (!alive) break;
        }
      }
      if constexpr (Cfg::HALVES == 2 && EPI == 8) {
        if (out_kind == (DRAIN == 1 ? 1 : 3) && p.ep.acc == nullptr &&
            p.ep.activation == KAPYB_ACT_NONE) {
          // 16-bit output of a two-half tile: drain to registers, store afterwards
          EpiTile et;
          et.tempty_addr = tempty_leader;
          et.remote_arrive = CTAS == 2;
          et.b = b;
          et.m0 = m0;
          et.n0 = n0;
          et.row = row;
          et.lane = lane;
          et.t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
          et.cpart = cpart;
          et.col_begin = 0;
          et.col_end = BN;
          et.stg = stg;
          et.bias_col = bias_col;
          et.bias_fast = bias_fast;
          et.bias_row = 0.0f;
          et.bias_lanes = false;
          et.bias8 = make_uint4(0u, 0u, 0u, 0u);
          et.bias8_hi = make_uint4(0u, 0u, 0u, 0u);
          et.abort_flag = abort_flag;
          et.prof = (kEpilogueProbes && timeline && blockIdx.x == 0 && e == 0) ? p.status + 9 : nullptr;
          if (p.ep.bias != nullptr && p.ep.bias_axis == 0 && row < p.M)
            et.bias_row = load_as_f32(p.ep.bias, p.ep.bias_dtype, row);
          const bool active = m0 < p.M && !debug_on<4>(p.debug);
          const uint32_t tf0 = ptx::smem_u32(&tfull_bar[0]);
          // 12 KB of the operand ring per warp, once the CTA's last tile has let go of it
          static_assert(Cfg::STAGES * Cfg::STAGE_BYTES >= EPI * 12288, "operand ring too small");
          uint8_t *spare = w.last(p) ? smem + e * 12288 : nullptr;
          alive = epilogue_two_halves<EPI, DRAIN>(p, tmC, et, tf0, acc_phase, abort_flag, active, spare);
          if (!alive) break;
          acc_phase ^= 1u;
          continue;
        }
      }
      bool bias_lanes = false;
      uint4 bias8 = make_uint4(0u, 0u, 0u, 0u), bias8_hi = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (Cfg::HALVES == 1 && EPI == 4) {
        if (bias_col && p.ep.bias_dtype == KAPYB_F32 && m0 < p.M) {
          // an f32 bias: eight values per lane in two words of four
          bias_lanes = true;
          const int col = n0 + lane * 8;
          const float *bp = static_cast<const float *>(p.ep.bias);
          uint32_t wv[8];
#pragma unroll
          for (int k = 0; k < 8; ++k)
            wv[k] = (lane * 8 < BN && col + k < p.N) ? __float_as_uint(__ldg(bp + col + k)) : 0u;
          bias8 = make_uint4(wv[0], wv[1], wv[2], wv[3]);
          bias8_hi = make_uint4(wv[4], wv[5], wv[6], wv[7]);
        } else if (bias_col && bias_fast && m0 < p.M) {
          bias_lanes = true;
          const int col = n0 + lane * 8;
          const uint16_t *bp = static_cast<const uint16_t *>(p.ep.bias);
          if (lane * 8 < BN && col + 8 <= p.N) {
            bias8 = __ldg(reinterpret_cast<const uint4 *>(bp + col));
          } else if (lane * 8 < BN) {
            uint32_t wv[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (col + k < p.N) wv[k >> 1] |= static_cast<uint32_t>(__ldg(bp + col + k)) << (16 * (k & 1));
            bias8 = make_uint4(wv[0], wv[1], wv[2], wv[3]);
          }
        }
      }
#pragma unroll 1
      for (int hh = 0; hh < Cfg::HALVES; ++hh) {
        // slot: with two halves, half hh of this tile; otherwise the tile's slot
        const int slot = Cfg::HALVES == 2 ? hh : acc;
        const uint32_t w0 = prof ? static_cast<uint32_t>(clock()) : 0u;
        // warp vote after the wait: the lanes leave together or not at all
        if (!__all_sync(0xffffffffu,
                        ptx::mbar_wait(ptx::smem_u32(&tfull_bar[slot]), acc_phase, abort_flag))) {
          alive = false;
          break;
        }
        if (prof && lane == 0) atomicAdd(prof + 4, static_cast<uint32_t>(clock()) - w0);
        ptx::tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                               (Cfg::HALVES == 2 ? 0u : static_cast<uint32_t>(acc * BN));
        bool handed_back = false;
        const uint32_t slot_bar = tempty_leader + static_cast<uint32_t>(slot * 8);
        if (m0 < p.M && !debug_on<4>(p.debug)) {
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
          et.col_begin = hh * Cfg::SLOT_COLS;
          et.col_end = (hh + 1) * Cfg::SLOT_COLS;
          et.stg = stg;
          et.bias_col = bias_col;
          et.bias_fast = bias_fast;
          et.bias_row = 0.0f;
          et.bias_lanes = bias_lanes;
          et.bias8 = bias8;
          et.bias8_hi = bias8_hi;
          et.abort_flag = abort_flag;
          et.prof = prof;
          if (p.ep.bias != nullptr && p.ep.bias_axis == 0 && row < p.M)
            et.bias_row = load_as_f32(p.ep.bias, p.ep.bias_dtype, row);
          // One specialised copy of the chunk loop per (output kind, plain/full
          // epilogue): the switch runs once per slot, the loops inside are tight.
          switch (out_kind * 2 + (plain ? 1 : 0)) {
          case 0: handed_back = epilogue_tile<BN, EPI, 0, false, REDUCE>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 1: handed_back = epilogue_tile<BN, EPI, 0, true>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 2: handed_back = epilogue_tile<BN, EPI, 1, false, REDUCE>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 3: handed_back = epilogue_tile<BN, EPI, 1, true>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 4: handed_back = epilogue_tile<BN, EPI, 2, false, REDUCE>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 5: handed_back = epilogue_tile<BN, EPI, 2, true>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 6: handed_back = epilogue_tile<BN, EPI, 3, false, REDUCE>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 7: handed_back = epilogue_tile<BN, EPI, 3, true>(p, tmC, et, buf, acc_bar, acc_parity); break;
          case 8: handed_back = epilogue_tile<BN, EPI, 4, false, REDUCE>(p, tmC, et, buf, acc_bar, acc_parity); break;
          default: handed_back = epilogue_tile<BN, EPI, 4, true>(p, tmC, et, buf, acc_bar, acc_parity); break;
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
    if (timeline && lane == 0)
      atomicMax(p.status + 8, static_cast<uint32_t>(ptx::globaltimer_ns()));
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (timeline && blockIdx.x == 0 && threadIdx.x == 0) {
    for (int i = 0; i < 5; ++i) atomicAdd(p.status + 9 + i, prof_words[i]);
  }
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
