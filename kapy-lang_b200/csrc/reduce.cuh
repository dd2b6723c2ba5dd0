// kapy.reduce over a whole 2-D tensor (Ops.td:441-457).  The reference folds
// within a lane, then butterflies across the warp with shfl.sync.bfly
// (ReduceOpToLLVM.cpp:76-119); here one warp owns one row (axis 1), reads it
// with 256-bit coalesced loads, folds in registers and finishes with the same
// xor-shuffle tree.
//
// The lambda runs at the element type of the tensor it reduces
// (ReduceOpToLLVM.cpp:76-119 calls the region on values of that type).  When
// the destination is f32 the source is widened first (arith.extf ahead of the
// reduce) and the combiner works in f32.  When source and destination are the
// same 16-bit type (reduce_sum.mlir:10-25 adds in f16) every combination is
// rounded to that type, as the reference's add.f16 / fma.rn.bf16 would: the
// accumulators then hold values of the 16-bit type at every step (NARROW).
#pragma once

#include "common.cuh"

namespace kapyb {

struct ReduceParams {
  const void *src;  // element (0,0)
  void *dst;        // element 0
  int rows, cols;   // rows = number of results, cols = length of each reduction
  long long src_row_stride, src_col_stride, dst_stride;
  int src_dtype, dst_dtype, combiner;
};

// One rounding at a 16-bit type (operands exactly representable in it):
// add = fma(a, 1, b), mul = fma(a, b, -0) as ElementwiseOpToLLVM.cpp:771-892.
template <int DT>
__device__ __forceinline__ float fma16(float a, float b, float c) {
  if constexpr (DT == KAPYB_BF16)
    return __bfloat162float(
        __hfma(__float2bfloat16_rn(a), __float2bfloat16_rn(b), __float2bfloat16_rn(c)));
  else
    return __half2float(__hfma(__float2half_rn(a), __float2half_rn(b), __float2half_rn(c)));
}

// NT: KAPYB_F32 combines in f32; KAPYB_F16 / KAPYB_BF16 round every result to that type.
template <int COMB, int NT = KAPYB_F32>
__device__ __forceinline__ float combine(float a, float b) {
  if constexpr (NT != KAPYB_F32) {
    if (COMB == KAPYB_RED_ADD) return fma16<NT>(a, 1.0f, b);
    if (COMB == KAPYB_RED_MUL) return fma16<NT>(a, b, -0.0f);
  }
  if (COMB == KAPYB_RED_ADD) return __fadd_rn(a, b);
  if (COMB == KAPYB_RED_MUL) return __fmul_rn(a, b);
  if (COMB == KAPYB_RED_MAX) return (a != a || b != b) ? __uint_as_float(0x7fffffffu) : fmaxf(a, b);
  return (a != a || b != b) ? __uint_as_float(0x7fffffffu) : fminf(a, b);
}

template <int COMB>
__device__ __forceinline__ float identity() {
  if (COMB == KAPYB_RED_ADD) return 0.0f;
  if (COMB == KAPYB_RED_MUL) return 1.0f;
  if (COMB == KAPYB_RED_MAX) return __uint_as_float(0xff800000u);
  return __uint_as_float(0x7f800000u);
}

template <int COMB, int NT = KAPYB_F32>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1)
    v = combine<COMB, NT>(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

struct Vec32B {
  uint32_t w[8];
};

// 256-bit streaming load (sm_100): 32 bytes per lane, 1 KB per warp instruction.
__device__ __forceinline__ Vec32B ld_nc_v8(const void *p) {
  Vec32B v;
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]),
                 "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}

template <int COMB, int DT, int NT>
__device__ __forceinline__ float fold_vec(float acc, const Vec32B &v) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if constexpr (DT == KAPYB_F32) {
      acc = combine<COMB, NT>(acc, __uint_as_float(v.w[k]));
    } else {
      float lo, hi;
      unpack2_16<DT>(v.w[k], lo, hi);
      acc = combine<COMB, NT>(combine<COMB, NT>(acc, lo), hi);
    }
  }
  return acc;
}

constexpr int kReduceUnroll = 8;

// One warp per row; the reduced axis is contiguous.  VEC: every row starts on a
// 32-byte boundary, so the row is read with 256-bit loads, eight in flight per
// lane (8 KB per warp: one whole row of 4096 16-bit values).  !VEC: scalar loads
// with any strides.  NARROW: combine at DT (a 16-bit type) with a rounding per step.
// Order of combination (fixed, so a result is the same bits from run to run):
// lane l folds its elements in ascending order into up to four accumulators,
// which are joined as (a0 + a1) + (a2 + a3); the lanes then meet in a butterfly
// over lane distances 16, 8, 4, 2, 1.
template <int COMB, bool VEC, int DT, bool NARROW = false>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const ReduceParams p) {
  constexpr int NT = NARROW ? DT : KAPYB_F32;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long warp_global =
      static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const long long warp_step = static_cast<long long>(gridDim.x) * warps_per_block;
  constexpr int esz = DT == KAPYB_F32 ? 4 : 2;
  for (long long row = warp_global; row < p.rows; row += warp_step) {
    const char *base = static_cast<const char *>(p.src) + row * p.src_row_stride * esz;
    float acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = identity<COMB>();
    if constexpr (VEC) {
      constexpr int per = 32 / esz;
      const int n_vec = p.cols / per;
      int i = lane;
      for (; i + 32 * (kReduceUnroll - 1) < n_vec; i += 32 * kReduceUnroll) {
        Vec32B v[kReduceUnroll];
#pragma unroll
        for (int u = 0; u < kReduceUnroll; ++u) v[u] = ld_nc_v8(base + (i + 32 * u) * 32ll);
#pragma unroll
        for (int u = 0; u < kReduceUnroll; ++u) acc[u & 3] = fold_vec<COMB, DT, NT>(acc[u & 3], v[u]);
      }
      for (; i < n_vec; i += 32) acc[0] = fold_vec<COMB, DT, NT>(acc[0], ld_nc_v8(base + i * 32ll));
      for (int e = n_vec * per + lane; e < p.cols; e += 32)
        acc[1] = combine<COMB, NT>(acc[1], load_as_f32(base, DT, e));
    } else {
      for (int e = lane; e < p.cols; e += 32)
        acc[0] = combine<COMB, NT>(acc[0], load_as_f32(base, DT, e * p.src_col_stride));
    }
    float r = combine<COMB, NT>(combine<COMB, NT>(acc[0], acc[1]), combine<COMB, NT>(acc[2], acc[3]));
    r = warp_reduce<COMB, NT>(r);
    if (lane == 0) store_from_f32(p.dst, p.dst_dtype, row * p.dst_stride, r, 1);
  }
}

// Reduction along the strided axis (column results of a row-major tensor):
// 32 consecutive results per warp so loads stay coalesced; the 8 warps of a
// block split the reduced axis and meet in shared memory.
// NT as in combine(): KAPYB_F32, or the 16-bit type every combination is rounded to.
template <int COMB, int NT = KAPYB_F32>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const ReduceParams p) {
  __shared__ float part[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (long long r0 = static_cast<long long>(blockIdx.x) * 32; r0 < p.rows;
       r0 += static_cast<long long>(gridDim.x) * 32) {
    const long long r = r0 + lane;
    float acc = identity<COMB>();
    if (r < p.rows) {
      for (int e = w; e < p.cols; e += 8)
        acc = combine<COMB, NT>(acc, load_as_f32(p.src, p.src_dtype,
                                                 r * p.src_row_stride + e * p.src_col_stride));
    }
    part[w][lane] = acc;
    __syncthreads();
    if (w == 0 && r < p.rows) {
      float t = part[0][lane];
#pragma unroll
      for (int k = 1; k < 8; ++k) t = combine<COMB, NT>(t, part[k][lane]);
      store_from_f32(p.dst, p.dst_dtype, r * p.dst_stride, t, 1);
    }
    __syncthreads();
  }
}

// The same reduction for a source whose RESULT axis has the unit stride (column
// sums of a row-major matrix), first pass: the reduced axis is cut into slabs
// (grid.y) so that the whole GPU streams, a lane covers EPL adjacent results with
// one 16-byte load per reduced step and keeps four loads in flight, and the eight
// warps of a block share a slab's steps.  Writes one f32 row of partial results
// per slab (values already rounded to NT where NT is a 16-bit type); the kernel
// above finishes over the slabs.  (reduce_cols_kernel alone moved 0.2-0.5 TB/s on
// a 65536 x 4096 source: 64-byte requests, one dependent chain per thread, 128
// blocks.)
template <int COMB, int DT, int NT>
__global__ void __launch_bounds__(256)
reduce_cols_slab_kernel(const void *src, long long step_bytes, int results, int reduced,
                        int slab_len, float *partial) {
  constexpr int EPL = DT == KAPYB_F32 ? 4 : 8;  // results per lane: one 16-byte load
  __shared__ float part[8][32 * EPL + 4];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int r0 = (blockIdx.x * 32 + lane) * EPL;
  const int e0 = blockIdx.y * slab_len, e1 = min(reduced, e0 + slab_len);
  float acc[EPL];
#pragma unroll
  for (int k = 0; k < EPL; ++k) acc[k] = identity<COMB>();
  auto take = [&](const uint4 &q) {
    if constexpr (DT == KAPYB_F32) {
      acc[0] = combine<COMB, NT>(acc[0], __uint_as_float(q.x));
      acc[1] = combine<COMB, NT>(acc[1], __uint_as_float(q.y));
      acc[2] = combine<COMB, NT>(acc[2], __uint_as_float(q.z));
      acc[3] = combine<COMB, NT>(acc[3], __uint_as_float(q.w));
    } else {
      const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float lo, hi;
        unpack2_16<DT>(ws[t], lo, hi);
        acc[2 * t] = combine<COMB, NT>(acc[2 * t], lo);
        acc[2 * t + 1] = combine<COMB, NT>(acc[2 * t + 1], hi);
      }
    }
  };
  if (r0 < results) {  // results is a multiple of EPL: a lane is inside or outside as a whole
    const char *base = static_cast<const char *>(src) + static_cast<size_t>(r0) * (DT == KAPYB_F32 ? 4 : 2);
    int e = e0 + w;
    for (; e + 24 < e1; e += 32) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        q[u] = __ldcs(reinterpret_cast<const uint4 *>(base + static_cast<long long>(e + 8 * u) * step_bytes));
#pragma unroll
      for (int u = 0; u < 4; ++u) take(q[u]);
    }
    for (; e < e1; e += 8)
      take(__ldcs(reinterpret_cast<const uint4 *>(base + static_cast<long long>(e) * step_bytes)));
  }
#pragma unroll
  for (int k = 0; k < EPL; ++k) part[w][lane * EPL + k] = acc[k];
  __syncthreads();
  for (int t = threadIdx.x; t < 32 * EPL; t += 256) {
    const int r = blockIdx.x * 32 * EPL + t;
    if (r < results) {
      float v = part[0][t];
#pragma unroll
      for (int k = 1; k < 8; ++k) v = combine<COMB, NT>(v, part[k][t]);
      partial[static_cast<size_t>(blockIdx.y) * results + r] = v;
    }
  }
}

}  // namespace kapyb
