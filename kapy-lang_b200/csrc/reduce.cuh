// kapy.reduce over a whole 2-D tensor (Ops.td:441-457).  The reference folds
// within a lane, then butterflies across the warp with shfl.sync.bfly
// (ReduceOpToLLVM.cpp:76-119); here one warp owns one row (axis 1), reads it
// with 128-bit coalesced loads, folds in registers and finishes with the same
// xor-shuffle tree.  Values are widened to f32 before combining; a 16-bit
// destination is rounded once at the end.
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

template <int COMB>
__device__ __forceinline__ float combine(float a, float b) {
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

template <int COMB>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = combine<COMB>(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

__device__ __forceinline__ uint4 ld_nc_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int COMB>
__device__ __forceinline__ float fold_word16(float acc, uint32_t w, int dt) {
  acc = combine<COMB>(acc, cvt_16_to_f32(static_cast<uint16_t>(w & 0xffffu), dt));
  return combine<COMB>(acc, cvt_16_to_f32(static_cast<uint16_t>(w >> 16), dt));
}

// One warp per row; rows are contiguous along the reduced axis and every row
// starts on a 16-byte boundary (VEC) or anything else (!VEC).
template <int COMB, bool VEC>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const ReduceParams p) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long warp_global = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const long long warp_step = static_cast<long long>(gridDim.x) * warps_per_block;
  const int esz = dtype_size(p.src_dtype);
  for (long long row = warp_global; row < p.rows; row += warp_step) {
    const char *base = static_cast<const char *>(p.src) + row * p.src_row_stride * esz;
    float acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = identity<COMB>();
    if (VEC) {
      const int per = 16 / esz;
      const int n_vec = p.cols / per;
      const uint4 *v = reinterpret_cast<const uint4 *>(base);
      int i = lane;
      for (; i + 96 < n_vec; i += 128) {
        uint4 w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) w[u] = ld_nc_v4(v + i + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (p.src_dtype == KAPYB_F32) {
            acc[u] = combine<COMB>(acc[u], __uint_as_float(w[u].x));
            acc[u] = combine<COMB>(acc[u], __uint_as_float(w[u].y));
            acc[u] = combine<COMB>(acc[u], __uint_as_float(w[u].z));
            acc[u] = combine<COMB>(acc[u], __uint_as_float(w[u].w));
          } else {
            acc[u] = fold_word16<COMB>(acc[u], w[u].x, p.src_dtype);
            acc[u] = fold_word16<COMB>(acc[u], w[u].y, p.src_dtype);
            acc[u] = fold_word16<COMB>(acc[u], w[u].z, p.src_dtype);
            acc[u] = fold_word16<COMB>(acc[u], w[u].w, p.src_dtype);
          }
        }
      }
      for (; i < n_vec; i += 32) {
        const uint4 w = ld_nc_v4(v + i);
        if (p.src_dtype == KAPYB_F32) {
          acc[0] = combine<COMB>(acc[0], __uint_as_float(w.x));
          acc[0] = combine<COMB>(acc[0], __uint_as_float(w.y));
          acc[0] = combine<COMB>(acc[0], __uint_as_float(w.z));
          acc[0] = combine<COMB>(acc[0], __uint_as_float(w.w));
        } else {
          acc[0] = fold_word16<COMB>(acc[0], w.x, p.src_dtype);
          acc[0] = fold_word16<COMB>(acc[0], w.y, p.src_dtype);
          acc[0] = fold_word16<COMB>(acc[0], w.z, p.src_dtype);
          acc[0] = fold_word16<COMB>(acc[0], w.w, p.src_dtype);
        }
      }
      for (int e = n_vec * per + lane; e < p.cols; e += 32)
        acc[1] = combine<COMB>(acc[1], load_as_f32(base, p.src_dtype, e));
    } else {
      for (int e = lane; e < p.cols; e += 32)
        acc[0] = combine<COMB>(acc[0], load_as_f32(base, p.src_dtype, e * p.src_col_stride));
    }
    float r = combine<COMB>(combine<COMB>(acc[0], acc[1]), combine<COMB>(acc[2], acc[3]));
    r = warp_reduce<COMB>(r);
    if (lane == 0) store_from_f32(p.dst, p.dst_dtype, row * p.dst_stride, r, 1);
  }
}

// Reduction along the strided axis (column results of a row-major tensor):
// 32 consecutive results per warp so loads stay coalesced; the 8 warps of a
// block split the reduced axis and meet in shared memory.
template <int COMB>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const ReduceParams p) {
  __shared__ float part[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (long long r0 = static_cast<long long>(blockIdx.x) * 32; r0 < p.rows;
       r0 += static_cast<long long>(gridDim.x) * 32) {
    const long long r = r0 + lane;
    float acc = identity<COMB>();
    if (r < p.rows) {
      for (int e = w; e < p.cols; e += 8)
        acc = combine<COMB>(acc, load_as_f32(p.src, p.src_dtype,
                                             r * p.src_row_stride + e * p.src_col_stride));
    }
    part[w][lane] = acc;
    __syncthreads();
    if (w == 0 && r < p.rows) {
      float t = part[0][lane];
#pragma unroll
      for (int k = 1; k < 8; ++k) t = combine<COMB>(t, part[k][lane]);
      store_from_f32(p.dst, p.dst_dtype, r * p.dst_stride, t, 1);
    }
    __syncthreads();
  }
}

}  // namespace kapyb
