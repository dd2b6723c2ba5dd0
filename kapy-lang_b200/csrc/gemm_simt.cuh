// CUDA-core matmul for operands the TMA path cannot describe (a base address or
// a leading dimension that is not a multiple of 16 bytes, or two non-unit
// strides).  Same arithmetic contract as the tcgen05 kernel: operands widened
// exactly to f32, products accumulated in f32 in ascending k, fused epilogue.
// It is a correctness path, not a fast one.
#pragma once

#include "common.cuh"

namespace kapyb {

struct SimtGemmParams {
  const void *a;
  const void *b;
  void *c;
  int M, N, K, batch;
  long long a_s0, a_s1, a_bs;  // element strides (row, column, batch)
  long long b_s0, b_s1, b_bs;
  long long c_s0, c_s1, c_bs;
  int in_dtype, in_dtype_b, out_dtype;
  int tf32;  // f32 operands multiplied as tf32: the low 13 mantissa bits are dropped
  EpilogueArgs ep;
};

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;

__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtGemmParams p) {
  __shared__ float sa[kSimtK][kSimtTile + 1];
  __shared__ float sb[kSimtK][kSimtTile + 1];
  const int bz = blockIdx.z;
  const int m0 = blockIdx.y * kSimtTile, n0 = blockIdx.x * kSimtTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < p.K; k0 += kSimtK) {
    for (int e = threadIdx.x; e < kSimtK * kSimtTile; e += 256) {
      const int kk = e / kSimtTile, mm = e % kSimtTile;
      const int gm = m0 + mm, gk = k0 + kk;
      float va = 0.0f;
      if (gm < p.M && gk < p.K)
        va = load_as_f32(p.a, p.in_dtype, bz * p.a_bs + gm * p.a_s0 + gk * p.a_s1);
      if (p.tf32) va = __uint_as_float(__float_as_uint(va) & 0xffffe000u);
      sa[kk][mm] = va;
      const int gn = n0 + mm;
      float vb = 0.0f;
      if (gn < p.N && gk < p.K)
        vb = load_as_f32(p.b, p.in_dtype_b, bz * p.b_bs + gk * p.b_s0 + gn * p.b_s1);
      if (p.tf32) vb = __uint_as_float(__float_as_uint(vb) & 0xffffe000u);
      sb[kk][mm] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtK; ++kk) {
      float ra[4], rb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) ra[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) rb[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(ra[i], rb[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= p.N) continue;
      float v = acc[i][j] * p.ep.alpha;
      if (p.ep.bias != nullptr)
        v += load_as_f32(p.ep.bias, p.ep.bias_dtype, p.ep.bias_axis == 1 ? gn : gm);
      if (p.ep.acc != nullptr)
        v += load_as_f32(p.ep.acc, p.ep.acc_dtype,
                         bz * p.ep.acc_batch_stride + gm * p.ep.acc_stride0 +
                             gn * p.ep.acc_stride1);
      v = apply_activation(p.ep.activation, v);
      store_from_f32(p.c, p.out_dtype, bz * p.c_bs + gm * p.c_s0 + gn * p.c_s1, v,
                     p.ep.rounding);
    }
  }
}

}  // namespace kapyb
