// Device helpers shared by every kernel: element loads/stores at the three
// element types, the arithmetic primitives whose rounding kapy's lowering fixes,
// and the fused activations.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kapyb.h"

namespace kapyb {

// Status word layout (one uint32 in device memory per handle).
enum : uint32_t { kStatusOk = 0, kStatusTimeout = 1 };

__host__ __device__ inline int dtype_size(int dtype) {
  return dtype == KAPYB_F32 ? 4 : (dtype == KAPYB_F8E4M3 || dtype == KAPYB_F8E5M2) ? 1 : 2;
}

// ---- primitives with the reference's instruction choice --------------------

// math.exp on f32 = ex2.approx.f32(x * log2(e))  (ElementwiseOpToLLVM.cpp:1039-1073)
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float kapy_exp(float x) {
  return ex2_approx(__fmul_rn(x, 1.4426950408889634f));
}
// arith.divf on f32 = div.full.f32  (ElementwiseOpToLLVM.cpp:730-769)
__device__ __forceinline__ float div_full(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// gelu_tanh as the cancellation-free composite u / (1 + exp(-2k)),
// k = c0 * fma(c1*u*u, u, u).  Every step is an explicit single-rounding f32 op
// so the rounding points are those of the op-by-op graph.
__device__ __forceinline__ float gelu_tanh_f32(float u) {
  const float c0 = 0.7978845608f, c1 = 0.044715f;
  float t = __fmul_rn(__fmul_rn(c1, u), u);
  float k = __fmul_rn(c0, __fmaf_rn(t, u, u));
  float e = kapy_exp(__fmul_rn(-2.0f, k));
  return div_full(u, __fadd_rn(1.0f, e));
}

// The same with the activation known at compile time (callers that finish many
// values at once branch once per group, not once per value).
template <int ACT>
__device__ __forceinline__ float apply_activation_t(float v) {
  if constexpr (ACT == KAPYB_ACT_RELU) return v > 0.0f ? v : (v != v ? v : 0.0f);
  if constexpr (ACT == KAPYB_ACT_GELU_TANH) return gelu_tanh_f32(v);
  if constexpr (ACT == KAPYB_ACT_SILU) return div_full(v, __fadd_rn(1.0f, kapy_exp(-v)));
  return v;
}

__device__ __forceinline__ float apply_activation(int act, float v) {
  switch (act) {
  case KAPYB_ACT_RELU: return v > 0.0f ? v : (v != v ? v : 0.0f);
  case KAPYB_ACT_GELU_TANH: return gelu_tanh_f32(v);
  case KAPYB_ACT_SILU: return div_full(v, __fadd_rn(1.0f, kapy_exp(-v)));
  default: return v;
  }
}

// ---- conversions (cvt.{rn,rz}.{bf16,f16}.f32, ElementwiseOpToLLVM.cpp:381-417)

__device__ __forceinline__ uint16_t cvt_f32_to_16(float v, int dtype, int rn) {
  uint16_t r;
  if (dtype == KAPYB_BF16) {
    if (rn)
      asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(v));
    else
      asm("cvt.rz.bf16.f32 %0, %1;" : "=h"(r) : "f"(v));
  } else {
    if (rn)
      asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
    else
      asm("cvt.rz.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
  }
  return r;
}

// Two floats -> one packed 32-bit word (lo in bits [0,16)).
__device__ __forceinline__ uint32_t cvt_pack2(float lo, float hi, int dtype, int rn) {
  uint32_t r;
  if (dtype == KAPYB_BF16) {
    if (rn)
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else
      asm("cvt.rz.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    if (rn)
      asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else
      asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

// Compile-time variants for hot loops (a run-time dtype inside an unrolled loop
// turns into four predicated conversions per value).
template <int DT, int RN>
__device__ __forceinline__ uint32_t cvt_pack2_t(float lo, float hi) {
  uint32_t r;
  if constexpr (DT == KAPYB_BF16) {
    if constexpr (RN)
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else
      asm("cvt.rz.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    if constexpr (RN)
      asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else
      asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

// Both halves of a packed 16-bit pair, widened exactly.
template <int DT>
__device__ __forceinline__ void unpack2_16(uint32_t w, float &lo, float &hi) {
  if constexpr (DT == KAPYB_BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    lo = f.x;
    hi = f.y;
  }
}

__device__ __forceinline__ float cvt_16_to_f32(uint16_t h, int dtype) {
  if (dtype == KAPYB_BF16) return __uint_as_float(static_cast<uint32_t>(h) << 16);
  return __half2float(__ushort_as_half(h));
}

// fp8 -> f32, exact (E4M3 has no infinities; its all-ones pattern is NaN).
__device__ __forceinline__ float cvt_fp8_to_f32(uint8_t v, int dtype) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(
      static_cast<__nv_fp8_storage_t>(v), dtype == KAPYB_F8E4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(__half(h));
}

// f32 -> fp8, the reference's down casts (ElementwiseOpToLLVM.cpp:83-289, :583-650):
// rn = cvt.rn.satfinite (beyond the largest finite value, infinities included, gives
// that value; NaN stays NaN); rz exists for E5M2 only and is the high byte of the
// value truncated to f16.
__device__ __forceinline__ uint8_t cvt_f32_to_fp8(float v, int dtype, int rn) {
  uint16_t r;
  if (dtype == KAPYB_F8E4M3) {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
    return static_cast<uint8_t>(r & 0xffu);
  }
  if (rn) {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
    return static_cast<uint8_t>(r & 0xffu);
  }
  asm("cvt.rz.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
  return static_cast<uint8_t>(r >> 8);
}

__device__ __forceinline__ bool is_fp8_dtype(int dtype) {
  return dtype == KAPYB_F8E4M3 || dtype == KAPYB_F8E5M2;
}

__device__ __forceinline__ float load_as_f32(const void *base, int dtype, int64_t idx) {
  if (dtype == KAPYB_F32) return static_cast<const float *>(base)[idx];
  if (dtype == KAPYB_F8E4M3 || dtype == KAPYB_F8E5M2)
    return cvt_fp8_to_f32(static_cast<const uint8_t *>(base)[idx], dtype);
  return cvt_16_to_f32(static_cast<const uint16_t *>(base)[idx], dtype);
}

__device__ __forceinline__ void store_from_f32(void *base, int dtype, int64_t idx, float v,
                                               int rn) {
  if (dtype == KAPYB_F32)
    static_cast<float *>(base)[idx] = v;
  else if (is_fp8_dtype(dtype))
    static_cast<uint8_t *>(base)[idx] = cvt_f32_to_fp8(v, dtype, rn);
  else
    static_cast<uint16_t *>(base)[idx] = cvt_f32_to_16(v, dtype, rn);
}

// Epilogue parameters as the kernels see them.
struct EpilogueArgs {
  float alpha;
  const void *bias;
  int bias_dtype;
  int bias_axis;
  int activation;
  int rounding;
  const void *acc;  // optional [M,N] addend (already offset to element 0,0)
  int acc_dtype;
  long long acc_stride0, acc_stride1, acc_batch_stride;
};

}  // namespace kapyb
