// Elementwise kernels.
//
//  * elt_interp_kernel: executes a recorded op list per element with a rounding
//    to the op's element type after every op -- the semantics of the reference's
//    per-op lowering (ElementwiseOpToLLVM.cpp:424-485; bf16/f16 mul/add/sub/fma
//    as single-rounding fma, :771-892).  Handles any strides, broadcast inputs
//    and out-of-bounds padding.  Correct for every valid program; not tuned.
//  * elt_unary16_kernel / elt_binary_kernel: the same op sequences for the
//    canonical graphs, as streaming kernels with 128-bit coalesced accesses.
//    They execute exactly the ops the interpreter would, in the same order, so
//    both produce identical bits.
#pragma once

#include "common.cuh"

namespace kapyb {

struct EltTensor {
  const void *ptr;  // element (0,0)
  long long s0, s1;
  int size0, size1;
  int dtype;
  int padding;
  int cache;        // KAPYB_CACHE_HINTS of the ld_global / st_global on this tensor
};

// ld.global / st.global in the forms the reference emits for a cache operator or
// an eviction priority (LdGlobalOpToLLVM.cpp:101-110, StGlobalOpToLLVM.cpp:100-108):
// volatile wins, then the cache operator, then "L1::<priority>".  A hint never
// changes the value moved.
// X(form index, qualifier before ".global", qualifier after it)
#define KAPYB_LD_FORMS(X)                                                                    \
  X(0, "", "") X(1, "", ".ca") X(2, "", ".cg") X(3, "", ".cs") X(4, "", ".lu") X(5, "", ".cv") \
  X(6, ".volatile", "") X(7, "", ".L1::evict_first") X(8, "", ".L1::evict_last")             \
  X(9, "", ".L1::evict_unchanged") X(10, "", ".L1::no_allocate")
#define KAPYB_ST_FORMS(X)                                                                    \
  X(0, "", "") X(1, "", ".wb") X(2, "", ".cg") X(3, "", ".cs") X(4, "", ".wt")               \
  X(6, ".volatile", "") X(7, "", ".L1::evict_first") X(8, "", ".L1::evict_last")             \
  X(9, "", ".L1::evict_unchanged") X(10, "", ".L1::no_allocate")

// form index of a load (0 = plain) from the packed hints
__host__ __device__ inline int ld_form(int cache) {
  if (cache & (1 << 16)) return 6;
  switch (cache & 0xff) {
  case KAPYB_CACHE_CA: return 1;
  case KAPYB_CACHE_CG: return 2;
  case KAPYB_CACHE_CS: return 3;
  case KAPYB_CACHE_LU: return 4;
  case KAPYB_CACHE_CV: return 5;
  default: break;  // NONE; WB / WT are store operators
  }
  switch ((cache >> 8) & 0xff) {
  case KAPYB_EVICT_FIRST: return 7;
  case KAPYB_EVICT_LAST: return 8;
  case KAPYB_EVICT_UNCHANGED: return 9;
  case KAPYB_NO_ALLOCATE: return 10;
  default: return 0;
  }
}
__host__ __device__ inline int st_form(int cache) {
  if (cache & (1 << 16)) return 6;
  switch (cache & 0xff) {
  case KAPYB_CACHE_WB: return 1;
  case KAPYB_CACHE_CG: return 2;
  case KAPYB_CACHE_CS: return 3;
  case KAPYB_CACHE_WT: return 4;
  default: break;  // NONE; CA / LU / CV are load operators
  }
  switch ((cache >> 8) & 0xff) {
  case KAPYB_EVICT_FIRST: return 7;
  case KAPYB_EVICT_LAST: return 8;
  case KAPYB_EVICT_UNCHANGED: return 9;
  case KAPYB_NO_ALLOCATE: return 10;
  default: return 0;
  }
}

// the bits of one element (8, 16 or 32 of them), loaded / stored with form `form`
__device__ __forceinline__ uint32_t ld_bits_form(const void *p, int bytes, int form) {
  uint32_t v = 0;
  uint16_t h = 0;
#define KAPYB_X(ID, PRE, POST)                                                                    \
  case ID:                                                                                  \
    if (bytes == 4)                                                                         \
      asm volatile("ld" PRE ".global" POST ".u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");      \
    else if (bytes == 2) {                                                                  \
      asm volatile("ld" PRE ".global" POST ".u16 %0, [%1];" : "=h"(h) : "l"(p) : "memory");      \
      v = h;                                                                                \
    } else {                                                                                \
      asm volatile("ld" PRE ".global" POST ".u8 %0, [%1];" : "=h"(h) : "l"(p) : "memory");       \
      v = h & 0xffu;                                                                        \
    }                                                                                       \
    break;
  switch (form) { KAPYB_LD_FORMS(KAPYB_X) default: break; }
#undef KAPYB_X
  return v;
}
__device__ __forceinline__ void st_bits_form(void *p, int bytes, int form, uint32_t v) {
  const uint16_t h = static_cast<uint16_t>(v);
#define KAPYB_X(ID, PRE, POST)                                                                    \
  case ID:                                                                                  \
    if (bytes == 4)                                                                         \
      asm volatile("st" PRE ".global" POST ".u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");         \
    else if (bytes == 2)                                                                    \
      asm volatile("st" PRE ".global" POST ".u16 [%0], %1;" ::"l"(p), "h"(h) : "memory");         \
    else                                                                                    \
      asm volatile("st" PRE ".global" POST ".u8 [%0], %1;" ::"l"(p), "h"(h) : "memory");          \
    break;
  switch (form) { KAPYB_ST_FORMS(KAPYB_X) default: break; }
#undef KAPYB_X
}

__device__ __forceinline__ float load_as_f32_form(const void *base, int dtype, long long idx,
                                                  int form) {
  if (form == 0) return load_as_f32(base, dtype, idx);
  const int bytes = dtype_size(dtype);
  const uint32_t v = ld_bits_form(static_cast<const char *>(base) + idx * bytes, bytes, form);
  if (dtype == KAPYB_F32) return __uint_as_float(v);
  if (is_fp8_dtype(dtype)) return cvt_fp8_to_f32(static_cast<uint8_t>(v), dtype);
  return cvt_16_to_f32(static_cast<uint16_t>(v), dtype);
}
__device__ __forceinline__ void store_from_f32_form(void *base, int dtype, long long idx, float x,
                                                    int rn, int form) {
  if (form == 0) {
    store_from_f32(base, dtype, idx, x, rn);
    return;
  }
  const int bytes = dtype_size(dtype);
  uint32_t v;
  if (dtype == KAPYB_F32)
    v = __float_as_uint(x);
  else if (is_fp8_dtype(dtype))
    v = cvt_f32_to_fp8(x, dtype, rn);
  else
    v = cvt_f32_to_16(x, dtype, rn);
  st_bits_form(static_cast<char *>(base) + idx * bytes, bytes, form, v);
}

struct EltProgram {
  kapyb_inst inst[KAPYB_MAX_INSTS];
  int n_inst;
  EltTensor in[KAPYB_MAX_INPUTS];
  int n_in;
  EltTensor out;
};

__device__ __forceinline__ float round_to_dtype(float v, int dtype, int rn) {
  if (dtype == KAPYB_F32) return v;
  if (is_fp8_dtype(dtype)) return cvt_fp8_to_f32(cvt_f32_to_fp8(v, dtype, rn), dtype);
  return cvt_16_to_f32(cvt_f32_to_16(v, dtype, rn), dtype);
}

// a*b + c with ONE rounding at `dtype`; operands are exactly representable.
__device__ __forceinline__ float fma_at(float a, float b, float c, int dtype) {
  if (dtype == KAPYB_F32) return __fmaf_rn(a, b, c);
  if (dtype == KAPYB_BF16)
    return __bfloat162float(
        __hfma(__float2bfloat16_rn(a), __float2bfloat16_rn(b), __float2bfloat16_rn(c)));
  return __half2float(__hfma(__float2half_rn(a), __float2half_rn(b), __float2half_rn(c)));
}

__device__ __forceinline__ float pad_value(int padding) {
  switch (padding) {
  case KAPYB_PAD_QNAN: return __uint_as_float(0x7fffffffu);
  case KAPYB_PAD_PINF: return __uint_as_float(0x7f800000u);
  case KAPYB_PAD_NINF: return __uint_as_float(0xff800000u);
  default: return 0.0f;
  }
}

__device__ __forceinline__ float maximum_f(float a, float b) {
  if (a != a || b != b) return __uint_as_float(0x7fffffffu);
  return fmaxf(a, b);  // fmaxf orders -0 < +0
}
__device__ __forceinline__ float minimum_f(float a, float b) {
  if (a != a || b != b) return __uint_as_float(0x7fffffffu);
  return fminf(a, b);
}

// arith.cmpf: ordered predicates are false, unordered ones true, when an operand is NaN.
__device__ __forceinline__ bool cmp_f(int pred, float a, float b) {
  const bool un = a != a || b != b;
  switch (pred) {
  case KAPYB_CMP_OLT: return a < b;
  case KAPYB_CMP_OGT: return a > b;
  case KAPYB_CMP_OLE: return a <= b;
  case KAPYB_CMP_OGE: return a >= b;
  case KAPYB_CMP_OEQ: return a == b;
  case KAPYB_CMP_ONE: return !un && a != b;
  case KAPYB_CMP_ULT: return un || a < b;
  case KAPYB_CMP_UGT: return un || a > b;
  case KAPYB_CMP_ULE: return un || a <= b;
  case KAPYB_CMP_UGE: return un || a >= b;
  case KAPYB_CMP_UEQ: return un || a == b;
  default: return un || a != b;  // UNE
  }
}

__device__ float interp_one(const EltProgram &P, int i, int j, bool *stored, float *store_val) {
  float r[KAPYB_MAX_REGS];
#pragma unroll
  for (int t = 0; t < KAPYB_MAX_REGS; ++t) r[t] = 0.0f;
  float last = 0.0f;
  for (int pc = 0; pc < P.n_inst; ++pc) {
    const kapyb_inst in = P.inst[pc];
    const float a = in.a >= 0 ? r[in.a & (KAPYB_MAX_REGS - 1)] : 0.0f;
    const float b = in.b >= 0 ? r[in.b & (KAPYB_MAX_REGS - 1)] : 0.0f;
    const float c = in.c >= 0 ? r[in.c & (KAPYB_MAX_REGS - 1)] : 0.0f;
    float v = 0.0f;
    const int dt = in.dtype;
    switch (in.op) {
    case KAPYB_OP_LOAD: {
      const EltTensor &t = P.in[in.flags & (KAPYB_MAX_INPUTS - 1)];
      const int ii = t.size0 == 1 ? 0 : i, jj = t.size1 == 1 ? 0 : j;
      if (ii >= t.size0 || jj >= t.size1)
        v = pad_value(t.padding);
      else
        v = load_as_f32_form(t.ptr, t.dtype, ii * t.s0 + jj * t.s1, ld_form(t.cache));
      break;
    }
    case KAPYB_OP_CONST: v = round_to_dtype(in.imm, dt, 1); break;
    case KAPYB_OP_CVT: v = round_to_dtype(a, dt, in.flags); break;
    case KAPYB_OP_ADD: v = dt == KAPYB_F32 ? __fadd_rn(a, b) : fma_at(a, 1.0f, b, dt); break;
    case KAPYB_OP_SUB: v = dt == KAPYB_F32 ? __fsub_rn(a, b) : fma_at(b, -1.0f, a, dt); break;
    case KAPYB_OP_MUL: v = dt == KAPYB_F32 ? __fmul_rn(a, b) : fma_at(a, b, -0.0f, dt); break;
    case KAPYB_OP_FMA: v = fma_at(a, b, c, dt); break;
    case KAPYB_OP_DIV:
      v = dt == KAPYB_F32 ? div_full(a, b) : round_to_dtype(__fdiv_rn(a, b), dt, 1);
      break;
    case KAPYB_OP_MAXIMUM: v = maximum_f(a, b); break;
    case KAPYB_OP_MINIMUM: v = minimum_f(a, b); break;
    case KAPYB_OP_MAXNUM: v = fmaxf(a, b); break;
    case KAPYB_OP_MINNUM: v = fminf(a, b); break;
    case KAPYB_OP_CLAMP:
      v = in.flags ? minimum_f(maximum_f(a, b), c) : fminf(fmaxf(a, b), c);
      break;
    case KAPYB_OP_ABS: v = fabsf(a); break;
    case KAPYB_OP_NEG: v = -a; break;
    case KAPYB_OP_EXP: v = dt == KAPYB_F32 ? kapy_exp(a) : round_to_dtype(expf(a), dt, 1); break;
    case KAPYB_OP_EXP2: v = round_to_dtype(exp2f(a), dt, 1); break;
    case KAPYB_OP_LOG: v = round_to_dtype(logf(a), dt, 1); break;
    case KAPYB_OP_LOG2: v = round_to_dtype(log2f(a), dt, 1); break;
    case KAPYB_OP_SQRT: v = round_to_dtype(__fsqrt_rn(a), dt, 1); break;
    case KAPYB_OP_RSQRT: v = round_to_dtype(rsqrtf(a), dt, 1); break;
    case KAPYB_OP_ERF: v = round_to_dtype(erff(a), dt, 1); break;
    case KAPYB_OP_SIN: v = round_to_dtype(sinf(a), dt, 1); break;
    case KAPYB_OP_COS: v = round_to_dtype(cosf(a), dt, 1); break;
    case KAPYB_OP_FLOOR: v = floorf(a); break;
    case KAPYB_OP_CEIL: v = ceilf(a); break;
    case KAPYB_OP_TANH: v = round_to_dtype(tanhf(a), dt, 1); break;
    case KAPYB_OP_STORE:
      *stored = true;
      *store_val = a;
      break;
    // conditions (i1) live in the float registers as 0 / 1
    case KAPYB_OP_CMP: v = cmp_f(in.flags, a, b) ? 1.0f : 0.0f; break;
    case KAPYB_OP_SELECT: v = a != 0.0f ? b : c; break;
    case KAPYB_OP_AND: v = (a != 0.0f && b != 0.0f) ? 1.0f : 0.0f; break;
    case KAPYB_OP_OR: v = (a != 0.0f || b != 0.0f) ? 1.0f : 0.0f; break;
    case KAPYB_OP_XOR: v = ((a != 0.0f) != (b != 0.0f)) ? 1.0f : 0.0f; break;
    default: break;
    }
    if (in.op != KAPYB_OP_STORE && in.dst >= 0) r[in.dst & (KAPYB_MAX_REGS - 1)] = v;
    last = v;
  }
  return last;
}

__global__ void __launch_bounds__(256) elt_interp_kernel(const EltProgram P) {
  const long long total = static_cast<long long>(P.out.size0) * P.out.size1;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
       e += step) {
    // walk along the unit-stride axis of the output for coalescing
    int i, j;
    if (P.out.s1 == 1 || P.out.size0 == 1) {
      i = static_cast<int>(e / P.out.size1);
      j = static_cast<int>(e - static_cast<long long>(i) * P.out.size1);
    } else {
      j = static_cast<int>(e / P.out.size0);
      i = static_cast<int>(e - static_cast<long long>(j) * P.out.size0);
    }
    bool stored = false;
    float sv = 0.0f;
    interp_one(P, i, j, &stored, &sv);
    if (stored) {
      void *o = const_cast<void *>(P.out.ptr);
      const long long idx = i * P.out.s0 + j * P.out.s1;
      // the stored register already holds a value of the output's type
      // (f8E5M2: the truncating encoder, which keeps an infinity; the rounding
      // one saturates it)
      store_from_f32_form(o, P.out.dtype, idx, sv, P.out.dtype == KAPYB_F8E5M2 ? 0 : 1,
                          st_form(P.out.cache));
    }
  }
}

// ------------------------------------------------------------ fused kernels

// Packed f32x2 arithmetic (sm_100): each half is an independent IEEE
// round-to-nearest op, so the bits equal those of the scalar instruction; one
// issue slot does the work of two.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// y = cvt16( act( fma(ext(x), s, b) ) ): the "affine (+ gelu_tanh)" graph.
// The gelu constants come from the program so the kernel reproduces whatever
// constants the caller recorded.  Two elements are processed per call, with the
// same op sequence per element as the op-by-op interpreter:
//   u = fma(x,s,b); t = (c1*u)*u; k = c0*fma(t,u,u); e = ex2(( m2*k )*log2e);
//   y = u / (one + e)
struct AffineGelu {
  float s, b;
  int gelu;        // 0: affine only
  float c0, c1;    // k = c0 * fma(c1*u*u, u, u)
  float m2, one;   // y = u / (one + exp(m2 * k))
  int ftz_ok;      // |one| is large enough that a subnormal exp() cannot change one + exp()
  __device__ __forceinline__ float ex2(float z) const {
    // ex2.approx.f32 handles subnormals with extra scaling instructions.  When the
    // sum that follows absorbs any subnormal (one + e == one), the flush-to-zero
    // form gives the same bits for one instruction.
    if (ftz_ok) {
      float r;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(z));
      return r;
    }
    return ex2_approx(z);
  }
  __device__ __forceinline__ void operator()(float &x0, float &x1) const {
    const uint64_t u = fma2(pack2(x0, x1), pack2(s, s), pack2(b, b));
    if (!gelu) {
      unpack2(u, x0, x1);
      return;
    }
    const uint64_t t = mul2(mul2(pack2(c1, c1), u), u);
    const uint64_t k = mul2(pack2(c0, c0), fma2(t, u, u));
    const uint64_t z = mul2(mul2(pack2(m2, m2), k),
                            pack2(1.4426950408889634f, 1.4426950408889634f));
    float z0, z1, u0, u1, d0, d1;
    unpack2(z, z0, z1);
    const uint64_t d = add2(pack2(one, one), pack2(ex2(z0), ex2(z1)));
    unpack2(u, u0, u1);
    unpack2(d, d0, d1);
    x0 = div_full(u0, d0);
    x1 = div_full(u1, d1);
  }
};

__device__ __forceinline__ uint4 ld_stream(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(uint4 *p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

template <class F, int DT, int RN>
__device__ __forceinline__ uint32_t apply2_16(uint32_t w, const F &f) {
  float lo, hi;
  unpack2_16<DT>(w, lo, hi);
  f(lo, hi);
  return cvt_pack2_t<DT, RN>(lo, hi);
}

constexpr int kEltUnroll = 4;

// One streaming access of W x 16 bytes (W = 2 uses the 256-bit ld/st forms).
template <int W>
struct StreamVec {
  uint4 q[W];
};
template <int W>
__device__ __forceinline__ StreamVec<W> ld_stream_vec(const uint4 *p) {
  StreamVec<W> v;
  if constexpr (W == 1) {
    v.q[0] = ld_stream(p);
  } else {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.q[0].x), "=r"(v.q[0].y), "=r"(v.q[0].z), "=r"(v.q[0].w),
                   "=r"(v.q[1].x), "=r"(v.q[1].y), "=r"(v.q[1].z), "=r"(v.q[1].w)
                 : "l"(p));
  }
  return v;
}
template <int W>
__device__ __forceinline__ void st_stream_vec(uint4 *p, const StreamVec<W> &v) {
  if constexpr (W == 1) {
    st_stream(p, v.q[0]);
  } else {
    asm volatile("st.global.cs.v8.u32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p),
                 "r"(v.q[0].x), "r"(v.q[0].y), "r"(v.q[0].z), "r"(v.q[0].w), "r"(v.q[1].x),
                 "r"(v.q[1].y), "r"(v.q[1].z), "r"(v.q[1].w)
                 : "memory");
  }
}

// One 16-bit element type in and out (DT), downcast rounding RN, contiguous;
// both pointers aligned to W x 16 bytes.  n_acc accesses of W*8 elements plus a
// scalar tail handled by the last block.  One block per contiguous chunk of
// kEltUnroll x 256 accesses, as many blocks as there are chunks: the block
// scheduler keeps every SM on neighbouring addresses, which streams about 14 %
// faster from HBM than a resident grid striding through the array.
template <class F, int W, int DT, int RN>
__global__ void __launch_bounds__(256)
elt_unary16_kernel(const uint4 *__restrict__ x, uint4 *__restrict__ y, long long n_acc,
                   long long n_elems, F f) {
  const long long base = static_cast<long long>(blockIdx.x) * (kEltUnroll * 256) + threadIdx.x;
  auto apply = [&](const StreamVec<W> &v) {
    StreamVec<W> o;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      o.q[w].x = apply2_16<F, DT, RN>(v.q[w].x, f);
      o.q[w].y = apply2_16<F, DT, RN>(v.q[w].y, f);
      o.q[w].z = apply2_16<F, DT, RN>(v.q[w].z, f);
      o.q[w].w = apply2_16<F, DT, RN>(v.q[w].w, f);
    }
    return o;
  };
  if (base + (kEltUnroll - 1) * 256 < n_acc) {
    StreamVec<W> v[kEltUnroll];
#pragma unroll
    for (int u = 0; u < kEltUnroll; ++u) v[u] = ld_stream_vec<W>(x + (base + u * 256) * W);
#pragma unroll
    for (int u = 0; u < kEltUnroll; ++u) st_stream_vec<W>(y + (base + u * 256) * W, apply(v[u]));
  } else {
    for (long long i = base; i < n_acc; i += 256)
      st_stream_vec<W>(y + i * W, apply(ld_stream_vec<W>(x + i * W)));
  }
  if (blockIdx.x == gridDim.x - 1) {
    const uint16_t *xs = reinterpret_cast<const uint16_t *>(x);
    uint16_t *ys = reinterpret_cast<uint16_t *>(y);
    for (long long e = n_acc * (8 * W) + threadIdx.x; e < n_elems; e += blockDim.x) {
      float a = cvt_16_to_f32(xs[e], DT), unused = 0.0f;
      f(a, unused);
      ys[e] = cvt_f32_to_16(a, DT, RN);
    }
  }
}

// ------------------------------------------------------------ f8 casts
//
// y = cast(x) where one side is an 8-bit float type: contiguous, both pointers
// 16-byte aligned.  A thread converts 16 consecutive elements (16 to 64 bytes
// on either side, moved as 128-bit vectors); one block per contiguous chunk of
// kCastUnroll x 256 such groups; the last block also does the scalar tail.
constexpr int kCastUnroll = 2;

template <int DT>
__device__ __forceinline__ void load16_as_f32(const uint8_t *p, float (&f)[16]) {
  if constexpr (DT == KAPYB_F32) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint4 v = ld_stream(reinterpret_cast<const uint4 *>(p) + k);
      f[4 * k] = __uint_as_float(v.x);
      f[4 * k + 1] = __uint_as_float(v.y);
      f[4 * k + 2] = __uint_as_float(v.z);
      f[4 * k + 3] = __uint_as_float(v.w);
    }
  } else if constexpr (DT == KAPYB_F16 || DT == KAPYB_BF16) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint4 v = ld_stream(reinterpret_cast<const uint4 *>(p) + k);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) unpack2_16<DT>(w[t], f[8 * k + 2 * t], f[8 * k + 2 * t + 1]);
    }
  } else {
    const uint4 v = ld_stream(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int b = 0; b < 4; ++b)
        f[4 * t + b] = cvt_fp8_to_f32(static_cast<uint8_t>(w[t] >> (8 * b)), DT);
  }
}

template <int DT, int RN>
__device__ __forceinline__ void store16_from_f32(uint8_t *p, const float (&f)[16]) {
  if constexpr (DT == KAPYB_F32) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      st_stream(reinterpret_cast<uint4 *>(p) + k,
                make_uint4(__float_as_uint(f[4 * k]), __float_as_uint(f[4 * k + 1]),
                           __float_as_uint(f[4 * k + 2]), __float_as_uint(f[4 * k + 3])));
  } else if constexpr (DT == KAPYB_F16 || DT == KAPYB_BF16) {
#pragma unroll
    for (int k = 0; k < 2; ++k)
      st_stream(reinterpret_cast<uint4 *>(p) + k,
                make_uint4(cvt_pack2_t<DT, RN>(f[8 * k], f[8 * k + 1]),
                           cvt_pack2_t<DT, RN>(f[8 * k + 2], f[8 * k + 3]),
                           cvt_pack2_t<DT, RN>(f[8 * k + 4], f[8 * k + 5]),
                           cvt_pack2_t<DT, RN>(f[8 * k + 6], f[8 * k + 7])));
  } else {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      w[t] = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b)
        w[t] |= static_cast<uint32_t>(cvt_f32_to_fp8(f[4 * t + b], DT, RN)) << (8 * b);
    }
    st_stream(reinterpret_cast<uint4 *>(p), make_uint4(w[0], w[1], w[2], w[3]));
  }
}

template <int SD, int DD, int RN>
__global__ void __launch_bounds__(256)
elt_cast_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, long long n_groups,
                long long n_elems) {
  constexpr int ssz = SD == KAPYB_F32 ? 4 : (SD == KAPYB_F16 || SD == KAPYB_BF16) ? 2 : 1;
  constexpr int dsz = DD == KAPYB_F32 ? 4 : (DD == KAPYB_F16 || DD == KAPYB_BF16) ? 2 : 1;
  const long long base = static_cast<long long>(blockIdx.x) * (kCastUnroll * 256) + threadIdx.x;
#pragma unroll
  for (int u = 0; u < kCastUnroll; ++u) {
    const long long g = base + u * 256;
    if (g < n_groups) {
      float f[16];
      load16_as_f32<SD>(x + g * (16 * ssz), f);
      store16_from_f32<DD, RN>(y + g * (16 * dsz), f);
    }
  }
  if (blockIdx.x == gridDim.x - 1) {
    for (long long e = n_groups * 16 + threadIdx.x; e < n_elems; e += blockDim.x)
      store_from_f32(y, DD, e, load_as_f32(x, SD, e), RN);
  }
}

// z = a (op) b at one element type, contiguous and 16-byte aligned.
template <int OP>
__device__ __forceinline__ float binop_at(float a, float b, int dt) {
  if (OP == KAPYB_OP_ADD) return dt == KAPYB_F32 ? __fadd_rn(a, b) : fma_at(a, 1.0f, b, dt);
  if (OP == KAPYB_OP_SUB) return dt == KAPYB_F32 ? __fsub_rn(a, b) : fma_at(b, -1.0f, a, dt);
  if (OP == KAPYB_OP_DIV) return dt == KAPYB_F32 ? div_full(a, b) : round_to_dtype(__fdiv_rn(a, b), dt, 1);
  if (OP == KAPYB_OP_MAXIMUM) return maximum_f(a, b);
  if (OP == KAPYB_OP_MINIMUM) return minimum_f(a, b);
  if (OP == KAPYB_OP_MAXNUM) return fmaxf(a, b);
  if (OP == KAPYB_OP_MINNUM) return fminf(a, b);
  return dt == KAPYB_F32 ? __fmul_rn(a, b) : fma_at(a, b, -0.0f, dt);
}

template <int OP>
__device__ __forceinline__ uint32_t binop_word(uint32_t wa, uint32_t wb, int dt) {
  if (dt == KAPYB_F32)
    return __float_as_uint(binop_at<OP>(__uint_as_float(wa), __uint_as_float(wb), dt));
  if constexpr (OP != KAPYB_OP_ADD && OP != KAPYB_OP_SUB && OP != KAPYB_OP_MUL) {
    // the interpreter's own arithmetic on each half (results are values of the type:
    // the repacking conversion is exact)
    float alo, ahi, blo, bhi;
    if (dt == KAPYB_BF16) {
      unpack2_16<KAPYB_BF16>(wa, alo, ahi);
      unpack2_16<KAPYB_BF16>(wb, blo, bhi);
    } else {
      unpack2_16<KAPYB_F16>(wa, alo, ahi);
      unpack2_16<KAPYB_F16>(wb, blo, bhi);
    }
    return cvt_pack2(binop_at<OP>(alo, blo, dt), binop_at<OP>(ahi, bhi, dt), dt, 1);
  }
  if (dt == KAPYB_BF16) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&wa);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162 *>(&wb);
    __nv_bfloat162 r;
    if (OP == KAPYB_OP_ADD)
      r = __hfma2(a, __float2bfloat162_rn(1.0f), b);
    else if (OP == KAPYB_OP_SUB)
      r = __hfma2(b, __float2bfloat162_rn(-1.0f), a);
    else
      r = __hfma2(a, b, __float2bfloat162_rn(-0.0f));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
  const __half2 a = *reinterpret_cast<const __half2 *>(&wa);
  const __half2 b = *reinterpret_cast<const __half2 *>(&wb);
  __half2 r;
  if (OP == KAPYB_OP_ADD)
    r = __hadd2(a, b);
  else if (OP == KAPYB_OP_SUB)
    r = __hsub2(a, b);
  else
    r = __hmul2(a, b);
  return *reinterpret_cast<const uint32_t *>(&r);
}

constexpr int kBinUnroll = 2;

// One block per contiguous chunk of kBinUnroll x 256 vectors (see elt_unary16_kernel).
template <int OP>
__global__ void __launch_bounds__(256)
elt_binary_kernel(const uint4 *__restrict__ a, const uint4 *__restrict__ b, uint4 *__restrict__ z,
                  long long n_vec, long long n_elems, int dt) {
  const long long base = static_cast<long long>(blockIdx.x) * (kBinUnroll * 256) + threadIdx.x;
  uint4 va[kBinUnroll], vb[kBinUnroll];
#pragma unroll
  for (int u = 0; u < kBinUnroll; ++u) {
    if (base + u * 256 < n_vec) {
      va[u] = ld_stream(a + base + u * 256);
      vb[u] = ld_stream(b + base + u * 256);
    }
  }
#pragma unroll
  for (int u = 0; u < kBinUnroll; ++u) {
    if (base + u * 256 < n_vec) {
      uint4 o;
      o.x = binop_word<OP>(va[u].x, vb[u].x, dt);
      o.y = binop_word<OP>(va[u].y, vb[u].y, dt);
      o.z = binop_word<OP>(va[u].z, vb[u].z, dt);
      o.w = binop_word<OP>(va[u].w, vb[u].w, dt);
      st_stream(z + base + u * 256, o);
    }
  }
  if (blockIdx.x == gridDim.x - 1) {
    const int per = dt == KAPYB_F32 ? 4 : 8;
    for (long long e = n_vec * per + threadIdx.x; e < n_elems; e += blockDim.x) {
      const float x = load_as_f32(a, dt, e), y = load_as_f32(b, dt, e);
      store_from_f32(z, dt, e, binop_at<OP>(x, y, dt), 1);
    }
  }
}

}  // namespace kapyb
