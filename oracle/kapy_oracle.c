/*
 * kapy_oracle.c -- CPU restatement of kapy-lang's matmul / elementwise / reduce
 * op semantics.  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA path is
 * compared with and the timed CPU baseline; nothing in the product imports,
 * links or calls it.
 *
 * PARITY UNPINNED: the reference ships no golden vectors, known-answer tests or
 * numerical fixtures for this path (the .mlir files under test/Conversion/KapyToKgpu carry no
 * CHECK lines and no data) and cannot be built here (needs LLVM/MLIR 19.1.7),
 * so this restatement is pinned only by closed-form cases and by the PTX ISA
 * semantics of the mnemonics the reference emits.
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/kapyb.h"

#define KO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------
 * Float formats.  bf16: p=8, emin=-126, emax=127.  f16: p=11, emin=-14,
 * emax=15.  f32: p=24, emin=-126, emax=127.
 * ---------------------------------------------------------------------- */

typedef struct {
  int p, emin, emax;
} ko_format;

static const ko_format KO_FMT[3] = {
    {11, -14, 15},   /* KAPYB_F16 */
    {8, -126, 127},  /* KAPYB_BF16 */
    {24, -126, 127}, /* KAPYB_F32 */
};

/* Rounds a double to the given format; the result is returned as a double that
 * is exactly representable in the format.  rn != 0: round to nearest even
 * (cvt.rn); rn == 0: toward zero (cvt.rz), which never turns a finite value
 * into an infinity.  Follows ElementwiseOpToLLVM.cpp:381-417 (cvt.{rn,rz}.
 * {f16,bf16}.f32) and :1006-1037 (truncf = cvt.rn). */
static double ko_round_to_f8(double x, int dtype, int rn);

static double ko_round_to(double x, int dtype, int rn) {
  if (dtype == KAPYB_F8E4M3 || dtype == KAPYB_F8E5M2) return ko_round_to_f8(x, dtype, rn);
  if (x == 0.0 || isnan(x) || isinf(x)) return x;
  const ko_format f = KO_FMT[dtype];
  int e;
  (void)frexp(fabs(x), &e);
  int lead = e - 1;
  int q = (lead < f.emin ? f.emin : lead) - (f.p - 1); /* exponent of one ulp */
  double scaled = ldexp(fabs(x), -q);                  /* exact */
  double r = rn ? nearbyint(scaled) : trunc(scaled);
  double res = ldexp(r, q);
  double limit = ldexp(1.0, f.emax + 1);
  if (res >= limit) {
    if (rn)
      res = INFINITY;
    else
      res = limit - ldexp(1.0, f.emax - (f.p - 1));
  }
  return copysign(res, x);
}

static float ko_bits_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint32_t ko_f32_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* cvt.f32.bf16 (ElementwiseOpToLLVM.cpp:973-1004): exact widening. */
KO_API float ko_bf16_to_f32(uint16_t h) { return ko_bits_f32((uint32_t)h << 16); }

/* cvt.f32.f16: exact widening. */
KO_API float ko_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  int exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  float v;
  if (exp == 0) {
    v = ldexpf((float)man, -24);
  } else if (exp == 31) {
    return ko_bits_f32(sign | 0x7f800000u | (man << 13));
  } else {
    v = ldexpf((float)(man | 0x400u), exp - 25);
  }
  return sign ? -v : v;
}

/* Encodes a double that is exactly representable in bf16. */
static uint16_t ko_enc_bf16(double v) {
  float f = (float)v;
  uint32_t u = ko_f32_bits(f);
  if (isnan(f)) return (uint16_t)((u >> 16) | 0x40u);
  return (uint16_t)(u >> 16);
}

/* Encodes a double that is exactly representable in f16. */
static uint16_t ko_enc_f16(double v) {
  uint16_t sign = signbit(v) ? 0x8000u : 0;
  double a = fabs(v);
  if (isnan(v)) return (uint16_t)(sign | 0x7e00u);
  if (isinf(v)) return (uint16_t)(sign | 0x7c00u);
  if (a == 0.0) return sign;
  int e;
  double m = frexp(a, &e); /* a = m * 2^e, m in [0.5, 1) */
  int lead = e - 1;
  if (lead < -14) {
    uint32_t man = (uint32_t)ldexp(a, 24); /* multiples of 2^-24 */
    return (uint16_t)(sign | man);
  }
  uint32_t man = (uint32_t)ldexp(m, 11) & 0x3ffu;
  return (uint16_t)(sign | ((uint32_t)(lead + 15) << 10) | man);
}

KO_API uint16_t ko_f32_to_bf16(float x, int rn) {
  if (isnan(x)) return 0x7fffu; /* cvt.*.bf16.f32 returns the canonical NaN */
  return ko_enc_bf16(ko_round_to((double)x, KAPYB_BF16, rn));
}

KO_API uint16_t ko_f32_to_f16(float x, int rn) {
  if (isnan(x)) return 0x7fffu;
  return ko_enc_f16(ko_round_to((double)x, KAPYB_F16, rn));
}

/* Down casts to the two 8-bit types (FPToFPOp lowering,
 * ElementwiseOpToLLVM.cpp:83-289 and :583-600, conversion table :628-650):
 *   rn: cvt.rn.satfinite.{e4m3x2,e5m2x2}.{f16x2,f32} -- nearest even, and
 *       anything beyond the largest finite value (448 / 57344), infinities
 *       included, becomes that value; NaN stays NaN.  bf16 sources are widened
 *       to f32 first (exact), f16 sources convert directly: one rounding either
 *       way, so the rule is a function of the source VALUE.
 *   rz: exists for f8E5M2 only (:104-112): the high byte of the f16 pattern,
 *       i.e. truncation toward zero with f16's specials kept (an f32 source is
 *       first truncated to f16, :583-600, which cannot produce an infinity). */
static double ko_round_to_f8(double x, int dtype, int rn) {
  const int p = dtype == KAPYB_F8E4M3 ? 4 : 3;          /* significand bits */
  const int emin = dtype == KAPYB_F8E4M3 ? -6 : -14;    /* smallest normal exponent */
  const double maxv = dtype == KAPYB_F8E4M3 ? 448.0 : 57344.0;
  if (isnan(x) || x == 0.0) return x;
  if (!rn) {
    /* f32 -> f16 toward zero, then drop the low 8 bits of the f16 pattern */
    double h = isinf(x) ? x : ko_round_to(x, KAPYB_F16, 0);
    if (isinf(h)) return h; /* only from an infinite source */
    int e;
    (void)frexp(fabs(h), &e);
    int lead = e - 1;
    int q = (lead < -14 ? -14 : lead) - 2; /* f16 exponent rules, 2 stored mantissa bits */
    return copysign(ldexp(trunc(ldexp(fabs(h), -q)), q), x);
  }
  if (isinf(x)) return copysign(maxv, x);
  int e;
  (void)frexp(fabs(x), &e);
  int lead = e - 1;
  int q = (lead < emin ? emin : lead) - (p - 1);
  double res = ldexp(nearbyint(ldexp(fabs(x), -q)), q);
  if (res > maxv) res = maxv;
  return copysign(res, x);
}

/* Encodes a double that is exactly representable in the 8-bit format. */
static uint8_t ko_enc_f8(double v, int dtype) {
  const int mbits = dtype == KAPYB_F8E4M3 ? 3 : 2;
  const int bias = dtype == KAPYB_F8E4M3 ? 7 : 15;
  uint8_t sign = signbit(v) ? 0x80u : 0;
  if (isnan(v)) return 0x7fu;
  if (isinf(v)) return (uint8_t)(sign | 0x7cu); /* f8E5M2 only */
  double a = fabs(v);
  if (a == 0.0) return sign;
  int e;
  double m = frexp(a, &e);
  int lead = e - 1;
  if (lead < 1 - bias) return (uint8_t)(sign | (uint8_t)ldexp(a, bias - 1 + mbits));
  uint32_t man = (uint32_t)ldexp(m, mbits + 1) & ((1u << mbits) - 1u);
  return (uint8_t)(sign | ((uint32_t)(lead + bias) << mbits) | man);
}

KO_API uint8_t ko_f32_to_f8(float x, int dtype, int rn) {
  return ko_enc_f8(ko_round_to_f8((double)x, dtype, rn), dtype);
}

/* The two 8-bit operand types of the matmul verifier (Kapy.cpp:484-487,
 * 548-564).  f8E4M3 is the finite-only "FN" variant: bias 7, no infinities,
 * S.1111.111 is NaN.  f8E5M2 is a truncated f16: bias 15, IEEE specials. */
static double ko_f8e4m3_to_f64(uint8_t b) {
  int e = (b >> 3) & 15, m = b & 7;
  double v;
  if (e == 15 && m == 7) return NAN;
  v = e == 0 ? ldexp((double)m, -9) : ldexp((double)(8 + m), e - 10);
  return (b & 0x80) ? -v : v;
}

static double ko_f8e5m2_to_f64(uint8_t b) {
  int e = (b >> 2) & 31, m = b & 3;
  double v;
  if (e == 31) v = m ? NAN : INFINITY;
  else v = e == 0 ? ldexp((double)m, -16) : ldexp((double)(4 + m), e - 17);
  return (b & 0x80) ? -v : v;
}

static double ko_load(const void *base, int dtype, int64_t idx) {
  switch (dtype) {
  case KAPYB_F16: return (double)ko_f16_to_f32(((const uint16_t *)base)[idx]);
  case KAPYB_BF16: return (double)ko_bf16_to_f32(((const uint16_t *)base)[idx]);
  case KAPYB_F8E4M3: return ko_f8e4m3_to_f64(((const uint8_t *)base)[idx]);
  case KAPYB_F8E5M2: return ko_f8e5m2_to_f64(((const uint8_t *)base)[idx]);
  default: return (double)((const float *)base)[idx];
  }
}

static void ko_store(void *base, int dtype, int64_t idx, double v) {
  switch (dtype) {
  case KAPYB_F16: ((uint16_t *)base)[idx] = isnan(v) ? 0x7fffu : ko_enc_f16(v); break;
  case KAPYB_BF16: ((uint16_t *)base)[idx] = isnan(v) ? 0x7fffu : ko_enc_bf16(v); break;
  case KAPYB_F8E4M3:
  case KAPYB_F8E5M2: ((uint8_t *)base)[idx] = ko_enc_f8(v, dtype); break;
  default: ((float *)base)[idx] = (float)v; break;
  }
}

/* Element (i,j) of a mk_global descriptor, with the out-of-bounds padding of
 * ld_global (LdGlobalOpToLLVM.cpp:83-98; constants ConvertUtils.cpp:267-334). */
static double ko_tensor_get(const kapyb_tensor2d *t, int64_t i, int64_t j) {
  if (i >= t->size0 || j >= t->size1 || i < 0 || j < 0) {
    switch (t->padding) {
    case KAPYB_PAD_QNAN: return NAN;
    case KAPYB_PAD_PINF: return INFINITY;
    case KAPYB_PAD_NINF: return -INFINITY;
    default: return 0.0;
    }
  }
  return ko_load(t->ptr, t->dtype, t->offset_elems + i * (int64_t)t->stride0 + j * (int64_t)t->stride1);
}

/* ------------------------------------------------------------------------
 * Single-rounding arithmetic at a tensor's element type.
 * ---------------------------------------------------------------------- */

/* RN(a*b + c) for operands exactly representable in `dtype` (f16 or bf16): the
 * product is exact in double (<= 22 significant bits); the sum is formed with
 * TwoSum and forced to round-to-odd before the final rounding, so the result is
 * the single rounding fma.rn.bf16 / fma.rn.f16 perform
 * (ElementwiseOpToLLVM.cpp:771-892: mul = fma(a,b,-0), add = fma(a,1,b),
 * sub = fma(b,-1,a)). */
static double ko_fma_small(double a, double b, double c, int dtype) {
  double p = a * b;
  double s = p + c;
  if (isfinite(s)) {
    double bb = s - p;
    double err = (p - (s - bb)) + (c - bb);
    if (err != 0.0) {
      uint64_t u;
      memcpy(&u, &s, 8);
      if ((u & 1u) == 0) {
        s = nextafter(s, err > 0 ? INFINITY : -INFINITY);
      }
    }
  }
  return ko_round_to(s, dtype, 1);
}

static double ko_arith(int op, double a, double b, double c, int dtype) {
  if (dtype == KAPYB_F32) {
    float fa = (float)a, fb = (float)b, fc = (float)c;
    switch (op) {
    case KAPYB_OP_ADD: return (double)(fa + fb);
    case KAPYB_OP_SUB: return (double)(fa - fb);
    case KAPYB_OP_MUL: return (double)(fa * fb);
    case KAPYB_OP_FMA: return (double)fmaf(fa, fb, fc);
    }
  } else {
    switch (op) {
    case KAPYB_OP_ADD: return ko_fma_small(a, 1.0, b, dtype);
    case KAPYB_OP_SUB: return ko_fma_small(b, -1.0, a, dtype);
    case KAPYB_OP_MUL: return ko_fma_small(a, b, -0.0, dtype);
    case KAPYB_OP_FMA: return ko_fma_small(a, b, c, dtype);
    }
  }
  return NAN;
}

static double ko_maximum(double a, double b) {
  if (isnan(a) || isnan(b)) return NAN;
  if (a == 0.0 && b == 0.0) return signbit(a) ? b : a;
  return a > b ? a : b;
}
static double ko_minimum(double a, double b) {
  if (isnan(a) || isnan(b)) return NAN;
  if (a == 0.0 && b == 0.0) return signbit(a) ? a : b;
  return a < b ? a : b;
}
static double ko_maxnum(double a, double b) {
  if (isnan(a)) return b;
  if (isnan(b)) return a;
  return ko_maximum(a, b);
}
static double ko_minnum(double a, double b) {
  if (isnan(a)) return b;
  if (isnan(b)) return a;
  return ko_minimum(a, b);
}

/* arith.cmpf with the predicates Builder.create_cmpf_* binds (ir.cc:941-1000):
 * ordered predicates are false and unordered ones true when an operand is NaN. */
static int ko_cmpf(int pred, double a, double b) {
  const int un = isnan(a) || isnan(b);
  switch (pred) {
  case KAPYB_CMP_OLT: return !un && a < b;
  case KAPYB_CMP_OGT: return !un && a > b;
  case KAPYB_CMP_OLE: return !un && a <= b;
  case KAPYB_CMP_OGE: return !un && a >= b;
  case KAPYB_CMP_OEQ: return !un && a == b;
  case KAPYB_CMP_ONE: return !un && a != b;
  case KAPYB_CMP_ULT: return un || a < b;
  case KAPYB_CMP_UGT: return un || a > b;
  case KAPYB_CMP_ULE: return un || a <= b;
  case KAPYB_CMP_UGE: return un || a >= b;
  case KAPYB_CMP_UEQ: return un || a == b;
  default: return un || a != b;
  }
}

/* The gelu_tanh composite in the form the benchmark graph pins:
 * u / (1 + exp(-2k)), k = c0 * fma(c1*u*u, u, u), evaluated here in double from
 * a given u (transcendental step exact, as the tolerance rule requires). */
static double ko_gelu_tanh_f64(double u) {
  const double c0 = (double)0.7978845608f, c1 = (double)0.044715f;
  double k = c0 * (c1 * u * u * u + u);
  return u / (1.0 + exp(-2.0 * k));
}

static double ko_activation(int act, double v) {
  switch (act) {
  case KAPYB_ACT_RELU: return v > 0 ? v : (isnan(v) ? v : 0.0);
  case KAPYB_ACT_GELU_TANH: return ko_gelu_tanh_f64(v);
  case KAPYB_ACT_SILU: return v / (1.0 + exp(-v));
  default: return v;
  }
}

/* ------------------------------------------------------------------------
 * Elementwise interpreter: applies each recorded op and rounds to the op's
 * tensor element type after every op (generic per-element pattern,
 * ElementwiseOpToLLVM.cpp:424-485).  exp/div/... are evaluated in double from
 * the exactly rounded operand and rounded once to the op's dtype, so that a
 * device result can be held to "<= 2 ulp of the output dtype".
 * ---------------------------------------------------------------------- */

KO_API int ko_eltwise(const kapyb_inst *prog, int n_inst, const kapyb_tensor2d *inputs,
                      int n_inputs, const kapyb_tensor2d *out) {
  if (n_inst <= 0 || n_inst > KAPYB_MAX_INSTS || n_inputs > KAPYB_MAX_INPUTS) return KAPYB_INVALID_ARG;
  const int64_t rows = out->size0, cols = out->size1;
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t i = 0; i < rows; ++i) {
    for (int64_t j = 0; j < cols; ++j) {
      double r[KAPYB_MAX_REGS];
      for (int t = 0; t < KAPYB_MAX_REGS; ++t) r[t] = 0.0;
      for (int pc = 0; pc < n_inst; ++pc) {
        const kapyb_inst in = prog[pc];
        double a = in.a >= 0 ? r[in.a] : 0.0;
        double b = in.b >= 0 ? r[in.b] : 0.0;
        double c = in.c >= 0 ? r[in.c] : 0.0;
        double v = 0.0;
        switch (in.op) {
        case KAPYB_OP_LOAD: {
          if (in.flags < 0 || in.flags >= n_inputs) { bad |= 1; break; }
          const kapyb_tensor2d *t = &inputs[in.flags];
          v = ko_tensor_get(t, t->size0 == 1 ? 0 : i, t->size1 == 1 ? 0 : j);
          break;
        }
        case KAPYB_OP_CONST: v = ko_round_to((double)in.imm, in.dtype, 1); break;
        case KAPYB_OP_CVT: v = ko_round_to(a, in.dtype, in.flags); break;
        case KAPYB_OP_ADD:
        case KAPYB_OP_SUB:
        case KAPYB_OP_MUL:
        case KAPYB_OP_FMA: v = ko_arith(in.op, a, b, c, in.dtype); break;
        case KAPYB_OP_DIV: v = ko_round_to(a / b, in.dtype, 1); break;
        case KAPYB_OP_MAXIMUM: v = ko_maximum(a, b); break;
        case KAPYB_OP_MINIMUM: v = ko_minimum(a, b); break;
        case KAPYB_OP_MAXNUM: v = ko_maxnum(a, b); break;
        case KAPYB_OP_MINNUM: v = ko_minnum(a, b); break;
        case KAPYB_OP_CLAMP:
          /* ClampFOpConversion, ElementwiseOpToLLVM.cpp:699-728 */
          v = in.flags ? ko_minimum(ko_maximum(a, b), c) : ko_minnum(ko_maxnum(a, b), c);
          break;
        case KAPYB_OP_ABS: v = fabs(a); break;
        case KAPYB_OP_NEG: v = -a; break;
        case KAPYB_OP_EXP: v = ko_round_to(exp(a), in.dtype, 1); break;
        case KAPYB_OP_EXP2: v = ko_round_to(exp2(a), in.dtype, 1); break;
        case KAPYB_OP_LOG: v = ko_round_to(log(a), in.dtype, 1); break;
        case KAPYB_OP_LOG2: v = ko_round_to(log2(a), in.dtype, 1); break;
        case KAPYB_OP_SQRT: v = ko_round_to(sqrt(a), in.dtype, 1); break;
        case KAPYB_OP_RSQRT: v = ko_round_to(1.0 / sqrt(a), in.dtype, 1); break;
        case KAPYB_OP_ERF: v = ko_round_to(erf(a), in.dtype, 1); break;
        case KAPYB_OP_SIN: v = ko_round_to(sin(a), in.dtype, 1); break;
        case KAPYB_OP_COS: v = ko_round_to(cos(a), in.dtype, 1); break;
        case KAPYB_OP_FLOOR: v = floor(a); break;
        case KAPYB_OP_CEIL: v = ceil(a); break;
        case KAPYB_OP_TANH: v = ko_round_to(tanh(a), in.dtype, 1); break;
        case KAPYB_OP_CMP: v = ko_cmpf(in.flags, a, b) ? 1.0 : 0.0; break;
        case KAPYB_OP_SELECT: v = a != 0.0 ? b : c; break; /* arith.select (ir.cc:1162) */
        case KAPYB_OP_AND: v = (a != 0.0 && b != 0.0) ? 1.0 : 0.0; break;
        case KAPYB_OP_OR: v = (a != 0.0 || b != 0.0) ? 1.0 : 0.0; break;
        case KAPYB_OP_XOR: v = ((a != 0.0) != (b != 0.0)) ? 1.0 : 0.0; break;
        case KAPYB_OP_STORE:
          ko_store(out->ptr, out->dtype,
                   out->offset_elems + i * (int64_t)out->stride0 + j * (int64_t)out->stride1, a);
          break;
        default: bad |= 1; break;
        }
        if (in.op != KAPYB_OP_STORE && in.dst >= 0 && in.dst < KAPYB_MAX_REGS) r[in.dst] = v;
      }
    }
  }
  return bad ? KAPYB_INVALID_ARG : KAPYB_OK;
}

/* Fast restatement of the benchmark graph for the timed CPU baseline:
 *   y = truncf_rn( gelu_tanh( fma(extf(x), s, b) ) ), all in f32 arithmetic with
 * exp taken as expf.  n contiguous bf16 elements.  When `linear_only` is set the
 * gelu step is skipped (the transcendental-free variant whose device result
 * must be bit-exact).  Same op order as ko_eltwise would execute. */
KO_API void ko_affine_gelu_bf16(const uint16_t *x, uint16_t *y, int64_t n, float s, float b,
                                int linear_only) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float xf = ko_bf16_to_f32(x[i]);
    float u = fmaf(xf, s, b);
    float v = u;
    if (!linear_only) {
      const float c0 = 0.7978845608f, c1 = 0.044715f;
      float k = c0 * fmaf(c1 * u * u, u, u);
      v = u / (1.0f + expf(-2.0f * k));
    }
    /* cvt.rn.bf16.f32 */
    uint32_t bits = ko_f32_bits(v);
    uint16_t o;
    if (isnan(v)) {
      o = 0x7fffu;
    } else {
      uint32_t lsb = (bits >> 16) & 1u;
      bits += 0x7fffu + lsb;
      o = (uint16_t)(bits >> 16);
    }
    y[i] = o;
  }
}

/* ------------------------------------------------------------------------
 * Reduce (ReduceOpToLLVM.cpp:76-119; result shape Kapy.cpp:613-626): the
 * reference fixes no order of combination, so the checker is the f64 result
 * plus, for sums, sum|x| so a caller can form the 4*eps*sum|x| bound.
 * out64 and abs64 have size0 (axis 1) or size1 (axis 0) entries.
 * ---------------------------------------------------------------------- */

KO_API int ko_reduce_f64(const kapyb_tensor2d *src, int axis, int combiner, double *out64,
                         double *abs64) {
  if (axis != 0 && axis != 1) return KAPYB_INVALID_ARG;
  const int64_t outer = axis == 1 ? src->size0 : src->size1;
  const int64_t inner = axis == 1 ? src->size1 : src->size0;
#pragma omp parallel for schedule(static)
  for (int64_t o = 0; o < outer; ++o) {
    double acc = 0.0, aabs = 0.0;
    for (int64_t k = 0; k < inner; ++k) {
      double v = axis == 1 ? ko_tensor_get(src, o, k) : ko_tensor_get(src, k, o);
      if (k == 0) {
        acc = v;
      } else {
        switch (combiner) {
        case KAPYB_RED_ADD: acc += v; break;
        case KAPYB_RED_MUL: acc *= v; break;
        case KAPYB_RED_MAX: acc = ko_maximum(acc, v); break;
        case KAPYB_RED_MIN: acc = ko_minimum(acc, v); break;
        }
      }
      aabs += fabs(v);
    }
    out64[o] = acc;
    if (abs64) abs64[o] = aabs;
  }
  return KAPYB_OK;
}

/* Row sums of a contiguous [rows, cols] bf16 matrix with an f32 accumulator,
 * ascending column order: the timed CPU baseline of the row-reduce workload
 * (extf then addf in f32, as the warp loop of reduce_sum.mlir:10-25 would). */
KO_API void ko_rowsum_bf16_f32(const uint16_t *x, float *out, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const uint16_t *p = x + r * cols;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t k = 0;
    for (; k + 8 <= cols; k += 8)
      for (int t = 0; t < 8; ++t) acc[t] += ko_bits_f32((uint32_t)p[k + t] << 16);
    float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    for (; k < cols; ++k) s += ko_bits_f32((uint32_t)p[k] << 16);
    out[r] = s;
  }
}

/* ------------------------------------------------------------------------
 * Matmul.  Semantics: Ops.td:416-439 (result = lhs . rhs + acc), legal dtypes
 * Kapy.cpp:451-574, accumulation in the accumulator type in ascending k
 * (MatmulOpToLLVM.cpp:125-170), bias as accumulator init (Combine.td:38-88),
 * RN/RZ downcast (ElementwiseOpToLLVM.cpp:381-417).
 * ---------------------------------------------------------------------- */

/* Exact-as-possible checker: every requested entry in f64.
 *   ref[r*ncols + c] = act(alpha * sum_k A[rows[r],k]*B[k,cols[c]] + bias [+ acc])
 * rows == NULL means 0..nrows-1 (same for cols).  No final rounding: the caller
 * compares the device output with a relative tolerance. */
KO_API int ko_matmul_f64(const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
                         const kapyb_tensor2d *acc, const kapyb_epilogue *ep, const int32_t *rows,
                         int32_t nrows, const int32_t *cols, int32_t ncols, double *ref) {
  const int64_t K = lhs->size1;
  if (rhs->size0 != K) return KAPYB_INVALID_ARG;
  /* gather the requested rows of A and columns of B into dense f64 panels */
  double *pa = (double *)malloc(sizeof(double) * (size_t)nrows * (size_t)K);
  double *pb = (double *)malloc(sizeof(double) * (size_t)ncols * (size_t)K);
  if (!pa || !pb) {
    free(pa);
    free(pb);
    return KAPYB_INVALID_ARG;
  }
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < nrows; ++r) {
    int64_t i = rows ? rows[r] : r;
    for (int64_t k = 0; k < K; ++k) pa[r * K + k] = ko_tensor_get(lhs, i, k);
  }
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < ncols; ++c) {
    int64_t j = cols ? cols[c] : c;
    for (int64_t k = 0; k < K; ++k) pb[c * K + k] = ko_tensor_get(rhs, k, j);
  }
  const double alpha = ep ? (double)ep->alpha : 1.0;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t r = 0; r < nrows; ++r) {
    const double *a = pa + r * K;
    int64_t i = rows ? rows[r] : r;
    for (int64_t c = 0; c < ncols; ++c) {
      const double *b = pb + c * K;
      int64_t j = cols ? cols[c] : c;
      double s = 0.0;
#pragma omp simd reduction(+ : s)
      for (int64_t k = 0; k < K; ++k) s += a[k] * b[k];
      s *= alpha;
      if (ep && ep->bias) s += ko_load(ep->bias, ep->bias_dtype, ep->bias_axis == 1 ? j : i);
      if (acc) s += ko_tensor_get(acc, i, j);
      ref[r * (int64_t)ncols + c] = ko_activation(ep ? ep->activation : KAPYB_ACT_NONE, s);
    }
  }
  free(pa);
  free(pb);
  return KAPYB_OK;
}

/* The reference's arithmetic at full size, as a timed CPU baseline: operands
 * widened to f32, products accumulated in an f32 accumulator in ascending k
 * starting from the bias (accumulator init), alpha and activation applied in
 * f32, then the RN/RZ downcast.  Computes rows [row_begin, row_end) of `out`.
 * Blocked i-k-j so each output keeps its ascending-k order. */
KO_API int ko_matmul_f32acc(const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
                            const kapyb_tensor2d *out, const kapyb_epilogue *ep,
                            int32_t row_begin, int32_t row_end) {
  const int64_t N = rhs->size1, K = lhs->size1;
  if (rhs->size0 != K) return KAPYB_INVALID_ARG;
  const int64_t MR = row_end - row_begin;
  if (MR <= 0) return KAPYB_OK;
  float *fb = (float *)malloc(sizeof(float) * (size_t)K * (size_t)N);
  float *fa = (float *)malloc(sizeof(float) * (size_t)MR * (size_t)K);
  if (!fa || !fb) {
    free(fa);
    free(fb);
    return KAPYB_INVALID_ARG;
  }
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < K; ++k)
    for (int64_t j = 0; j < N; ++j) fb[k * N + j] = (float)ko_tensor_get(rhs, k, j);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < MR; ++i)
    for (int64_t k = 0; k < K; ++k) fa[i * K + k] = (float)ko_tensor_get(lhs, row_begin + i, k);
  const float alpha = ep ? ep->alpha : 1.0f;
  const int rn = ep ? ep->rounding : 1;
  const int act = ep ? ep->activation : KAPYB_ACT_NONE;
  enum { BI = 8, BJ = 512 };
  const int64_t nbj = (N + BJ - 1) / BJ, nbi = (MR + BI - 1) / BI;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
  for (int64_t bi = 0; bi < nbi; ++bi) {
    for (int64_t bj = 0; bj < nbj; ++bj) {
      float accbuf[BI][BJ];
      const int64_t i0 = bi * BI, j0 = bj * BJ;
      const int64_t ni = MR - i0 < BI ? MR - i0 : BI;
      const int64_t nj = N - j0 < BJ ? N - j0 : BJ;
      for (int64_t i = 0; i < ni; ++i)
        for (int64_t j = 0; j < nj; ++j) accbuf[i][j] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float *brow = fb + k * N + j0;
        for (int64_t i = 0; i < ni; ++i) {
          const float a = fa[(i0 + i) * K + k];
          float *crow = accbuf[i];
#pragma omp simd
          for (int64_t j = 0; j < nj; ++j) crow[j] += a * brow[j];
        }
      }
      for (int64_t i = 0; i < ni; ++i) {
        for (int64_t j = 0; j < nj; ++j) {
          float v = accbuf[i][j] * alpha;
          if (ep && ep->bias)
            v += (float)ko_load(ep->bias, ep->bias_dtype,
                                ep->bias_axis == 1 ? (j0 + j) : (row_begin + i0 + i));
          if (act != KAPYB_ACT_NONE) v = (float)ko_activation(act, (double)v);
          double rv = ko_round_to((double)v, out->dtype, rn);
          ko_store(out->ptr, out->dtype,
                   out->offset_elems + (row_begin + i0 + i) * (int64_t)out->stride0 +
                       (j0 + j) * (int64_t)out->stride1,
                   rv);
        }
      }
    }
  }
  free(fa);
  free(fb);
  return KAPYB_OK;
}

/* max_i |c_i - ref_i| / max(|ref_i|, tau), tau = 2^-6 * rms(ref): the matmul
 * parity metric.  `c` holds device outputs already widened to f64. */
KO_API double ko_max_rel_err(const double *c, const double *ref, int64_t n, double *tau_out) {
  double ss = 0.0;
#pragma omp parallel for reduction(+ : ss)
  for (int64_t i = 0; i < n; ++i) ss += ref[i] * ref[i];
  double tau = sqrt(ss / (double)(n > 0 ? n : 1)) / 64.0;
  if (tau == 0.0) tau = 1e-30;
  double worst = 0.0;
#pragma omp parallel for reduction(max : worst)
  for (int64_t i = 0; i < n; ++i) {
    double d = fabs(c[i] - ref[i]);
    double den = fabs(ref[i]) > tau ? fabs(ref[i]) : tau;
    double e = d / den;
    if (isnan(e)) e = INFINITY;
    if (e > worst) worst = e;
  }
  if (tau_out) *tau_out = tau;
  return worst;
}

/* Sets the number of OpenMP threads later calls use (n <= 0: one per processor
 * this process may run on).  A launcher may have exported OMP_NUM_THREADS=1;
 * the timed CPU baseline must not inherit that. */
KO_API int ko_set_num_threads(int n) {
#ifdef _OPENMP
  if (n <= 0) n = omp_get_num_procs();
  omp_set_num_threads(n);
  return n;
#else
  (void)n;
  return 1;
#endif
}

KO_API int ko_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
