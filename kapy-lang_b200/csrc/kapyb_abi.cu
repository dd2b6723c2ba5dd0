// C ABI of the library (include/kapyb.h): handle management, verifier-equivalent
// validation, kernel selection and launch.  Everything here runs on the host;
// the arithmetic lives in the .cuh kernels.  There is no CPU compute path: a
// call either launches CUDA kernels or returns an error status.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/kapyb.h"
#include "eltwise.cuh"
#include "gather_sync.cuh"
#include "gemm_simt.cuh"
#include "gemm_skinny_sm100.cuh"
#include "gemm_sm100.cuh"
#include "reduce.cuh"

using namespace kapyb;

// ------------------------------------------------------------------ context

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

enum MatmulPath { PATH_AUTO = 0, PATH_1CTA, PATH_2CTA, PATH_SKINNY, PATH_SIMT };
constexpr int kMaxDevices = 64;

struct kapyb_context {
  int device = 0;
  int sm_count = 0;
  uint32_t *status = nullptr;  // device word written by kernels that give up
  void *workspace = nullptr;
  size_t workspace_bytes = 0;
  EncodeTiledFn encode = nullptr;
  std::string last_error;
  const char *last_kernel = "none";
  int64_t launches = 0;
  int forced_path = PATH_AUTO;
  int forced_bn = 0;
  int debug = 0;
  uint32_t wait_limit_us = 0;
  int forced_epi = 0;  // 0: by K; 4 or 8: that many epilogue warps (single-CTA kernels)
  int skinny_stages = 0;  // 0: the default depth
  uint32_t skinny_epoch = 0;  // number of the last decode-kernel launch that used the workspace
  int forced_group_m = 0; // 0: the default raster group (row blocks walked together); else that many
  int skinny_split = -1;  // -1: by shape; 0: whole weight tiles only; 1: split leftover tiles between SMs
  int tile_split = -1;    // tcgen05 kernels, the same three choices for the last wave's tiles
  void *split_scratch = nullptr;  // their partial accumulators and flag words
  size_t split_scratch_bytes = 0;
  uint32_t split_epoch = 0;       // number of the last launch that used them
  // host-buffer calls: copy streams and events for the chunked pipeline
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t ev[2 * 16 + 2] = {};
  bool pipe_ready = false;
  // sharded host-buffer calls: the stream that forwards this rank's rows to its peers
  cudaStream_t push = nullptr;
  cudaEvent_t ev_push[16 + 1] = {};
  bool push_ready = false;
};

static thread_local std::string g_create_error;

static kapyb_status fail(kapyb_handle h, kapyb_status st, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (h)
    h->last_error = buf;
  else
    g_create_error = buf;
  return st;
}

#define CUDA_TRY(h, expr)                                                                  \
  do {                                                                                     \
    cudaError_t e_ = (expr);                                                               \
    if (e_ != cudaSuccess)                                                                 \
      return fail(h, KAPYB_CUDA_ERROR, "%s failed: %s", #expr, cudaGetErrorString(e_));    \
  } while (0)

extern "C" KAPYB_API int kapyb_version(void) { return 110; }

extern "C" KAPYB_API kapyb_status kapyb_create(kapyb_handle *out, int device) {
  if (!out) return fail(nullptr, KAPYB_INVALID_ARG, "kapyb_create: out is NULL");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fail(nullptr, KAPYB_CUDA_ERROR,
                "kapyb_create: no CUDA device (%s); this library has no CPU path",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  if (device < 0 || device >= n || device >= kMaxDevices)
    return fail(nullptr, KAPYB_INVALID_ARG, "kapyb_create: device %d out of range [0,%d)", device,
                std::min(n, kMaxDevices));
  cudaDeviceProp prop;
  CUDA_TRY(nullptr, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(nullptr, KAPYB_CUDA_ERROR,
                "kapyb_create: device %d is sm_%d%d; kernels are built for sm_100a only", device,
                prop.major, prop.minor);
  CUDA_TRY(nullptr, cudaSetDevice(device));
  kapyb_context *c = new kapyb_context();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  cudaDriverEntryPointQueryResult q;
  void *fn = nullptr;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess) {
    delete c;
    return fail(nullptr, KAPYB_CUDA_ERROR, "kapyb_create: cuTensorMapEncodeTiled not available");
  }
  c->encode = reinterpret_cast<EncodeTiledFn>(fn);
  // word 0: status; words 2..15: the profiling probes read by kapyb_probe_read
  e = cudaMalloc(&c->status, 16 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(c->status, 0, 16 * sizeof(uint32_t));
  if (e != cudaSuccess) {
    delete c;
    return fail(nullptr, KAPYB_CUDA_ERROR, "kapyb_create: status word: %s", cudaGetErrorString(e));
  }
  *out = c;
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_destroy(kapyb_handle h) {
  if (!h) return KAPYB_OK;
  cudaSetDevice(h->device);
  if (h->workspace) cudaFree(h->workspace);
  if (h->split_scratch) cudaFree(h->split_scratch);
  if (h->status) cudaFree(h->status);
  if (h->push_ready) {
    cudaStreamDestroy(h->push);
    for (cudaEvent_t e : h->ev_push)
      if (e) cudaEventDestroy(e);
  }
  if (h->pipe_ready) {
    cudaStreamDestroy(h->copy_in);
    cudaStreamDestroy(h->copy_out);
    for (cudaEvent_t e : h->ev)
      if (e) cudaEventDestroy(e);
  }
  delete h;
  return KAPYB_OK;
}

extern "C" KAPYB_API const char *kapyb_last_error_string(kapyb_handle h) {
  return h ? h->last_error.c_str() : g_create_error.c_str();
}

extern "C" KAPYB_API const char *kapyb_last_kernel(kapyb_handle h) {
  return h ? h->last_kernel : "none";
}

extern "C" KAPYB_API int64_t kapyb_launch_count(kapyb_handle h) { return h ? h->launches : 0; }

extern "C" KAPYB_API kapyb_status kapyb_probe_read(kapyb_handle h, void *stream, uint32_t *words,
                                                   int32_t n) {
  if (!h || !words || n < 0 || n > 14)
    return fail(h, KAPYB_INVALID_ARG, "kapyb_probe_read: NULL argument or n outside 0..14");
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (n > 0)
    CUDA_TRY(h, cudaMemcpy(words, h->status + 2, n * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  // probes accumulate with max/min across CTAs: start each measurement from zero
  CUDA_TRY(h, cudaMemset(h->status + 2, 0, 14 * sizeof(uint32_t)));
  return KAPYB_OK;
}

// A dispatch choice in text form: "auto" | "1cta" | "2cta" | "skinny" | "simt",
// optionally followed by ":<tile width>" and options ":e<epilogue warps>",
// ":s<stages>" and ":k<0|1>" (skinny: whole tiles only | split leftover tiles),
// ":g<n>" (tcgen05: row blocks per raster group), ":x<0|1>" (tcgen05: the tiles of a
// partly filled last wave stay whole | are split between the CTAs),
// ":d<debug bits>", ":w<wait limit, ms>".
struct PathChoice {
  int path = PATH_AUTO, bn = 0, epi = 0, skinny_stages = 0, skinny_split = -1, debug = 0, group_m = 0;
  int tile_split = -1;
  uint32_t wait_limit_us = 0;
};

static bool parse_path(const std::string &text, PathChoice &c, const char **why) {
  c = PathChoice{};
  auto option = [&](const char *tag, size_t from) -> int {
    const size_t at = text.find(tag, from);
    return at == std::string::npos ? -1 : atoi(text.c_str() + at + 2);
  };
  const size_t colon = text.find(':');
  const std::string family = text.substr(0, colon);
  if (family == "auto")
    c.path = PATH_AUTO;
  else if (family == "1cta")
    c.path = PATH_1CTA;
  else if (family == "2cta")
    c.path = PATH_2CTA;
  else if (family == "skinny")
    c.path = PATH_SKINNY;
  else if (family == "simt")
    c.path = PATH_SIMT;
  else {
    *why = "unknown path";
    return false;
  }
  if (colon == std::string::npos) return true;
  const char first = text[colon + 1];  // text[size()] is the terminator: in bounds
  if (first >= '0' && first <= '9') {
    c.bn = atoi(text.c_str() + colon + 1);
    if (c.bn != 64 && c.bn != 128 && c.bn != 256 && c.bn != 512) {
      *why = "tile width must be 64/128/256/512";
      return false;
    }
  }
  c.debug = std::max(0, option(":d", colon));
  c.epi = std::max(0, option(":e", colon));
  c.skinny_stages = std::max(0, option(":s", colon));
  c.skinny_split = option(":k", colon);
  c.group_m = std::max(0, option(":g", colon));
  c.tile_split = option(":x", colon);
  const int w = option(":w", colon);
  c.wait_limit_us = w > 0 ? 1000u * static_cast<uint32_t>(w) : 0u;
  return true;
}

extern "C" KAPYB_API kapyb_status kapyb_set_matmul_path(kapyb_handle h, const char *name) {
  if (!h || !name) return fail(h, KAPYB_INVALID_ARG, "kapyb_set_matmul_path: NULL argument");
  PathChoice c;
  const char *why = "";
  if (!parse_path(name, c, &why))
    return fail(h, KAPYB_INVALID_ARG, "kapyb_set_matmul_path: %s ('%s')", why, name);
  if (c.debug & ~kDebugMask)
    return fail(h, KAPYB_UNSUPPORTED,
                "kapyb_set_matmul_path: debug bits %d make results garbage and exist only in a "
                "library built with -DKAPYB_DEBUG_SWITCHES ('%s')", c.debug & ~kDebugMask, name);
  h->forced_path = c.path;
  h->forced_bn = c.bn;
  h->forced_epi = c.epi;
  h->skinny_stages = c.skinny_stages;
  h->skinny_split = c.skinny_split;
  h->forced_group_m = c.group_m;
  h->tile_split = c.tile_split;
  h->debug = c.debug;
  h->wait_limit_us = c.wait_limit_us;
  return KAPYB_OK;
}

static int dtype_from_name(const std::string &n) {
  if (n == "f16") return KAPYB_F16;
  if (n == "bf16") return KAPYB_BF16;
  if (n == "f32") return KAPYB_F32;
  if (n == "f8E4M3") return KAPYB_F8E4M3;
  if (n == "f8E5M2") return KAPYB_F8E5M2;
  return -1;
}

extern "C" KAPYB_API kapyb_status kapyb_check(kapyb_handle h, void *stream) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_check: NULL handle");
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  uint32_t st = 0;
  CUDA_TRY(h, cudaMemcpy(&st, h->status, sizeof(st), cudaMemcpyDeviceToHost));
  if (st != kStatusOk) {
    cudaMemset(h->status, 0, sizeof(uint32_t));
    return fail(h, KAPYB_TIMEOUT, "a kernel gave up on a bounded wait (status %u)", st);
  }
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_reserve_workspace(kapyb_handle h, size_t bytes) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_reserve_workspace: NULL handle");
  if (bytes <= h->workspace_bytes) return KAPYB_OK;
  CUDA_TRY(h, cudaSetDevice(h->device));
  CUDA_TRY(h, cudaDeviceSynchronize());
  if (h->workspace) {
    cudaFree(h->workspace);
    h->workspace = nullptr;
    h->workspace_bytes = 0;
  }
  size_t want = (bytes + (1u << 20) - 1) & ~static_cast<size_t>((1u << 20) - 1);
  CUDA_TRY(h, cudaMalloc(&h->workspace, want));
  // The decode kernel's partial sums carry the number of the launch that wrote
  // them; zero is the one number no launch uses.
  CUDA_TRY(h, cudaMemset(h->workspace, 0, want));
  h->workspace_bytes = want;
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_shard_range(int64_t total, int32_t parts, int32_t rank,
                                                    int64_t align, int64_t *begin,
                                                    int64_t *end) {
  if (!begin || !end || total < 0 || parts <= 0 || rank < 0 || rank >= parts || align <= 0)
    return KAPYB_INVALID_ARG;
  const int64_t blocks = (total + align - 1) / align;
  const int64_t base = blocks / parts, extra = blocks % parts;
  const int64_t b0 = rank * base + std::min<int64_t>(rank, extra);
  const int64_t b1 = b0 + base + (rank < extra ? 1 : 0);
  *begin = std::min(total, b0 * align);
  *end = std::min(total, b1 * align);
  return KAPYB_OK;
}

// --------------------------------------------------------------- validation

// kapyb_tensor2d.cache: cache operator 0..7, eviction priority 0..4, volatile bit
static bool valid_cache(int c) {
  return (c & ~0x1ffff) == 0 && (c & 0xff) <= KAPYB_CACHE_CV && ((c >> 8) & 0xff) <= KAPYB_NO_ALLOCATE;
}

static bool valid_dtype(int d) { return d == KAPYB_F16 || d == KAPYB_BF16 || d == KAPYB_F32; }
static bool is_fp8(int d) { return d == KAPYB_F8E4M3 || d == KAPYB_F8E5M2; }
static bool valid_operand_dtype(int d) { return valid_dtype(d) || is_fp8(d); }

static const char *dtype_name(int d) {
  return d == KAPYB_F16     ? "f16"
         : d == KAPYB_BF16  ? "bf16"
         : d == KAPYB_F32   ? "f32"
         : d == KAPYB_F8E4M3 ? "f8E4M3"
         : d == KAPYB_F8E5M2 ? "f8E5M2"
         : d == KAPYB_I1     ? "i1"
                             : "?";
}

static const void *elem_ptr(const kapyb_tensor2d *t) {
  return static_cast<const char *>(t->ptr) + t->offset_elems * dtype_size(t->dtype);
}

// The checks of MatmulOp::verify (Kapy.cpp:459-565) that apply at whole-problem
// scope, with the reference's diagnostics.
static kapyb_status verify_matmul(kapyb_handle h, const kapyb_tensor2d *lhs,
                                  const kapyb_tensor2d *rhs, const kapyb_tensor2d *acc,
                                  const kapyb_tensor2d *out, const kapyb_epilogue *ep,
                                  int impl_way) {
  if (!lhs || !rhs || !out) return fail(h, KAPYB_INVALID_ARG, "matmul: NULL tensor descriptor");
  auto empty = [](const kapyb_tensor2d *t) { return t->size0 == 0 || t->size1 == 0; };
  if ((!lhs->ptr && !empty(lhs)) || (!rhs->ptr && !empty(rhs)) || (!out->ptr && !empty(out)))
    return fail(h, KAPYB_INVALID_ARG, "matmul: NULL data pointer");
  if (!valid_operand_dtype(lhs->dtype) || !valid_operand_dtype(rhs->dtype) || !valid_dtype(out->dtype))
    return fail(h, KAPYB_INVALID_ARG, "matmul: unknown element type");
  if (lhs->size0 < 0 || lhs->size1 < 0 || rhs->size0 < 0 || rhs->size1 < 0)
    return fail(h, KAPYB_INVALID_ARG, "matmul: negative size");
  // Out-of-bounds lanes of a matmul operand are filled with zeros (TMA fill, and
  // the zero accumulator contribution that implies).  The other padding options
  // of ld_global (Enums.td:52-61) would put NaN or infinities into every output
  // whose K range is ragged against the kernel's tile, which depends on a tile
  // size the caller cannot see: refuse them instead of ignoring them.
  if (!valid_cache(lhs->cache) || !valid_cache(rhs->cache) || !valid_cache(out->cache))
    return fail(h, KAPYB_INVALID_ARG, "matmul: unknown cache operator or eviction priority");
  if (lhs->padding != KAPYB_PAD_ZERO || rhs->padding != KAPYB_PAD_ZERO)
    return fail(h, KAPYB_UNSUPPORTED,
                "matmul: operands are padded with zeros only (padding option %d requested)",
                lhs->padding != KAPYB_PAD_ZERO ? lhs->padding : rhs->padding);
  if (lhs->size1 != rhs->size0)
    return fail(h, KAPYB_INVALID_ARG,
                "matmul: number of columns of lhs must be equal to number of rows of rhs");
  if (out->size0 != lhs->size0)
    return fail(h, KAPYB_INVALID_ARG,
                "matmul: number of rows of acc must be equal to number of rows of lhs");
  if (out->size1 != rhs->size1)
    return fail(h, KAPYB_INVALID_ARG,
                "matmul: number of columns of acc must be equal to number of columns of rhs");
  if (dtype_size(lhs->dtype) != dtype_size(rhs->dtype))
    return fail(h, KAPYB_INVALID_ARG, "matmul: lhs and rhs must have same element bit width");
  if (!is_fp8(lhs->dtype) && lhs->dtype != rhs->dtype)
    return fail(h, KAPYB_INVALID_ARG,
                "matmul: lhs and rhs must have same element type unless they have f8 element type");
  if (acc) {
    if (!acc->ptr || (acc->dtype != KAPYB_F16 && acc->dtype != KAPYB_F32))
      return fail(h, KAPYB_INVALID_ARG, "matmul: result must have f16 or f32 element type");
    if (lhs->dtype == KAPYB_BF16 && acc->dtype == KAPYB_F16)
      return fail(h, KAPYB_INVALID_ARG,
                  "matmul: result must have f32 element type when operands are bf16 element type");
    if (acc->size0 != out->size0 || acc->size1 != out->size1)
      return fail(h, KAPYB_INVALID_ARG, "matmul: acc shape must match the result shape");
  }
  const bool half_ops = lhs->dtype == KAPYB_F16 || lhs->dtype == KAPYB_BF16;
  switch (impl_way) {
  case KAPYB_MMA_ANY: break;
  case KAPYB_MMA_M16N8K8_F16:
    if (!half_ops)
      return fail(h, KAPYB_INVALID_ARG, "matmul: mma_m16n8k8_f16 operands must have f16 or bf16 element type");
    break;
  case KAPYB_MMA_M16N8K16_F16:
    if (!half_ops)
      return fail(h, KAPYB_INVALID_ARG, "matmul: mma_m16n8k16_f16 operands must have f16 or bf16 element type");
    break;
  case KAPYB_MMA_M16N8K8_TF32:
    if (lhs->dtype != KAPYB_F32)
      return fail(h, KAPYB_INVALID_ARG, "matmul: mma_m16n8k8_tf32 operands must have f32 element type");
    break;
  case KAPYB_MMA_M16N8K16_F8:
    if (!is_fp8(lhs->dtype) || !is_fp8(rhs->dtype))
      return fail(h, KAPYB_INVALID_ARG,
                  "matmul: mma_m16n8k16_f8 operands must have f8E4M3 or f8E5M2 element type");
    break;
  default: return fail(h, KAPYB_INVALID_ARG, "matmul: unknown MatmulImplWay %d", impl_way);
  }
  if (ep) {
    if (ep->bias && !valid_dtype(ep->bias_dtype)) return fail(h, KAPYB_INVALID_ARG, "matmul: bad bias dtype");
    if (ep->bias_axis != 0 && ep->bias_axis != 1) return fail(h, KAPYB_INVALID_ARG, "matmul: bias_axis must be 0 or 1");
    if (ep->activation < KAPYB_ACT_NONE || ep->activation > KAPYB_ACT_SILU)
      return fail(h, KAPYB_INVALID_ARG, "matmul: unknown activation %d", ep->activation);
    if (ep->rounding != KAPYB_RZ && ep->rounding != KAPYB_RN)
      return fail(h, KAPYB_INVALID_ARG, "matmul: rounding mode must be set for down cast");
  }
  return KAPYB_OK;
}

// ------------------------------------------------------------- tensor maps

static CUtensorMapDataType tmap_dtype(int dtype) {
  return dtype == KAPYB_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
         : dtype == KAPYB_F16  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
         : dtype == KAPYB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                               : CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

// 3-D map over a matrix whose unit-stride axis has `inner` elements and whose
// other axis has `outer` rows `ld` elements apart, repeated `batch` times.
static kapyb_status make_tmap(kapyb_handle h, CUtensorMap *map, const void *base, int dtype,
                              uint64_t inner, uint64_t outer, uint64_t batch, uint64_t ld,
                              uint64_t batch_stride, uint32_t box_inner, uint32_t box_outer,
                              bool swizzle_32b_units = false) {
  const uint64_t esz = dtype_size(dtype);
  cuuint64_t dims[3] = {inner, outer, batch};
  uint64_t bs = batch_stride * esz;
  if (batch <= 1 || bs == 0) bs = ((std::max<uint64_t>(outer, 1) * ld * esz) + 15) / 16 * 16;
  cuuint64_t strides[2] = {ld * esz, bs};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = h->encode(map, tmap_dtype(dtype), 3, const_cast<void *>(base), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle_32b_units ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                           : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(h, KAPYB_CUDA_ERROR,
                "cuTensorMapEncodeTiled failed (%d): dims=%llu,%llu,%llu ld=%llu box=%u,%u", (int)r,
                (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)batch,
                (unsigned long long)ld, box_inner, box_outer);
  return KAPYB_OK;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// A 2-D operand is TMA-describable when one stride is 1, its base is 16-byte
// aligned and the other stride (and the batch stride) are multiples of 16 bytes.
static bool tma_ok(const void *base, int dtype, int64_t unit_extent, int64_t other_extent,
                   int64_t ld, int64_t batch, int64_t batch_stride) {
  const int64_t esz = dtype_size(dtype);
  if (!aligned16(base)) return false;
  if (unit_extent <= 0 || other_extent <= 0) return false;
  if (other_extent > 1 && ((ld * esz) % 16 != 0 || ld < unit_extent)) return false;
  if (other_extent == 1 && (ld * esz) % 16 != 0) return false;
  if (batch > 1 && ((batch_stride * esz) % 16 != 0 || batch_stride <= 0)) return false;
  if (ld * esz >= (1ll << 40)) return false;
  return true;
}

// ------------------------------------------------------------------ matmul

struct MatmulProblem {
  const void *a, *b;
  void *c;
  int M, N, K, batch;
  long long a_s0, a_s1, a_bs, b_s0, b_s1, b_bs, c_s0, c_s1, c_bs;
  int in_dtype, in_dtype_b, out_dtype;
  EpilogueArgs ep;
  int a_l2 = 0, b_l2 = 0, c_l2 = 0;  // L2 policy of each tensor's TMA traffic (see l2_policy_of)
};

// kapyb_tensor2d.cache -> L2 policy of the tensor's TMA loads / stores: 0 default,
// 1 evict_first, 2 evict_last.  Tiles always pass through L2, so NO_ALLOCATE (and a
// streaming cache operator) become evict_first.
static int l2_policy_of(int cache) {
  const int mod = cache & 0xff, prio = (cache >> 8) & 0xff;
  if (prio == KAPYB_EVICT_FIRST || prio == KAPYB_NO_ALLOCATE) return 1;
  if (prio == KAPYB_EVICT_LAST) return 2;
  if (mod == KAPYB_CACHE_CS || mod == KAPYB_CACHE_LU) return 1;
  return 0;
}

static EpilogueArgs make_ep(const kapyb_epilogue *ep, const kapyb_tensor2d *acc) {
  EpilogueArgs e;
  e.alpha = ep ? ep->alpha : 1.0f;
  e.bias = ep ? ep->bias : nullptr;
  e.bias_dtype = ep ? ep->bias_dtype : KAPYB_F32;
  e.bias_axis = ep ? ep->bias_axis : 1;
  e.activation = ep ? ep->activation : KAPYB_ACT_NONE;
  e.rounding = ep ? ep->rounding : KAPYB_RN;
  e.acc = acc ? elem_ptr(acc) : nullptr;
  e.acc_dtype = acc ? acc->dtype : KAPYB_F32;
  e.acc_stride0 = acc ? acc->stride0 : 0;
  e.acc_stride1 = acc ? acc->stride1 : 0;
  e.acc_batch_stride = 0;
  return e;
}

static void transpose_problem(MatmulProblem &p) {
  // C^T = B^T . A^T
  std::swap(p.a, p.b);
  std::swap(p.in_dtype, p.in_dtype_b);
  std::swap(p.M, p.N);
  long long a0 = p.a_s0, a1 = p.a_s1, ab = p.a_bs;
  p.a_s0 = p.b_s1;
  p.a_s1 = p.b_s0;
  p.a_bs = p.b_bs;
  p.b_s0 = a1;
  p.b_s1 = a0;
  p.b_bs = ab;
  std::swap(p.c_s0, p.c_s1);
  std::swap(p.a_l2, p.b_l2);
  std::swap(p.ep.acc_stride0, p.ep.acc_stride1);
  p.ep.bias_axis ^= 1;
}

static kapyb_status launch_simt(kapyb_handle h, const MatmulProblem &p, cudaStream_t stream) {
  SimtGemmParams sp;
  sp.a = p.a;
  sp.b = p.b;
  sp.c = p.c;
  sp.M = p.M;
  sp.N = p.N;
  sp.K = p.K;
  sp.batch = p.batch;
  sp.a_s0 = p.a_s0;
  sp.a_s1 = p.a_s1;
  sp.a_bs = p.a_bs;
  sp.b_s0 = p.b_s0;
  sp.b_s1 = p.b_s1;
  sp.b_bs = p.b_bs;
  sp.c_s0 = p.c_s0;
  sp.c_s1 = p.c_s1;
  sp.c_bs = p.c_bs;
  sp.in_dtype = p.in_dtype;
  sp.in_dtype_b = p.in_dtype_b;
  sp.tf32 = p.in_dtype == KAPYB_F32 ? 1 : 0;
  sp.out_dtype = p.out_dtype;
  sp.ep = p.ep;
  dim3 grid((p.N + kSimtTile - 1) / kSimtTile, (p.M + kSimtTile - 1) / kSimtTile, p.batch);
  if (grid.y > 65535 || grid.z > 65535)
    return fail(h, KAPYB_UNSUPPORTED, "matmul (simt path): problem too large");
  gemm_simt_kernel<<<grid, 256, 0, stream>>>(sp);
  CUDA_TRY(h, cudaGetLastError());
  h->launches++;
  h->last_kernel = "simt";
  return KAPYB_OK;
}

// The last wave of a tcgen05 launch: `leftover` tiles for `units` CTAs (pairs).
// Split between all of them (each takes one contiguous span of the tiles' K
// blocks), every SM works to the end instead of a part of them for a whole
// tile's time.  Measured on the column shards of the 8192^3 problem (34, 54 and
// 64 tiles of 256 x 512 left for 74 pairs) this does NOT pay on a B200: the part
// runs at its power cap, so SMs that sit out the last wave hand their share of
// the power to the rest as clock, and the split adds traffic (a 512 KB partial
// accumulator per tile through L2, read back on the critical path) and scatters
// the tiles' K offsets, which costs operand reuse in L2: 8192 x 1024 x 8192 took
// 110 us split against 97 us whole, and 96.6 us with the partial sums' traffic
// compiled out.  So the split runs only when asked for (":x1"); the default
// keeps whole tiles.
struct TileSplit {
  bool on = false;
  int first_tile = 0;   // tiles below are dealt whole
  int k_blocks = 0;     // K blocks of the split tiles, all together
};

// the instantiations the split variant of the kernel is built for
constexpr bool split_built(int bn, int ctas, int epi) {
  return ctas == 2 ? (bn == 512 || epi == 4) : (bn == 256);
}

static TileSplit tile_split_of(int forced, long long tiles, int num_kb, int units, int bn, int ctas,
                               int epi) {
  TileSplit s;
  const int leftover = static_cast<int>(tiles % units);
  const long long blocks = static_cast<long long>(leftover) * num_kb;
  if (forced == 0 || leftover == 0 || !split_built(bn, ctas, epi) || blocks < units ||
      blocks > 0x3fffffff)
    return s;
  if (forced < 0) return s;  // not by default: see above
  s.on = true;
  s.first_tile = static_cast<int>(tiles - leftover);
  s.k_blocks = static_cast<int>(blocks);
  return s;
}

constexpr size_t kSplitFlagBytes = 65536;  // 8 words per CTA, up to 2048 CTAs

static kapyb_status reserve_split_scratch(kapyb_handle h, size_t bytes) {
  if (bytes <= h->split_scratch_bytes) return KAPYB_OK;
  CUDA_TRY(h, cudaDeviceSynchronize());
  if (h->split_scratch) {
    cudaFree(h->split_scratch);
    h->split_scratch = nullptr;
    h->split_scratch_bytes = 0;
  }
  CUDA_TRY(h, cudaMalloc(&h->split_scratch, bytes));
  // flag words carry launch numbers; zero is the one number no launch uses
  CUDA_TRY(h, cudaMemset(h->split_scratch, 0, kSplitFlagBytes));
  h->split_scratch_bytes = bytes;
  return KAPYB_OK;
}

template <int BN, int CTAS, int EPI>
static void tcgen05_launch_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute (&attr)[2],
                                  cudaStream_t stream) {
  using Cfg = GemmCfg<BN, CTAS, EPI>;
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // the kernel's set-up may overlap the tail of the kernel ahead of it in the
  // stream; it waits (griddepcontrol.wait) before it touches global memory
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
}

// CTAs (pairs) of this instantiation the device holds at once.  The tile loop is
// statically strided, so every CTA (pair) of the grid must be resident: a pair
// that only starts when another retires would run its whole share afterwards.
// Pairs need two free SMs in one GPC, which can be fewer than sm_count / 2.
template <int BN, int CTAS, int EPI, bool REDUCE, bool SK, int DRAIN>
static kapyb_status tcgen05_resident(kapyb_handle h, int &resident) {
  using Cfg = GemmCfg<BN, CTAS, EPI>;
  auto kern = gemm_tcgen05_kernel<BN, CTAS, EPI, REDUCE, SK, DRAIN>;
  static int cached[kMaxDevices] = {};
  if (cached[h->device] == 0) {
    CUDA_TRY(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::SMEM_BYTES));
    int n = h->sm_count / CTAS;
    if (CTAS == 2) {
      cudaLaunchConfig_t cfg = {};
      cudaLaunchAttribute attr[2];
      tcgen05_launch_config<BN, CTAS, EPI>(cfg, attr, nullptr);
      cfg.gridDim = dim3(h->sm_count / CTAS * CTAS, 1, 1);
      int clusters = 0;
      CUDA_TRY(h, cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg));
      n = std::min(n, std::max(1, clusters));
    }
    cached[h->device] = std::max(1, n);
  }
  resident = cached[h->device];
  return KAPYB_OK;
}

// DRAIN: the 16-bit output type the register-drain epilogue of the 512-wide tile is
// compiled for (1 bf16, 2 f16); other outputs of that tile, and every other tile,
// go chunk by chunk whatever it says.
template <int BN, int CTAS, int EPI, bool REDUCE = false, bool SK = false, int DRAIN = 1>
static kapyb_status launch_tcgen05(kapyb_handle h, const MatmulProblem &p, bool a_mn, bool b_mn,
                                   void *const *outs, int n_out, cudaStream_t stream,
                                   float *red = nullptr, int red_axis = 1) {
  using Cfg = GemmCfg<BN, CTAS, EPI>;
  CUtensorMap tmA, tmB;
  TmapArray tmC;
  kapyb_status st;
  if constexpr (BN == 512 && EPI == 8 && DRAIN == 1) {
    if (p.out_dtype == KAPYB_F16)
      return launch_tcgen05<BN, CTAS, EPI, REDUCE, SK, 2>(h, p, a_mn, b_mn, outs, n_out, stream, red,
                                                         red_axis);
  }
  if constexpr (!SK && !REDUCE && split_built(BN, CTAS, EPI)) {
    // the same kernel with the last wave's tiles split between the CTAs, when that pays
    int resident = 0;
    st = tcgen05_resident<BN, CTAS, EPI, false, true, DRAIN>(h, resident);
    if (st != KAPYB_OK) return st;
    const long long tiles = static_cast<long long>((p.M + Cfg::TILE_M - 1) / Cfg::TILE_M) *
                            ((p.N + BN - 1) / BN) * p.batch;
    const int num_kb = (p.K + 128 / static_cast<int>(dtype_size(p.in_dtype)) - 1) /
                       (128 / static_cast<int>(dtype_size(p.in_dtype)));
    if (tile_split_of(h->tile_split, tiles, num_kb, resident, BN, CTAS, EPI).on)
      return launch_tcgen05<BN, CTAS, EPI, false, true, DRAIN>(h, p, a_mn, b_mn, outs, n_out, stream);
  }
  // A shared-memory row is 128 bytes: `ce` elements of the operand type.
  // A: K-major -> inner K, rows M, box {ce, 128}; MN-major -> inner M, rows K, box {ce, ce}.
  const uint32_t ce = 128 / dtype_size(p.in_dtype);
  // A 32-bit operand whose unit stride is on M / N has to sit in shared memory
  // swizzled in 32-byte units (4-row pattern); everything else uses 16-byte units.
  const bool mn32 = dtype_size(p.in_dtype) == 4;
  if (!a_mn)
    st = make_tmap(h, &tmA, p.a, p.in_dtype, p.K, p.M, p.batch, p.a_s0, p.a_bs, ce, Cfg::BM);
  else
    st = make_tmap(h, &tmA, p.a, p.in_dtype, p.M, p.K, p.batch, p.a_s1, p.a_bs, ce, ce, mn32);
  if (st != KAPYB_OK) return st;
  // B [K,N]: MN-major (N contiguous) -> inner N, rows K, box {ce, ce};
  //          K-major (K contiguous)  -> inner K, rows N, box {ce, columns per CTA and half}.
  if (b_mn)
    st = make_tmap(h, &tmB, p.b, p.in_dtype_b, p.N, p.K, p.batch, p.b_s0, p.b_bs, ce, ce, mn32);
  else
    st = make_tmap(h, &tmB, p.b, p.in_dtype_b, p.K, p.N, p.batch, p.b_s1, p.b_bs, ce,
                   Cfg::MMA_N / CTAS);
  if (st != KAPYB_OK) return st;
  const uint32_t cw = p.out_dtype == KAPYB_F32 ? 32 : 64;
  for (int o = 0; o < n_out; ++o) {
    st = make_tmap(h, &tmC.m[o], outs[o], p.out_dtype, p.N, p.M, p.batch, p.c_s0, p.c_bs, cw, 32);
    if (st != KAPYB_OK) return st;
  }
  for (int o = n_out; o < kMaxOutputs; ++o) tmC.m[o] = tmC.m[0];

  GemmParams gp;
  gp.M = p.M;
  gp.N = p.N;
  gp.K = p.K;
  gp.batch = p.batch;
  gp.tiles_m = (p.M + Cfg::TILE_M - 1) / Cfg::TILE_M;
  gp.tiles_n = (p.N + BN - 1) / BN;
  gp.num_tiles = gp.tiles_m * gp.tiles_n * p.batch;
  gp.bk_elems = static_cast<int>(ce);
  gp.num_kb = (p.K + gp.bk_elems - 1) / gp.bk_elems;
  gp.kind = p.in_dtype == KAPYB_F32 ? 1 : is_fp8(p.in_dtype) ? 2 : 0;
  gp.mn_lbo = ce * 128u;                                 // ce K rows of 128 bytes per chunk
  gp.mn_kadv = (32u / dtype_size(p.in_dtype)) * 128u;    // K rows per MMA step x 128 bytes
  gp.mn_sbo = mn32 ? 512u : 1024u;
  gp.mn_layout = mn32 ? 1u : 2u;
  gp.group_m = std::max(1, std::min(gp.tiles_m, 16 / CTAS));
  gp.a_mn_major = a_mn ? 1 : 0;
  gp.b_mn_major = b_mn ? 1 : 0;
  gp.out_dtype = p.out_dtype;
  gp.n_out = n_out;
  gp.out_col_offset = 0;
  auto fmt = [](int dt) {
    return dt == KAPYB_BF16 ? 1 : dt == KAPYB_F32 ? 2 : dt == KAPYB_F8E5M2 ? 1 : 0;
  };
  gp.idesc = ptx::make_idesc(fmt(p.in_dtype), fmt(p.in_dtype_b), a_mn, b_mn, Cfg::TILE_M, Cfg::MMA_N);
  if (BN == 512) gp.group_m = std::max(1, std::min(gp.tiles_m, 12));
  if (h->forced_group_m > 0) gp.group_m = std::max(1, std::min(gp.tiles_m, h->forced_group_m));
  gp.div_per_batch = FastDiv::make(static_cast<uint32_t>(gp.tiles_m * gp.tiles_n));
  gp.div_in_group = FastDiv::make(static_cast<uint32_t>(gp.group_m * gp.tiles_n));
  gp.div_group_m = FastDiv::make(static_cast<uint32_t>(gp.group_m));
  gp.div_last_group = FastDiv::make(static_cast<uint32_t>(std::max(1, gp.tiles_m % gp.group_m)));
  gp.status = h->status;
  gp.debug = h->debug;
  gp.wait_limit_us = h->wait_limit_us;
  gp.ep = p.ep;
  gp.red = red;
  gp.red_axis = red_axis;
  gp.a_l2 = p.a_l2;
  gp.b_l2 = p.b_l2;
  gp.c_l2 = p.c_l2;

  gp.acc_tma = 0;
  if (p.ep.acc != nullptr && n_out < kMaxOutputs && p.ep.acc_dtype == p.out_dtype &&
      (p.ep.acc_stride1 == 1 || p.N == 1) &&
      tma_ok(p.ep.acc, p.ep.acc_dtype, p.N, p.M, p.ep.acc_stride0, p.batch, p.ep.acc_batch_stride)) {
    // the addend as tiles of the output's shape: fetched by TMA in the epilogue
    st = make_tmap(h, &tmC.m[kMaxOutputs - 1], p.ep.acc, p.ep.acc_dtype, p.N, p.M, p.batch,
                   p.ep.acc_stride0, p.ep.acc_batch_stride, cw, 32);
    if (st != KAPYB_OK) return st;
    gp.acc_tma = 1;
  }
  gp.sk_first_tile = gp.num_tiles;
  gp.sk_total = 0;
  gp.sk_scratch = nullptr;
  gp.sk_flags = nullptr;
  gp.sk_epoch = 0;

  int resident = 0;
  st = tcgen05_resident<BN, CTAS, EPI, REDUCE, SK, DRAIN>(h, resident);
  if (st != KAPYB_OK) return st;
  auto kern = gemm_tcgen05_kernel<BN, CTAS, EPI, REDUCE, SK, DRAIN>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  tcgen05_launch_config<BN, CTAS, EPI>(cfg, attr, stream);
  int units = std::min(gp.num_tiles, resident);
  if constexpr (SK) {
    const TileSplit ts = tile_split_of(h->tile_split, gp.num_tiles, gp.num_kb, resident, BN, CTAS, EPI);
    units = resident;
    const size_t slot_bytes = static_cast<size_t>(CTAS) * 128 * BN * sizeof(float);
    st = reserve_split_scratch(h, kSplitFlagBytes + static_cast<size_t>(units) * slot_bytes);
    if (st != KAPYB_OK) return st;
    if (static_cast<size_t>(units) * CTAS * 8 * sizeof(uint32_t) > kSplitFlagBytes)
      return fail(h, KAPYB_UNSUPPORTED, "matmul: more CTAs than the split tiles' flag words cover");
    gp.sk_first_tile = ts.first_tile;
    gp.sk_total = ts.k_blocks;
    gp.sk_flags = static_cast<uint32_t *>(h->split_scratch);
    gp.sk_scratch = reinterpret_cast<float *>(static_cast<char *>(h->split_scratch) + kSplitFlagBytes);
    if (++h->split_epoch == 0) h->split_epoch = 1;
    gp.sk_epoch = h->split_epoch;
  }
  cfg.gridDim = dim3(units * CTAS, 1, 1);
  CUDA_TRY(h, cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, gp));
  h->launches++;
  h->last_kernel = CTAS == 2 ? (SK ? "tcgen05_2cta_split" : "tcgen05_2cta")
                             : (SK ? "tcgen05_1cta_split" : "tcgen05_1cta");
  return KAPYB_OK;
}

static size_t skinny_workspace_bytes() { return kSkinnyScratchBytes; }

// Partial sums of split weight tiles: one slot of [roundup16(M)][128] (fp32, launch
// number) pairs per CTA.
static size_t skinny_partial_bytes(int sm_count, int M) {
  const int m_pad = (M + 15) / 16 * 16;
  return static_cast<size_t>(sm_count) * m_pad * 128 * sizeof(uint2);
}

static bool skinny_supported(int sm_count, int M, int N, int K) {
  return M >= 1 && M <= kSkinnyMaxM && K >= 1 && N >= 1 &&
         skinny_partial_bytes(sm_count, M) <= kSkinnyScratchBytes;
}

// Whether leftover weight tiles are split between SMs (stream-K) or every tile
// stays whole.  forced: -1 decide here, 0 never, 1 always.
static bool skinny_splits(int forced, int n_tiles, int sm_count) {
  if (forced == 0) return false;
  if (forced == 1) return true;
  // One whole tile per SM on 80-100 % of the SMs streams as fast as all SMs on
  // equal spans, and has no reduction at its end (measured at M = 16, K = 8192: 130
  // tiles 41.9 us whole against 46.4 us split; 112 tiles 40.4 / 41.0; 100 tiles
  // 40.3 / 38.0).  Everything else splits the leftover tiles.
  return !(n_tiles <= sm_count && n_tiles * 5 > sm_count * 4);
}

// Launches the weight-streaming kernel.  `scratch` holds (partial sum, launch
// number) pairs; `epoch` is this launch's number: not 0 and not a number that
// may still sit in the scratch (callers count up).
static kapyb_status launch_skinny_on(kapyb_handle h, const MatmulProblem &p, bool a_mn, bool b_mn,
                                     uint2 *scratch, uint32_t epoch, cudaStream_t stream) {
  SkinnyParams sp;
  sp.M = p.M;
  sp.N = p.N;
  sp.K = p.K;
  sp.m_pad = (p.M + 15) / 16 * 16;
  sp.num_kb = (p.K + 63) / 64;
  sp.n_tiles = (p.N + 127) / 128;
  sp.w_mn_major = b_mn ? 1 : 0;
  sp.x_mn_major = a_mn ? 1 : 0;
  sp.x_bytes = a_mn ? 8192 : sp.m_pad * 128;
  int cols = 32;
  while (cols < 2 * sp.m_pad) cols *= 2;
  sp.tmem_cols = cols;
  sp.out_dtype = p.out_dtype;
  sp.c_s0 = p.c_s0;
  sp.c_s1 = p.c_s1;
  sp.c = p.c;
  sp.scratch = scratch;
  sp.epoch = epoch;
  sp.idesc = ptx::make_idesc_f16(p.in_dtype == KAPYB_BF16, b_mn, a_mn, 128, sp.m_pad);
  sp.status = h->status;
  sp.wait_limit_us = h->wait_limit_us;
  sp.debug = h->debug;
  sp.ep = p.ep;
  // The weights are read once per call: unless the caller's descriptor says
  // otherwise they stream through L2 as evict_first, which alone is worth 2-4 % of
  // the kernel's time (72.8 -> 71.2 us at N = 28672, 78.8 -> 75.9 us at M = 64,
  // interleaved bursts); the activations, which every CTA re-reads, stay as they are.
  sp.w_l2 = p.b_l2 ? p.b_l2 : 1;
  sp.x_l2 = p.a_l2;
  // Whole tiles round-robin while they fill the GPU evenly; the leftover tiles
  // (all of them when there are fewer tiles than SMs) are split into equal spans.
  int grid;
  const bool split = skinny_splits(h->skinny_split, sp.n_tiles, h->sm_count);
  if (!split) {
    // whole tiles only, dealt round-robin (the last round may be ragged)
    grid = std::min(sp.n_tiles, h->sm_count);
    sp.dp_per_cta = (sp.n_tiles + grid - 1) / grid;
    sp.sk_tiles = 0;
    sp.span = 0;
  } else if (sp.n_tiles >= h->sm_count) {
    grid = h->sm_count;
    sp.dp_per_cta = sp.n_tiles / grid;
    sp.sk_tiles = sp.n_tiles % grid;
    const long long units = static_cast<long long>(sp.sk_tiles) * sp.num_kb;
    sp.span = static_cast<int>((units + grid - 1) / grid);
  } else {
    const long long units = static_cast<long long>(sp.n_tiles) * sp.num_kb;
    const int ctas = static_cast<int>(std::min<long long>(h->sm_count, units));
    sp.dp_per_cta = 0;
    sp.sk_tiles = sp.n_tiles;
    sp.span = static_cast<int>((units + ctas - 1) / ctas);
    grid = static_cast<int>((units + sp.span - 1) / sp.span);
  }
  const int stage_bytes = 128 * 64 * 2 + sp.x_bytes;
  const int budget = 232448 - 1024 - 1024;
  sp.stages = std::max(2, std::min(kSkinnyMaxStages, budget / stage_bytes));
  sp.stages = std::min(sp.stages, h->skinny_stages >= 2 ? h->skinny_stages : kSkinnyStages);
  const int smem = 1024 + sp.stages * stage_bytes + 1024;

  CUtensorMap tmW, tmX;
  kapyb_status st;
  if (b_mn)
    st = make_tmap(h, &tmW, p.b, p.in_dtype, p.N, p.K, 1, p.b_s0, 0, 64, 64);
  else
    st = make_tmap(h, &tmW, p.b, p.in_dtype, p.K, p.N, 1, p.b_s1, 0, 64, 128);
  if (st != KAPYB_OK) return st;
  if (a_mn)
    st = make_tmap(h, &tmX, p.a, p.in_dtype, p.M, p.K, 1, p.a_s1, 0, 64, 64);
  else
    st = make_tmap(h, &tmX, p.a, p.in_dtype, p.K, p.M, 1, p.a_s0, 0, 64, sp.m_pad);
  if (st != KAPYB_OK) return st;
  static bool attr_set[kMaxDevices] = {};
  if (!attr_set[h->device]) {
    CUDA_TRY(h, cudaFuncSetAttribute(gemm_skinny_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    attr_set[h->device] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kSkinnyThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see launch_tcgen05
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(h, cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, tmW, tmX, sp));
  h->launches++;
  h->last_kernel = "tcgen05_skinny";
  return KAPYB_OK;
}

static kapyb_status launch_skinny(kapyb_handle h, const MatmulProblem &p, bool a_mn, bool b_mn,
                                  cudaStream_t stream) {
  if (!skinny_supported(h->sm_count, p.M, p.N, p.K))
    return fail(h, KAPYB_UNSUPPORTED, "matmul: shape outside the skinny kernel's range");
  kapyb_status st = kapyb_reserve_workspace(h, skinny_workspace_bytes());
  if (st != KAPYB_OK) return st;
  if (++h->skinny_epoch == 0) ++h->skinny_epoch;  // 0 marks scratch no launch has written
  return launch_skinny_on(h, p, a_mn, b_mn, static_cast<uint2 *>(h->workspace), h->skinny_epoch, stream);
}

// What run_matmul decided for a problem: the kernel family, the tile, and the
// facts the choice rests on.  Computed on the host without touching the GPU.
struct MatmulPlan {
  int path = PATH_SIMT;        // PATH_SIMT / PATH_SKINNY / PATH_1CTA / PATH_2CTA
  bool transposed = false;     // the transposed problem is computed (out has its unit stride on axis 0)
  bool tuned = false;          // the choice came from the tuning table
  bool a_mn = false, b_mn = false;  // operand majors as the kernel sees them
  bool tma = false;            // operands and output are TMA-describable
  int bn = 0, epi = 4;         // tile width and epilogue warps (tcgen05 paths)
  const char *error = nullptr; // set with a non-OK status
};

struct PlanOptions {
  int sm_count;
  int forced_path, forced_bn, forced_epi;
};

// ---- tuned dispatch choices (process-wide; see kapyb_tuning_load)
struct TuneEntry {
  int M, N, K, batch, in_dtype, a_mn, b_mn;
  PathChoice choice;
};
static std::mutex g_tune_mu;
static std::vector<TuneEntry> g_tune;

static bool tuned_choice(const MatmulProblem &p, bool a_mn, bool b_mn, PathChoice &c) {
  std::lock_guard<std::mutex> lock(g_tune_mu);
  for (const TuneEntry &e : g_tune)
    if (e.M == p.M && e.N == p.N && e.K == p.K && e.batch == p.batch && e.in_dtype == p.in_dtype &&
        e.a_mn == (a_mn ? 1 : 0) && e.b_mn == (b_mn ? 1 : 0)) {
      c = e.choice;
      return true;
    }
  return false;
}

static kapyb_status plan_decide(const PlanOptions &o, const MatmulProblem &p, void *const *peer_outs,
                                int n_peers, MatmulPlan &plan);

// Decides how `p` runs.  `p` is transposed in place when the output's unit
// stride is on axis 0.  Without a forced path, a tuned choice for exactly this
// problem (shape, batch, operand type and majors) is tried first; if it does not
// apply after all, the built-in heuristics decide.
static kapyb_status plan_matmul(const PlanOptions &o, MatmulProblem &p, void *const *peer_outs,
                                int n_peers, MatmulPlan &plan) {
  // Put the output's unit stride on axis 1 (compute the transposed problem otherwise).
  const bool transposed = p.c_s1 != 1 && p.c_s0 == 1 && n_peers == 0;
  if (transposed) transpose_problem(p);
  if (o.forced_path == PATH_AUTO && o.forced_bn == 0) {
    const bool a_k = p.a_s1 == 1 || p.K == 1, a_m = p.a_s0 == 1 || p.M == 1;
    const bool b_n = p.b_s1 == 1 || p.N == 1;
    PathChoice c;
    if (tuned_choice(p, !a_k && a_m, b_n, c) && c.path != PATH_AUTO) {
      PlanOptions t = o;
      t.forced_path = c.path;
      t.forced_bn = c.bn;
      t.forced_epi = c.epi;
      MatmulPlan tuned;
      if (plan_decide(t, p, peer_outs, n_peers, tuned) == KAPYB_OK) {
        plan = tuned;
        plan.transposed = transposed;
        plan.tuned = true;
        return KAPYB_OK;
      }
    }
  }
  const kapyb_status st = plan_decide(o, p, peer_outs, n_peers, plan);
  plan.transposed = transposed;
  return st;
}

static kapyb_status plan_decide(const PlanOptions &o, const MatmulProblem &p, void *const *peer_outs,
                                int n_peers, MatmulPlan &plan) {
  const bool c_unit = p.c_s1 == 1 || p.N == 1;
  const bool a_k = p.a_s1 == 1 || p.K == 1, a_m = p.a_s0 == 1 || p.M == 1;
  const bool b_n = p.b_s1 == 1 || p.N == 1, b_k = p.b_s0 == 1 || p.K == 1;
  const bool a_mn = !a_k && a_m;
  const bool b_mn = b_n;  // prefer N-contiguous when both hold
  plan.a_mn = a_mn;
  plan.b_mn = b_mn;
  bool tma = c_unit && (a_k || a_m) && (b_n || b_k) && p.K > 0;
  if (tma) {
    tma = tma_ok(p.a, p.in_dtype, a_mn ? p.M : p.K, a_mn ? p.K : p.M, a_mn ? p.a_s1 : p.a_s0,
                 p.batch, p.a_bs) &&
          tma_ok(p.b, p.in_dtype_b, b_mn ? p.N : p.K, b_mn ? p.K : p.N, b_mn ? p.b_s0 : p.b_s1,
                 p.batch, p.b_bs) &&
          tma_ok(p.c, p.out_dtype, p.N, p.M, p.c_s0, p.batch, p.c_bs);
    for (int i = 0; tma && i < n_peers; ++i)
      tma = tma_ok(peer_outs[i], p.out_dtype, p.N, p.M, p.c_s0, 1, 0);
  }
  plan.tma = tma;
  int path = o.forced_path;
  if (path == PATH_SIMT || !tma) {
    if (n_peers > 0) {
      plan.error = "matmul_push: operands must be TMA-describable (16-byte aligned bases and "
                   "leading dimensions)";
      return KAPYB_UNSUPPORTED;
    }
    if (path != PATH_AUTO && path != PATH_SIMT && !tma) {
      plan.error = "matmul: forced tcgen05 path but operands are not TMA-describable";
      return KAPYB_UNSUPPORTED;
    }
    plan.path = PATH_SIMT;  // also K == 0: the epilogue of a zero accumulator
    return KAPYB_OK;
  }
  if (path == PATH_AUTO) {
    // CTA pairs halve the B traffic per SM and win once there is at least about
    // a quarter wave of pair tiles and a K loop long enough to amortise the
    // pair's start-up; everything else runs on single CTAs.
    const long long pair_tiles =
        static_cast<long long>((p.M + 255) / 256) * ((p.N + 255) / 256) * p.batch;
    if (p.M <= kSkinnyMaxM && n_peers == 0 && p.batch == 1 && dtype_size(p.in_dtype) == 2 &&
        skinny_supported(o.sm_count, p.M, p.N, p.K))
      path = PATH_SKINNY;
    else if (p.M >= 256 && p.N >= 256 && p.K >= 512 && pair_tiles * 5 >= o.sm_count && o.forced_bn == 0)
      path = PATH_2CTA;
    else
      path = PATH_1CTA;
  }
  if (path == PATH_SKINNY) {
    if (n_peers > 0 || p.batch != 1 || p.M > kSkinnyMaxM || dtype_size(p.in_dtype) != 2) {
      plan.error = "matmul: skinny path needs M <= 64, batch 1, 16-bit operands";
      return KAPYB_UNSUPPORTED;
    }
    if (!skinny_supported(o.sm_count, p.M, p.N, p.K)) {
      plan.error = "matmul: shape outside the skinny kernel's range";
      return KAPYB_UNSUPPORTED;
    }
    plan.path = PATH_SKINNY;
    return KAPYB_OK;
  }
  // Tile width for single CTAs: waves of tiles x the time of one tile.  A tile's
  // main loop is load latency per K block, so a narrower tile is only a little
  // quicker (measured 1.0 : 0.9 : 0.76 for 256 : 128 : 64 columns); it pays when
  // it saves a wave or fills more SMs in the only wave there is.
  int bn = o.forced_bn;
  if (bn == 0) {
    const long long tm = (p.M + 127) / 128;
    double best = 0.0;
    const int widths[3] = {256, 128, 64};
    const double tile_time[3] = {1.0, 0.9, 0.76};
    for (int i = 0; i < 3; ++i) {
      const int w = widths[i];
      if (w > 64 && p.N <= w / 2) continue;  // mostly padding
      const long long t = tm * ((p.N + w - 1) / w) * p.batch;
      const double cost = static_cast<double>((t + o.sm_count - 1) / o.sm_count) * tile_time[i];
      if (bn == 0 || cost < best - 1e-9) {
        bn = w;
        best = cost;
      }
    }
  }
  // An N-contiguous B arrives in chunks of 128 bytes of N: the columns one CTA
  // loads for one MMA (tile width / column halves / CTAs) have to hold at least
  // one chunk (128 columns of an 8-bit type).
  const int min_cols = b_mn ? 128 / static_cast<int>(dtype_size(p.in_dtype_b)) : 0;
  auto group_cols = [](int w, int ctas) { return w / (w == 512 ? 2 : 1) / ctas; };
  if (path == PATH_2CTA && group_cols(512, 2) >= min_cols && p.N < 512 &&
      group_cols(std::max(bn, 128), 2) < min_cols)
    path = PATH_1CTA;  // only the 512-wide pair tile would do, and N is too narrow for it
  while (path == PATH_1CTA && bn < 256 && group_cols(bn, 1) < min_cols) bn *= 2;
  if (path == PATH_2CTA) {
    if (o.forced_bn == 0) {
      // 256 x 512 pair tiles move a quarter fewer operand bytes per flop than
      // 256 x 256 and keep the tensor pipe fuller (two accumulators in turn): measured
      // about 1.25x per tile-wave, so take them unless they fill the waves that much worse.
      const int pairs = std::max(1, o.sm_count / 2);
      auto wave_eff = [&](int w) {
        const long long t = static_cast<long long>((p.M + 255) / 256) * ((p.N + w - 1) / w) * p.batch;
        return static_cast<double>(t) / static_cast<double>((t + pairs - 1) / pairs * pairs);
      };
      bn = (p.N >= 512 && p.K >= 1024 && wave_eff(512) >= 0.8 * wave_eff(256)) ? 512 : 256;
      // The wide tile's drain is not hidden behind the next tile's main loop, which
      // costs the more the shorter the K loop and the fewer the waves: measured
      // 256-wide against 512-wide, 4096 x 4096 x 1024 30.7 : 34.0 us, 4096 x 2048 x 2048
      // 29.6 : 32.3, 2048 x 4096 x 4096 51.3 : 53.3; the other way round 8192 x 8192 x 2048
      // 190 : 184, 4096^3 99.5 : 97.5, 8192 x 1024 x 8192 102 : 96.
      const long long t512 = static_cast<long long>((p.M + 255) / 256) * ((p.N + 511) / 512) * p.batch;
      if (bn == 512 && ((p.K <= 2048 && t512 < 3 * pairs) || (p.K <= 4096 && t512 <= pairs))) bn = 256;
      // less than half a wave of 256-wide pair tiles: 128-wide ones put more SMs to work
      const long long t256 = static_cast<long long>((p.M + 255) / 256) * ((p.N + 255) / 256) * p.batch;
      if (bn == 256 && t256 * 2 <= pairs) bn = 128;
      // Push epilogue: a tile's stores to the peers can only leave when its K loop is
      // over, so more, smaller tiles start the NVLink traffic earlier, which outweighs
      // their slower main loop once there is a wave of them (full output on every rank,
      // 8192^3, 256-wide against 512-wide: 2 GPUs 0.410 : 0.422 ms, 4 GPUs 0.289 : 0.312,
      // 8 GPUs 0.268 : 0.278; 128-wide tiles are slower again: 0.303 at 8 GPUs).
      if (n_peers > 0 && bn == 512 && t256 >= pairs) bn = 256;
    }
    if (bn == 64) bn = 128;
    if (group_cols(bn, 2) < min_cols) bn = 512;
    plan.path = PATH_2CTA;
    plan.bn = bn;
    plan.epi = bn == 512 && o.forced_epi != 4 ? 8 : 4;
    return KAPYB_OK;
  }
  // Short K loops cannot hide the epilogue behind the next tile's main loop:
  // give those problems eight epilogue warps instead of four.
  const bool epi8 = (p.K + 63) / 64 <= 8 || o.forced_epi == 8;
  plan.path = PATH_1CTA;
  plan.bn = bn;
  plan.epi = epi8 && o.forced_epi != 4 ? 8 : 4;
  return KAPYB_OK;
}

// Pipeline depth of a tcgen05 configuration (GemmCfg::STAGES of the instantiation).
static int stages_of(int bn, int ctas, int epi) {
  if (ctas == 2) {
    if (bn == 128) return GemmCfg<128, 2, 4>::STAGES;
    if (bn == 256) return GemmCfg<256, 2, 4>::STAGES;
    return epi == 8 ? GemmCfg<512, 2, 8>::STAGES : GemmCfg<512, 2, 4>::STAGES;
  }
  if (epi == 8)
    return bn == 64 ? GemmCfg<64, 1, 8>::STAGES : bn == 128 ? GemmCfg<128, 1, 8>::STAGES
                                                             : GemmCfg<256, 1, 8>::STAGES;
  return bn == 64 ? GemmCfg<64, 1, 4>::STAGES : bn == 128 ? GemmCfg<128, 1, 4>::STAGES
                                                           : GemmCfg<256, 1, 4>::STAGES;
}

static kapyb_status run_matmul(kapyb_handle h, MatmulProblem p, void *const *peer_outs,
                               int n_peers, cudaStream_t stream) {
  if (p.M == 0 || p.N == 0 || p.batch == 0) return KAPYB_OK;  // empty result
  CUDA_TRY(h, cudaSetDevice(h->device));
  MatmulPlan plan;
  const PlanOptions opt{h->sm_count, h->forced_path, h->forced_bn, h->forced_epi};
  kapyb_status st = plan_matmul(opt, p, peer_outs, n_peers, plan);
  if (st != KAPYB_OK) return fail(h, st, "%s", plan.error);
  const bool a_mn = plan.a_mn, b_mn = plan.b_mn;
  if (plan.path == PATH_SIMT) return launch_simt(h, p, stream);
  if (plan.path == PATH_SKINNY) return launch_skinny(h, p, a_mn, b_mn, stream);
  void *own[1] = {p.c};
  void *const *outs = n_peers > 0 ? peer_outs : own;
  const int n_out = n_peers > 0 ? n_peers : 1;
  const int bn = plan.bn;
  if (plan.path == PATH_2CTA) {
    if (bn == 128) return launch_tcgen05<128, 2, 4>(h, p, a_mn, b_mn, outs, n_out, stream);
    if (bn == 512) {
      if (plan.epi == 4) return launch_tcgen05<512, 2, 4>(h, p, a_mn, b_mn, outs, n_out, stream);
      return launch_tcgen05<512, 2, 8>(h, p, a_mn, b_mn, outs, n_out, stream);
    }
    return launch_tcgen05<256, 2, 4>(h, p, a_mn, b_mn, outs, n_out, stream);
  }
  if (plan.epi == 8) {
    if (bn == 64) return launch_tcgen05<64, 1, 8>(h, p, a_mn, b_mn, outs, n_out, stream);
    if (bn == 128) return launch_tcgen05<128, 1, 8>(h, p, a_mn, b_mn, outs, n_out, stream);
    return launch_tcgen05<256, 1, 8>(h, p, a_mn, b_mn, outs, n_out, stream);
  }
  if (bn == 64) return launch_tcgen05<64, 1, 4>(h, p, a_mn, b_mn, outs, n_out, stream);
  if (bn == 128) return launch_tcgen05<128, 1, 4>(h, p, a_mn, b_mn, outs, n_out, stream);
  return launch_tcgen05<256, 1, 4>(h, p, a_mn, b_mn, outs, n_out, stream);
}

static MatmulProblem make_problem(const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
                                  const kapyb_tensor2d *acc, const kapyb_tensor2d *out,
                                  const kapyb_epilogue *ep) {
  MatmulProblem p;
  p.a = elem_ptr(lhs);
  p.b = elem_ptr(rhs);
  p.c = const_cast<void *>(elem_ptr(out));
  p.M = lhs->size0;
  p.K = lhs->size1;
  p.N = rhs->size1;
  p.batch = 1;
  p.a_s0 = lhs->stride0;
  p.a_s1 = lhs->stride1;
  p.b_s0 = rhs->stride0;
  p.b_s1 = rhs->stride1;
  p.c_s0 = out->stride0;
  p.c_s1 = out->stride1;
  p.a_bs = p.b_bs = p.c_bs = 0;
  p.in_dtype = lhs->dtype;
  p.in_dtype_b = rhs->dtype;
  p.out_dtype = out->dtype;
  p.ep = make_ep(ep, acc);
  p.a_l2 = l2_policy_of(lhs->cache);
  p.b_l2 = l2_policy_of(rhs->cache);
  p.c_l2 = l2_policy_of(out->cache);
  return p;
}

extern "C" KAPYB_API kapyb_status kapyb_matmul_plan(kapyb_handle h, int32_t sm_count,
                                                    const kapyb_tensor2d *lhs,
                                                    const kapyb_tensor2d *rhs,
                                                    const kapyb_tensor2d *out, int32_t batch,
                                                    char *text, size_t capacity) {
  if (!text || capacity == 0) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_plan: no text buffer");
  text[0] = 0;
  if (!h && sm_count <= 0)
    return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_plan: give a handle or an SM count");
  kapyb_status st = verify_matmul(h, lhs, rhs, nullptr, out, nullptr, KAPYB_MMA_ANY);
  if (st != KAPYB_OK) return st;
  if (batch < 1) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_plan: batch must be >= 1");
  MatmulProblem p = make_problem(lhs, rhs, nullptr, out, nullptr);
  p.batch = batch;
  if (batch > 1) {  // densely packed batch entries
    p.a_bs = static_cast<long long>(p.M) * p.K;
    p.b_bs = static_cast<long long>(p.K) * p.N;
    p.c_bs = static_cast<long long>(p.M) * p.N;
  }
  PlanOptions opt{sm_count > 0 ? sm_count : h->sm_count, h ? h->forced_path : PATH_AUTO,
                  h ? h->forced_bn : 0, h ? h->forced_epi : 0};
  MatmulPlan plan;
  if (p.M == 0 || p.N == 0) {
    snprintf(text, capacity, "path: none (empty result)\n");
    return KAPYB_OK;
  }
  st = plan_matmul(opt, p, nullptr, 0, plan);
  if (st != KAPYB_OK) return fail(h, st, "%s", plan.error);
  const char *amaj = plan.a_mn ? "M contiguous (MN-major)" : "K contiguous (K-major)";
  const char *bmaj = plan.b_mn ? "N contiguous (MN-major)" : "K contiguous (K-major)";
  int n = 0;
  auto add = [&](const char *fmt, auto... args) {
    if (n < static_cast<int>(capacity))
      n += snprintf(text + n, capacity - n, fmt, args...);
  };
  if (plan.path == PATH_SIMT) {
    add("path: simt (CUDA cores; %s)\n",
        plan.tma ? "forced" : "an operand or the output has no unit stride, a base off 16 bytes or a "
                              "leading dimension that is not a multiple of 16 bytes");
    add("tile: 64 x 64 x 16 elements, 256 threads, grid %d x %d x %d\n", (p.N + 63) / 64,
        (p.M + 63) / 64, p.batch);
  } else if (plan.path == PATH_SKINNY) {
    const int num_kb = (p.K + 63) / 64, n_tiles = (p.N + 127) / 128;
    const bool split = skinny_splits(h ? h->skinny_split : -1, n_tiles, opt.sm_count);
    const int grid = split ? static_cast<int>(std::min<long long>(opt.sm_count, static_cast<long long>(n_tiles) * num_kb))
                           : std::min(n_tiles, opt.sm_count);
    const int dp = !split ? (n_tiles + grid - 1) / grid : n_tiles >= opt.sm_count ? n_tiles / opt.sm_count : 0;
    const int sk = !split ? 0 : n_tiles >= opt.sm_count ? n_tiles % opt.sm_count : n_tiles;
    add("path: %s\n", "tcgen05_skinny (weights on the 128-row side of the MMA, activations on its N side)");
    add("tile: 128 weight columns x %d rows x 64 k; %d weight tiles x %d k-blocks on %d CTAs\n",
        (p.M + 15) / 16 * 16, n_tiles, num_kb, grid);
    add("schedule: %d split tile(s) first, in spans of %lld k-block(s); then %d whole tile(s) per CTA\n",
        sk, sk ? (static_cast<long long>(sk) * num_kb + grid - 1) / grid : 0ll, dp);
  } else {
    const int ctas = plan.path == PATH_2CTA ? 2 : 1;
    const int tile_m = 128 * ctas;
    const int tiles_m = (p.M + tile_m - 1) / tile_m, tiles_n = (p.N + plan.bn - 1) / plan.bn;
    const long long tiles = static_cast<long long>(tiles_m) * tiles_n * p.batch;
    const int units = std::max(1, opt.sm_count / ctas);
    const long long waves = (tiles + units - 1) / units;
    add("path: %s\n", ctas == 2 ? "tcgen05_2cta (CTA pairs, cta_group::2)" : "tcgen05_1cta");
    add("tile: %d x %d x 128 bytes of K%s; stages %d, epilogue warps %d, TMEM columns %d\n", tile_m,
        plan.bn, plan.bn == 512 ? " (two 256-column halves, one accumulator each)" : "",
        stages_of(plan.bn, ctas, plan.epi), plan.epi,
        plan.bn == 512 ? 512 : std::max(32, 2 * plan.bn));
    add("grid: %d x %d x %d = %lld tile(s) on %d %s: %lld wave(s), %.0f %% of their slots used\n",
        tiles_m, tiles_n, p.batch, tiles, units, ctas == 2 ? "CTA pairs" : "CTAs", waves,
        100.0 * static_cast<double>(tiles) / static_cast<double>(waves * units));
    const int num_kb = (p.K + 128 / static_cast<int>(dtype_size(p.in_dtype)) - 1) /
                       (128 / static_cast<int>(dtype_size(p.in_dtype)));
    const TileSplit ts = tile_split_of(h ? h->tile_split : -1, tiles, num_kb, units, plan.bn, ctas, plan.epi);
    if (ts.on)
      add("last wave: %lld tile(s) x %d k-blocks split between the %d %s in spans of %d-%d k-blocks "
          "(partial sums added in CTA order)\n",
          tiles - ts.first_tile, num_kb, units, ctas == 2 ? "CTA pairs" : "CTAs", ts.k_blocks / units,
          (ts.k_blocks + units - 1) / units);
    add("lanes: accumulator row r of a tile -> CTA r / 128 of the %s, TMEM lane r %% 128; "
        "column c -> TMEM column c%s\n",
        ctas == 2 ? "pair" : "tile (always 0)", plan.bn == 512 ? "" : " + slot * tile width");
  }
  add("operands: A %s, B %s%s\n", amaj, bmaj,
      plan.transposed ? "; the transposed problem is computed (out has its unit stride on axis 0)" : "");
  if (plan.tuned) add("%s\n", "choice: from the tuning table");
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_tuning_clear(void) {
  std::lock_guard<std::mutex> lock(g_tune_mu);
  g_tune.clear();
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_tuning_load(const char *file, int32_t *n_entries) {
  if (n_entries) *n_entries = 0;
  if (!file) return fail(nullptr, KAPYB_INVALID_ARG, "kapyb_tuning_load: NULL file name");
  std::ifstream in(file);
  if (!in) return fail(nullptr, KAPYB_INVALID_ARG, "kapyb_tuning_load: cannot read '%s'", file);
  std::vector<TuneEntry> loaded;
  std::string line;
  int lineno = 0;
  while (std::getline(in, line)) {
    ++lineno;
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.resize(hash);
    std::istringstream ls(line);
    TuneEntry e{};
    std::string dt, amaj, bmaj, path;
    if (!(ls >> e.M)) continue;  // blank or comment line
    const char *why = "";
    if (!(ls >> e.N >> e.K >> e.batch >> dt >> amaj >> bmaj >> path) || e.M < 1 || e.N < 1 ||
        e.K < 1 || e.batch < 1 || (e.in_dtype = dtype_from_name(dt)) < 0 ||
        (amaj != "k" && amaj != "mn") || (bmaj != "k" && bmaj != "mn") ||
        !parse_path(path, e.choice, &why) || e.choice.debug != 0)
      return fail(nullptr, KAPYB_INVALID_ARG,
                  "kapyb_tuning_load: %s line %d is not 'M N K batch dtype k|mn k|mn path'", file,
                  lineno);
    e.a_mn = amaj == "mn";
    e.b_mn = bmaj == "mn";
    loaded.push_back(e);
  }
  std::lock_guard<std::mutex> lock(g_tune_mu);
  for (const TuneEntry &e : loaded) {
    bool replaced = false;
    for (TuneEntry &old : g_tune)
      if (old.M == e.M && old.N == e.N && old.K == e.K && old.batch == e.batch &&
          old.in_dtype == e.in_dtype && old.a_mn == e.a_mn && old.b_mn == e.b_mn) {
        old = e;
        replaced = true;
      }
    if (!replaced) g_tune.push_back(e);
  }
  if (n_entries) *n_entries = static_cast<int32_t>(loaded.size());
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_matmul(kapyb_handle h, const kapyb_tensor2d *lhs,
                                               const kapyb_tensor2d *rhs,
                                               const kapyb_tensor2d *acc,
                                               const kapyb_tensor2d *out,
                                               const kapyb_epilogue *epilogue, int32_t impl_way,
                                               void *stream) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul: NULL handle");
  kapyb_status st = verify_matmul(h, lhs, rhs, acc, out, epilogue, impl_way);
  if (st != KAPYB_OK) return st;
  return run_matmul(h, make_problem(lhs, rhs, acc, out, epilogue), nullptr, 0,
                    static_cast<cudaStream_t>(stream));
}

extern "C" KAPYB_API kapyb_status kapyb_matmul_reduce(
    kapyb_handle h, const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs, const kapyb_tensor2d *out,
    const kapyb_tensor2d *reduced, int32_t axis, int32_t combiner, const kapyb_epilogue *epilogue,
    int32_t impl_way, void *stream_) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_reduce: NULL handle");
  kapyb_status st = verify_matmul(h, lhs, rhs, nullptr, out, epilogue, impl_way);
  if (st != KAPYB_OK) return st;
  if (!reduced || axis < 0 || axis > 1)
    return fail(h, KAPYB_INVALID_ARG, "matmul_reduce: axis must be 0 or 1 and `reduced` given");
  if (combiner != KAPYB_RED_ADD)
    return fail(h, KAPYB_UNSUPPORTED, "matmul_reduce: only the addf lambda is fused (combiner %d)", combiner);
  // ReduceOp::inferReturnTypes (Kapy.cpp:613-626): the reduced axis becomes 1
  const int want0 = axis == 0 ? 1 : out->size0, want1 = axis == 1 ? 1 : out->size1;
  if (reduced->size0 != want0 || reduced->size1 != want1)
    return fail(h, KAPYB_INVALID_ARG, "matmul_reduce: result shape must be [%d, %d]", want0, want1);
  const int len = axis == 1 ? out->size0 : out->size1;
  const int rstride = axis == 1 ? reduced->stride0 : reduced->stride1;
  if (reduced->dtype != KAPYB_F32 || (len > 1 && rstride != 1) || (len > 0 && !reduced->ptr))
    return fail(h, KAPYB_UNSUPPORTED, "matmul_reduce: `reduced` must be a dense f32 vector");
  if (len == 0) return KAPYB_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  CUDA_TRY(h, cudaSetDevice(h->device));
  float *red = static_cast<float *>(const_cast<void *>(elem_ptr(reduced)));
  // the sums are formed with atomic adds: they start from zero (and stay zero
  // when there is nothing to sum)
  CUDA_TRY(h, cudaMemsetAsync(red, 0, static_cast<size_t>(len) * sizeof(float), stream));
  if (out->size0 == 0 || out->size1 == 0) return KAPYB_OK;
  MatmulProblem p = make_problem(lhs, rhs, nullptr, out, epilogue);
  MatmulPlan plan;
  const PlanOptions opt{h->sm_count, PATH_1CTA, 128, 4};
  st = plan_decide(opt, p, nullptr, 0, plan);
  if (st != KAPYB_OK) return fail(h, st, "%s", plan.error);
  if (plan.path != PATH_1CTA || !plan.tma || p.c_s1 != 1 || p.K < 1)
    return fail(h, KAPYB_UNSUPPORTED,
                "matmul_reduce: operands and a row-major output must be TMA-describable "
                "(unit strides, 16-byte aligned bases and leading dimensions), K >= 1");
  void *own[1] = {p.c};
  if (plan.bn == 256)
    return launch_tcgen05<256, 1, 4, true>(h, p, plan.a_mn, plan.b_mn, own, 1, stream, red, axis);
  return launch_tcgen05<128, 1, 4, true>(h, p, plan.a_mn, plan.b_mn, own, 1, stream, red, axis);
}

extern "C" KAPYB_API kapyb_status kapyb_matmul_batched(
    kapyb_handle h, const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
    const kapyb_tensor2d *out, int32_t batch, int64_t batch_stride_lhs, int64_t batch_stride_rhs,
    int64_t batch_stride_out, const kapyb_epilogue *epilogue, int32_t impl_way, void *stream) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_batched: NULL handle");
  kapyb_status st = verify_matmul(h, lhs, rhs, nullptr, out, epilogue, impl_way);
  if (st != KAPYB_OK) return st;
  if (batch < 0 || batch > 65535) return fail(h, KAPYB_INVALID_ARG, "matmul_batched: batch must be in [0, 65535]");
  if (batch > 1 && (batch_stride_lhs < 0 || batch_stride_rhs < 0 || batch_stride_out <= 0))
    return fail(h, KAPYB_INVALID_ARG, "matmul_batched: bad batch stride");
  MatmulProblem p = make_problem(lhs, rhs, nullptr, out, epilogue);
  p.batch = batch;
  p.a_bs = batch_stride_lhs;
  p.b_bs = batch_stride_rhs;
  p.c_bs = batch_stride_out;
  return run_matmul(h, p, nullptr, 0, static_cast<cudaStream_t>(stream));
}

extern "C" KAPYB_API kapyb_status kapyb_matmul_push(
    kapyb_handle h, const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs, void *const *peer_out,
    int32_t n_peers, int32_t out_dtype, int32_t out_stride0, int32_t col_begin, int32_t n_total,
    const kapyb_epilogue *epilogue, int32_t impl_way, void *stream) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_push: NULL handle");
  if (!peer_out || n_peers < 1 || n_peers > kMaxOutputs)
    return fail(h, KAPYB_INVALID_ARG, "matmul_push: n_peers must be in [1, %d]", kMaxOutputs);
  if (!lhs || !rhs) return fail(h, KAPYB_INVALID_ARG, "matmul_push: NULL tensor descriptor");
  if (col_begin < 0 || col_begin + rhs->size1 > n_total || out_stride0 < n_total)
    return fail(h, KAPYB_INVALID_ARG, "matmul_push: column block [%d, %d) outside [0, %d)",
                col_begin, col_begin + rhs->size1, n_total);
  kapyb_tensor2d out;
  out.ptr = peer_out[0];
  out.offset_elems = col_begin;
  out.size0 = lhs->size0;
  out.size1 = rhs->size1;
  out.stride0 = out_stride0;
  out.stride1 = 1;
  out.dtype = out_dtype;
  out.padding = 0;
  out.cache = 0;
  out.reserved_ = 0;
  kapyb_status st = verify_matmul(h, lhs, rhs, nullptr, &out, epilogue, impl_way);
  if (st != KAPYB_OK) return st;
  void *outs[kMaxOutputs];
  for (int r = 0; r < n_peers; ++r) {
    if (!peer_out[r]) return fail(h, KAPYB_INVALID_ARG, "matmul_push: peer_out[%d] is NULL", r);
    outs[r] = static_cast<char *>(peer_out[r]) + static_cast<int64_t>(col_begin) * dtype_size(out_dtype);
  }
  MatmulProblem p = make_problem(lhs, rhs, nullptr, &out, epilogue);
  return run_matmul(h, p, outs, n_peers, static_cast<cudaStream_t>(stream));
}

// Number of bytes spanned by a host tensor starting at its element (0,0).
static size_t span_bytes(const kapyb_tensor2d *t) {
  if (t->size0 <= 0 || t->size1 <= 0) return 0;
  const int64_t last = static_cast<int64_t>(t->size0 - 1) * t->stride0 +
                       static_cast<int64_t>(t->size1 - 1) * t->stride1;
  return static_cast<size_t>(last + 1) * dtype_size(t->dtype);
}

static size_t round256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// Copy streams and events of the host-buffer pipelines, created on first use.
static kapyb_status ensure_pipe(kapyb_handle h) {
  if (h->pipe_ready) return KAPYB_OK;
  CUDA_TRY(h, cudaStreamCreateWithFlags(&h->copy_in, cudaStreamNonBlocking));
  CUDA_TRY(h, cudaStreamCreateWithFlags(&h->copy_out, cudaStreamNonBlocking));
  for (cudaEvent_t &e : h->ev) CUDA_TRY(h, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  h->pipe_ready = true;
  return KAPYB_OK;
}

// KAPYB_TRACE=1 in the environment makes the host-buffer calls record a timing
// event on the stream of each phase as the phase is issued and, when the call is
// over, print when each one completed on the device (milliseconds after the
// call's first event) next to the host time at which it had been issued.
// Nothing is synchronised while the call runs, so the overlap is the real one.
// A diagnosis aid: events are created per call, so leave it off in timed runs.
struct HostTrace {
  bool on;
  int rank;
  std::chrono::steady_clock::time_point t0;
  struct Mark {
    const char *what;
    int index;
    cudaEvent_t ev;
    double issued_ms;
  };
  std::vector<Mark> marks;
  explicit HostTrace(int rank_) : rank(rank_), t0(std::chrono::steady_clock::now()) {
    const char *e = getenv("KAPYB_TRACE");
    on = e && e[0] && e[0] != '0';
  }
  double ms() const {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  }
  void mark(const char *what, cudaStream_t s, int index = -1) {
    if (!on) return;
    cudaEvent_t ev;
    if (cudaEventCreate(&ev) != cudaSuccess) return;
    cudaEventRecord(ev, s);
    marks.push_back(Mark{what, index, ev, ms()});
  }
  // call after everything has completed
  void report() {
    if (!on || marks.empty()) return;
    for (const Mark &m : marks) {
      float dev_ms = 0.0f;
      cudaEventElapsedTime(&dev_ms, marks[0].ev, m.ev);
      if (m.index >= 0)
        fprintf(stderr, "[kapyb trace r%d] %-22s %d  issued %7.3f ms, done on device %7.3f ms\n", rank,
                m.what, m.index, m.issued_ms, dev_ms);
      else
        fprintf(stderr, "[kapyb trace r%d] %-24s issued %7.3f ms, done on device %7.3f ms\n", rank,
                m.what, m.issued_ms, dev_ms);
    }
    fprintf(stderr, "[kapyb trace r%d] call returns at %7.3f ms (host)\n", rank, ms());
    for (const Mark &m : marks) cudaEventDestroy(m.ev);
    marks.clear();
  }
};

extern "C" KAPYB_API kapyb_status kapyb_matmul_host(kapyb_handle h, const kapyb_tensor2d *lhs,
                                                    const kapyb_tensor2d *rhs,
                                                    const kapyb_tensor2d *out,
                                                    const kapyb_epilogue *epilogue,
                                                    int32_t impl_way, void *stream_) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_host: NULL handle");
  kapyb_status st = verify_matmul(h, lhs, rhs, nullptr, out, epilogue, impl_way);
  if (st != KAPYB_OK) return st;
  if (lhs->stride0 < 0 || lhs->stride1 < 0 || rhs->stride0 < 0 || rhs->stride1 < 0 ||
      out->stride0 < 0 || out->stride1 < 0)
    return fail(h, KAPYB_UNSUPPORTED, "matmul_host: negative strides are not supported");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t na = span_bytes(lhs), nb = span_bytes(rhs), nc = span_bytes(out);
  size_t nbias = 0;
  if (epilogue && epilogue->bias)
    nbias = static_cast<size_t>(epilogue->bias_axis == 1 ? rhs->size1 : lhs->size0) *
            dtype_size(epilogue->bias_dtype);
  const size_t skinny_ws = skinny_workspace_bytes();
  const size_t need = skinny_ws + round256(na) + round256(nb) + round256(nc) + round256(nbias);
  st = kapyb_reserve_workspace(h, need);
  if (st != KAPYB_OK) return st;
  CUDA_TRY(h, cudaSetDevice(h->device));
  char *w = static_cast<char *>(h->workspace) + skinny_ws;
  char *da = w, *db = da + round256(na), *dc = db + round256(nb), *dbias = dc + round256(nc);
  // Large row-major problems go up and come back in row chunks (see below).
  const bool can_pipe = lhs->stride1 == 1 && out->stride1 == 1 && out->stride0 == out->size1 &&
                        lhs->stride0 == lhs->size1 && lhs->size0 >= 2048 &&
                        (static_cast<size_t>(lhs->size0) * lhs->size1 >= (1u << 22));
  if (!can_pipe)
    CUDA_TRY(h, cudaMemcpyAsync(da, elem_ptr(lhs), na, cudaMemcpyHostToDevice, stream));
  CUDA_TRY(h, cudaMemcpyAsync(db, elem_ptr(rhs), nb, cudaMemcpyHostToDevice, stream));
  kapyb_epilogue ep;
  if (epilogue)
    ep = *epilogue;
  else {
    ep.alpha = 1.0f;
    ep.bias = nullptr;
    ep.bias_dtype = KAPYB_F32;
    ep.bias_axis = 1;
    ep.activation = KAPYB_ACT_NONE;
    ep.rounding = KAPYB_RN;
  }
  if (nbias) {
    CUDA_TRY(h, cudaMemcpyAsync(dbias, ep.bias, nbias, cudaMemcpyHostToDevice, stream));
    ep.bias = dbias;
  }
  kapyb_tensor2d dl = *lhs, dr = *rhs, dout = *out;
  dl.ptr = da;
  dl.offset_elems = 0;
  dr.ptr = db;
  dr.offset_elems = 0;
  dout.ptr = dc;
  dout.offset_elems = 0;
  // Large row-major problems: cut the rows into chunks and overlap the upload of
  // chunk i+1, the GEMM of chunk i and the download of chunk i-1 (PCIe is full
  // duplex; a single stream would serialise the three).
  constexpr int kMaxChunks = 16;
  if (can_pipe) {
    st = ensure_pipe(h);
    if (st != KAPYB_OK) return st;
    const int M = lhs->size0;
    // 1024-row chunks (8192^3 bf16: 5.87 ms with 1024 rows, 6.05 with 512, 6.00 with
    // 2048: smaller chunks lose more in copy and event overhead than they save; the
    // upload alone takes 4.92 ms, and each direction runs about 20 % slower while
    // the other is busy).  What stays exposed at the end is the last chunk's GEMM
    // and download, so the LAST chunk's rows go as a half and two quarters.
    const int chunks = std::min(kMaxChunks - 2, std::max(2, M / 1024));
    const int rows_per = ((M + chunks - 1) / chunks + 255) / 256 * 256;
    int plan_rows[kMaxChunks + 2];
    int n_plan = 0;
    {
      int r0 = 0;
      while (M - r0 > rows_per + 255) {   // whole chunks while more than one is left
        plan_rows[n_plan++] = rows_per;
        r0 += rows_per;
      }
      int left = M - r0;                  // the last chunk: 256 .. rows_per + 255 rows
      for (int div = 2; div <= 4 && left >= 512; div += 2) {
        const int part = (left / 2 + 255) / 256 * 256;
        if (left - part < 256) break;
        plan_rows[n_plan++] = part;
        left -= part;
      }
      plan_rows[n_plan++] = left;         // never fewer than 256 rows (no decode-kernel chunk,
                                          // whose sums run in another order than the tiles')
    }
    cudaEvent_t ev_start = h->ev[2 * kMaxChunks], ev_done = h->ev[2 * kMaxChunks + 1];
    HostTrace trace(0);
    trace.mark("start", stream);
    // B and the bias are already on their way on `stream`; A goes up chunk by chunk
    CUDA_TRY(h, cudaEventRecord(ev_start, stream));
    trace.mark("rhs uploaded", stream);
    CUDA_TRY(h, cudaStreamWaitEvent(h->copy_in, ev_start, 0));
    CUDA_TRY(h, cudaStreamWaitEvent(h->copy_out, ev_start, 0));
    const size_t esz_a = dtype_size(lhs->dtype), esz_c = dtype_size(out->dtype);
    const char *ha = static_cast<const char *>(elem_ptr(lhs));
    char *hc = static_cast<char *>(const_cast<void *>(elem_ptr(out)));
    int n_chunks = 0;
    for (int r0 = 0, rows = 0; n_chunks < n_plan; r0 += rows, ++n_chunks) {
      rows = plan_rows[n_chunks];
      const size_t a_off = static_cast<size_t>(r0) * lhs->stride0 * esz_a;
      const size_t c_off = static_cast<size_t>(r0) * out->stride0 * esz_c;
      CUDA_TRY(h, cudaMemcpyAsync(da + a_off, ha + a_off,
                                  static_cast<size_t>(rows) * lhs->stride0 * esz_a,
                                  cudaMemcpyHostToDevice, h->copy_in));
      CUDA_TRY(h, cudaEventRecord(h->ev[2 * n_chunks], h->copy_in));
      trace.mark("chunk uploaded", h->copy_in, n_chunks);
      CUDA_TRY(h, cudaStreamWaitEvent(stream, h->ev[2 * n_chunks], 0));
      kapyb_tensor2d cl = dl, co = dout;
      cl.offset_elems = static_cast<int64_t>(r0) * lhs->stride0;
      cl.size0 = rows;
      co.offset_elems = static_cast<int64_t>(r0) * out->stride0;
      co.size0 = rows;
      kapyb_epilogue cep = ep;
      if (cep.bias && cep.bias_axis == 0)
        cep.bias = static_cast<const char *>(cep.bias) + static_cast<size_t>(r0) * dtype_size(cep.bias_dtype);
      st = run_matmul(h, make_problem(&cl, &dr, nullptr, &co, &cep), nullptr, 0, stream);
      if (st != KAPYB_OK) return st;
      CUDA_TRY(h, cudaEventRecord(h->ev[2 * n_chunks + 1], stream));
      trace.mark("chunk multiplied", stream, n_chunks);
      CUDA_TRY(h, cudaStreamWaitEvent(h->copy_out, h->ev[2 * n_chunks + 1], 0));
      CUDA_TRY(h, cudaMemcpyAsync(hc + c_off, dc + c_off,
                                  static_cast<size_t>(rows) * out->stride0 * esz_c,
                                  cudaMemcpyDeviceToHost, h->copy_out));
      trace.mark("chunk downloaded", h->copy_out, n_chunks);
    }
    CUDA_TRY(h, cudaEventRecord(ev_done, h->copy_out));
    CUDA_TRY(h, cudaStreamWaitEvent(stream, ev_done, 0));
    const kapyb_status done = kapyb_check(h, stream);
    if (trace.on) {
      cudaDeviceSynchronize();
      trace.report();
    }
    return done;
  }
  st = run_matmul(h, make_problem(&dl, &dr, nullptr, &dout, &ep), nullptr, 0, stream);
  if (st != KAPYB_OK) return st;
  // Only the elements the kernel wrote are defined; the caller's buffer keeps
  // its gaps when `out` is a strided view, so copy row by row in that case.
  const bool dense = (out->stride1 == 1 && out->stride0 == out->size1) ||
                     (out->stride0 == 1 && out->stride1 == out->size0);
  void *hc = const_cast<void *>(elem_ptr(out));
  if (dense) {
    CUDA_TRY(h, cudaMemcpyAsync(hc, dc, nc, cudaMemcpyDeviceToHost, stream));
  } else if (out->stride1 == 1) {
    const size_t esz = dtype_size(out->dtype);
    CUDA_TRY(h, cudaMemcpy2DAsync(hc, out->stride0 * esz, dc, out->stride0 * esz,
                                  out->size1 * esz, out->size0, cudaMemcpyDeviceToHost, stream));
  } else if (out->stride0 == 1) {
    const size_t esz = dtype_size(out->dtype);
    CUDA_TRY(h, cudaMemcpy2DAsync(hc, out->stride1 * esz, dc, out->stride1 * esz,
                                  out->size0 * esz, out->size1, cudaMemcpyDeviceToHost, stream));
  } else {
    return fail(h, KAPYB_UNSUPPORTED, "matmul_host: out needs one unit stride");
  }
  return kapyb_check(h, stream);
}

// ------------------------------------------------- cross-GPU completion flags

extern "C" KAPYB_API kapyb_status kapyb_gather_signal(kapyb_handle h, void *const *peer_flags,
                                                      int32_t n_ranks, int32_t my_rank,
                                                      uint32_t seq, void *stream) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_gather_signal: NULL handle");
  if (!peer_flags || n_ranks < 1 || n_ranks > kMaxGatherRanks || my_rank < 0 || my_rank >= n_ranks)
    return fail(h, KAPYB_INVALID_ARG, "gather_signal: need 1..%d ranks and a rank inside them",
                kMaxGatherRanks);
  GatherFlagPtrs fp;
  for (int r = 0; r < n_ranks; ++r) {
    if (!peer_flags[r] || (reinterpret_cast<uintptr_t>(peer_flags[r]) & 3u))
      return fail(h, KAPYB_INVALID_ARG, "gather_signal: peer_flags[%d] is NULL or misaligned", r);
    fp.p[r] = static_cast<uint32_t *>(peer_flags[r]);
  }
  for (int r = n_ranks; r < kMaxGatherRanks; ++r) fp.p[r] = nullptr;
  CUDA_TRY(h, cudaSetDevice(h->device));
  gather_signal_kernel<<<1, kMaxGatherRanks, 0, static_cast<cudaStream_t>(stream)>>>(fp, n_ranks,
                                                                                      my_rank, seq);
  CUDA_TRY(h, cudaGetLastError());
  h->launches++;
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_gather_wait(kapyb_handle h, const void *my_flags,
                                                    int32_t n_ranks, uint32_t seq,
                                                    uint32_t limit_ms, void *stream) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_gather_wait: NULL handle");
  if (!my_flags || (reinterpret_cast<uintptr_t>(my_flags) & 3u) || n_ranks < 1 ||
      n_ranks > kMaxGatherRanks)
    return fail(h, KAPYB_INVALID_ARG, "gather_wait: need an aligned flag array of 1..%d words",
                kMaxGatherRanks);
  CUDA_TRY(h, cudaSetDevice(h->device));
  const unsigned long long limit_ns = (limit_ms ? limit_ms : 2000u) * 1000000ull;
  gather_wait_kernel<<<1, kMaxGatherRanks, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t *>(my_flags), n_ranks, seq, limit_ns, h->status);
  CUDA_TRY(h, cudaGetLastError());
  h->launches++;
  return KAPYB_OK;
}

// ------------------------------------------- host buffers, rows of A sharded


extern "C" KAPYB_API kapyb_status kapyb_matmul_host_sharded(
    kapyb_handle h, const kapyb_tensor2d *lhs_rows, int32_t m_total, int32_t row_begin,
    const kapyb_tensor2d *rhs, const kapyb_tensor2d *out, const kapyb_epilogue *epilogue,
    const kapyb_shard_ctx *ctx, int32_t impl_way, void *stream_) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_matmul_host_sharded: NULL handle");
  if (!lhs_rows || !rhs || !out || !ctx)
    return fail(h, KAPYB_INVALID_ARG, "matmul_host_sharded: NULL argument");
  const int world = ctx->world, rank = ctx->rank;
  if (world < 1 || world > kMaxGatherRanks || rank < 0 || rank >= world || !ctx->peer_lhs ||
      !ctx->peer_flags)
    return fail(h, KAPYB_INVALID_ARG, "matmul_host_sharded: bad rank / world / peer tables");
  const int K = lhs_rows->size1, rows_mine = lhs_rows->size0;
  if (m_total < 0 || row_begin < 0 || rows_mine < 0 || row_begin + rows_mine > m_total)
    return fail(h, KAPYB_INVALID_ARG, "matmul_host_sharded: rows [%d, %d) outside [0, %d)",
                row_begin, row_begin + rows_mine, m_total);
  // the whole problem as the kernels will see it: lhs [m_total, K] in the staging buffer
  kapyb_tensor2d full = *lhs_rows;
  full.size0 = m_total;
  full.stride0 = K;
  full.stride1 = 1;
  kapyb_status st = verify_matmul(h, &full, rhs, nullptr, out, epilogue, impl_way);
  if (st != KAPYB_OK) return st;
  if ((rows_mine > 0 && (lhs_rows->stride1 != 1 || lhs_rows->stride0 != K)) ||
      out->stride1 != 1 || out->stride0 != out->size1)
    return fail(h, KAPYB_UNSUPPORTED,
                "matmul_host_sharded: this rank's rows of lhs and the output must be dense row-major");
  if (rhs->stride0 < 0 || rhs->stride1 < 0)
    return fail(h, KAPYB_UNSUPPORTED, "matmul_host_sharded: negative strides are not supported");
  const size_t esz_a = dtype_size(lhs_rows->dtype), esz_c = dtype_size(out->dtype);
  if ((static_cast<size_t>(K) * esz_a) % 16 != 0)
    return fail(h, KAPYB_UNSUPPORTED, "matmul_host_sharded: a row of lhs must be a multiple of 16 bytes");
  for (int r = 0; r < world; ++r)
    if (!ctx->peer_lhs[r] || !ctx->peer_flags[r] || !aligned16(ctx->peer_lhs[r]))
      return fail(h, KAPYB_INVALID_ARG, "matmul_host_sharded: peer table entry %d is NULL or misaligned", r);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  CUDA_TRY(h, cudaSetDevice(h->device));

  const size_t nb = span_bytes(rhs), nc = span_bytes(out);
  size_t nbias = 0;
  if (epilogue && epilogue->bias)
    nbias = static_cast<size_t>(epilogue->bias_axis == 1 ? rhs->size1 : m_total) *
            dtype_size(epilogue->bias_dtype);
  const size_t skinny_ws = skinny_workspace_bytes();
  st = kapyb_reserve_workspace(h, skinny_ws + round256(nb) + round256(nc) + round256(nbias));
  if (st != KAPYB_OK) return st;
  st = ensure_pipe(h);
  if (st != KAPYB_OK) return st;
  if (!h->push_ready) {
    CUDA_TRY(h, cudaStreamCreateWithFlags(&h->push, cudaStreamNonBlocking));
    for (cudaEvent_t &e : h->ev_push) CUDA_TRY(h, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    h->push_ready = true;
  }
  char *w = static_cast<char *>(h->workspace) + skinny_ws;
  char *db = w, *dc = db + round256(nb), *dbias = dc + round256(nc);
  // Two staging copies of lhs per rank, used in turn: a peer may still multiply
  // out of one while the next call's rows arrive in the other (calls are at most
  // one apart across ranks, because each waits for every peer's rows of ITS call).
  const size_t a_bytes = static_cast<size_t>(m_total) * K * esz_a;
  const size_t half = (ctx->seq & 1u) ? ((a_bytes + 255) & ~static_cast<size_t>(255)) : 0;
  char *da = static_cast<char *>(ctx->peer_lhs[rank]) + half;

  constexpr int kMaxChunks = 16;
  cudaEvent_t ev_start = h->ev[2 * kMaxChunks], ev_done = h->ev[2 * kMaxChunks + 1];
  CUDA_TRY(h, cudaEventRecord(ev_start, stream));
  CUDA_TRY(h, cudaStreamWaitEvent(h->copy_in, ev_start, 0));
  CUDA_TRY(h, cudaStreamWaitEvent(h->copy_out, ev_start, 0));
  CUDA_TRY(h, cudaStreamWaitEvent(h->push, ev_start, 0));

  HostTrace trace(rank);
  trace.mark("start", stream);
  // The rows of lhs travel in `pieces` pieces per rank, and the staging copy keeps
  // them PIECE-MAJOR: piece j of every rank side by side (staging row of rank r,
  // piece j, row i = (j * world + r) * P + i).  Every rank uploads its piece j at
  // about the same time, so piece j of the whole matrix is complete long before
  // piece j+1, and its product and download overlap the upload of the next piece
  // (PCIe is full duplex; the download is the longer leg when all GPUs of a box
  // transfer at once).  A per-row bias would have to be permuted the same way, and
  // ragged row blocks do not tile: both run as one piece (natural row order).
  const int R = world > 0 ? m_total / world : 0;
  const bool uniform = m_total % world == 0 && rows_mine == R && row_begin == rank * R;
  if (!uniform) {
    // every rank must own the same number of rows for the staging layout to tile
    return fail(h, KAPYB_UNSUPPORTED,
                "matmul_host_sharded: every rank must own m_total / world rows, rank r the r-th block");
  }
  int pieces = 1;
  const bool row_bias = epilogue && epilogue->bias && epilogue->bias_axis == 0;
  if (!row_bias)
    for (int p : {4, 2})
      if (R % p == 0 && (R / p) % 64 == 0 && static_cast<long long>(R / p) * world >= 1024) {
        pieces = p;
        break;
      }
  const int P = R / pieces;                      // rows per rank and piece
  const size_t row_bytes = static_cast<size_t>(K) * esz_a;
  const size_t piece_bytes = static_cast<size_t>(P) * row_bytes;
  const char *ha = static_cast<const char *>(elem_ptr(lhs_rows));
  // flag words carry (seq, piece): they only ever grow
  auto flag_value = [&](int j) { return (ctx->seq << 6) | static_cast<uint32_t>(j + 1); };

  // 1. the column shard of rhs and the bias go up first: every product needs them
  CUDA_TRY(h, cudaMemcpyAsync(db, elem_ptr(rhs), nb, cudaMemcpyHostToDevice, h->copy_in));
  kapyb_epilogue ep;
  if (epilogue)
    ep = *epilogue;
  else {
    ep.alpha = 1.0f;
    ep.bias = nullptr;
    ep.bias_dtype = KAPYB_F32;
    ep.bias_axis = 1;
    ep.activation = KAPYB_ACT_NONE;
    ep.rounding = KAPYB_RN;
  }
  if (nbias) {
    CUDA_TRY(h, cudaMemcpyAsync(dbias, ep.bias, nbias, cudaMemcpyHostToDevice, h->copy_in));
    ep.bias = dbias;
  }
  CUDA_TRY(h, cudaEventRecord(h->ev_push[16], h->copy_in));
  CUDA_TRY(h, cudaStreamWaitEvent(stream, h->ev_push[16], 0));
  trace.mark("rhs shard uploaded", h->copy_in);
  // 2. this rank's rows, piece by piece; each piece is forwarded to every peer's
  //    staging copy over NVLink (copy engines, stores only) as soon as it has
  //    landed, and announced
  for (int j = 0; j < pieces; ++j) {
    const size_t off = (static_cast<size_t>(j) * world + rank) * piece_bytes;
    CUDA_TRY(h, cudaMemcpyAsync(da + off, ha + static_cast<size_t>(j) * piece_bytes, piece_bytes,
                                cudaMemcpyHostToDevice, h->copy_in));
    CUDA_TRY(h, cudaEventRecord(h->ev_push[j], h->copy_in));
    trace.mark("own piece uploaded", h->copy_in, j);
    CUDA_TRY(h, cudaStreamWaitEvent(h->push, h->ev_push[j], 0));
    if (piece_bytes % 16 == 0 && world - 1 < kMaxGatherRanks) {
      ForwardPeers fw;
      fw.n = world - 1;
      for (int i = 1; i < world; ++i) {
        const int peer = (rank + i) % world;  // ranks start with different peers
        fw.dst[i - 1] = reinterpret_cast<uint4 *>(static_cast<char *>(ctx->peer_lhs[peer]) + half + off);
      }
      // a quarter of the SMs: NVLink, not the SMs, bounds it, and the products of the
      // pieces before run beside it
      const int grid = std::max(8, h->sm_count / 4);
      forward_to_peers_kernel<<<grid, 256, 0, h->push>>>(reinterpret_cast<const uint4 *>(da + off),
                                                         piece_bytes / 16, fw);
      CUDA_TRY(h, cudaGetLastError());
      h->launches++;
    } else {
      for (int i = 1; i < world; ++i) {
        const int peer = (rank + i) % world;
        CUDA_TRY(h, cudaMemcpyAsync(static_cast<char *>(ctx->peer_lhs[peer]) + half + off, da + off,
                                    piece_bytes, cudaMemcpyDeviceToDevice, h->push));
      }
    }
    st = kapyb_gather_signal(h, ctx->peer_flags, world, rank, flag_value(j), h->push);
    if (st != KAPYB_OK) return st;
    // (this rank's own word is set by that kernel: the compute stream is ordered
    // after it by an event, never by polling for a kernel of the same GPU)
    CUDA_TRY(h, cudaEventRecord(h->ev_push[8 + j], h->push));
    trace.mark("own piece forwarded", h->push, j);
  }
  // 3. per piece: wait (bounded) until every rank's rows of the piece have landed
  //    here, multiply, and send the piece's rows of the output home
  kapyb_tensor2d dl = full, dr = *rhs, dout = *out;
  dl.ptr = da;
  dl.offset_elems = 0;
  dr.ptr = db;
  dr.offset_elems = 0;
  dout.ptr = dc;
  dout.offset_elems = 0;
  char *hc = static_cast<char *>(const_cast<void *>(elem_ptr(out)));
  const size_t out_row_bytes = static_cast<size_t>(out->stride0) * esz_c;
  for (int j = 0; j < pieces; ++j) {
    CUDA_TRY(h, cudaStreamWaitEvent(stream, h->ev_push[8 + j], 0));
    st = kapyb_gather_wait(h, ctx->peer_flags[rank], world, flag_value(j), ctx->wait_limit_ms, stream);
    if (st != KAPYB_OK) return st;
    trace.mark("piece complete here", stream, j);
    const int rows = P * world;                  // piece j of every rank, adjacent in staging
    const int64_t first = static_cast<int64_t>(j) * rows;
    kapyb_tensor2d cl = dl, co = dout;
    cl.offset_elems = first * K;
    cl.size0 = rows;
    co.offset_elems = first * out->stride0;
    co.size0 = rows;
    st = run_matmul(h, make_problem(&cl, &dr, nullptr, &co, &ep), nullptr, 0, stream);
    if (st != KAPYB_OK) return st;
    CUDA_TRY(h, cudaEventRecord(h->ev[2 * j + 1], stream));
    trace.mark("piece multiplied", stream, j);
    CUDA_TRY(h, cudaStreamWaitEvent(h->copy_out, h->ev[2 * j + 1], 0));
    // staging rows of (rank r, piece j) -> rows r * R + j * P of the caller's output
    if (out->stride0 == out->size1) {
      // the P rows of a rank are one contiguous block on both sides: all ranks'
      // blocks of the piece go home as one pitched copy (one block per "row")
      // instead of `world` small ones
      const size_t block = static_cast<size_t>(P) * out_row_bytes;
      CUDA_TRY(h, cudaMemcpy2DAsync(hc + static_cast<size_t>(j) * block, static_cast<size_t>(R) * out_row_bytes,
                                    dc + static_cast<size_t>(first) * out_row_bytes, block, block,
                                    static_cast<size_t>(world), cudaMemcpyDeviceToHost, h->copy_out));
    } else {
      for (int r = 0; r < world; ++r) {
        const size_t src = (static_cast<size_t>(first) + static_cast<size_t>(r) * P) * out_row_bytes;
        const size_t dst = (static_cast<size_t>(r) * R + static_cast<size_t>(j) * P) * out_row_bytes;
        CUDA_TRY(h, cudaMemcpyAsync(hc + dst, dc + src, static_cast<size_t>(P) * out_row_bytes,
                                    cudaMemcpyDeviceToHost, h->copy_out));
      }
    }
    trace.mark("piece downloaded", h->copy_out, j);
  }
  CUDA_TRY(h, cudaEventRecord(ev_done, h->copy_out));
  CUDA_TRY(h, cudaStreamWaitEvent(stream, ev_done, 0));
  const kapyb_status done = kapyb_check(h, stream);
  if (trace.on) {
    cudaDeviceSynchronize();
    trace.report();
  }
  return done;
}

// ------------------------------------------------------------- elementwise

static kapyb_status verify_program(kapyb_handle h, const kapyb_inst *prog, int n_inst,
                                   const kapyb_tensor2d *inputs, int n_inputs,
                                   const kapyb_tensor2d *out) {
  if (!prog || n_inst <= 0 || n_inst > KAPYB_MAX_INSTS)
    return fail(h, KAPYB_INVALID_ARG, "elementwise: program must have 1..%d ops", KAPYB_MAX_INSTS);
  if (n_inputs < 0 || n_inputs > KAPYB_MAX_INPUTS || (n_inputs > 0 && !inputs))
    return fail(h, KAPYB_INVALID_ARG, "elementwise: at most %d inputs", KAPYB_MAX_INPUTS);
  if (!out || !valid_operand_dtype(out->dtype) || out->size0 < 0 || out->size1 < 0 ||
      (!out->ptr && out->size0 != 0 && out->size1 != 0))
    return fail(h, KAPYB_INVALID_ARG, "elementwise: bad output descriptor");
  if (!valid_cache(out->cache))
    return fail(h, KAPYB_INVALID_ARG, "elementwise: unknown cache operator or eviction priority on the output");
  for (int k = 0; k < n_inputs; ++k) {
    const kapyb_tensor2d &t = inputs[k];
    if (!valid_operand_dtype(t.dtype) || t.size0 < 0 || t.size1 < 0 ||
        (!t.ptr && t.size0 != 0 && t.size1 != 0))
      return fail(h, KAPYB_INVALID_ARG, "elementwise: bad input descriptor %d", k);
    if (t.padding < KAPYB_PAD_ZERO || t.padding > KAPYB_PAD_NINF)
      return fail(h, KAPYB_INVALID_ARG, "elementwise: bad padding option on input %d", k);
    if (!valid_cache(t.cache))
      return fail(h, KAPYB_INVALID_ARG, "elementwise: unknown cache operator or eviction priority on input %d", k);
    if (t.dtype == KAPYB_F8E4M3 && (t.padding == KAPYB_PAD_PINF || t.padding == KAPYB_PAD_NINF))
      return fail(h, KAPYB_INVALID_ARG, "elementwise: f8E4M3 has no infinity to pad input %d with", k);
  }
  int reg_dtype[KAPYB_MAX_REGS];
  for (int r = 0; r < KAPYB_MAX_REGS; ++r) reg_dtype[r] = -1;
  int stores = 0;
  for (int pc = 0; pc < n_inst; ++pc) {
    const kapyb_inst &in = prog[pc];
    if (in.op < 0 || in.op >= KAPYB_OP_COUNT_)
      return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d at %d is unknown", in.op, pc);
    int nsrc = 0;
    switch (in.op) {
    case KAPYB_OP_LOAD:
    case KAPYB_OP_CONST: nsrc = 0; break;
    case KAPYB_OP_FMA:
    case KAPYB_OP_SELECT:
    case KAPYB_OP_CLAMP: nsrc = 3; break;
    case KAPYB_OP_CMP:
    case KAPYB_OP_AND:
    case KAPYB_OP_OR:
    case KAPYB_OP_XOR:
    case KAPYB_OP_ADD:
    case KAPYB_OP_SUB:
    case KAPYB_OP_MUL:
    case KAPYB_OP_DIV:
    case KAPYB_OP_MAXIMUM:
    case KAPYB_OP_MINIMUM:
    case KAPYB_OP_MAXNUM:
    case KAPYB_OP_MINNUM: nsrc = 2; break;
    default: nsrc = 1; break;
    }
    const int srcs[3] = {in.a, in.b, in.c};
    for (int s = 0; s < nsrc; ++s) {
      if (srcs[s] < 0 || srcs[s] >= KAPYB_MAX_REGS || reg_dtype[srcs[s]] < 0)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d reads an undefined value", pc);
    }
    if (in.op == KAPYB_OP_STORE) {
      if (reg_dtype[in.a] != out->dtype)
        return fail(h, KAPYB_INVALID_ARG,
                    "elementwise: st_global source is %s but the target tensor is %s",
                    dtype_name(reg_dtype[in.a]), dtype_name(out->dtype));
      ++stores;
      continue;
    }
    if (in.dst < 0 || in.dst >= KAPYB_MAX_REGS)
      return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d writes register %d", pc, in.dst);
    // Conditions: arith.cmpf yields i1 from two operands of one float type;
    // and/or/xor combine conditions; arith.select picks between two values of
    // the result type.
    if (in.op == KAPYB_OP_CMP) {
      const int ot = reg_dtype[in.a];
      if (in.dtype != KAPYB_I1 || !valid_dtype(ot) || reg_dtype[in.b] != ot)
        return fail(h, KAPYB_INVALID_ARG,
                    "elementwise: op %d (cmpf) needs two operands of one f16/bf16/f32 type and an i1 result", pc);
      if (in.flags < KAPYB_CMP_OLT || in.flags > KAPYB_CMP_UNE)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d has an unknown cmpf predicate %d", pc, in.flags);
      reg_dtype[in.dst] = KAPYB_I1;
      continue;
    }
    if (in.op == KAPYB_OP_AND || in.op == KAPYB_OP_OR || in.op == KAPYB_OP_XOR) {
      if (in.dtype != KAPYB_I1 || reg_dtype[in.a] != KAPYB_I1 || reg_dtype[in.b] != KAPYB_I1)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d combines i1 conditions only", pc);
      reg_dtype[in.dst] = KAPYB_I1;
      continue;
    }
    if (in.op == KAPYB_OP_SELECT) {
      if (reg_dtype[in.a] != KAPYB_I1)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d (select) needs an i1 condition", pc);
      if (!valid_dtype(in.dtype) || reg_dtype[in.b] != in.dtype || reg_dtype[in.c] != in.dtype)
        return fail(h, KAPYB_INVALID_ARG,
                    "elementwise: op %d (select) requires the same element type for both values and the result", pc);
      reg_dtype[in.dst] = in.dtype;
      continue;
    }
    if (!valid_operand_dtype(in.dtype))
      return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d has a bad element type", pc);
    // the 8-bit types exist in memory and across casts only
    if (is_fp8(in.dtype) && in.op != KAPYB_OP_LOAD && in.op != KAPYB_OP_CVT)
      return fail(h, KAPYB_INVALID_ARG, "elementwise: op %d cannot compute in an f8 element type", pc);
    if (in.op == KAPYB_OP_LOAD) {
      if (in.flags < 0 || in.flags >= n_inputs)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: ld_global of input %d, but %d given", in.flags, n_inputs);
      if (inputs[in.flags].dtype != in.dtype)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: ld_global result type differs from its source");
    } else if (in.op == KAPYB_OP_CVT) {
      // FPToFPOp::verify (Kapy.cpp:272-287): a downcast must name a rounding mode.
      if (dtype_size(in.dtype) < dtype_size(reg_dtype[in.a]) && in.flags != KAPYB_RZ && in.flags != KAPYB_RN)
        return fail(h, KAPYB_INVALID_ARG, "elementwise: rounding mode must be set for down cast");
      const int from = reg_dtype[in.a];
      if (is_fp8(from) && is_fp8(in.dtype))
        return fail(h, KAPYB_INVALID_ARG, "elementwise: convert f8 to f8 is not supported");
      if (is_fp8(in.dtype) && in.flags == KAPYB_RZ) {
        if (from == KAPYB_BF16)
          return fail(h, KAPYB_INVALID_ARG,
                      "elementwise: unsupported rounding mode when convert bf16 to f8");
        // no rz entry for f8E4M3 in the reference's conversion table
        // (ElementwiseOpToLLVM.cpp:628-650)
        if (in.dtype == KAPYB_F8E4M3)
          return fail(h, KAPYB_UNSUPPORTED, "elementwise: no toward-zero conversion to f8E4M3");
      }
    } else {
      for (int s = 0; s < nsrc; ++s)
        if (reg_dtype[srcs[s]] != in.dtype)
          return fail(h, KAPYB_INVALID_ARG,
                      "elementwise: op %d requires the same element type for all operands and results", pc);
    }
    reg_dtype[in.dst] = in.dtype;
  }
  if (stores != 1) return fail(h, KAPYB_INVALID_ARG, "elementwise: a program stores exactly once (%d found)", stores);
  return KAPYB_OK;
}

// Expression-tree view of a program, used to recognise the canonical graphs.
struct ExprNode {
  int op, dtype, a, b, c, flags;
  float imm;
};

static int build_nodes(const kapyb_inst *prog, int n, ExprNode *nodes, int *store_src) {
  int reg_node[KAPYB_MAX_REGS];
  for (int r = 0; r < KAPYB_MAX_REGS; ++r) reg_node[r] = -1;
  int cnt = 0;
  *store_src = -1;
  for (int pc = 0; pc < n; ++pc) {
    const kapyb_inst &in = prog[pc];
    if (in.op == KAPYB_OP_STORE) {
      *store_src = reg_node[in.a];
      continue;
    }
    ExprNode nd;
    nd.op = in.op;
    nd.dtype = in.dtype;
    nd.a = in.a >= 0 ? reg_node[in.a] : -1;
    nd.b = in.b >= 0 ? reg_node[in.b] : -1;
    nd.c = in.c >= 0 ? reg_node[in.c] : -1;
    nd.flags = in.flags;
    nd.imm = in.imm;
    nodes[cnt] = nd;
    reg_node[in.dst] = cnt++;
  }
  return cnt;
}

struct Matcher {
  const ExprNode *n;
  bool is(int i, int op, int dt) const { return i >= 0 && n[i].op == op && n[i].dtype == dt; }
  bool cst(int i, float *v) const {
    if (!is(i, KAPYB_OP_CONST, KAPYB_F32)) return false;
    *v = n[i].imm;
    return true;
  }
  // mul(f32) with one constant operand; returns the other operand
  bool mul_const(int i, float *cv, int *other) const {
    if (!is(i, KAPYB_OP_MUL, KAPYB_F32)) return false;
    if (cst(n[i].a, cv)) {
      *other = n[i].b;
      return true;
    }
    if (cst(n[i].b, cv)) {
      *other = n[i].a;
      return true;
    }
    return false;
  }
  // u = fma(ext(load), s, b)
  bool affine(int i, float *s, float *b, int *load) const {
    if (!is(i, KAPYB_OP_FMA, KAPYB_F32)) return false;
    const int x = n[i].a;
    if (!is(x, KAPYB_OP_CVT, KAPYB_F32)) return false;
    const int ld = n[x].a;
    if (ld < 0 || n[ld].op != KAPYB_OP_LOAD || n[ld].dtype == KAPYB_F32) return false;
    if (!cst(n[i].b, s) || !cst(n[i].c, b)) return false;
    *load = ld;
    return true;
  }
};

// Recognises  cvt16( fma(ext(x), s, b) )  and the gelu_tanh graph around it.
static bool match_affine_gelu(const ExprNode *nodes, int root, AffineGelu *f, int *load_input,
                              int *in_dtype, int *rounding) {
  Matcher m{nodes};
  if (root < 0 || nodes[root].op != KAPYB_OP_CVT || nodes[root].dtype == KAPYB_F32) return false;
  *rounding = nodes[root].flags;
  const int y = nodes[root].a;
  int ld = -1;
  if (m.affine(y, &f->s, &f->b, &ld)) {
    f->gelu = 0;
    f->c0 = f->c1 = f->m2 = f->one = 0.0f;
  } else {
    // y = u / (one + exp(m2 * k)), k = c0 * fma((c1*u)*u, u, u)
    if (!m.is(y, KAPYB_OP_DIV, KAPYB_F32)) return false;
    const int u = nodes[y].a, den = nodes[y].b;
    if (!m.affine(u, &f->s, &f->b, &ld)) return false;
    if (!m.is(den, KAPYB_OP_ADD, KAPYB_F32)) return false;
    int e = -1;
    if (m.cst(nodes[den].a, &f->one))
      e = nodes[den].b;
    else if (m.cst(nodes[den].b, &f->one))
      e = nodes[den].a;
    else
      return false;
    if (!m.is(e, KAPYB_OP_EXP, KAPYB_F32)) return false;
    int k = -1;
    if (!m.mul_const(nodes[e].a, &f->m2, &k)) return false;
    int inner = -1;
    if (!m.mul_const(k, &f->c0, &inner)) return false;
    if (!m.is(inner, KAPYB_OP_FMA, KAPYB_F32)) return false;
    if (nodes[inner].b != u || nodes[inner].c != u) return false;
    const int t2 = nodes[inner].a;  // (c1*u)*u
    if (!m.is(t2, KAPYB_OP_MUL, KAPYB_F32)) return false;
    int t1 = -1;
    if (nodes[t2].b == u)
      t1 = nodes[t2].a;
    else if (nodes[t2].a == u)
      t1 = nodes[t2].b;
    else
      return false;
    int uu = -1;
    if (!m.mul_const(t1, &f->c1, &uu) || uu != u) return false;
    f->gelu = 1;
  }
  *load_input = nodes[ld].flags;
  *in_dtype = nodes[ld].dtype;
  return true;
}

static bool contiguous_same(const kapyb_tensor2d &t, const kapyb_tensor2d &out) {
  if (t.size0 != out.size0 || t.size1 != out.size1) return false;
  const bool rm = (t.stride1 == 1 || t.size1 == 1) && (t.stride0 == t.size1 || t.size0 == 1);
  const bool orm = (out.stride1 == 1 || out.size1 == 1) && (out.stride0 == out.size1 || out.size0 == 1);
  return rm && orm;
}

// Grid of a streaming kernel whose blocks each take one contiguous chunk of
// `per_thread` x 256 vectors (at least one block: the last one owns the scalar tail).
static kapyb_status chunk_grid(kapyb_handle h, long long n_vec, int per_thread, int *grid) {
  const long long blocks = std::max(1ll, (n_vec + 256ll * per_thread - 1) / (256ll * per_thread));
  if (blocks > 0x7fffffffll) return fail(h, KAPYB_UNSUPPORTED, "elementwise: tensor too large");
  *grid = static_cast<int>(blocks);
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_elementwise(kapyb_handle h, const kapyb_inst *prog,
                                                    int32_t n_inst, const kapyb_tensor2d *inputs,
                                                    int32_t n_inputs, const kapyb_tensor2d *out,
                                                    void *stream_) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_elementwise: NULL handle");
  kapyb_status st = verify_program(h, prog, n_inst, inputs, n_inputs, out);
  if (st != KAPYB_OK) return st;
  const long long total = static_cast<long long>(out->size0) * out->size1;
  if (total == 0) return KAPYB_OK;
  CUDA_TRY(h, cudaSetDevice(h->device));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  // Output against inputs.  The streaming kernels read through the read-only
  // data path (ld.global.nc, __restrict__), which must not see memory the same
  // kernel writes.  An input that IS the output (same address, shape, strides
  // and element type: an in-place update, each element read before it is
  // written by the same thread) runs on the interpreter kernel, which uses plain
  // loads; any other overlap would make the result depend on thread timing and
  // is refused.
  bool in_place = false;
  {
    auto byte_range = [](const kapyb_tensor2d &t, uintptr_t *lo, uintptr_t *hi) {
      const int64_t e0 = static_cast<int64_t>(t.size0 - 1) * t.stride0;
      const int64_t e1 = static_cast<int64_t>(t.size1 - 1) * t.stride1;
      const int64_t mn = std::min<int64_t>(0, e0) + std::min<int64_t>(0, e1);
      const int64_t mx = std::max<int64_t>(0, e0) + std::max<int64_t>(0, e1);
      const int64_t esz = dtype_size(t.dtype);
      const uintptr_t base = reinterpret_cast<uintptr_t>(elem_ptr(&t));
      *lo = base + mn * esz;
      *hi = base + (mx + 1) * esz;
    };
    uintptr_t olo, ohi;
    byte_range(*out, &olo, &ohi);
    for (int k = 0; k < n_inputs; ++k) {
      const kapyb_tensor2d &t = inputs[k];
      if (t.size0 == 0 || t.size1 == 0) continue;
      uintptr_t ilo, ihi;
      byte_range(t, &ilo, &ihi);
      if (ihi <= olo || ohi <= ilo) continue;
      const bool same = elem_ptr(&t) == elem_ptr(out) && t.size0 == out->size0 &&
                        t.size1 == out->size1 && t.stride0 == out->stride0 &&
                        t.stride1 == out->stride1 && t.dtype == out->dtype;
      if (!same)
        return fail(h, KAPYB_INVALID_ARG,
                    "elementwise: the output overlaps input %d without being the same tensor "
                    "(only an exact in-place update is defined)", k);
      in_place = true;
    }
  }

  ExprNode nodes[KAPYB_MAX_INSTS];
  int root = -1;
  build_nodes(prog, n_inst, nodes, &root);

  // Fused path 0: a bare cast to or from an 8-bit float type, contiguous.
  if (!in_place && n_inst == 3 && prog[0].op == KAPYB_OP_LOAD && prog[1].op == KAPYB_OP_CVT &&
      prog[2].op == KAPYB_OP_STORE && prog[1].a == prog[0].dst && prog[2].a == prog[1].dst &&
      (is_fp8(prog[0].dtype) != is_fp8(prog[1].dtype))) {
    const kapyb_tensor2d &tin = inputs[prog[0].flags];
    if (contiguous_same(tin, *out) && aligned16(elem_ptr(&tin)) && aligned16(elem_ptr(out))) {
      const uint8_t *px = static_cast<const uint8_t *>(elem_ptr(&tin));
      uint8_t *py = static_cast<uint8_t *>(const_cast<void *>(elem_ptr(out)));
      const long long n_groups = total / 16;
      int grid = 1;
      st = chunk_grid(h, n_groups, kCastUnroll, &grid);
      if (st != KAPYB_OK) return st;
      const int sd = prog[0].dtype, dd = prog[1].dtype;
      const int rn = is_fp8(dd) ? (prog[1].flags == KAPYB_RN ? 1 : 0) : 1;
#define KAPYB_CAST(S, D, R)                                                                   \
  if (sd == S && dd == D && rn == R) {                                                        \
    elt_cast_kernel<S, D, R><<<grid, 256, 0, stream>>>(px, py, n_groups, total);              \
    launched = true;                                                                          \
  }
      bool launched = false;
      KAPYB_CAST(KAPYB_F8E4M3, KAPYB_F16, 1)
      KAPYB_CAST(KAPYB_F8E4M3, KAPYB_BF16, 1)
      KAPYB_CAST(KAPYB_F8E4M3, KAPYB_F32, 1)
      KAPYB_CAST(KAPYB_F8E5M2, KAPYB_F16, 1)
      KAPYB_CAST(KAPYB_F8E5M2, KAPYB_BF16, 1)
      KAPYB_CAST(KAPYB_F8E5M2, KAPYB_F32, 1)
      KAPYB_CAST(KAPYB_F16, KAPYB_F8E4M3, 1)
      KAPYB_CAST(KAPYB_BF16, KAPYB_F8E4M3, 1)
      KAPYB_CAST(KAPYB_F32, KAPYB_F8E4M3, 1)
      KAPYB_CAST(KAPYB_F16, KAPYB_F8E5M2, 1)
      KAPYB_CAST(KAPYB_BF16, KAPYB_F8E5M2, 1)
      KAPYB_CAST(KAPYB_F32, KAPYB_F8E5M2, 1)
      KAPYB_CAST(KAPYB_F16, KAPYB_F8E5M2, 0)
      KAPYB_CAST(KAPYB_F32, KAPYB_F8E5M2, 0)
#undef KAPYB_CAST
      if (launched) {
        CUDA_TRY(h, cudaGetLastError());
        h->launches++;
        h->last_kernel = "elt_cast_f8";
        return KAPYB_OK;
      }
    }
  }

  // Fused path 1: 16-bit -> 16-bit affine (+ gelu_tanh), contiguous.
  {
    AffineGelu f;
    int li = -1, din = 0, rn = 1;
    if (!in_place && match_affine_gelu(nodes, root, &f, &li, &din, &rn) &&
        (din == KAPYB_F16 || din == KAPYB_BF16) &&
        nodes[root].dtype == out->dtype && din == out->dtype && (rn == 0 || rn == 1) &&
        contiguous_same(inputs[li], *out) &&
        aligned16(elem_ptr(&inputs[li])) && aligned16(elem_ptr(out))) {
      const uint4 *px = static_cast<const uint4 *>(elem_ptr(&inputs[li]));
      uint4 *py = static_cast<uint4 *>(const_cast<void *>(elem_ptr(out)));
      const bool wide = ((reinterpret_cast<uintptr_t>(px) | reinterpret_cast<uintptr_t>(py)) & 31u) == 0;
      f.ftz_ok = (f.one >= 1e-30f || f.one <= -1e-30f) ? 1 : 0;
      const long long n_acc = total / (wide ? 16 : 8);
      int grid = 1;
      st = chunk_grid(h, n_acc, kEltUnroll, &grid);
      if (st != KAPYB_OK) return st;
#define KAPYB_LAUNCH_UNARY(W, DT, RN) \
  elt_unary16_kernel<AffineGelu, W, DT, RN><<<grid, 256, 0, stream>>>(px, py, n_acc, total, f)
      if (din == KAPYB_BF16) {
        if (wide) { if (rn) KAPYB_LAUNCH_UNARY(2, KAPYB_BF16, 1); else KAPYB_LAUNCH_UNARY(2, KAPYB_BF16, 0); }
        else      { if (rn) KAPYB_LAUNCH_UNARY(1, KAPYB_BF16, 1); else KAPYB_LAUNCH_UNARY(1, KAPYB_BF16, 0); }
      } else {
        if (wide) { if (rn) KAPYB_LAUNCH_UNARY(2, KAPYB_F16, 1); else KAPYB_LAUNCH_UNARY(2, KAPYB_F16, 0); }
        else      { if (rn) KAPYB_LAUNCH_UNARY(1, KAPYB_F16, 1); else KAPYB_LAUNCH_UNARY(1, KAPYB_F16, 0); }
      }
#undef KAPYB_LAUNCH_UNARY
      CUDA_TRY(h, cudaGetLastError());
      h->launches++;
      h->last_kernel = f.gelu ? "elt_affine_gelu" : "elt_affine";
      return KAPYB_OK;
    }
  }
  // Fused path 2: z = a (add|sub|mul|div|maximum|minimum|maxnum|minnum) b, one element type, contiguous.
  if (!in_place && root >= 0 && n_inputs >= 2) {
    const ExprNode &r = nodes[root];
    if ((r.op == KAPYB_OP_ADD || r.op == KAPYB_OP_SUB || r.op == KAPYB_OP_MUL ||
         r.op == KAPYB_OP_DIV || r.op == KAPYB_OP_MAXIMUM || r.op == KAPYB_OP_MINIMUM ||
         r.op == KAPYB_OP_MAXNUM || r.op == KAPYB_OP_MINNUM) && r.a >= 0 &&
        r.b >= 0 && nodes[r.a].op == KAPYB_OP_LOAD && nodes[r.b].op == KAPYB_OP_LOAD &&
        r.dtype == out->dtype) {
      const kapyb_tensor2d &ta = inputs[nodes[r.a].flags], &tb = inputs[nodes[r.b].flags];
      if (ta.dtype == r.dtype && tb.dtype == r.dtype && contiguous_same(ta, *out) &&
          contiguous_same(tb, *out) && aligned16(elem_ptr(&ta)) && aligned16(elem_ptr(&tb)) &&
          aligned16(elem_ptr(out))) {
        const int per = r.dtype == KAPYB_F32 ? 4 : 8;
        const long long n_vec = total / per;
        int grid = 1;
        st = chunk_grid(h, n_vec, kBinUnroll, &grid);
        if (st != KAPYB_OK) return st;
        const uint4 *pa = static_cast<const uint4 *>(elem_ptr(&ta));
        const uint4 *pb = static_cast<const uint4 *>(elem_ptr(&tb));
        uint4 *pz = static_cast<uint4 *>(const_cast<void *>(elem_ptr(out)));
        switch (r.op) {
#define KAPYB_BIN(OP) \
  case OP: elt_binary_kernel<OP><<<grid, 256, 0, stream>>>(pa, pb, pz, n_vec, total, r.dtype); break;
          KAPYB_BIN(KAPYB_OP_ADD) KAPYB_BIN(KAPYB_OP_SUB) KAPYB_BIN(KAPYB_OP_DIV)
          KAPYB_BIN(KAPYB_OP_MAXIMUM) KAPYB_BIN(KAPYB_OP_MINIMUM) KAPYB_BIN(KAPYB_OP_MAXNUM)
          KAPYB_BIN(KAPYB_OP_MINNUM)
#undef KAPYB_BIN
        default: elt_binary_kernel<KAPYB_OP_MUL><<<grid, 256, 0, stream>>>(pa, pb, pz, n_vec, total, r.dtype); break;
        }
        CUDA_TRY(h, cudaGetLastError());
        h->launches++;
        h->last_kernel = "elt_binary";
        return KAPYB_OK;
      }
    }
  }
  // Generic interpreter.
  EltProgram P;
  memset(&P, 0, sizeof(P));
  memcpy(P.inst, prog, sizeof(kapyb_inst) * n_inst);
  P.n_inst = n_inst;
  P.n_in = n_inputs;
  for (int k = 0; k < n_inputs; ++k) {
    P.in[k].ptr = elem_ptr(&inputs[k]);
    P.in[k].s0 = inputs[k].stride0;
    P.in[k].s1 = inputs[k].stride1;
    P.in[k].size0 = inputs[k].size0;
    P.in[k].size1 = inputs[k].size1;
    P.in[k].dtype = inputs[k].dtype;
    P.in[k].padding = inputs[k].padding;
    P.in[k].cache = inputs[k].cache;
  }
  P.out.ptr = elem_ptr(out);
  P.out.s0 = out->stride0;
  P.out.s1 = out->stride1;
  P.out.size0 = out->size0;
  P.out.size1 = out->size1;
  P.out.dtype = out->dtype;
  P.out.padding = 0;
  P.out.cache = out->cache;
  const int grid = static_cast<int>(std::max(1ll, std::min((total + 255) / 256,
                                                            static_cast<long long>(h->sm_count) * 32)));
  elt_interp_kernel<<<grid, 256, 0, stream>>>(P);
  CUDA_TRY(h, cudaGetLastError());
  h->launches++;
  h->last_kernel = "elt_interp";
  return KAPYB_OK;
}

// ------------------------------------------------------------------ reduce

template <int COMB, int DT>
static void launch_reduce_rows(const ReduceParams &p, bool vec, bool narrow, int grid,
                               cudaStream_t stream) {
  if constexpr (DT != KAPYB_F32) {
    if (narrow) {
      if (vec)
        reduce_rows_kernel<COMB, true, DT, true><<<grid, 256, 0, stream>>>(p);
      else
        reduce_rows_kernel<COMB, false, DT, true><<<grid, 256, 0, stream>>>(p);
      return;
    }
  }
  if (vec)
    reduce_rows_kernel<COMB, true, DT><<<grid, 256, 0, stream>>>(p);
  else
    reduce_rows_kernel<COMB, false, DT><<<grid, 256, 0, stream>>>(p);
}

template <int COMB>
static void launch_reduce(const ReduceParams &p, bool unit_inner, bool vec, int sm_count,
                          cudaStream_t stream) {
  // The lambda runs at the destination's element type: a 16-bit destination
  // (necessarily the source's type) means a rounding to that type per step.
  const bool narrow = p.dst_dtype != KAPYB_F32;
  if (unit_inner) {
    // One row per warp, as many blocks as that takes (capped far above a resident
    // wave): the block scheduler then walks the SMs through neighbouring rows,
    // which streams faster from HBM than a resident grid striding over the rows.
    const long long blocks = (static_cast<long long>(p.rows) + 7) / 8;
    const int grid = static_cast<int>(std::max(1ll, std::min(blocks, 1ll << 22)));
    (void)sm_count;
    if (p.src_dtype == KAPYB_F32)
      launch_reduce_rows<COMB, KAPYB_F32>(p, vec, false, grid, stream);
    else if (p.src_dtype == KAPYB_BF16)
      launch_reduce_rows<COMB, KAPYB_BF16>(p, vec, narrow, grid, stream);
    else
      launch_reduce_rows<COMB, KAPYB_F16>(p, vec, narrow, grid, stream);
  } else {
    const long long blocks = (static_cast<long long>(p.rows) + 31) / 32;
    const int grid = static_cast<int>(std::max(1ll, std::min(blocks, static_cast<long long>(sm_count) * 8)));
    if (narrow && p.dst_dtype == KAPYB_BF16)
      reduce_cols_kernel<COMB, KAPYB_BF16><<<grid, 256, 0, stream>>>(p);
    else if (narrow)
      reduce_cols_kernel<COMB, KAPYB_F16><<<grid, 256, 0, stream>>>(p);
    else
      reduce_cols_kernel<COMB><<<grid, 256, 0, stream>>>(p);
  }
}

extern "C" KAPYB_API kapyb_status kapyb_reduce(kapyb_handle h, const kapyb_tensor2d *src,
                                               const kapyb_tensor2d *dst, int32_t axis,
                                               int32_t combiner, void *stream_) {
  if (!h) return fail(h, KAPYB_INVALID_ARG, "kapyb_reduce: NULL handle");
  if (!src || !dst) return fail(h, KAPYB_INVALID_ARG, "reduce: NULL tensor");
  if ((!src->ptr && src->size0 != 0 && src->size1 != 0) || (!dst->ptr && dst->size0 != 0 && dst->size1 != 0))
    return fail(h, KAPYB_INVALID_ARG, "reduce: NULL data pointer");
  if (!valid_dtype(src->dtype) || !valid_dtype(dst->dtype)) return fail(h, KAPYB_INVALID_ARG, "reduce: unknown element type");
  if (axis != 0 && axis != 1) return fail(h, KAPYB_INVALID_ARG, "reduce: axis must be 0 or 1");
  if (combiner < KAPYB_RED_ADD || combiner > KAPYB_RED_MIN) return fail(h, KAPYB_INVALID_ARG, "reduce: unknown combiner %d", combiner);
  if (dst->dtype != KAPYB_F32 && dst->dtype != src->dtype)
    return fail(h, KAPYB_INVALID_ARG, "reduce: result element type must be f32 or the source's");
  // ReduceOp::inferReturnTypes (Kapy.cpp:613-626): the reduced axis becomes 1.
  const int want0 = axis == 0 ? 1 : src->size0, want1 = axis == 1 ? 1 : src->size1;
  if (dst->size0 != want0 || dst->size1 != want1)
    return fail(h, KAPYB_INVALID_ARG, "reduce: result shape must be [%d, %d]", want0, want1);
  if (src->size0 < 0 || src->size1 < 0) return fail(h, KAPYB_INVALID_ARG, "reduce: negative size");
  const int results = axis == 1 ? src->size0 : src->size1;
  const int length = axis == 1 ? src->size1 : src->size0;
  if (results == 0) return KAPYB_OK;
  if (length == 0) return fail(h, KAPYB_INVALID_ARG, "reduce: cannot reduce an empty axis");
  CUDA_TRY(h, cudaSetDevice(h->device));
  ReduceParams p;
  p.src = elem_ptr(src);
  p.dst = const_cast<void *>(elem_ptr(dst));
  p.rows = results;
  p.cols = length;
  p.src_row_stride = axis == 1 ? src->stride0 : src->stride1;
  p.src_col_stride = axis == 1 ? src->stride1 : src->stride0;
  p.dst_stride = axis == 1 ? dst->stride0 : dst->stride1;
  p.src_dtype = src->dtype;
  p.dst_dtype = dst->dtype;
  p.combiner = combiner;
  const bool unit_inner = p.src_col_stride == 1 || length == 1;
  const int esz = dtype_size(src->dtype);
  const bool vec = unit_inner && (reinterpret_cast<uintptr_t>(p.src) & 31u) == 0 &&
                   (p.src_row_stride * esz) % 32 == 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // Results on the unit-stride axis (column sums of a row-major tensor), long
  // enough to be worth two passes: slabs of the reduced axis first, then the slabs.
  const bool slabs = !unit_inner && p.src_row_stride == 1 && length >= 256 && results >= 64 &&
                     results % (esz == 4 ? 4 : 8) == 0 && (esz == 2 || esz == 4) &&
                     (reinterpret_cast<uintptr_t>(p.src) & 15u) == 0 && p.src_col_stride > 0 &&
                     (p.src_col_stride * esz) % 16 == 0;
  if (slabs) {
    const int epl = esz == 4 ? 4 : 8;
    const int blocks_x = (results + 32 * epl - 1) / (32 * epl);
    int n_slabs = std::max(1, std::min({64, h->sm_count * 4 / blocks_x, length / 64}));
    const int slab_len = ((length + n_slabs - 1) / n_slabs + 7) / 8 * 8;
    n_slabs = (length + slab_len - 1) / slab_len;
    const size_t skinny_ws = skinny_workspace_bytes();
    kapyb_status st = kapyb_reserve_workspace(h, skinny_ws + static_cast<size_t>(n_slabs) * results * sizeof(float));
    if (st != KAPYB_OK) return st;
    float *partial = reinterpret_cast<float *>(static_cast<char *>(h->workspace) + skinny_ws);
    const dim3 grid(blocks_x, n_slabs);
    const long long step_bytes = p.src_col_stride * esz;
    const bool narrow = p.dst_dtype != KAPYB_F32;
    ReduceParams q = p;
    q.src = partial;
    q.src_dtype = KAPYB_F32;
    q.cols = n_slabs;
    q.src_row_stride = 1;
    q.src_col_stride = results;
    const int grid2 = (results + 31) / 32;
#define KAPYB_SLAB(COMB)                                                                             \
  do {                                                                                               \
    if (p.src_dtype == KAPYB_F32) {                                                                  \
      reduce_cols_slab_kernel<COMB, KAPYB_F32, KAPYB_F32><<<grid, 256, 0, stream>>>(                 \
          p.src, step_bytes, results, length, slab_len, partial);                                    \
      reduce_cols_kernel<COMB><<<grid2, 256, 0, stream>>>(q);                                        \
    } else if (p.src_dtype == KAPYB_BF16 && narrow) {                                                \
      reduce_cols_slab_kernel<COMB, KAPYB_BF16, KAPYB_BF16><<<grid, 256, 0, stream>>>(               \
          p.src, step_bytes, results, length, slab_len, partial);                                    \
      reduce_cols_kernel<COMB, KAPYB_BF16><<<grid2, 256, 0, stream>>>(q);                            \
    } else if (p.src_dtype == KAPYB_BF16) {                                                          \
      reduce_cols_slab_kernel<COMB, KAPYB_BF16, KAPYB_F32><<<grid, 256, 0, stream>>>(                \
          p.src, step_bytes, results, length, slab_len, partial);                                    \
      reduce_cols_kernel<COMB><<<grid2, 256, 0, stream>>>(q);                                        \
    } else if (narrow) {                                                                             \
      reduce_cols_slab_kernel<COMB, KAPYB_F16, KAPYB_F16><<<grid, 256, 0, stream>>>(                 \
          p.src, step_bytes, results, length, slab_len, partial);                                    \
      reduce_cols_kernel<COMB, KAPYB_F16><<<grid2, 256, 0, stream>>>(q);                             \
    } else {                                                                                         \
      reduce_cols_slab_kernel<COMB, KAPYB_F16, KAPYB_F32><<<grid, 256, 0, stream>>>(                 \
          p.src, step_bytes, results, length, slab_len, partial);                                    \
      reduce_cols_kernel<COMB><<<grid2, 256, 0, stream>>>(q);                                        \
    }                                                                                                \
  } while (0)
    switch (combiner) {
    case KAPYB_RED_ADD: KAPYB_SLAB(KAPYB_RED_ADD); break;
    case KAPYB_RED_MUL: KAPYB_SLAB(KAPYB_RED_MUL); break;
    case KAPYB_RED_MAX: KAPYB_SLAB(KAPYB_RED_MAX); break;
    default: KAPYB_SLAB(KAPYB_RED_MIN); break;
    }
#undef KAPYB_SLAB
    CUDA_TRY(h, cudaGetLastError());
    h->launches += 2;
    h->last_kernel = "reduce_cols_slabs";
    return KAPYB_OK;
  }
  switch (combiner) {
  case KAPYB_RED_ADD: launch_reduce<KAPYB_RED_ADD>(p, unit_inner, vec, h->sm_count, stream); break;
  case KAPYB_RED_MUL: launch_reduce<KAPYB_RED_MUL>(p, unit_inner, vec, h->sm_count, stream); break;
  case KAPYB_RED_MAX: launch_reduce<KAPYB_RED_MAX>(p, unit_inner, vec, h->sm_count, stream); break;
  default: launch_reduce<KAPYB_RED_MIN>(p, unit_inner, vec, h->sm_count, stream); break;
  }
  CUDA_TRY(h, cudaGetLastError());
  h->launches++;
  h->last_kernel = unit_inner ? "reduce_rows" : "reduce_cols";
  return KAPYB_OK;
}

// ------------------------------------------- decode matmul without allocation

// Fixed scratch for kapyb_matmul_decode_static: the partial sums of split weight
// tiles, as (fp32 value, launch number) pairs, one slot per CTA (10 MiB hold them
// for 64 rows on a GPU of up to 160 SMs).  It lives in the library image, so
// every GPU that loads the library carries these bytes until the process exits;
// it starts zeroed, and zero is the one launch number never used.
constexpr size_t kStaticPartialBytes = 10u << 20;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticPartialBytes];
static __device__ uint32_t g_decode_status;

struct StaticDeviceState {
  std::atomic<bool> ready{false};    // written last, with release ordering
  unsigned char *scratch = nullptr;  // device address of g_decode_scratch on this device
  uint32_t *status = nullptr;        // device address of g_decode_status on this device
  int sm_count = 0;
  EncodeTiledFn encode = nullptr;
  std::atomic<uint32_t> epoch{0};    // launches so far on this device: the numbers in the scratch
};
static StaticDeviceState g_static_state[kMaxDevices];
static std::mutex g_static_mu;  // serialises the one-time set-up per device

// First call on device `dev` (which must be current): resolve where the static
// arrays live there.  In host code the symbol name is only a stand-in, not a
// device address, so the runtime is asked for the address.  Two threads that make
// their first call at once are serialised; later calls take no lock.
static kapyb_status static_state_init(int dev, StaticDeviceState &sd) {
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (sd.ready.load(std::memory_order_acquire)) return KAPYB_OK;
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: device properties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: device %d is sm_%d%d; kernels are built for sm_100a only", dev, prop.major, prop.minor);
  void *p_scratch = nullptr, *p_status = nullptr;
  e = cudaGetSymbolAddress(&p_scratch, g_decode_scratch);
  if (e != cudaSuccess) return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
  e = cudaGetSymbolAddress(&p_status, g_decode_status);
  if (e != cudaSuccess) return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
  cudaDriverEntryPointQueryResult q;
  void *fn = nullptr;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
    return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: cuTensorMapEncodeTiled not available");
  sd.scratch = static_cast<unsigned char *>(p_scratch);
  sd.status = static_cast<uint32_t *>(p_status);
  sd.sm_count = prop.multiProcessorCount;
  sd.encode = reinterpret_cast<EncodeTiledFn>(fn);
  sd.ready.store(true, std::memory_order_release);
  return KAPYB_OK;
}

extern "C" KAPYB_API kapyb_status kapyb_matmul_decode_static(const kapyb_tensor2d *lhs,
                                                             const kapyb_tensor2d *rhs,
                                                             const kapyb_tensor2d *out,
                                                             const kapyb_epilogue *epilogue,
                                                             int32_t sync_and_check,
                                                             void *stream_) {
  // A stack context lets this call share the launcher of the ordinary path
  // without creating a handle (which would allocate).
  kapyb_context ctx;
  auto bail = [&](kapyb_status st) {
    g_create_error = ctx.last_error;
    return st;
  };
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(nullptr, KAPYB_UNSUPPORTED, "matmul_decode_static: device index %d not supported", dev);
  StaticDeviceState &sd = g_static_state[dev];
  if (!sd.ready.load(std::memory_order_acquire)) {
    const kapyb_status ist = static_state_init(dev, sd);
    if (ist != KAPYB_OK) return ist;
  }
  ctx.device = dev;
  ctx.sm_count = sd.sm_count;
  ctx.status = sd.status;
  ctx.encode = sd.encode;

  kapyb_status st = verify_matmul(&ctx, lhs, rhs, nullptr, out, epilogue, KAPYB_MMA_ANY);
  if (st != KAPYB_OK) return bail(st);
  MatmulProblem p = make_problem(lhs, rhs, nullptr, out, epilogue);
  if (p.M == 0 || p.N == 0) return KAPYB_OK;
  if (dtype_size(p.in_dtype) != 2)
    return bail(fail(&ctx, KAPYB_UNSUPPORTED, "matmul_decode_static: operands must be f16 or bf16"));
  if (p.M > kSkinnyMaxM || p.K < 1)
    return bail(fail(&ctx, KAPYB_UNSUPPORTED, "matmul_decode_static: needs 1 <= M <= %d and K >= 1 (got M=%d, K=%d)", kSkinnyMaxM, p.M, p.K));
  const size_t need_partial = skinny_partial_bytes(ctx.sm_count, p.M);
  if (need_partial > kStaticPartialBytes)
    return bail(fail(&ctx, KAPYB_UNSUPPORTED,
                     "matmul_decode_static: problem needs %zu bytes of partial sums (SMs * roundup16(M) * "
                     "1024); the fixed scratch holds %zu",
                     need_partial, kStaticPartialBytes));
  if (p.c_s1 != 1 && p.N != 1)
    return bail(fail(&ctx, KAPYB_UNSUPPORTED, "matmul_decode_static: out must be row-major (unit stride on axis 1)"));
  const bool a_k = p.a_s1 == 1 || p.K == 1, a_m = p.a_s0 == 1 || p.M == 1;
  const bool b_n = p.b_s1 == 1 || p.N == 1, b_k = p.b_s0 == 1 || p.K == 1;
  const bool a_mn = !a_k && a_m, b_mn = b_n;
  if ( !(a_k || a_m) || !(b_n || b_k) ||
      !tma_ok(p.a, p.in_dtype, a_mn ? p.M : p.K, a_mn ? p.K : p.M, a_mn ? p.a_s1 : p.a_s0, 1, 0) ||
      !tma_ok(p.b, p.in_dtype, b_mn ? p.N : p.K, b_mn ? p.K : p.N, b_mn ? p.b_s0 : p.b_s1, 1, 0))
    return bail(fail(&ctx, KAPYB_UNSUPPORTED,
                     "matmul_decode_static: operands need a unit stride, 16-byte aligned bases and "
                     "leading dimensions that are multiples of 16 bytes"));
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // The array keeps the last call's contents.  Nothing in it has to be cleared:
  // every partial sum carries the number of the call that wrote it, and this
  // call only accepts its own number.  The status word is shared too and does
  // start from zero, so that a checked call never reports what an earlier
  // unchecked call left behind.
  e = cudaMemsetAsync(sd.status, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: clearing the status word: %s", cudaGetErrorString(e));
  uint32_t epoch = sd.epoch.fetch_add(1, std::memory_order_relaxed) + 1;
  if (epoch == 0) epoch = sd.epoch.fetch_add(1, std::memory_order_relaxed) + 1;
  st = launch_skinny_on(&ctx, p, a_mn, b_mn, reinterpret_cast<uint2 *>(sd.scratch), epoch, stream);
  if (st != KAPYB_OK) return bail(st);
  if (sync_and_check) {
    e = cudaStreamSynchronize(stream);
    uint32_t word = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&word, sd.status, sizeof(word), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(nullptr, KAPYB_CUDA_ERROR, "matmul_decode_static: %s", cudaGetErrorString(e));
    if (word != kStatusOk) {
      cudaMemset(sd.status, 0, sizeof(uint32_t));
      return fail(nullptr, KAPYB_TIMEOUT, "matmul_decode_static: the kernel gave up on a bounded wait");
    }
  }
  return KAPYB_OK;
}
