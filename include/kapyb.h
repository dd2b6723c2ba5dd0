/*
 * kapyb.h -- C ABI of the B200 (sm_100a) backend for kapy-lang's matmul /
 * elementwise / reduce operator surface.
 *
 * The reference turns a kernel built through python/src/ir.cc (Builder.create_*)
 * into a PTX string (python/src/passes.cc:69-262, PassManager.run ->
 * translate_llvm_to_ptx) and has no launcher.  A binding that wants the kernel
 * to *run* calls the entry points below instead of that pipeline: the operands
 * are the same seven-field global tensor descriptors kapy.mk_global builds
 * (python/src/ir.cc:1013-1025), the enums carry the numeric values of
 * include/kapy/Dialect/Kapy/IR/Enums.td:42-109, and errors come back as status
 * codes instead of C++ exceptions (python/src/passes.cc:72-75).
 *
 * Conventions
 *   - plain C, no torch / CUDA types in signatures; `stream` is a cudaStream_t
 *     passed as void* (NULL = the legacy default stream);
 *   - every pointer inside a kapyb_tensor2d is a DEVICE pointer unless the
 *     function name ends in `_host`;
 *   - calls are asynchronous with respect to the host and ordered on `stream`,
 *     except the `_host` variants, which return after the result is in the host
 *     buffer;
 *   - nothing here throws, aborts or traps the device; device-side waits are
 *     bounded and surface as KAPYB_TIMEOUT on the next kapyb_check().
 */
#ifndef KAPYB_H_
#define KAPYB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define KAPYB_API
#else
#define KAPYB_API __attribute__((visibility("default")))
#endif

/* ------------------------------------------------------------------ enums */

typedef enum {
  KAPYB_OK = 0,
  KAPYB_INVALID_ARG = 1, /* verifier-equivalent rejection (Kapy.cpp:451-574) */
  KAPYB_UNSUPPORTED = 2,
  KAPYB_CUDA_ERROR = 3,
  /* 4 is not used: the library calls no communication library; ranks meet
   * through the flags of kapyb_gather_signal / kapyb_gather_wait */
  KAPYB_TIMEOUT = 5      /* a bounded device-side wait gave up */
} kapyb_status;

/* Element types on the path (ir.cc get_*_type, :598-640). */
typedef enum {
  KAPYB_F16 = 0,
  KAPYB_BF16 = 1,
  KAPYB_F32 = 2,
  /* The two 8-bit types: matmul operands (MatmulImplWay MMA_M16N8K16_F8,
   * Kapy.cpp:547-564) and the two ends of a cast (FPToFPOp, Kapy.cpp:272-287);
   * nothing computes in them.  f8E4M3 bytes are read the way the MMA and cvt
   * instructions read them: finite-only, S.1111.111 is NaN, largest value 448. */
  KAPYB_F8E4M3 = 3,
  KAPYB_F8E5M2 = 4,
  /* i1, the result type of arith.cmpf (ir.cc:941-1000): a value inside an
   * elementwise program only (the condition of a select); no tensor in memory
   * has it. */
  KAPYB_I1 = 5
} kapyb_dtype;

/* Enums.td:52-61 -- value returned for out-of-bounds lanes of ld_global. */
typedef enum {
  KAPYB_PAD_ZERO = 0,
  KAPYB_PAD_QNAN = 1,
  KAPYB_PAD_PINF = 2,
  KAPYB_PAD_NINF = 3
} kapyb_padding;

/* Enums.td:63-76: the cache operator of ld_global / st_global (PTX .ca .cg .cs
 * .wb .wt .lu .cv). */
typedef enum {
  KAPYB_CACHE_NONE = 0,
  KAPYB_CACHE_CA = 1,
  KAPYB_CACHE_CG = 2,
  KAPYB_CACHE_CS = 3,
  KAPYB_CACHE_WB = 4,
  KAPYB_CACHE_WT = 5,
  KAPYB_CACHE_LU = 6,
  KAPYB_CACHE_CV = 7
} kapyb_cache_modifier;

/* Enums.td:78-88: the eviction priority of ld_global / st_global. */
typedef enum {
  KAPYB_EVICT_NORMAL = 0,
  KAPYB_EVICT_FIRST = 1,
  KAPYB_EVICT_LAST = 2,
  KAPYB_EVICT_UNCHANGED = 3,
  KAPYB_NO_ALLOCATE = 4
} kapyb_evict_priority;

/* kapyb_tensor2d.cache: cache operator, eviction priority and the volatile flag
 * of the ld_global / st_global that touches the tensor
 * (LdGlobalOpToLLVM.cpp:101-110, StGlobalOpToLLVM.cpp:100-108). */
#define KAPYB_CACHE_HINTS(modifier, priority, is_volatile) \
  ((int32_t)(modifier) | ((int32_t)(priority) << 8) | ((is_volatile) ? (1 << 16) : 0))

/* Enums.td:90-100.  Names an sm_80 instruction; validated against the operand
 * dtypes exactly as MatmulOp::verify does (Kapy.cpp:491-565) and otherwise
 * ignored: scheduling on sm_100a is tcgen05. */
typedef enum {
  KAPYB_MMA_ANY = 0,
  KAPYB_MMA_M16N8K8_F16 = 1,
  KAPYB_MMA_M16N8K16_F16 = 2,
  KAPYB_MMA_M16N8K8_TF32 = 3,
  KAPYB_MMA_M16N8K16_F8 = 4
} kapyb_matmul_impl_way;

/* Enums.td:102-109. */
typedef enum {
  KAPYB_RZ = 0,
  KAPYB_RN = 1
} kapyb_rounding;

/* Activation fused into the GEMM epilogue.  GELU_TANH is the composite
 * u / (1 + exp(-2k)), k = 0.7978845608f * fma(0.044715f*u*u, u, u), built from
 * the ops kapy has (exp -> ex2.approx, ElementwiseOpToLLVM.cpp:1039-1073;
 * divf -> div.full.f32, :730-769). */
typedef enum {
  KAPYB_ACT_NONE = 0,
  KAPYB_ACT_RELU = 1,
  KAPYB_ACT_GELU_TANH = 2,
  KAPYB_ACT_SILU = 3
} kapyb_activation;

/* Combiner of kapy.reduce's lambda region (Ops.td:441-457, Kapy.cpp:628-649);
 * the four single-op lambdas are recognised. */
typedef enum {
  KAPYB_RED_ADD = 0,
  KAPYB_RED_MUL = 1,
  KAPYB_RED_MAX = 2, /* arith.maximumf: NaN propagates */
  KAPYB_RED_MIN = 3  /* arith.minimumf */
} kapyb_combiner;

/* ------------------------------------------------------------ descriptors */

/* kapy.mk_global (Ops.td:95-111; lowered struct {ptr,start0,start1,end0,end1,
 * stride0,stride1}, TypeConverter.cpp:64-73).  Element (i, j) lives at
 * ptr + (offset_elems + i*stride0 + j*stride1) * sizeof(dtype).  Sizes and
 * strides are i32 as in the reference; a size of 1 broadcasts when the tensor
 * is an elementwise input. */
typedef struct {
  void *ptr;
  int64_t offset_elems;
  int32_t size0, size1;
  int32_t stride0, stride1;
  int32_t dtype; /* kapyb_dtype */
  int32_t padding; /* kapyb_padding: what an elementwise load returns out of bounds.
                      Matmul operands take KAPYB_PAD_ZERO only (anything else is
                      refused with KAPYB_UNSUPPORTED); outputs ignore it. */
  int32_t cache;   /* KAPYB_CACHE_HINTS(...), 0 = none.  Hints never change a
                      result.  Elementwise programs on the general kernel issue the
                      very ld / st forms the reference emits (a cache operator
                      wins over a priority, volatile over both).  Matmul operands
                      map the priority to an L2 policy on their TMA loads:
                      EVICT_FIRST -> L2::evict_first, EVICT_LAST -> L2::evict_last,
                      NO_ALLOCATE -> L2::evict_first (a tile is never loaded
                      around L2); other values leave the default, which is no
                      hint, except for the weight operand of the decode-shape
                      kernel (M <= 64): read once per call, it streams as
                      evict_first unless a priority is named.  The fused
                      streaming kernels and kapyb_reduce keep their own policy
                      (read-once loads that bypass L1, streaming stores). */
  int32_t reserved_; /* keeps the struct a multiple of 8 bytes; set to 0 */
} kapyb_tensor2d;

/* result = downcast(act(alpha * (lhs . rhs) + bias [+ acc])).
 * The product accumulates in fp32 (bf16 operands require it, Kapy.cpp:479-482);
 * bias enters in the accumulator type, which is what kapy-combine makes of
 * add(matmul(a,b,0), broadcast(bias)) (Combine.td:38-88); the downcast is
 * kapy.fptofp with a mandatory rounding mode (Kapy.cpp:272-287). */
typedef struct {
  float alpha;        /* 1.0f for plain matmul */
  const void *bias;   /* NULL, or device vector */
  int32_t bias_dtype; /* kapyb_dtype */
  int32_t bias_axis;  /* 1: one value per column ([1,N] broadcast over rows);
                         0: one value per row ([M,1]) */
  int32_t activation; /* kapyb_activation */
  int32_t rounding;   /* kapyb_rounding for the final downcast */
} kapyb_epilogue;

/* ----------------------------------------------- elementwise programs */

/* One op of a recorded elementwise graph; mirrors the arith/math/kapy ops
 * Builder.create_* can emit (ir.cc:744-1000, :1106-1157).  Every op rounds to
 * `dtype`, its tensor element type, as the reference's per-op lowering does
 * (ElementwiseOpToLLVM.cpp:424-485; bf16 mul/add/sub are single-rounding
 * fma.rn.bf16, :771-892). */
typedef enum {
  KAPYB_OP_LOAD = 0,   /* dst = inputs[flags]            (kapy.ld_global) */
  KAPYB_OP_CONST = 1,  /* dst = imm rounded to dtype     (arith.constant + kapy.splat) */
  KAPYB_OP_CVT = 2,    /* dst = cast(a), flags = kapyb_rounding (extf/truncf/fptofp) */
  KAPYB_OP_ADD = 3,
  KAPYB_OP_SUB = 4,
  KAPYB_OP_MUL = 5,
  KAPYB_OP_DIV = 6,
  KAPYB_OP_FMA = 7,    /* dst = a*b + c, one rounding    (math.fma) */
  KAPYB_OP_MAXIMUM = 8,  /* arith.maximumf: NaN if either is NaN */
  KAPYB_OP_MINIMUM = 9,
  KAPYB_OP_MAXNUM = 10,  /* arith.maxnumf: the non-NaN operand */
  KAPYB_OP_MINNUM = 11,
  KAPYB_OP_CLAMP = 12, /* clampf(a, low=b, high=c); flags = propagate_nan */
  KAPYB_OP_ABS = 13,
  KAPYB_OP_NEG = 14,
  KAPYB_OP_EXP = 15,
  KAPYB_OP_EXP2 = 16,
  KAPYB_OP_LOG = 17,
  KAPYB_OP_LOG2 = 18,
  KAPYB_OP_SQRT = 19,
  KAPYB_OP_RSQRT = 20,
  KAPYB_OP_ERF = 21,
  KAPYB_OP_SIN = 22,
  KAPYB_OP_COS = 23,
  KAPYB_OP_FLOOR = 24,
  KAPYB_OP_CEIL = 25,
  KAPYB_OP_TANH = 26,  /* elementwise_extern_lib "__nv_tanhf" (Ops.td:459-484) */
  KAPYB_OP_STORE = 27, /* output = a                      (kapy.st_global) */
  KAPYB_OP_CMP = 28,   /* dst(i1) = a <pred> b, flags = kapyb_cmp_predicate (arith.cmpf;
                          Builder.create_cmpf_*, ir.cc:941-1000); dtype = KAPYB_I1 */
  KAPYB_OP_SELECT = 29, /* dst = a(i1) ? b : c            (arith.select, ir.cc:1162) */
  KAPYB_OP_AND = 30,   /* i1 logic on conditions          (arith.andi / ori / xori on i1) */
  KAPYB_OP_OR = 31,
  KAPYB_OP_XOR = 32,
  KAPYB_OP_COUNT_
} kapyb_opcode;

/* Predicates of arith.cmpf as Builder.create_cmpf_* binds them (ir.cc:941-1000).
 * "Ordered" predicates are false when either operand is NaN, "unordered" ones
 * true. */
typedef enum {
  KAPYB_CMP_OLT = 0,
  KAPYB_CMP_OGT = 1,
  KAPYB_CMP_OLE = 2,
  KAPYB_CMP_OGE = 3,
  KAPYB_CMP_OEQ = 4,
  KAPYB_CMP_ONE = 5,
  KAPYB_CMP_ULT = 6,
  KAPYB_CMP_UGT = 7,
  KAPYB_CMP_ULE = 8,
  KAPYB_CMP_UGE = 9,
  KAPYB_CMP_UEQ = 10,
  KAPYB_CMP_UNE = 11
} kapyb_cmp_predicate;

#define KAPYB_MAX_REGS 16
#define KAPYB_MAX_INSTS 64
#define KAPYB_MAX_INPUTS 4

typedef struct {
  int32_t op;    /* kapyb_opcode */
  int32_t dtype; /* kapyb_dtype of the result */
  int32_t dst;   /* register 0..KAPYB_MAX_REGS-1 */
  int32_t a, b, c; /* source registers, -1 when unused */
  float imm;     /* KAPYB_OP_CONST */
  int32_t flags; /* see the opcode */
} kapyb_inst;

/* ------------------------------------------------------------------ handle */

typedef struct kapyb_context *kapyb_handle;

/* Library version (major*100 + minor). */
KAPYB_API int kapyb_version(void);

/* Creates a handle bound to CUDA device `device`.  Fails with KAPYB_CUDA_ERROR
 * when the device is absent or is not compute capability 10.x: there is no CPU
 * fallback.  The handle owns its workspace, its status word and its tensor-map
 * cache; the caller owns every tensor.  Not thread-safe: one handle per thread
 * and device.  Replaces the reference's MLIRContext + PassManager pair
 * (ir.cc:157-170, passes.cc:69-75). */
KAPYB_API kapyb_status kapyb_create(kapyb_handle *out, int device);
KAPYB_API kapyb_status kapyb_destroy(kapyb_handle h);

/* Text of the last non-OK status returned through `h` (also valid for
 * h == NULL: the last failure of kapyb_create on this thread).  Stands in for
 * the what() of the exceptions the reference throws (passes.cc:74,
 * ir.cc:257,431,588,677,1085). */
KAPYB_API const char *kapyb_last_error_string(kapyb_handle h);

/* Synchronises `stream` and reports what the device recorded: KAPYB_TIMEOUT if
 * a kernel gave up on a bounded wait, KAPYB_CUDA_ERROR on a sticky error. */
KAPYB_API kapyb_status kapyb_check(kapyb_handle h, void *stream);

/* Grows the handle's device workspace (split-K partials, host-call staging) to
 * at least `bytes`.  Called implicitly when needed; call it up front to keep
 * allocation out of a timed region. */
KAPYB_API kapyb_status kapyb_reserve_workspace(kapyb_handle h, size_t bytes);

/* ------------------------------------------------------------------ matmul */

/* kapy.matmul (Ops.td:416-439) at whole-problem scope:
 *   out[M,N] = epilogue( lhs[M,K] . rhs[K,N] (+ acc[M,N]) ).
 * lhs/rhs: both f16, both bf16, both f32 (multiplied as tf32: the tensor core
 * reads the upper 19 bits of each operand, as mma_m16n8k8_tf32 does), or each
 * one of the two fp8 types (Kapy.cpp:484-487, :530-564); either may be row- or
 * column-major (one unit stride, CoalesceAccess.cpp:32-40).  `acc` may be NULL
 * (= zero accumulator, the arith.constant dense<0.0> of matmul.mlir:6) or an
 * f16/f32 [M,N] tensor added in fp32 (fastest when it has out's element type,
 * unit stride on its columns, a 16-byte aligned base and a leading dimension
 * that is a multiple of 16 bytes: the epilogue then fetches it tile by tile;
 * anything else is read element by element, same result).  out: f16, bf16 or f32.
 * Returns KAPYB_INVALID_ARG for the shape/dtype violations MatmulOp::verify
 * rejects (Kapy.cpp:459-487). */
KAPYB_API kapyb_status kapyb_matmul(kapyb_handle h, const kapyb_tensor2d *lhs,
                                    const kapyb_tensor2d *rhs,
                                    const kapyb_tensor2d *acc,
                                    const kapyb_tensor2d *out,
                                    const kapyb_epilogue *epilogue,
                                    int32_t impl_way, void *stream);

/* kapyb_matmul with a kapy.reduce (Ops.td:441-457) of its result fused into the
 * epilogue: besides `out`, the f32 values the epilogue produces (scale, bias,
 * activation; before the downcast to out's type) are summed along `axis` into
 * `reduced`, a dense f32 vector of shape [M,1] (axis 1: one sum per row) or
 * [1,N] (axis 0: one per column).  This is what a kernel that follows its
 * matmul chain with `kapy.reduce ... lambda addf` on the accumulator tile
 * computes, without a second pass over the output.  `reduced` is cleared on
 * `stream` and then accumulated with fp32 atomic adds, so the order of
 * combination is unspecified (as in the reference, ReduceOpToLLVM.cpp:76-119)
 * and may differ from run to run in the last bits.  Only the addf lambda
 * (KAPYB_RED_ADD) is fused; operands and output must be TMA-describable. */
KAPYB_API kapyb_status kapyb_matmul_reduce(kapyb_handle h, const kapyb_tensor2d *lhs,
                                           const kapyb_tensor2d *rhs, const kapyb_tensor2d *out,
                                           const kapyb_tensor2d *reduced, int32_t axis,
                                           int32_t combiner, const kapyb_epilogue *epilogue,
                                           int32_t impl_way, void *stream);

/* `batch` independent matmuls; operand b of batch i starts batch_stride_*
 * elements after batch i-1.  In the reference the batch is the grid's z axis
 * (kapy.program_id axis 2, ir.cc:1091-1096). */
KAPYB_API kapyb_status kapyb_matmul_batched(
    kapyb_handle h, const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
    const kapyb_tensor2d *out, int32_t batch, int64_t batch_stride_lhs,
    int64_t batch_stride_rhs, int64_t batch_stride_out,
    const kapyb_epilogue *epilogue, int32_t impl_way, void *stream);

/* kapyb_matmul with HOST buffers: copies lhs/rhs (and bias) to the handle's
 * workspace, runs the same kernels, copies `out` back and returns when it has
 * landed.  This is the call a binding makes when the caller's arrays live in
 * host memory (numpy), and the one the end-to-end benchmark times. */
KAPYB_API kapyb_status kapyb_matmul_host(kapyb_handle h,
                                         const kapyb_tensor2d *lhs,
                                         const kapyb_tensor2d *rhs,
                                         const kapyb_tensor2d *out,
                                         const kapyb_epilogue *epilogue,
                                         int32_t impl_way, void *stream);

/* N-sharded matmul with the gather fused into the epilogue: this rank owns
 * columns [col_begin, col_begin + rhs->size1) of the full [M, n_total] output
 * and stores each finished tile of them into the full-size output of every
 * peer (peer_out[r] = base pointer of rank r's [M, n_total] buffer with row
 * stride out_stride0, reachable from this device; peer_out[my rank] included).
 * No loads from remote memory are issued.  The caller synchronises ranks
 * (stream-ordered barrier) before reading. */
KAPYB_API kapyb_status kapyb_matmul_push(
    kapyb_handle h, const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
    void *const *peer_out, int32_t n_peers, int32_t out_dtype,
    int32_t out_stride0, int32_t col_begin, int32_t n_total,
    const kapyb_epilogue *epilogue, int32_t impl_way, void *stream);

/* Completion flags between the GPUs of one box; no reference counterpart (the
 * reference has no multi-GPU code).  Every rank owns an array of n_ranks 32-bit
 * words in memory all ranks can reach (peer-mapped device memory, or pinned
 * host memory), zero at the start.  kapyb_gather_signal stores `seq` into word
 * my_rank of EVERY rank's array (peer_flags[r] = rank r's array), ordered after
 * everything issued on `stream` before it; kapyb_gather_wait returns (on
 * `stream`) once every word of this rank's own array has reached `seq` (wrapping
 * comparison; start at 1 and count up).  Only stores cross the link.  The wait
 * polls for at most limit_ms (0 = 2000): when that runs out the kernel gives
 * up, later work on the stream still runs, and kapyb_check returns
 * KAPYB_TIMEOUT.  A rank must order its own signal before its wait (same stream,
 * or an event): the wait is never the only thing keeping a kernel of the same
 * GPU from running. */
KAPYB_API kapyb_status kapyb_gather_signal(kapyb_handle h, void *const *peer_flags,
                                           int32_t n_ranks, int32_t my_rank, uint32_t seq,
                                           void *stream);
KAPYB_API kapyb_status kapyb_gather_wait(kapyb_handle h, const void *my_flags, int32_t n_ranks,
                                         uint32_t seq, uint32_t limit_ms, void *stream);

/* What a rank needs to meet its peers in kapyb_matmul_host_sharded. */
typedef struct {
  int32_t rank, world;
  /* [world] device pointers, entry r = rank r's staging area for the whole lhs,
   * reachable from this GPU (entry [rank] is this GPU's own memory).  Each area
   * holds TWO copies of [m_total, K], the second starting roundup256(m_total *
   * K * element size) bytes after the first; calls use them in turn (seq & 1). */
  void *const *peer_lhs;
  /* [world] device pointers to every rank's flag array (kapyb_gather_signal). */
  void *const *peer_flags;
  uint32_t seq;           /* 1 for the first call, then +1 per call, the same on all ranks
                             (the flag words carry seq * 64 + a piece number) */
  uint32_t wait_limit_ms; /* 0: 2000 */
} kapyb_shard_ctx;

/* kapyb_matmul_host for `world` GPUs that share one problem: the output is
 * sharded by columns (this rank computes out[m_total, n_local] = lhs . rhs with
 * rhs its own [K, n_local] column block of B), and the upload of lhs is sharded
 * by rows: this rank uploads only rows [row_begin, row_begin + lhs_rows->size0)
 * from host memory and forwards them to every peer's staging area over NVLink
 * (copy engines, stores only, no loads of remote memory), so each row of lhs
 * crosses PCIe once per box instead of once per GPU.  The rows travel in up to
 * four pieces per rank; the product of a piece and the download of its rows of
 * `out` overlap the upload of the next piece.  m_total must be a multiple of
 * world and rank r must own the r-th block of m_total / world rows.  Every rank
 * must make the matching call (same seq).  Returns when `out` has landed in host memory;
 * KAPYB_TIMEOUT when a peer's rows did not arrive within the limit.  No
 * reference counterpart. */
KAPYB_API kapyb_status kapyb_matmul_host_sharded(
    kapyb_handle h, const kapyb_tensor2d *lhs_rows, int32_t m_total, int32_t row_begin,
    const kapyb_tensor2d *rhs, const kapyb_tensor2d *out, const kapyb_epilogue *epilogue,
    const kapyb_shard_ctx *ctx, int32_t impl_way, void *stream);

/* The decode-shape (few-row) matmul for callers that must not allocate device
 * memory.  No counterpart in the reference.
 *
 * Who needs it: a host whose memory pool already owns the whole GPU (a serving
 * engine that reserved all of HBM up front, so a plugin's cudaMalloc fails or
 * steals from the pool), a latency-critical loop that cannot afford the
 * device-wide synchronisation cudaMalloc/cudaFree imply, or an embedding that
 * forbids allocation after start-up.  kapyb_matmul on this shape splits weight
 * tiles between SMs and passes the pieces through scratch memory taken from the
 * handle's workspace (a cudaMalloc); this variant takes no handle and keeps that
 * scratch in a fixed array inside the library image instead.
 *
 *   out[M,N] = epilogue(lhs[M,K] . rhs[K,N]),  1 <= M <= 64, f16/bf16 operands.
 *
 * Limits and rules:
 *  - the fixed scratch is 10 MiB of partial sums per GPU (held by every GPU that
 *    loads the library, until exit); a call needs SMs * roundup16(M) * 1024
 *    bytes of it (M = 64 fits on up to 160 SMs).  Larger problems, and M > 64,
 *    are refused with KAPYB_UNSUPPORTED and a message saying so; nothing is
 *    launched;
 *  - operands must be TMA-describable (one unit stride, 16-byte aligned base,
 *    leading dimension a multiple of 16 bytes); there is no fallback kernel;
 *  - the call runs on the CURRENT device.  Its first call on each device looks
 *    up the array's device address (cudaGetSymbolAddress) and the device's
 *    properties; make that first call outside any stream capture.  Threads that
 *    make their first call on one device at the same time are serialised;
 *  - it calls no cudaMalloc/cudaFree and no allocating library routine.  It
 *    clears the time-out word (cudaMemsetAsync on `stream`), then launches the
 *    kernel on `stream`.  The array keeps the previous call's partial sums and
 *    needs no clearing: each one carries the number of the call that wrote it,
 *    and a call only accepts its own;
 *  - all calls on one GPU share the one array: two calls whose kernels can
 *    overlap on the GPU (different streams, no dependency) race and give wrong
 *    results.  Keep them on one stream or order them yourself;
 *  - sync_and_check != 0 waits for `stream` and returns KAPYB_TIMEOUT if THIS
 *    call's kernel gave up on a bounded wait; with 0 the call returns after
 *    launching and a time-out of it goes unreported (the next call starts the
 *    word from zero again);
 *  - a tile split between SMs is summed in a fixed order, so the result is the
 *    same bits as kapyb_matmul's on the same problem and device.
 * Error text: kapyb_last_error_string(NULL) on the calling thread. */
KAPYB_API kapyb_status kapyb_matmul_decode_static(const kapyb_tensor2d *lhs,
                                                  const kapyb_tensor2d *rhs,
                                                  const kapyb_tensor2d *out,
                                                  const kapyb_epilogue *epilogue,
                                                  int32_t sync_and_check, void *stream);

/* --------------------------------------------------- elementwise / reduce */

/* Runs a recorded elementwise graph over out->size0 x out->size1 elements.
 * inputs[k] is what the k-th KAPYB_OP_LOAD reads; an input whose size on an
 * axis is 1 broadcasts along it (kapy.broadcast, Ops.td:342-356).  Canonical
 * graphs (affine, affine + gelu_tanh, binary add/sub/mul, casts to or from an
 * 8-bit type) run as fused vectorised kernels; any other valid program runs on
 * the generic device interpreter.  Casts involving f8E4M3 / f8E5M2 follow
 * ElementwiseOpToLLVM.cpp:83-289, :583-650: widening is exact; narrowing with
 * rn is cvt.rn.satfinite (beyond the largest finite value, infinities included,
 * gives that value); rz exists for f8E5M2 from f16 / f32 only (the high byte of
 * the value truncated to f16); f8 to f8 and rz from bf16 are refused with the
 * verifier's words (Kapy.cpp:272-287).  Programs are validated (register use before def, dtype
 * agreement, downcasts need a rounding mode) as the op verifiers would. */
KAPYB_API kapyb_status kapyb_elementwise(kapyb_handle h, const kapyb_inst *prog,
                                         int32_t n_inst,
                                         const kapyb_tensor2d *inputs,
                                         int32_t n_inputs,
                                         const kapyb_tensor2d *out,
                                         void *stream);

/* kapy.reduce (Ops.td:441-457; lowering ReduceOpToLLVM.cpp:76-119) over a whole
 * [size0,size1] tensor: axis 1 -> dst [size0,1], axis 0 -> dst [1,size1].
 * dst->dtype must be f32 or equal src->dtype.  The lambda runs at dst's element
 * type, as the reference calls the region on values of the tensor's type: with
 * an f32 destination a 16-bit source is widened first (arith.extf) and combined
 * in f32; with a 16-bit destination every combination is rounded to that type
 * (reduce_sum.mlir:10-25 adds in f16).  The order of combination is unspecified
 * in the reference; here it is fixed per shape, so results repeat bit for bit. */
KAPYB_API kapyb_status kapyb_reduce(kapyb_handle h, const kapyb_tensor2d *src,
                                    const kapyb_tensor2d *dst, int32_t axis,
                                    int32_t combiner, void *stream);

/* ------------------------------------------------------------- shard math */

/* Range [begin, end) of `total` units owned by `rank` of `parts` when units
 * are dealt in blocks of `align` (the last blocks may be short or empty).
 * Pure host arithmetic; no reference counterpart (the reference has no
 * multi-GPU code). */
KAPYB_API kapyb_status kapyb_shard_range(int64_t total, int32_t parts,
                                         int32_t rank, int64_t align,
                                         int64_t *begin, int64_t *end);

/* ------------------------------------------------------------ diagnostics */

/* Describes, as a few lines of text, how kapyb_matmul would run this problem:
 * kernel family, tile and pipeline depth, tile grid and waves, operand majors,
 * and where an accumulator element sits in tensor memory.  The counterpart of
 * the reference's layout printer (bin/kapy-layout.cpp:79-126): a debugging
 * aid.  Pure host code: only the descriptors' shapes, strides, dtypes and the
 * alignment of their addresses are looked at, nothing is launched.  `h` may be
 * NULL when `sm_count` > 0 (then no GPU is needed at all); with a handle,
 * sm_count = 0 means the handle's device and the path forced with
 * kapyb_set_matmul_path applies.  `batch` > 1 plans densely packed batches. */
KAPYB_API kapyb_status kapyb_matmul_plan(kapyb_handle h, int32_t sm_count,
                                         const kapyb_tensor2d *lhs, const kapyb_tensor2d *rhs,
                                         const kapyb_tensor2d *out, int32_t batch, char *text,
                                         size_t capacity);

/* Tuned dispatch choices, process-wide.  A file has one problem per line,
 *     M N K batch dtype k|mn k|mn path        # comment
 * (dtype of lhs: f16 bf16 f32 f8E4M3 f8E5M2; the majors of lhs and rhs as the
 * kernel sees them, "k" = K contiguous; path as in kapyb_set_matmul_path, e.g.
 * "2cta:256" or "1cta:128:e8").  kapyb_matmul consults the table when no path
 * is forced and the problem matches a line exactly; a choice that does not apply
 * (say, a tcgen05 path for operands TMA cannot describe) is ignored.  Loading
 * adds to the table (same problem: the later line wins); errors name the line.
 * kapyb_matmul_plan shows when a choice came from the table.  The reference
 * keeps no such cache; `kapy-lang_b200/runtime.py: tune_matmul` writes one. */
KAPYB_API kapyb_status kapyb_tuning_load(const char *file, int32_t *n_entries);
KAPYB_API kapyb_status kapyb_tuning_clear(void);

/* Name of the kernel family the last matmul on `h` dispatched to
 * ("tcgen05_1cta", "tcgen05_2cta", "tcgen05_skinny", "simt"). */
KAPYB_API const char *kapyb_last_kernel(kapyb_handle h);

/* Number of kernels this handle has launched since creation. */
KAPYB_API int64_t kapyb_launch_count(kapyb_handle h);

/* Profiling probes of the last matmul launched with debug bit 7 (":d128" in
 * kapyb_set_matmul_path), then cleared.  Copies n <= 14 words after
 * synchronising `stream`.  tcgen05 GEMM: word 0 = SM cycles, word 1 = wall
 * nanoseconds the first CTA's MMA-issuing thread spent in its tile loop (their
 * ratio is the SM clock in GHz while the kernel ran).  Both kernels: words 2..6
 * are readings of the nanosecond timer's low 32 bits: the
 * complement of the earliest CTA start, then the latest, over all CTAs, of: CTA
 * start, first operand stage landed, last MMA issued, epilogue done.  GEMM only
 * (zero unless the library was built with -DKAPYB_DEBUG_SWITCHES):
 * words 7..11 = clocks one epilogue warp of the first CTA spent per phase of its
 * chunk loop (for the register drain of the 256 x 512 tile: timer at which it saw
 * half 0, clocks in tcgen05.ld, clocks from there to handing half 1 back, clocks
 * in the two hand-overs, clocks issuing the first store); words 12, 13 = clocks the first CTA's MMA warp waited for operand
 * stages and for accumulator slots. */
KAPYB_API kapyb_status kapyb_probe_read(kapyb_handle h, void *stream, uint32_t *words, int32_t n);

/* Forces a kernel family for matmul ("auto", "1cta", "2cta", "skinny", "simt"),
 * optionally ":<tile width>", ":e<epilogue warps>", ":s<stages>", ":k<0|1>"
 * (decode kernel: whole weight tiles only | leftover tiles split between SMs),
 * ":g<row blocks per raster group>", ":x<0|1>" (tcgen05 kernels: the tiles of a
 * partly filled last wave stay whole, the default | are split between the CTAs,
 * their partial sums added in CTA order: the same bits on every run, though not
 * the bits of the whole-tile schedule; the first such call allocates 40 MB of
 * scratch, so make it before any stream capture), ":w<wait limit in ms>" and
 * ":d<debug bits>"; for tests and profiling.  Debug bit 16 silences
 * the producer (every bounded wait then runs out: the test of the time-out
 * path) and bit 128 switches the probes on; both leave correct kernels
 * correct.  The bits that make a kernel skip work (1, 2, 4, 8, 32) are refused
 * with KAPYB_UNSUPPORTED unless the library was built with
 * -DKAPYB_DEBUG_SWITCHES. */
KAPYB_API kapyb_status kapyb_set_matmul_path(kapyb_handle h, const char *name);

#ifdef __cplusplus
}
#endif
#endif /* KAPYB_H_ */
