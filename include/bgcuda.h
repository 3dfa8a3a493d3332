/*
 * bgcuda.h -- C ABI of the B200 (sm_100a) realizer bridge for browsergrad-jit.
 *
 * One bg_context is one bridge: the object `bg.register_webgpu_bridge(bridge)` stores
 * (packages/browsergrad-jit/src/python/_realize_webgpu.py:628-636) and whose methods the
 * realizers call (Protocol: packages/browsergrad-jit/src/python/_bridge.py:61-289; TypeScript
 * interface: packages/browsergrad-kernels/src/realizer.ts:77-280).  Each entry point below
 * names the bridge method it stands behind.  Host shims (Python ctypes, Node N-API) only
 * translate argument encodings; all scheduling, fusion and memory management is in the
 * library.
 *
 * Conventions
 *  - every function returns a bg_status (0 = ok); on failure bg_last_error(ctx) holds a UTF-8
 *    message prefixed "CUDA bridge: <op> ..."; nothing throws across the boundary;
 *  - a context is used from one thread at a time (the reference bridge is never shared
 *    between threads, realizer.ts:895-896); two contexts on one device are independent;
 *  - handles are positive, minted from 1 upward and never reused (realizer.ts:907, :925);
 *  - tensors are dense row-major little-endian, exactly the bytes of `ndarray.tobytes()`;
 *  - all work of one context is ordered on one CUDA stream; calls that return bytes
 *    synchronise that stream, calls that return handles do not.
 */
#ifndef BGCUDA_H
#define BGCUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BG_MAX_RANK 8
#define BG_MAX_STEP_INPUTS 8
#define BG_ABI_VERSION 1

typedef struct bg_context bg_context;
typedef int64_t bg_handle;

typedef enum bg_status {
  BG_OK = 0,
  BG_ERR_INVALID = 1,         /* malformed argument, shape/dtype/byte-length mismatch   */
  BG_ERR_UNSUPPORTED = 2,     /* opcode or variant outside the forward path              */
  BG_ERR_CUDA = 3,            /* a CUDA runtime/driver call failed                       */
  BG_ERR_OOM = 4,             /* device allocation failed                                */
  BG_ERR_UNKNOWN_HANDLE = 5,  /* handle was never minted or already released             */
  BG_ERR_DEVICE_TIMEOUT = 6,  /* a bounded device-side wait ran out                      */
  BG_ERR_INDEX_RANGE = 7      /* gather / cross-entropy index outside its axis           */
} bg_status;

/* dtype names of the IR (packages/browsergrad-jit/src/python/_ir.py:348-353) + bfloat16,
 * which the reference does not have (extension used by the bf16 autocast path). */
typedef enum bg_dtype {
  BG_F16 = 0, BG_F32 = 1, BG_F64 = 2,
  BG_I8 = 3, BG_I16 = 4, BG_I32 = 5, BG_I64 = 6,
  BG_U8 = 7, BG_U16 = 8, BG_U32 = 9, BG_U64 = 10,
  BG_BOOL = 11, BG_BF16 = 12
} bg_dtype;

/* Opcodes of the forward path (names as in _ir.py:203-247). */
typedef enum bg_opcode {
  BG_OP_BUFFER = 0, BG_OP_LOAD = 1, BG_OP_CONST = 2, BG_OP_CAST = 3,
  BG_OP_ADD = 4, BG_OP_MUL = 5, BG_OP_DIV = 6, BG_OP_NEG = 7, BG_OP_EXP = 8, BG_OP_LOG = 9,
  BG_OP_ABS = 10, BG_OP_SIGN = 11, BG_OP_SIN = 12, BG_OP_COS = 13, BG_OP_ISNAN = 14,
  BG_OP_CMP = 15, BG_OP_WHERE = 16,
  BG_OP_MATMUL = 17, BG_OP_REDUCE = 18, BG_OP_RESHAPE = 19, BG_OP_PERMUTE = 20,
  BG_OP_BROADCAST_TO = 21, BG_OP_LAYER_NORM = 22, BG_OP_CROSS_ENTROPY = 23, BG_OP_INDEX = 24,
  BG_OP_FUSED_ELEMENTWISE = 25, BG_OP_FUSED_SOFTMAX = 26, BG_OP_ATTENTION_FORWARD = 27,
  /* Data-movement opcodes beyond the 28 of the forward configs (_ir.py:93-99; handlers
     _realize.py:268-327): iarg[0] = axis (FLIP, CUMSUM, CONCAT) or diagonal (TRIL, TRIU);
     CUMSUM iarg[1] = reverse.  CONCAT takes up to BG_MAX_STEP_INPUTS inputs. */
  BG_OP_TRIL = 28, BG_OP_TRIU = 29, BG_OP_FLIP = 30, BG_OP_CONCAT = 31, BG_OP_CUMSUM = 32,
  /* Stable ordering along iarg[0] (_framework_contracts.py:4921-4936, :5063-5089), int64 positions out:
     SORT_INDICES iarg[1] = descending; TOPK_INDICES iarg[1] = k, iarg[2] = largest, iarg[3] = sorted (must be 1).
     The *_VALUES opcodes of the reference are gathers along the same axis and arrive as INDEX. */
  BG_OP_SORT_INDICES = 33, BG_OP_TOPK_INDICES = 34,
  /* Overwrite scatter along iarg[0] (_realize.py:1179-1189; contract _framework_contracts.py:5494-5630):
     inputs (target, int64 index, source of the index's shape or a scalar constant); the result is a copy
     of the target with source values stored at the indexed places.  An index outside the axis or two
     index entries naming one destination end the plan with BG_ERR_INDEX_RANGE, as the reference raises. */
  BG_OP_SCATTER = 35,
  /* Basic slicing x[start:stop:step, ...] (_realize.py:1124-1128; NARROW, _realize.py:309-314, arrives as the same
     opcode): a strided view of the input, iarg[d] = start_d + (step_d << 40) per input axis (start >= 0,
     step >= 1, the declared shape gives the extents).  Never a copy unless the view is the plan's root. */
  BG_OP_SLICE = 36,
  BG_OP_COUNT = 37
} bg_opcode;

typedef enum bg_cmp { BG_CMP_EQ = 0, BG_CMP_NE = 1, BG_CMP_LT = 2, BG_CMP_LE = 3,
                      BG_CMP_GT = 4, BG_CMP_GE = 5 } bg_cmp;
typedef enum bg_reduce { BG_RED_SUM = 0, BG_RED_MAX = 1, BG_RED_MIN = 2, BG_RED_MEAN = 3,
                         BG_RED_ARGMAX = 4, BG_RED_ARGMIN = 5, BG_RED_ANY = 6,
                         BG_RED_ALL = 7, BG_RED_PROD = 8 } bg_reduce;

/*
 * One scheduled step of a tensor plan: the C form of one entry of
 * `GpuExecutionPlan.summary()["steps"]` (packages/browsergrad-jit/src/python/_gpu_plan.py:176-209).
 * value ids equal step indices (webgpu_realizer.test.ts:1114-1161), inputs precede users.
 * The live Python `arg` is flattened by the shim into iarg/farg/ext:
 *   CONST            farg[0] = value as double; iarg[0] = value as int64 (integer/bool dtypes)
 *   CAST             target dtype = .dtype
 *   CMP              iarg[0] = bg_cmp
 *   REDUCE           iarg[0] = bg_reduce; iarg[1] = bit mask of reduced input axes;
 *                    iarg[2] = keepdims
 *   PERMUTE          iarg[0..rank-1] = axes
 *   FUSED_SOFTMAX    iarg[0] = axis (non-negative)
 *   LAYER_NORM       iarg[0] = rows, iarg[1] = cols, farg[0] = eps
 *   INDEX            iarg[0] = gather dimension
 *   CROSS_ENTROPY    iarg[0] = 0 none / 1 mean / 2 sum; iarg[1] = ignore_index; iarg[2] = batch_rank (0);
 *                    iarg[3] = bit 0 probability targets (else int64 class indices), bit 1 class weights
 *                    as a third input; farg[0] = label smoothing
 *   ATTENTION_FORWARD farg[0] = scale
 *   FUSED_ELEMENTWISE ext[ext_offset .. +3*ext_count) = (bg_opcode, lhs_ref, rhs_ref) triples;
 *                    refs < 0 name input -ref-1, refs >= 0 an earlier triple
 *                    (_fusion.py:184-232); rhs_ref = BG_REF_NONE for unary ops.
 */
#define BG_REF_NONE INT32_MIN

typedef struct bg_plan_step {
  int32_t op;       /* bg_opcode */
  int32_t dtype;    /* bg_dtype of the step's value */
  int32_t rank;
  int32_t n_inputs;
  int64_t shape[BG_MAX_RANK];
  int32_t input_ids[BG_MAX_STEP_INPUTS];
  int64_t iarg[BG_MAX_RANK];
  double farg[2];
  int32_t ext_offset;
  int32_t ext_count;
} bg_plan_step;

typedef struct bg_plan {
  const bg_plan_step* steps;
  int32_t n_steps;
  int32_t root_id;
  const int32_t* ext;
  int32_t n_ext;
} bg_plan;

/* Binding of one BUFFER step: an existing handle, or host bytes to upload for this run
 * (`{value_id, handle}` | `{value_id, data}`, _realize_webgpu.py:490-519). */
typedef struct bg_plan_input {
  int32_t value_id;
  int32_t reserved;
  bg_handle handle;   /* 0 when `data` is given */
  const void* data;
  size_t nbytes;
} bg_plan_input;

/* Byte-exact accounting, the fields of `resourceSnapshot()` (realizer.ts:287-298). */
typedef struct bg_resource_stats {
  int64_t current_bytes;
  int64_t peak_bytes;
  int64_t total_allocated_bytes;
  int64_t total_released_bytes;
  int64_t alive_handles;
  int64_t logical_tensor_plan_peak_bytes;
  int64_t kernel_launches;      /* kernels of this library launched so far */
  int64_t plan_cache_hits;
  int64_t plan_cache_misses;
} bg_resource_stats;

/* One timed launch, the role of `DirectDispatchProfile` (runner.ts:409-507). */
typedef struct bg_profile_entry {
  char name[64];
  float ms;
  int32_t launches;
} bg_profile_entry;

/* -- lifecycle: createWebGpuRealizerBridge(device, {profiling}) (realizer.ts:902-1006) ---- */
int bg_create(int device_ordinal, bg_context** out);
int bg_destroy(bg_context* ctx);
const char* bg_last_error(bg_context* ctx);
int bg_abi_version(void);
/* options: "profiling" (0/1), "f64_contraction" (0 = exact fp64 FMA, 1 = fp32-faithful tensor
 * path, 2 = automatic: tensor path when no fp64 leaf enters the plan), "fusion" (0/1), "tensor_cores" (0/1),
 * "static_patterns" (0/1: the kernels specialised for whole expressions -- the dominant chains, residual + LayerNorm
 * rows -- and the producer-side operand formats that go with them; 0 leaves every elementwise / row group to the
 * generic interpreter and every value in the type the graph gives it), "gemm_groups" (0/1), "gemm_cta_pairs" (0/1/2), "gemm_pair_tile_width" (0/256/192/128),
 * "attention16_kernel" (bit set: 1 two query tiles per CTA, 2 V as an MN-major operand, 4 P in tensor memory,
 * 8 fp32 K / V converted inside the kernel; 0 one query tile per CTA; -1 restores the default),
 * "dependent_launch" (0/1, default 1: the tensor-core GEMMs, the fused attentions, the LayerNorm rows, the small GEMM,
 * the one-launch cross entropy and the embedding lookup are launched with programmatic stream serialization -- each is
 * set up on the SMs the kernel before it has left and waits for that whole kernel before its first access to global
 * memory; 0 restores plain stream order),
 * "attention32_kernel" (3xTF32 attention: 0 two threads per row, 1 one thread per row with P and O in tensor
 * memory, 3 the same with fp32 Q / K rows split into planes inside the kernel; -1 restores the default). */
int bg_set_option(bg_context* ctx, const char* key, int64_t value);

/* -- buffers: upload / materialize / release (_bridge.py:65-71; realizer.ts:1006-1041) ----- */
int bg_upload(bg_context* ctx, const void* data, size_t nbytes, const int64_t* shape, int rank,
              int dtype, bg_handle* out);
int bg_materialize(bg_context* ctx, bg_handle h, void* out, size_t nbytes);
/* A buffer of the given shape and dtype whose contents the caller writes itself, on the context's stream (bg_stream),
 * through bg_device_pointer: the destination of a device-side collective (the all-gather of row shards or of the
 * column blocks of a wide Linear across GPUs).  No counterpart in the reference bridge, which has one device
 * (the only "collective" there is a single-device simulation, semantic_host_graph_wgsl.ts:143-160). */
int bg_alloc(bg_context* ctx, const int64_t* shape, int rank, int dtype, bg_handle* out);
int bg_release(bg_context* ctx, bg_handle h);     /* idempotent; unknown handle is a no-op */
int bg_handle_nbytes(bg_context* ctx, bg_handle h, int64_t* out);

/* -- per-op methods (_bridge.py:74-105; realizer.ts:1043-1151) --------------------------- */
int bg_matmul(bg_context* ctx, bg_handle a, bg_handle b, int64_t m, int64_t k, int64_t n,
              int dtype, bg_handle* out);
int bg_fused_elementwise(bg_context* ctx, const bg_handle* inputs, int n_inputs,
                         const int32_t* op_triples, int n_ops, const int64_t* shape, int rank,
                         int dtype, bg_handle* out);
int bg_cast(bg_context* ctx, bg_handle h, int src_dtype, int dst_dtype, const int64_t* shape,
            int rank, bg_handle* out);
/* mask = 0 for none, else an additive mask handle of shape mask_shape[4] = [B'|1,H'|1,Sq,Sk]
 * (packages/browsergrad-kernels/src/kernels/flash_attention.ts:8-9). */
int bg_flash_attention(bg_context* ctx, bg_handle q, bg_handle k, bg_handle v, bg_handle mask,
                       const int64_t* mask_shape, int64_t b, int64_t h, int64_t sq, int64_t sk,
                       int64_t d, double scale, int dtype, bg_handle* out);

/* -- whole-plan methods: run_tensor_plan[_resident] (_bridge.py:262-289;
 *    realizer.ts:1557-1652).  The *_semantic variants differ only in the shim, which checks
 *    the dense-permutation-view-copy requests (_gpu_plan.py:668-734) and writes their axes
 *    into the PERMUTE steps before calling these. -------------------------------------- */
int bg_run_tensor_plan(bg_context* ctx, const bg_plan* plan, const bg_plan_input* inputs,
                       int n_inputs, void* out_host, size_t out_nbytes);
int bg_run_tensor_plan_resident(bg_context* ctx, const bg_plan* plan,
                                const bg_plan_input* inputs, int n_inputs, bg_handle* out);

/* -- diagnostics: aliveHandleCount / resourceSnapshot / flushProfiles
 *    (realizer.ts:273-279, :287-298, :945-993) ------------------------------------------ */
int bg_alive_handle_count(bg_context* ctx, int64_t* out);
int bg_resource_snapshot(bg_context* ctx, bg_resource_stats* out);
int bg_flush_profiles(bg_context* ctx, bg_profile_entry* out, int capacity, int* n_out);
/* Text listing of the kernels the most recent plan compiled to, one per line: the unit's kind, what was folded into
 * it ("+bias", "+gelu", "+mask", "+merge"), the operand format it stores for its readers ("+split": operand planes of
 * the split products that read it; "+cast16": the 16-bit type of the autocast Linears that read it; "+f32store": the
 * fp32 values of an fp64-typed product that only the fused attention reads), and the dtype of the graph node. */
int bg_last_plan_trace(bg_context* ctx, char* out, size_t capacity);
/*
 * Cross entropy over class-index targets with no allocation of any kind (no counterpart in the
 * reference).  For callers that may not allocate device memory while running -- a process whose
 * own arena already owns the GPU, or a loop that cannot afford cudaMalloc's device-wide stall.
 * logits [rows, classes, inner] fp32, targets [rows, inner] int64, out: one fp32; all three are
 * DEVICE pointers owned by the caller.  reduction: 1 = mean over valid targets, 2 = sum.
 * The per-position scratch is a static device array: rows * inner <= 1 048 576 (larger problems
 * are refused with BG_ERR_UNSUPPORTED and a message in `err`); every GPU that loads the library
 * holds those 4 MiB + 256 B until the process exits.  The first call on a device looks the array's
 * device address up and should therefore come before any stream capture.  All calls share the
 * array: calls that overlap on the GPU race, so order them on one stream.  The call synchronises
 * `stream` (a cudaStream_t) and reports an out-of-range target as BG_ERR_INDEX_RANGE.
 */
int bg_cross_entropy_noalloc(const float* logits, const int64_t* targets, float* out, int64_t rows,
                             int64_t classes, int64_t inner, int reduction, int64_t ignore_index,
                             void* stream, char* err, size_t err_capacity);
/* Host-only diagnostic: compiles `plan` into its kernel list (one name per line) without a
 * device or a context; `fusion` bit 0 enables group formation, bit 1 lowers as on a B200 (tensor-core
 * kernels selectable).  Used to test the plan compiler
 * on machines without a GPU. */
int bg_compile_plan_dry(const bg_plan* plan, int fusion, char* out, size_t capacity);
/* Diagnostics of the failure paths.  One small kernel waits `limit_cycles` SM cycles, with the bounded wait of the
 * tensor-core kernels, on a barrier nothing arrives on and gives up: the call returns BG_ERR_DEVICE_TIMEOUT through the
 * same status word those kernels use, and the context stays usable.  (Option "fail_allocation_after" = n makes the
 * n-th device allocation from now fail with BG_ERR_OOM.)  No counterpart in the reference bridge. */
int bg_selftest_wait_timeout(bg_context* ctx, int64_t limit_cycles);
/* The CUDA stream all work of this context is ordered on (a cudaStream_t). */
void* bg_stream(bg_context* ctx);
/* Raw device pointer behind a handle, for callers that time kernels themselves. */
int bg_device_pointer(bg_context* ctx, bg_handle h, void** out);

#ifdef __cplusplus
}
#endif
#endif /* BGCUDA_H */
