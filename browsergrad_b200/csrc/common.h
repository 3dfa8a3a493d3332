// Internal declarations shared by the translation units of libbgcuda.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/bgcuda.h"

namespace bg {

constexpr int kMaxRank = BG_MAX_RANK;

inline int dtype_size(int dt) {
  switch (dt) {
    case BG_F16: case BG_BF16: case BG_I16: case BG_U16: return 2;
    case BG_F32: case BG_I32: case BG_U32: return 4;
    case BG_F64: case BG_I64: case BG_U64: return 8;
    case BG_I8: case BG_U8: case BG_BOOL: return 1;
  }
  return 0;
}
inline bool dtype_is_float(int dt) { return dt == BG_F16 || dt == BG_F32 || dt == BG_F64 || dt == BG_BF16; }
inline bool dtype_is_int(int dt) { return dt >= BG_I8 && dt <= BG_U64; }
const char* dtype_name(int dt);
const char* op_name(int op);

// ---------------------------------------------------------------------------------------
// Elementwise program: the descriptor the generic kernel interprets.  It is passed as a
// __grid_constant__ kernel parameter, i.e. it lives in the constant bank.
// ---------------------------------------------------------------------------------------
enum EwType : uint8_t { T_F32 = 0, T_F64 = 1, T_I64 = 2, T_B = 3 };

enum EwOp : uint8_t {
  E_LOAD = 0,   // dst <- inputs[aux], converted to `type`
  E_CONST,      // dst <- consts[aux] (double bits for floats, int64 bits for T_I64/T_B)
  E_ADD, E_MUL, E_DIV, E_NEG, E_EXP, E_LOG, E_ABS, E_SIGN, E_SIN, E_COS,
  E_ISNAN,      // dst(T_B) <- isnan(a) ; type = class of a
  E_CMP,        // dst(T_B) <- a (aux = bg_cmp) b ; type = class of a, b
  E_WHERE,      // dst <- a(T_B) ? b : c
  E_CVT,        // dst(type) <- a (aux low 4 bits = source class); applies narrowing
  E_NARROW,     // dst <- round/wrap a to the storage dtype in aux (f16, bf16, i8..u32, bool)
  E_AND, E_OR,  // bool arithmetic (NumPy: bool*bool = and, bool+bool = or)
  E_STORE,      // outputs[aux] <- a
  // fp32 super-instructions formed by the compiler's peephole pass
  E_SUB,        // dst <- a - b            (ADD of a NEG)
  E_RELU,       // dst <- a > 0 ? a : +0   (CONST 0, CMP gt, WHERE)
  E_EXPNEG,     // dst <- exp(-a)          (NEG, EXP)
  E_COPY,       // dst <- a                (a dense fp32 LOAD or STORE after operand folding; a float64 output widens)
  E_GELU,       // dst <- a / (1 + exp(-2 k (a + 0.044715 a^3))), k = sqrt(2/pi): the tanh GELU of an fp32 value, which
                // replaces its float64 evaluation 0.5 a (1 + tanh(k (a + 0.044715 a^3))) in plans without a float64 leaf
  E_OPCOUNT
};

// Register fields of fp32 instructions may name something else than a shared-memory register:
//   0x80|k   source: input k (dense fp32, vector-aligned) read at the element's own linear index;
//            destination: output k written there.  The compiler folds single-use LOADs and final
//            STOREs this way, so a value that is consumed once never round-trips through shared memory;
//   0xC0|k   source: consts[k] as an fp32 splat;
//   kEwAcc   the accumulator: the value the previous instruction left in real registers.  A result
//            whose only reader is the next instruction goes there and nowhere else.
constexpr uint8_t kEwDirect = 0x80;
constexpr uint8_t kEwConst = 0xC0;
constexpr uint8_t kEwAcc = 0x7e;

struct EwInstr {
  uint8_t op, type, dst, a, b, c;
  uint16_t aux;
};

constexpr int kEwMaxInstr = 160;
constexpr int kEwMaxInputs = 12;
constexpr int kEwMaxOutputs = 4;
constexpr int kEwMaxConsts = 24;
constexpr int kEwMaxDims = 5;

enum EwAddr : int32_t { A_CONTIG = 0, A_SCALAR = 1, A_STRIDED = 2 };

struct EwOperand {
  const void* ptr;
  int32_t dtype;
  int32_t mode;                 // EwAddr
  int32_t vec_ok;               // 16-byte (or natural 4-element) vector access allowed
  int32_t pad;
  int64_t stride[kEwMaxDims];   // element strides per collapsed iteration dim (A_STRIDED)
};

struct EwOutput {
  void* ptr;
  int32_t dtype;
  int32_t vec_ok;
};

enum RowTail : int32_t {
  TAIL_NONE = 0,
  TAIL_REDUCE = 1,     // tail_arg = bg_reduce; result per row -> outputs[tail_out]
  TAIL_SOFTMAX = 2,    // softmax over the row of register tail_reg -> outputs[tail_out]
  TAIL_LAYERNORM = 3,  // (x-mean)*rsqrt(var+eps)*w+b; w = inputs[tail_w], b = inputs[tail_b]
  TAIL_LOGSOFTMAX_PICK = 4  // cross entropy per row: -(log_softmax(x)[target]); target = inputs[tail_w]
};

struct EwProgram {
  int32_t n_instr;
  int32_t n_regs;
  int32_t wide;                 // any 8-byte register class in use
  int32_t ndim;                 // collapsed iteration rank (>= 1)
  int64_t shape[kEwMaxDims];    // collapsed iteration shape, row-major
  int64_t numel;
  int32_t n_inputs, n_outputs, n_consts;
  // row mode
  int32_t tail;                 // RowTail
  int32_t tail_arg;
  int32_t tail_reg;             // register holding the row values
  int32_t tail_type;            // EwType of tail_reg
  int32_t tail_out;             // output index of the tail result
  int32_t tail_w, tail_b;       // operand indices (layer norm weight/bias, CE target)
  int32_t tail_out_dtype;
  float tail_eps;
  int32_t tail_acc;             // the last instruction is an fp32 one that produces tail_reg: its accumulator holds the row values
  int32_t pad0;
  int64_t rows, cols;           // row mode: numel = rows * cols
  int64_t tail_aux;             // CE: ignore_index
  EwInstr instr[kEwMaxInstr];
  EwOperand inputs[kEwMaxInputs];
  EwOutput outputs[kEwMaxOutputs];
  int64_t consts[kEwMaxConsts];  // raw 64-bit patterns
};

// Kernel launchers (defined in the .cu files).  All return cudaError_t of the launch.
cudaError_t launch_elementwise(const EwProgram& p, cudaStream_t s, int sm_count);
cudaError_t launch_rowwise(const EwProgram& p, cudaStream_t s, int sm_count, int* status_flag);
// Row-mode capacity: how many 1024-element chunks per row the shared-memory register file holds.
int rowwise_max_chunks(int n_regs, int wide);

// Specialised fp32 pattern kernels (ew_static.cu).
struct StaticArgs {
  const float* in[4];
  float* out;
  int64_t rows, cols, numel;
};
enum StaticKind { SK_FLAT = 0, SK_ROWSUM = 1, SK_SOFTMAX = 2 };
int static_pattern_id(const std::string& signature, int* n_inputs);
bool static_shape_ok(int kind, int64_t rows, int64_t cols, int64_t numel, int sm_count);
cudaError_t launch_static(int pattern, int kind, const StaticArgs& a, int arg, cudaStream_t s, int sm_count);

// Layer-norm rows over a sum of terms (ln_static.cu): h = term0 + term1 + ..; out = LN(f32(h)) * w + b.
struct LnArgs {
  const void* term[4];
  int32_t term_dtype[4];     // BG_F32 or BG_F64
  int32_t term_rowvec[4];    // 1: a [cols] vector repeated on every row
  int32_t n_terms;
  int32_t wide;              // the sum is fp64 (else fp32; then every term is fp32)
  void* sum_out;             // optional h, stored in the sum type
  void* out;
  int32_t out_dtype;         // BG_F32 or BG_F64
  int32_t w_dtype, b_dtype;
  float eps;
  const void* w;
  const void* b;
  int64_t rows, cols;
  // non-null: `out` is not written; the rows are stored as the planes launch_tf32_split(out, ...) would have made
  void* planes_hi;
  void* planes_lo;
  // non-null: `out` is not written; the rows are stored rounded to out16_dtype (BG_F16 / BG_BF16), as a CAST of `out`
  // would have given
  void* out16;
  int32_t out16_dtype;
};
bool static_ln_shape_ok(int64_t rows, int64_t cols);
cudaError_t launch_static_ln(const LnArgs& a, cudaStream_t s, int sm_count);

struct StridedView {
  const void* ptr;
  int32_t dtype;
  int32_t rank;
  int64_t shape[kMaxRank];
  int64_t stride[kMaxRank];   // elements
};

// Data-movement kernels over a strided input view and a dense output (shape_kernels.cu).
// tri: keep the lower (upper = 0) or upper triangle of the last two dims relative to `diagonal`, zero elsewhere.
cudaError_t launch_tri(const StridedView& in, void* out, int64_t numel, int upper, int64_t diagonal, cudaStream_t s);
// flip: out[..., i, ...] = in[..., n - 1 - i, ...] along `axis`.
cudaError_t launch_flip(const StridedView& in, void* out, int64_t numel, int axis, cudaStream_t s);
// place: copies `in` (converted to out_dtype) into the block of the dense output `out_shape` that starts at
// `axis_offset` along `axis` (one launch per CONCAT input).  With `fill` the block is set to that constant
// and `in` only gives the block's shape (a broadcast scalar as a CONCAT input: the borders of a constant PAD).
struct PlaceFill { int is_int; double f; long long n; };
cudaError_t launch_place(const StridedView& in, void* out, int out_dtype, const int64_t* out_shape, int axis, int64_t axis_offset,
                         cudaStream_t s, const PlaceFill* fill = nullptr);
// scatter: out (already a dense copy of the target) receives src[i] (or the constant) at the place index entry i
// names along `dim`; `claim` is scratch of one int per output element.  Bad or repeated destinations set *status.
cudaError_t launch_scatter(const int64_t* idx, const void* src, void* out, int* claim, int esize, int rank, const int64_t* out_shape,
                           const int64_t* idx_shape, int dim, bool src_is_const, unsigned long long const_bits, int* status, cudaStream_t s);
// cumsum along `axis` in the output dtype, sequential per line as NumPy's add.accumulate.
cudaError_t launch_cumsum(const StridedView& in, void* out, int out_dtype, int axis, int reverse, cudaStream_t s);

// Stable argsort of every line along `axis` (at most kSortMaxLine elements per line); the first `keep` positions of
// each sorted line are written as int64 to the dense output (keep = line length for a full sort, k for top-k).
constexpr int kSortMaxLine = 4096;
cudaError_t launch_sort_lines(const StridedView& in, int64_t* out, int axis, int descending, int64_t keep, cudaStream_t s);

// out[...] = in[view] : dense copy of a strided view (permute / broadcast materialisation).
cudaError_t launch_strided_copy(const StridedView& in, void* out, int64_t numel, cudaStream_t s);
// Generic [outer, R, inner] reductions / softmax on dense data (any inner), fp32/fp64/int64.
cudaError_t launch_reduce_generic(const void* in, void* out, int in_dtype, int out_dtype, int red_op,
                                  int64_t outer, int64_t R, int64_t inner, cudaStream_t s);
cudaError_t launch_softmax_generic(const void* in, void* out, int dtype, int64_t outer, int64_t R,
                                   int64_t inner, cudaStream_t s);
// gather along `dim` (torch.gather semantics); out-of-range indices set *status = BG_ERR_INDEX_RANGE.
cudaError_t launch_gather(const void* x, const int64_t* idx, void* out, int esize, int rank,
                          const int64_t* x_shape, const int64_t* idx_shape, int dim, int* status,
                          cudaStream_t s);
// Cross entropy (misc_kernels.cu).  launch_ce_rows writes one loss per position of logits [outer, C, inner] (class axis
// strided by inner): class-index targets (int64, `ignore_index` skipped, values outside [0, C) set *status) or
// probability targets of the logits' shape and type; optional class weights [C] of the logits' type and label
// smoothing.  `sel_w`, when given, receives each position's target weight (0 for ignored targets).
struct CeProblem {
  const void* logits;
  const void* targets;
  const void* weight;
  void* per_pos;
  void* sel_w;
  int dtype;                 // BG_F32 or BG_F64
  int prob_targets;
  int64_t outer, C, inner, ignore_index;
  double label_smoothing;
  int* status;
};
cudaError_t launch_ce_rows(const CeProblem& c, cudaStream_t s);
// Per-position losses -> sum (reduction 2) or mean (1): the mean divides by the summed `sel_w` when given, else by the
// number of `targets` that differ from ignore_index when given, else by `fixed_count`.
// Losses and their mean / sum in one launch of one CTA, for at most 256 positions with a short class axis; the bits
// launch_ce_rows + launch_ce_reduce give.
bool ce_small_usable(const CeProblem& c);
cudaError_t launch_ce_small(const CeProblem& c, void* out, int reduction, double fixed_count, cudaStream_t s);
cudaError_t launch_ce_reduce(const void* per_pos, const int64_t* targets, const void* sel_w, void* out, int dtype, int64_t n,
                             int reduction, int64_t ignore_index, double fixed_count, cudaStream_t s);

struct GemmOperand {
  const void* ptr;
  int32_t dtype;
  int64_t row_stride, col_stride;   // elements
  int64_t batch_stride[4];          // per broadcast batch dim (0 where broadcast)
};
struct GemmProblem {
  int64_t m, n, k;
  int32_t n_batch_dims;
  int64_t batch_shape[4];
  GemmOperand a, b;
  void* c;            // dense [batch..., m, n]
  int32_t c_dtype;
};
// Reference-order SIMT GEMM for every dtype (fp32 FMA, fp64 FMA, exact int64).
cudaError_t launch_gemm_simt(const GemmProblem& p, cudaStream_t s);

// Split-K kernel for small 2-D fp32 problems (gemm_simt.cu), with an fp32 bias row and ReLU folded.  gemm_small_plan
// says whether the problem qualifies, into how many K slices it is cut and how many bytes of partial tiles it needs;
// `counters` are 1024 device ints that are zero between launches.
bool gemm_small_plan(const GemmProblem& p, int sm_count, int* splits, int64_t* partial_bytes);
cudaError_t launch_gemm_small(const GemmProblem& p, const void* bias, int act, void* partials, int* counters, int splits, cudaStream_t s);

// Tensor-core GEMM (gemm_tc.cu): C[M,N] = epilogue(A[M,K] . B[N,K]^T), operands dense row-major.
enum TcAct { TC_ACT_NONE = 0, TC_ACT_RELU = 1, TC_ACT_GELU = 2 };
struct TcGemm {
  int64_t M, N, K;
  const void* A;        // [M,K]: f16 / bf16, or the tf32-rounded "hi" part of an fp32 operand
  const void* B;        // [N,K]
  const void* A_lo;     // fp32 residual parts (3xTF32 only)
  const void* B_lo;
  int ab_dtype;         // BG_F16, BG_BF16, or BG_F32 (3xTF32)
  void* C;              // [M,N] dense
  int c_dtype;          // BG_F32, BG_F16, BG_BF16, BG_F64
  const void* bias;     // [N] or null
  int bias_dtype;
  int act;              // TcAct
  int round_acc;        // 0, or dtype + 1: round the accumulator through f16 / bf16 before the epilogue
  int wide;             // activation arithmetic in fp64 (for fp64 results)
  // Non-null (single problems, N a multiple of 8, pointers 32-byte aligned): C is not written; the epilogue stores
  // the result as the planes launch_tf32_split(C, c_dtype, planes_hi, planes_lo, M*N, N) would have made of it.
  void* planes_hi;
  void* planes_lo;
};
// Set by the host-only dry compile so that plans can be lowered as they would be on a B200.
extern bool g_tc_assume_available;
// CTA-pair (cta_group::2) GEMM tiles: 0 never, 1 for problems that fill the device (default), 2 whenever legal.
extern int g_tc_pair_mode;
extern int g_tc_pair_width;
// Programmatic dependent launch of the decoder's kernels (1 = on): a kernel of the chain may be set up on the SMs the
// kernel before it has left, while that kernel's last CTAs still run; it waits for the whole grid before it (and for
// its memory) at grid_dependency_wait(), which it reaches before its first access to global memory.  Only kernels that
// contain that wait are ever launched this way.
extern int g_dependent_launch;
bool tc_gemm_supported(int64_t M, int64_t N, int64_t K, int ab_dtype);
cudaError_t launch_gemm_tc(const TcGemm& g, int* status, cudaStream_t s);
// 1 to 3 problems that share A, M, N, K, dtypes and the epilogue kind and differ in B, bias and C, as one launch.
cudaError_t launch_gemm_tc_group(const TcGemm* gs, int n_prob, int* status, cudaStream_t s);
// Self test of the bounded device wait: a wait of `limit_cycles` on a barrier nothing arrives on; sets *status.
cudaError_t launch_wait_timeout_selftest(long long limit_cycles, int* status, cudaStream_t s);
// hi = tf32(x) (round to nearest), lo = x - hi, for fp32 or fp64 input; optional transpose is not done here.
cudaError_t launch_tf32_split(const void* src, int src_dtype, float* hi, float* lo, int64_t n, int64_t k, cudaStream_t s);
// dst (f16 / bf16) = round-to-nearest-even(src fp32), dense, eight elements per thread step.
cudaError_t launch_convert16(const void* src, int src_dtype, void* dst, int64_t n, int dtype16, cudaStream_t s);

// Fused attention (attn_tc.cu).  Operands are [B,H,S,D] views with element strides; D = 64.
struct AttnOperand {
  const void* ptr;
  int dtype;
  int64_t stride[4];
};
struct AttnProblem {
  int B, H, Sq, Sk, D;
  AttnOperand q, k, v;
  const float* scale_buf;   // [B,H,Sq,Sk] multiplier or null (then `scale`)
  float scale;
  const void* mask;         // additive fp32 or bool, rows Sk apart, or null
  int mask_is_bool;
  int64_t mask_sb, mask_sh; // element strides over batch / head, 0 when broadcast
  void* out;                // [B,H,Sq,D] addressed through out_sb / out_sh / out_ss; rows of D are dense
  int64_t out_sb, out_sh, out_ss;   // element strides over batch / head / query row
  int out_dtype;
  int mode;                 // 0: 16-bit operands (ab_dtype), 1: 3xTF32
  int ab_dtype;
  // 3xTF32 only, non-null when the result only feeds split products as their A operand: the planes
  // launch_tf32_split would make of the B*H*Sq*D result values (same element offsets as `out`, which must then
  // cover its elements densely).  `out` is written only when the kernel in use cannot store planes.
  void* planes_hi;
  void* planes_lo;
};
bool attn_tc_supported(const AttnProblem& a);
void attn_scratch_sizes(const AttnProblem& a, int64_t bytes[8]);
// scratch[7] is the device flag "scale_buf is uniform"; it is (re)computed when check_uniform is set.
cudaError_t launch_attention_tc(const AttnProblem& a, void* const scratch[8], bool check_uniform, bool classify_mask, int* status, cudaStream_t s);
// Which 16-bit attention kernel runs (attn_tc.cu): bit 0 the two-query-tile kernel, bit 1 V as an MN-major operand,
// bit 2 P kept in tensor memory, bit 3 (with bits 1 and 2) fp32 K / V converted inside the kernel; 0 is the single-tile kernel.
extern int g_attn16_variant;
constexpr int kAttn16DefaultVariant = 15;
// Which 3xTF32 attention kernel runs: 0 two threads per row, P through shared memory; 1 one thread per row, P and O in
// tensor memory; 3 as 1, and fp32 Q / K rows are split into their hi / lo planes inside the kernel.
extern int g_attn32_variant;
constexpr int kAttn32DefaultVariant = 3;

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch of a kernel that calls grid_dependency_wait() before it touches global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at{};
  at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &at;
  cfg.numAttrs = g_dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

}  // namespace bg
