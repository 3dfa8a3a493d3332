// Tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in tensor memory, operand tiles
// staged in shared memory by TMA, fused bias / activation / conversion epilogue.
//
//   C[M,N] = epilogue( A[M,K] . B[N,K]^T )          both operands K-major (row-major [rows, K])
//
// One CTA computes one 128 x BN output tile (BN = 128 or 256) with three specialised roles:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of 128-byte-swizzled A / B tiles into a
//              ring of shared-memory stages, completion counted on "full" mbarriers;
//   warp 1     MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 32 bytes of K per
//              instruction) into the TMEM accumulator and releases stages with tcgen05.commit;
//   warps 2-9  epilogue: tcgen05.ld of the 128 accumulator lanes, bias / activation / rounding,
//              vector stores of the result rows.
// Loads carry no cluster multicast.  Two operand encodings share the kernel:
//   * 16-bit (f16 / bf16) operands, fp32 accumulate;
//   * a split product for fp32-faithful results ("3xTF32" in kernel names): A and B are pre-split into hi = tf32(x),
//     bf16(x) and bf16(x - hi); hi.hi runs on the tf32 path, the two correction products on the bf16 path;
//     the K loop runs three passes (residual.bf16, bf16.residual, hi.hi - small terms first) into one accumulator.
// Every wait is bounded by a clock deadline; on expiry the kernel records
// BG_ERR_DEVICE_TIMEOUT in the status word, lets copies in flight land, frees its tensor memory
// and returns.
#include "common.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tc_common.cuh"

namespace bg {
namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int kStageRowBytes = 128;          // one swizzle row: 64 x 16-bit or 32 x tf32
constexpr int kTf32ChunkBlocks = 16;         // 3xTF32: K blocks (of 32 floats) summed in tensor memory before a register add
// Sixteen epilogue warps in the 16-bit kernels, twelve in the split-product kernels (four / three per TMEM lane
// quarter, taking the 32-column chunks of a tile in turn): with short K loops the epilogue's instruction issue, not
// the tensor pipe, sets the pace.  A split-product warp holds up to three chunks of partial sums in registers, which
// is what limits its count.
template <bool TF32> struct EpiCfg {
  static constexpr int kWarps = TF32 ? 12 : 16;
  static constexpr int kThreads = 64 + 32 * kWarps;
};

struct TcParams {
  int M, N;
  int num_k_blocks;     // K blocks of 128 bytes per pass
  int passes;           // 1, or 3 for the hi/lo split
  int chunk_blocks;     // K blocks accumulated in tensor memory before the epilogue warps take the partial sum over
  int elems_per_block;  // K elements per 128-byte block (64 or 32)
  void* C;
  int c_dtype;
  const void* bias;     // per-column (length N) or null
  int bias_dtype;
  int act;              // TcAct
  int round_acc;        // 0: none, BG_F16 + 1 / BG_BF16 + 1: round the accumulator through that dtype first
  int wide;             // activation arithmetic in fp64
  uint32_t idesc;
  uint32_t idesc16;     // split product: the instruction descriptor of its two bf16 passes
  int mixed;            // split product: 1 = correction passes on bf16 planes; 0 = on the fp32 residual plane (tf32), for row
                        // lengths whose bf16 rows would not start on 16-byte boundaries
  int group_m;
  int* status;
  // grouped launch of the CTA-pair kernel: n_prob problems that share A, M, N, K and the epilogue kind and
  // differ in B, bias and C (the q / k / v projections of one activation); tiles of all problems form one grid
  int n_prob;
  void* Cg[3];
  const void* biasg[3];
  // The result is the A operand of split products only: instead of C the epilogue stores its planes (tf32(x) as
  // fp32; then, in the 16-bit area, bf16(x) and bf16(x - tf32(x)), M*N elements each).  N is a multiple of 8.
  float* planes_hi;
  __nv_bfloat16* planes_16;
};
constexpr int kMaxGroup = 3;
struct PairBMaps { CUtensorMap m[3 * kMaxGroup]; };   // per problem: B (or its tf32 plane), then its bf16 plane and its bf16 residual plane

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// gelu(x) = 0.5 x (1 + tanh(u)), u = k (x + 0.044715 x^3), of the reference graph, evaluated as x / (1 + e^(-2u)):
// one exponential on the exp2 unit, no cancellation for negative x.  The graph writes tanh as
// (e^u - e^-u) / (e^u + e^-u), which is inf / inf = NaN once e^|u| overflows the graph's arithmetic type; `u_max` is
// that type's largest exponent argument (88.72 for fp32 graphs, 709.78 for float64 tails) and the result is NaN
// beyond it, as the reference's is.
__device__ __forceinline__ float gelu_one_exp(float x, float u_max) {
  const float x2 = x * x;
  const float u = x * fmaf(0.7978845608028654f * 0.044715f, x2, 0.7978845608028654f);
  const float e = ex2_fast(u * (-2.0f * 1.4426950408889634f));
  const float g = x * rcp_fast(1.0f + e);
  return fabsf(u) > u_max ? __int_as_float(0x7fc00000) : g;
}
// fp32 graphs reach the epilogue through the 16-bit autocast path (tolerance 2e-2)
template <typename T>
__device__ __forceinline__ T gelu_graph(T x) { return (T)gelu_one_exp((float)x, 88.72f); }
// results stored as float64: the product is fp32-accurate (split product), so the activation is evaluated in fp32
// (about 1e-6 relative) and widened
__device__ __forceinline__ float gelu_accurate(float x) { return gelu_one_exp(x, 709.78f); }

// One 32-byte store per lane: an epilogue thread owns a row of the tile, so a 16-byte store fills half a sector per
// lane; the 256-bit form (sm_100) writes whole sectors with half the instructions.  `p` is 32-byte aligned.
__device__ __forceinline__ void st_global_256(void* p, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
               "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

__device__ __forceinline__ float load_bias(const void* b, int dt, int col) {
  switch (dt) {
    case BG_F32: return reinterpret_cast<const float*>(b)[col];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(b)[col]);
    case BG_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[col]);
    default: return (float)reinterpret_cast<const double*>(b)[col];
  }
}

// Epilogue of one 32-column chunk of one accumulator row: rounding, bias, activation, store.
// SPLIT: the kernel computes split products, whose results may leave as operand planes (p.planes_hi).
template <bool SPLIT>
__device__ __forceinline__ void epilogue_chunk(const TcParams& p, const uint32_t* r, int row, int col0, void* C, const void* bias) {
  // (the choices that are the same for every element -- rounding, activation, store type -- are taken outside the
  // element loops: inside them the compiler predicates, and every element then issues the instructions of all branches)
  float v[32];
  if (p.round_acc == BG_F16 + 1) {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float2 f = __half22float2(__floats2half2_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
      v[j] = f.x; v[j + 1] = f.y;
    }
  } else if (p.round_acc == BG_BF16 + 1) {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float2 f = __bfloat1622float2(__floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
      v[j] = f.x; v[j + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  }
  if (bias) {
    if (p.bias_dtype == BG_F32 && col0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(bias) & 15) == 0 && (col0 & 3) == 0) {
      const float4* b4 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(bias) + col0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 bb = __ldg(b4 + j);
        v[4 * j] = __fadd_rn(v[4 * j], bb.x);
        v[4 * j + 1] = __fadd_rn(v[4 * j + 1], bb.y);
        v[4 * j + 2] = __fadd_rn(v[4 * j + 2], bb.z);
        v[4 * j + 3] = __fadd_rn(v[4 * j + 3], bb.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] = __fadd_rn(v[j], load_bias(bias, p.bias_dtype, col0 + j));
    }
  }
  const bool full = col0 + 32 <= p.N;
  const size_t base = (size_t)row * p.N + col0;
  if ((SPLIT && p.planes_hi) || p.c_dtype == BG_F64) {
    // fp64 results and operand planes hold the fp32 value of the activation
    if (p.act == TC_ACT_RELU) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
    } else if (p.act == TC_ACT_GELU) {
      if (p.c_dtype == BG_F64) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_accurate(v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_graph<float>(v[j]);
      }
    }
  }
  if (SPLIT && p.planes_hi) {
    // the value the C store would have held (an fp32 value also when C is fp64), split as launch_tf32_split does
    float* hi = p.planes_hi + base;
    __nv_bfloat16* x16 = p.planes_16 + base;
    __nv_bfloat16* lo16 = x16 + (size_t)p.M * p.N;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (col0 + j + 8 > p.N) break;
      uint32_t wh[8], wx[4], wl[4];
      float xs[8], ls[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float x = v[j + t];
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(wh[t]) : "f"(x));
        xs[t] = x;
        ls[t] = __fadd_rn(x, -__uint_as_float(wh[t]));
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        __nv_bfloat162 a = __floats2bfloat162_rn(xs[2 * t], xs[2 * t + 1]), l = __floats2bfloat162_rn(ls[2 * t], ls[2 * t + 1]);
        wx[t] = *reinterpret_cast<uint32_t*>(&a);
        wl[t] = *reinterpret_cast<uint32_t*>(&l);
      }
      st_global_256(hi + j, wh);
      *reinterpret_cast<uint4*>(x16 + j) = make_uint4(wx[0], wx[1], wx[2], wx[3]);
      *reinterpret_cast<uint4*>(lo16 + j) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
    }
    return;
  }
  const bool al32 = (reinterpret_cast<uintptr_t>(C) & 31) == 0;      // 32-byte stores need the tensor to start on a sector
  if (p.c_dtype == BG_F64 && full && al32 && (p.N & 3) == 0) {
    double* out = reinterpret_cast<double*>(C) + base;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      uint32_t w[8];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const double x = (double)v[j + t];
        const unsigned long long b = (unsigned long long)__double_as_longlong(x);
        w[2 * t] = (uint32_t)b;
        w[2 * t + 1] = (uint32_t)(b >> 32);
      }
      st_global_256(out + j, w);
    }
    return;
  }
  if (p.c_dtype == BG_F64) {
    double* out = reinterpret_cast<double*>(C) + base;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      double w[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        w[t] = (double)v[j + t];
      }
      if (full && (p.N & 1) == 0) *reinterpret_cast<double2*>(out + j) = make_double2(w[0], w[1]);
      else {
        if (col0 + j < p.N) out[j] = w[0];
        if (col0 + j + 1 < p.N) out[j + 1] = w[1];
      }
    }
    return;
  }
  if (p.act == TC_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
  } else if (p.act == TC_ACT_GELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_graph<float>(v[j]);
  }
  if (p.c_dtype == BG_F32) {
    float* out = reinterpret_cast<float*>(C) + base;
    if (full && al32 && (p.N & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint32_t w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = __float_as_uint(v[j + t]);
        st_global_256(out + j, w);
      }
    } else if (full && (p.N & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) out[j] = v[j];
    }
  } else if (p.c_dtype == BG_F16) {
    __half* out = reinterpret_cast<__half*>(C) + base;
    if (full && al32 && (p.N & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 16) {
        uint32_t w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          __half2 h = __floats2half2_rn(v[j + 2 * t], v[j + 2 * t + 1]);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
        }
        st_global_256(out + j, w);
      }
    } else if (full && (p.N & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        __half2 h[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __floats2half2_rn(v[j + 2 * t], v[j + 2 * t + 1]);
        *reinterpret_cast<uint4*>(out + j) = *reinterpret_cast<uint4*>(h);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) out[j] = __float2half_rn(v[j]);
    }
  } else {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C) + base;
    if (full && al32 && (p.N & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 16) {
        uint32_t w[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[j + 2 * t], v[j + 2 * t + 1]);
          w[t] = *reinterpret_cast<uint32_t*>(&h);
        }
        st_global_256(out + j, w);
      }
    } else if (full && (p.N & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(v[j + 2 * t], v[j + 2 * t + 1]);
        *reinterpret_cast<uint4*>(out + j) = *reinterpret_cast<uint4*>(h);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) out[j] = __float2bfloat16_rn(v[j]);
    }
  }
}

// The tensor core adds into its fp32 accumulator with truncation, so a long K loop drifts by about
// 2^-24 of the accumulated magnitude per instruction (2e-5 relative at K = 8192 with three passes).  The
// 3xTF32 kernels therefore accumulate at most `chunk_blocks` K blocks in tensor memory; the epilogue warps
// add each partial sum into registers with round-to-nearest fp32 adds (one warp owns NC x 32 columns of 32
// rows) and apply the epilogue to the total.  `use` counts accumulator buffers consumed by this CTA.
// This warp owns the 32-column chunks first_chunk_col, first_chunk_col + chunk_stride, ... below n_cols_chunks.
template <int NC>
__device__ __forceinline__ bool drain_chunks(const TcParams& p, uint64_t* acc_full, uint32_t tmem_lane_base, int buf_cols, int first_chunk_col,
                                             int chunk_stride, int n_cols_chunks, int n_chunks, int& use, volatile int* abort_flag,
                                             float (&acc)[NC][32], int lane, uint32_t acc_empty_addr0, bool remote_arrive,
                                             uint64_t* acc_empty_local) {
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[c][j] = 0.f;
  for (int ch = 0; ch < n_chunks; ++ch, ++use) {
    const int buf = use & 1;
    if (!mbar_wait(&acc_full[buf], (uint32_t)(use >> 1) & 1u, abort_flag)) return false;
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int cc = first_chunk_col + c * chunk_stride;
      if (cc < n_cols_chunks) {          // the same for every lane of the warp
        uint32_t r[32];
        tmem_ld32(tmem_lane_base + (uint32_t)(buf * buf_cols + cc * 32), r);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c][j] = __fadd_rn(acc[c][j], __uint_as_float(r[j]));
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (remote_arrive) mbar_arrive_at(acc_empty_addr0 + (uint32_t)(buf * 8));
      else mbar_arrive(&acc_empty_local[buf]);
    }
  }
  return true;
}

// Persistent kernel: each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The accumulator is
// double-buffered in tensor memory, so the epilogue of tile t overlaps the MMAs of tile t + 1.
template <int BN, bool TF32>
__global__ void __launch_bounds__(EpiCfg<TF32>::kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmA2,
               const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
               const __grid_constant__ TcParams p) {
  constexpr int kABytes = BM * kStageRowBytes;
  constexpr int kBBytes = BN * kStageRowBytes;
  constexpr int kStageBytes = kABytes + kBBytes;
  constexpr int kStages = (BN == 256) ? 4 : 6;
  constexpr int kTmemCols = 2 * BN;   // two accumulators; a power of two >= 32

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;    // [2] MMAs of a tile have completed
  uint64_t* acc_empty = acc_full + 2;          // [2] the epilogue has drained the buffer
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int gsz = p.group_m * num_n;
  // tile id -> block coordinates: groups of `group_m` row blocks share their B column blocks in L2
  auto tile_origin = [&](int tile, int& m0, int& n0) {
    const int g = tile / gsz;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, num_m - first_m);
    m0 = (first_m + (tile % gsz) % gm) * BM;
    n0 = ((tile % gsz) / gm) * BN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EpiCfg<TF32>::kWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int n_chunks = p.num_k_blocks > 0 ? (p.num_k_blocks + p.chunk_blocks - 1) / p.chunk_blocks : 0;
  grid_dependency_wait();       // barriers and tensor memory are set up; nothing of global memory has been touched
  grid_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m0, n0;
        tile_origin(tile, m0, n0);
        for (int ch = 0; ch < n_chunks && ok; ++ch) {
          const int kb0 = ch * p.chunk_blocks, kb1 = min(kb0 + p.chunk_blocks, p.num_k_blocks);
          for (int pass = 0; pass < p.passes && ok; ++pass) {
            // passes of the split product: residual(A).B and A.residual(B) on bf16 planes (64 k per block), then
            // tf32(A).tf32(B) (32 k per block); a single pass uses map 0 of each operand
            const bool p16 = p.passes == 3 && p.mixed && pass < 2;
            const bool legacy = p.passes == 3 && !p.mixed;      // maps 1 hold the fp32 residual planes
            const CUtensorMap* ma = p16 ? (pass == 0 ? &tmA2 : &tmA1) : ((legacy && pass == 0) ? &tmA1 : &tmA0);
            const CUtensorMap* mb = p16 ? (pass == 0 ? &tmB1 : &tmB2) : ((legacy && pass == 1) ? &tmB1 : &tmB0);
            const int b0 = p16 ? kb0 >> 1 : kb0, b1 = p16 ? (kb1 + 1) >> 1 : kb1, per = p16 ? 64 : p.elems_per_block;
            for (int kb = b0; kb < b1; ++kb, ++it) {
              const int s = it % kStages;
              const uint32_t ph = (uint32_t)(it / kStages) & 1u;
              if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
              unsigned char* sa = smem + s * kStageBytes;
              mbar_expect_tx(&full_bar[s], kStageBytes);
              tma_load_2d(ma, sa, &full_bar[s], kb * per, m0);
              tma_load_2d(mb, sa + kABytes, &full_bar[s], kb * per, n0);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, use = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int ch = 0; ch < n_chunks && ok; ++ch, ++use) {
          const int buf = use & 1;
          if (!mbar_wait(&acc_empty[buf], ((uint32_t)(use >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
          const int kb0 = ch * p.chunk_blocks, kb1 = min(kb0 + p.chunk_blocks, p.num_k_blocks);
          uint32_t accumulate = 0;
          // stages of this chunk: two bf16 passes of ceil(blocks / 2) stages, then the tf32 pass (one pass otherwise)
          const int n16 = (p.passes == 3 && p.mixed) ? ((kb1 + 1) >> 1) - (kb0 >> 1) : 0;
          const int n_stage = p.passes == 3 ? (p.mixed ? 2 * n16 + (kb1 - kb0) : 3 * (kb1 - kb0)) : kb1 - kb0;
          for (int k = 0; k < n_stage; ++k, ++it) {
            const int s = it % kStages;
            const uint32_t ph = (uint32_t)(it / kStages) & 1u;
            if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * kStageBytes);
            const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + kABytes);
            const bool tf32 = TF32 && k >= 2 * n16;
#pragma unroll
            for (int kk = 0; kk < kStageRowBytes / 32; ++kk) {
              // each instruction consumes 32 bytes of K; the start address advances inside the swizzle row
              if (TF32) umma_sel(tmem_acc, da + (uint64_t)(kk * 32 >> 4), db + (uint64_t)(kk * 32 >> 4), tf32 ? p.idesc : p.idesc16, accumulate, tf32);
              else umma<false>(tmem_acc, da + (uint64_t)(kk * 32 >> 4), db + (uint64_t)(kk * 32 >> 4), p.idesc, accumulate);
              accumulate = 1;
            }
            umma_commit(&empty_bar[s]);
          }
          if (ok) umma_commit(&acc_full[buf]);
        }
      }
    }
  } else {
    // epilogue: warp w may read TMEM lanes 32*(w%4) .. +31; the two warps of a quarter split the columns
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int use = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m0, n0;
      tile_origin(tile, m0, n0);
      const int row = m0 + q * 32 + lane;
      const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
      if (TF32) {
        constexpr int kParts = EpiCfg<TF32>::kWarps / 4;
        constexpr int NC = (BN / 32 + kParts - 1) / kParts;
        float acc[NC][32];
        ok = drain_chunks<NC>(p, acc_full, lane_base, BN, half, kParts, BN / 32, n_chunks, use, abort_flag, acc, lane, 0u, false, acc_empty);
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int cc = half + c * kParts;
          const int col0 = n0 + cc * 32;
          if (cc < BN / 32 && row < p.M && col0 < p.N) epilogue_chunk<TF32>(p, reinterpret_cast<const uint32_t*>(acc[c]), row, col0, p.C, p.bias);
        }
      } else {
        const int buf = use & 1;
        if (n_chunks > 0) ok = mbar_wait(&acc_full[buf], (uint32_t)(use >> 1) & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = lane_base + (uint32_t)(buf * BN);
#pragma unroll 1
        for (int c = half; c < BN / 32; c += EpiCfg<TF32>::kWarps / 4) {      // the warps of a lane quarter take the 32-column chunks in turn
          uint32_t r[32];
          if (n_chunks > 0) tmem_ld32(tmem_acc + (uint32_t)(c * 32), r);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N) epilogue_chunk<TF32>(p, r, row, col0, p.C, p.bias);
        }
        // the buffer's values are in registers / memory: hand it back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && n_chunks > 0) mbar_arrive(&acc_empty[buf]);
        use += n_chunks;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out: report, give copies in flight time to land before shared memory is released
    if (threadIdx.x == 0) atomicExch(p.status, BG_ERR_DEVICE_TIMEOUT);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// CTA-pair variant: a cluster of two CTAs computes one 256 x 256 tile with tcgen05 cta_group::2.
// Each CTA stages its own 128 rows of A and its own 128 rows (output columns) of B, so a pair reads
// 64 KB of operands per K block where two independent 128 x 256 CTAs read 96 KB - the single-CTA
// kernel is limited by shared-memory fill from L2, not by the tensor pipe.  CTA 0 of the pair issues
// every MMA; the instruction reads both CTAs' shared memory and writes rows 0..127 of the tile into
// CTA 0's tensor memory and rows 128..255 into CTA 1's.  Barrier protocol (s = stage, b = buffer):
//   full[s]      lives in CTA 0; both producers arrive with their byte counts, both CTAs' copies
//                complete on it (count 2 + 64 KB);
//   empty[s]     one per CTA; CTA 0's MMA thread commits to its own and to CTA 1's;
//   acc_full[b]  one per CTA, committed the same way after a tile's last MMA;
//   acc_empty[b] lives in CTA 0; the sixteen epilogue warps of the pair arrive on it.
// The two CTAs meet at a cluster barrier after set-up and before tear-down, so no remote arrive or
// MMA ever targets a CTA that has exited.
constexpr int kPairStages = 6;

template <bool TF32, int TN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(EpiCfg<TF32>::kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmA2,
                    const __grid_constant__ PairBMaps tmB, const __grid_constant__ TcParams p) {
  constexpr int kHalf = 128;                           // rows of A each CTA stages
  constexpr int kBHalf = TN / 2;                       // rows of B each CTA stages
  constexpr int kABytes = kHalf * kStageRowBytes;
  constexpr int kStageBytes = kABytes + kBHalf * kStageRowBytes;
  constexpr int kTile = 256;                           // tile rows; the tile is kTile x TN
  constexpr int kTmemCols = TN > 128 ? 512 : 256;      // two accumulators of TN columns; a power of two

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kPairStages;
  uint64_t* acc_full = empty_bar + kPairStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + kTile - 1) / kTile, num_n1 = (p.N + TN - 1) / TN;
  const int num_n = num_n1 * p.n_prob;              // column tiles of all problems of the group, side by side
  const int num_tiles = num_m * num_n;
  const int gsz = p.group_m * num_n;
  auto tile_origin = [&](int tile, int& m0, int& n0, int& prob) {
    const int g = tile / gsz;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, num_m - first_m);
    m0 = (first_m + (tile % gsz) % gm) * kTile;
    const int nt = (tile % gsz) / gm;
    prob = nt / num_n1;
    n0 = (nt - prob * num_n1) * TN;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(&full_bar[s], 2); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * EpiCfg<TF32>::kWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // the same warp of both CTAs allocates; each CTA receives the same column range of its own tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int n_chunks = p.num_k_blocks > 0 ? (p.num_k_blocks + p.chunk_blocks - 1) / p.chunk_blocks : 0;
  grid_dependency_wait();       // barriers and tensor memory are set up; nothing of global memory has been touched
  grid_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m0, n0, prob;
        tile_origin(tile, m0, n0, prob);
        for (int ch = 0; ch < n_chunks && ok; ++ch) {
          const int kb0 = ch * p.chunk_blocks, kb1 = min(kb0 + p.chunk_blocks, p.num_k_blocks);
          for (int pass = 0; pass < p.passes && ok; ++pass) {
            // residual(A).B and A.residual(B) on bf16 planes (64 k per block), then tf32(A).tf32(B) (32 k per block)
            const bool p16 = p.passes == 3 && p.mixed && pass < 2;
            const bool legacy = p.passes == 3 && !p.mixed;      // maps 1 hold the fp32 residual planes
            const CUtensorMap* ma = p16 ? (pass == 0 ? &tmA2 : &tmA1) : ((legacy && pass == 0) ? &tmA1 : &tmA0);
            const CUtensorMap* mb = &tmB.m[3 * prob + (p16 ? (pass == 0 ? 1 : 2) : ((legacy && pass == 1) ? 1 : 0))];
            const int b0 = p16 ? kb0 >> 1 : kb0, b1 = p16 ? (kb1 + 1) >> 1 : kb1, per = p16 ? 64 : p.elems_per_block;
            for (int kb = b0; kb < b1; ++kb, ++it) {
              const int s = it % kPairStages;
              const uint32_t ph = (uint32_t)(it / kPairStages) & 1u;
              if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) { ok = false; break; }
              unsigned char* sa = smem + s * kStageBytes;
              const uint32_t full0 = map_to_cta(smem_u32(&full_bar[s]), 0);
              mbar_expect_tx_at(full0, kStageBytes);
              tma_load_2d_pair(ma, sa, full0, kb * per, m0 + (int)rank * kHalf);
              tma_load_2d_pair(mb, sa + kABytes, full0, kb * per, n0 + (int)rank * kBHalf);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      int it = 0, use = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        for (int ch = 0; ch < n_chunks && ok; ++ch, ++use) {
          const int buf = use & 1;
          if (!mbar_wait(&acc_empty[buf], ((uint32_t)(use >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * TN);
          const int kb0 = ch * p.chunk_blocks, kb1 = min(kb0 + p.chunk_blocks, p.num_k_blocks);
          uint32_t accumulate = 0;
          const int n16 = (p.passes == 3 && p.mixed) ? ((kb1 + 1) >> 1) - (kb0 >> 1) : 0;
          const int n_stage = p.passes == 3 ? (p.mixed ? 2 * n16 + (kb1 - kb0) : 3 * (kb1 - kb0)) : kb1 - kb0;
          for (int k = 0; k < n_stage; ++k, ++it) {
            const int s = it % kPairStages;
            const uint32_t ph = (uint32_t)(it / kPairStages) & 1u;
            if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * kStageBytes);
            const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + kABytes);
            const bool tf32 = TF32 && k >= 2 * n16;
#pragma unroll
            for (int kk = 0; kk < kStageRowBytes / 32; ++kk) {
              if (TF32) umma_pair_sel(tmem_acc, da + (uint64_t)(kk * 32 >> 4), db + (uint64_t)(kk * 32 >> 4), tf32 ? p.idesc : p.idesc16, accumulate, tf32);
              else umma_pair<false>(tmem_acc, da + (uint64_t)(kk * 32 >> 4), db + (uint64_t)(kk * 32 >> 4), p.idesc, accumulate);
              accumulate = 1;
            }
            const uint32_t e = smem_u32(&empty_bar[s]);
            umma_commit_pair(map_to_cta(e, 0));
            umma_commit_pair(map_to_cta(e, 1));
          }
          if (ok) {
            const uint32_t f = smem_u32(&acc_full[buf]);
            umma_commit_pair(map_to_cta(f, 0));
            umma_commit_pair(map_to_cta(f, 1));
          }
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int use = 0;
    bool ok = true;
    const uint32_t acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);   // the barriers live in CTA 0, 8 bytes apart
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int m0, n0, prob;
      tile_origin(tile, m0, n0, prob);
      void* const Cp = p.Cg[prob];
      const void* const biasp = p.biasg[prob];
      const int row = m0 + (int)rank * kHalf + q * 32 + lane;
      const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
      if (TF32) {
        constexpr int kParts = EpiCfg<TF32>::kWarps / 4;
        constexpr int NC = (TN / 32 + kParts - 1) / kParts;
        float acc[NC][32];
        ok = drain_chunks<NC>(p, acc_full, lane_base, TN, half, kParts, TN / 32, n_chunks, use, abort_flag, acc, lane, acc_empty0, true, nullptr);
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int cc = half + c * kParts;
          const int col0 = n0 + cc * 32;
          if (cc < TN / 32 && row < p.M && col0 < p.N) epilogue_chunk<TF32>(p, reinterpret_cast<const uint32_t*>(acc[c]), row, col0, Cp, biasp);
        }
      } else {
        const int buf = use & 1;
        if (n_chunks > 0) ok = mbar_wait(&acc_full[buf], (uint32_t)(use >> 1) & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_acc = lane_base + (uint32_t)(buf * TN);
#pragma unroll 1
        for (int c = half; c < TN / 32; c += EpiCfg<TF32>::kWarps / 4) {
          uint32_t r[32];
          if (n_chunks > 0) tmem_ld32(tmem_acc + (uint32_t)(c * 32), r);
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N) epilogue_chunk<TF32>(p, r, row, col0, Cp, biasp);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && n_chunks > 0) mbar_arrive_at(acc_empty0 + (uint32_t)(buf * 8));
        use += n_chunks;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, BG_ERR_DEVICE_TIMEOUT);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
    __syncthreads();
  }
  // both CTAs are past their last remote arrive / MMA before either frees tensor memory or exits
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// Rows of k elements can travel as bf16 planes when they start on 16-byte boundaries.
__host__ __device__ inline bool split_is_mixed(int64_t k) { return (k * 2) % 16 == 0; }

// The fp32 residual plane (lo = x - tf32(x)) for row lengths that cannot use bf16 planes: three tf32 passes.
__global__ void tf32_split_legacy_kernel(const void* src, int src_dtype, float* hi, float* lo, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float x;
    double xd = 0.0;
    if (src_dtype == BG_F64) { xd = reinterpret_cast<const double*>(src)[i]; x = (float)xd; }
    else x = reinterpret_cast<const float*>(src)[i];
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    const float fh = __uint_as_float(h);
    hi[i] = fh;
    lo[i] = src_dtype == BG_F64 ? (float)(xd - (double)fh) : __fadd_rn(x, -fh);
  }
}

// Planes of an operand of the split product, n elements each: hi = tf32(x) as fp32, then (in the 16-bit area)
// bf16(x) and bf16(x - hi).  x.y is computed as hi_x.hi_y on the tf32 path plus residual(x).bf16(y) and
// bf16(x).residual(y) on the bf16 path: the residual is below 2^-11 |x|, so the 2^-9 relative rounding of the bf16
// factors leaves about 2^-20 |x.y| per product -- the error level of an fp32 accumulation -- at two thirds of the
// tensor-pipe time of three tf32 passes (a bf16 instruction covers twice the k of a tf32 one).
__global__ void tf32_split_kernel(const void* src, int src_dtype, float* hi, __nv_bfloat16* x16, __nv_bfloat16* lo16, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float x;
    double xd = 0.0;
    if (src_dtype == BG_F64) { xd = reinterpret_cast<const double*>(src)[i]; x = (float)xd; }
    else x = reinterpret_cast<const float*>(src)[i];
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    const float fh = __uint_as_float(h);
    hi[i] = fh;
    x16[i] = __float2bfloat16_rn(x);
    // the residual is exact in fp32; for fp64 sources it also carries the bits fp32 dropped
    lo16[i] = __float2bfloat16_rn(src_dtype == BG_F64 ? (float)(xd - (double)fh) : __fadd_rn(x, -fh));
  }
}

// The same for a dense fp32 or float64 source whose length is a multiple of 4: 16-byte loads and stores.
template <typename S>
__global__ void tf32_split4_kernel(const S* __restrict__ src, float4* __restrict__ hi, uint2* __restrict__ x16, uint2* __restrict__ lo16,
                                   int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    double xd[4];
    float xs[4];
    if (sizeof(S) == 8) {
      const double2 a = __ldcs(reinterpret_cast<const double2*>(src) + 2 * i), b = __ldcs(reinterpret_cast<const double2*>(src) + 2 * i + 1);
      xd[0] = a.x; xd[1] = a.y; xd[2] = b.x; xd[3] = b.y;
    } else {
      const float4 x = __ldcs(reinterpret_cast<const float4*>(src) + i);
      xd[0] = x.x; xd[1] = x.y; xd[2] = x.z; xd[3] = x.w;
    }
    float hs[4], ls[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      xs[e] = (float)xd[e];
      uint32_t h;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(xs[e]));
      hs[e] = __uint_as_float(h);
      // for float64 sources the residual also carries the bits fp32 dropped
      ls[e] = sizeof(S) == 8 ? (float)(xd[e] - (double)hs[e]) : __fadd_rn(xs[e], -hs[e]);
    }
    hi[i] = make_float4(hs[0], hs[1], hs[2], hs[3]);
    __nv_bfloat162 a0 = __floats2bfloat162_rn(xs[0], xs[1]), a1 = __floats2bfloat162_rn(xs[2], xs[3]);
    __nv_bfloat162 l0 = __floats2bfloat162_rn(ls[0], ls[1]), l1 = __floats2bfloat162_rn(ls[2], ls[3]);
    x16[i] = make_uint2(*reinterpret_cast<uint32_t*>(&a0), *reinterpret_cast<uint32_t*>(&a1));
    lo16[i] = make_uint2(*reinterpret_cast<uint32_t*>(&l0), *reinterpret_cast<uint32_t*>(&l1));
  }
}

template <typename S>
__global__ void convert16_kernel(const S* __restrict__ src, void* dst, int64_t n, int bf16) {
  const int64_t n8 = n >> 3;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    float4 a, b;
    if (sizeof(S) == 8) {
      // float64 source: rounded to fp32 first and then to the 16-bit type, as the interpreter's CAST does
      const double2* q = reinterpret_cast<const double2*>(src) + 4 * i;
      const double2 d0 = __ldcs(q), d1 = __ldcs(q + 1), d2 = __ldcs(q + 2), d3 = __ldcs(q + 3);
      a = make_float4((float)d0.x, (float)d0.y, (float)d1.x, (float)d1.y);
      b = make_float4((float)d2.x, (float)d2.y, (float)d3.x, (float)d3.y);
    } else {
      a = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i);
      b = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    }
    uint32_t w[4];
    if (bf16) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
      w[0] = *reinterpret_cast<uint32_t*>(&p0); w[1] = *reinterpret_cast<uint32_t*>(&p1);
      w[2] = *reinterpret_cast<uint32_t*>(&p2); w[3] = *reinterpret_cast<uint32_t*>(&p3);
    } else {
      __half2 p0 = __floats2half2_rn(a.x, a.y), p1 = __floats2half2_rn(a.z, a.w);
      __half2 p2 = __floats2half2_rn(b.x, b.y), p3 = __floats2half2_rn(b.z, b.w);
      w[0] = *reinterpret_cast<uint32_t*>(&p0); w[1] = *reinterpret_cast<uint32_t*>(&p1);
      w[2] = *reinterpret_cast<uint32_t*>(&p2); w[3] = *reinterpret_cast<uint32_t*>(&p3);
    }
    reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // ragged end
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const int64_t i = (n8 << 3) + threadIdx.x;
    if (bf16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn((float)src[i]);
    else reinterpret_cast<__half*>(dst)[i] = __float2half_rn((float)src[i]);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// [rows, K] row-major operand, box = one 128-byte swizzle row x box_rows; out-of-range elements read as zero.
bool make_operand_map(CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int es = dtype_size(dtype);
  CUtensorMapDataType dt = dtype == BG_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : dtype == BG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * es};
  cuuint32_t box[2] = {(cuuint32_t)(kStageRowBytes / es), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool TF32>
cudaError_t launch_variant(const TcGemm& g, int* status, cudaStream_t s) {
  CUtensorMap a0, a1, a2, b0, b1, b2;
  if (!make_operand_map(&a0, g.A, g.ab_dtype, g.M, g.K, BM)) return cudaErrorInvalidValue;
  if (!make_operand_map(&b0, g.B, g.ab_dtype, g.N, g.K, BN)) return cudaErrorInvalidValue;
  a1 = a2 = a0;
  b1 = b2 = b0;
  const bool mixed = TF32 && split_is_mixed(g.K);
  if (mixed) {
    // the 16-bit area of a split operand: the bf16 plane, then the bf16 residual plane
    const char* a16 = reinterpret_cast<const char*>(g.A_lo);
    const char* b16 = reinterpret_cast<const char*>(g.B_lo);
    if (!make_operand_map(&a1, a16, BG_BF16, g.M, g.K, BM)) return cudaErrorInvalidValue;
    if (!make_operand_map(&a2, a16 + g.M * g.K * 2, BG_BF16, g.M, g.K, BM)) return cudaErrorInvalidValue;
    if (!make_operand_map(&b1, b16, BG_BF16, g.N, g.K, BN)) return cudaErrorInvalidValue;
    if (!make_operand_map(&b2, b16 + g.N * g.K * 2, BG_BF16, g.N, g.K, BN)) return cudaErrorInvalidValue;
  } else if (TF32) {
    if (!make_operand_map(&a1, g.A_lo, g.ab_dtype, g.M, g.K, BM)) return cudaErrorInvalidValue;
    if (!make_operand_map(&b1, g.B_lo, g.ab_dtype, g.N, g.K, BN)) return cudaErrorInvalidValue;
  }
  TcParams p{};
  p.M = (int)g.M;
  p.N = (int)g.N;
  const int es = dtype_size(g.ab_dtype);
  p.elems_per_block = kStageRowBytes / es;
  p.num_k_blocks = (int)((g.K + p.elems_per_block - 1) / p.elems_per_block);
  p.passes = TF32 ? 3 : 1;
  p.chunk_blocks = TF32 ? (p.num_k_blocks < kTf32ChunkBlocks ? (p.num_k_blocks > 0 ? p.num_k_blocks : 1) : kTf32ChunkBlocks) : (p.num_k_blocks > 0 ? p.num_k_blocks : 1);
  p.C = g.C;
  p.c_dtype = g.c_dtype;
  p.bias = g.bias;
  p.bias_dtype = g.bias_dtype;
  p.act = g.act;
  p.round_acc = g.round_acc;
  p.wide = g.wide;
  p.status = status;
  p.planes_hi = reinterpret_cast<float*>(g.planes_hi);
  p.planes_16 = reinterpret_cast<__nv_bfloat16*>(g.planes_lo);
  p.group_m = 8;
  const uint32_t fmt = TF32 ? 2u : (g.ab_dtype == BG_BF16 ? 1u : 0u);
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  p.idesc16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  p.mixed = mixed ? 1 : 0;
  constexpr int kStages = (BN == 256) ? 4 : 6;
  const size_t smem = (size_t)kStages * (BM + BN) * kStageRowBytes + 256 + 1024;
  auto kern = gemm_tc_kernel<BN, TF32>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int64_t tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t grid = tiles < sms ? tiles : sms;
  return launch_dependent(kern, dim3((unsigned)grid), dim3(EpiCfg<TF32>::kThreads), smem, s, a0, a1, a2, b0, b1, b2, p);
}

template <bool TF32, int TN>
cudaError_t launch_pair(const TcGemm* gs, int n_prob, int* status, cudaStream_t s, bool* launched) {
  *launched = false;
  const TcGemm& g = gs[0];
  CUtensorMap a0, a1, a2;
  PairBMaps bm;
  if (!make_operand_map(&a0, g.A, g.ab_dtype, g.M, g.K, 128)) return cudaErrorInvalidValue;
  a1 = a2 = a0;
  const bool mixed = TF32 && split_is_mixed(g.K);
  if (mixed) {
    const char* a16 = reinterpret_cast<const char*>(g.A_lo);     // bf16 plane, then bf16 residual plane
    if (!make_operand_map(&a1, a16, BG_BF16, g.M, g.K, 128)) return cudaErrorInvalidValue;
    if (!make_operand_map(&a2, a16 + g.M * g.K * 2, BG_BF16, g.M, g.K, 128)) return cudaErrorInvalidValue;
  } else if (TF32) {
    if (!make_operand_map(&a1, g.A_lo, g.ab_dtype, g.M, g.K, 128)) return cudaErrorInvalidValue;
  }
  for (int i = 0; i < kMaxGroup; ++i) {
    const TcGemm& gi = gs[i < n_prob ? i : 0];
    if (!make_operand_map(&bm.m[3 * i], gi.B, gi.ab_dtype, gi.N, gi.K, TN / 2)) return cudaErrorInvalidValue;
    bm.m[3 * i + 1] = bm.m[3 * i + 2] = bm.m[3 * i];
    if (mixed) {
      const char* b16 = reinterpret_cast<const char*>(gi.B_lo);
      if (!make_operand_map(&bm.m[3 * i + 1], b16, BG_BF16, gi.N, gi.K, TN / 2)) return cudaErrorInvalidValue;
      if (!make_operand_map(&bm.m[3 * i + 2], b16 + gi.N * gi.K * 2, BG_BF16, gi.N, gi.K, TN / 2)) return cudaErrorInvalidValue;
    } else if (TF32) {
      if (!make_operand_map(&bm.m[3 * i + 1], gi.B_lo, gi.ab_dtype, gi.N, gi.K, TN / 2)) return cudaErrorInvalidValue;
    }
  }
  TcParams p{};
  p.M = (int)g.M;
  p.N = (int)g.N;
  const int es = dtype_size(g.ab_dtype);
  p.elems_per_block = kStageRowBytes / es;
  p.num_k_blocks = (int)((g.K + p.elems_per_block - 1) / p.elems_per_block);
  p.passes = TF32 ? 3 : 1;
  p.chunk_blocks = TF32 ? (p.num_k_blocks < kTf32ChunkBlocks ? (p.num_k_blocks > 0 ? p.num_k_blocks : 1) : kTf32ChunkBlocks) : (p.num_k_blocks > 0 ? p.num_k_blocks : 1);
  p.C = g.C;
  p.c_dtype = g.c_dtype;
  p.bias = g.bias;
  p.bias_dtype = g.bias_dtype;
  p.act = g.act;
  p.round_acc = g.round_acc;
  p.wide = g.wide;
  p.status = status;
  p.planes_hi = reinterpret_cast<float*>(g.planes_hi);
  p.planes_16 = reinterpret_cast<__nv_bfloat16*>(g.planes_lo);
  p.group_m = 4;
  p.n_prob = n_prob;
  for (int i = 0; i < kMaxGroup; ++i) { p.Cg[i] = gs[i < n_prob ? i : 0].C; p.biasg[i] = gs[i < n_prob ? i : 0].bias; }
  const uint32_t fmt = TF32 ? 2u : (g.ab_dtype == BG_BF16 ? 1u : 0u);
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  p.idesc16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  p.mixed = mixed ? 1 : 0;
  const size_t smem = (size_t)kPairStages * (128 + TN / 2) * kStageRowBytes + 256 + 1024;
  auto kern = gemm_tc_pair_kernel<TF32, TN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  // how many pairs the device can hold at once (two SMs of one TPC each)
  static int max_pairs = -1;
  if (max_pairs < 0) {
    cudaLaunchConfig_t qc{};
    qc.gridDim = dim3(2, 1, 1);
    qc.blockDim = dim3(EpiCfg<TF32>::kThreads, 1, 1);
    qc.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    qc.attrs = &attr;
    qc.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &qc) != cudaSuccess) { cudaGetLastError(); n = 0; }
    max_pairs = n;
  }
  if (max_pairs <= 0) return cudaSuccess;   // not launched: the caller falls back to single CTAs
  const int64_t tiles = ((g.M + 255) / 256) * ((g.N + TN - 1) / TN) * n_prob;
  const int64_t pairs = tiles < max_pairs ? tiles : max_pairs;
  *launched = true;
  return launch_dependent(kern, dim3((unsigned)(2 * pairs)), dim3(EpiCfg<TF32>::kThreads), smem, s, a0, a1, a2, bm, p);
}

}  // namespace

bool g_tc_assume_available = false;

bool tc_gemm_supported(int64_t M, int64_t N, int64_t K, int ab_dtype) {
  if (!g_tc_assume_available && !encode_fn()) return false;
  if (ab_dtype != BG_F16 && ab_dtype != BG_BF16 && ab_dtype != BG_F32) return false;
  const int es = dtype_size(ab_dtype);
  if (M <= 0 || N <= 0 || K <= 0) return false;
  if ((K * es) % 16 != 0) return false;                 // TMA row pitch
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return false;
  return true;
}

int g_dependent_launch = 1;
int g_tc_pair_mode = 1;   // 0: never, 1: when the problem fills the device with 256 x 256 tiles, 2: whenever legal

// Width of the CTA-pair tile (256 rows x TN columns).  A pair works through ceil(tiles / pairs) tiles one
// after the other; a tile costs about TN + 64 (the A half of every stage does not shrink with TN), so a
// narrower tile wins when it removes a mostly idle last round: M = 8192, N = 768 is 96 tiles of 256 columns
// (two rounds on 74 pairs, the second a third full) but 128 tiles of 192 columns (two shorter rounds).  A tile of
// the split product carries a larger cost that does not shrink with its width (the folds of its accumulation chunks
// and its final epilogue by the same warps): TN + 256 reproduces the measured order of the widths on the decoder's
// shapes ([8192, 768] x 768 / 2304 / 3072 and 4096^3), where TN + 64 chose 192 columns for N = 3072 (202 us against 192).
static int pair_tile_width(int64_t M, int64_t N, int pairs, bool split, int n_prob = 1) {
  int best = 256;
  int64_t best_cost = -1;
  const int widths[3] = {256, 192, 128};
  for (int w : widths) {
    const int64_t tiles = ((M + 255) / 256) * ((N + w - 1) / w) * n_prob;
    const int64_t rounds = (tiles + pairs - 1) / pairs;
    const int64_t cost = rounds * (w + (split ? 256 : 64));
    if (best_cost < 0 || cost < best_cost) { best = w; best_cost = cost; }
  }
  return best;
}

template <bool TF32>
static cudaError_t launch_pair_width(int tn, const TcGemm* gs, int n_prob, int* status, cudaStream_t s, bool* launched) {
  if (tn == 192) return launch_pair<TF32, 192>(gs, n_prob, status, s, launched);
  if (tn == 128) return launch_pair<TF32, 128>(gs, n_prob, status, s, launched);
  return launch_pair<TF32, 256>(gs, n_prob, status, s, launched);
}

int g_tc_pair_width = 0;   // 0: chosen by pair_tile_width; 256 / 192 / 128: forced

// Problems that share A, the shape and the epilogue kind (checked by the caller) as one launch of the CTA-pair
// kernel: their column tiles lie side by side, so the last round of the grid is shared (three N = 768
// projections: 3 x 2 rounds alone, 4 rounds together).  Falls back to one launch per problem.
cudaError_t launch_gemm_tc_group(const TcGemm* gs, int n_prob, int* status, cudaStream_t s) {
  if (n_prob < 1 || n_prob > kMaxGroup) return cudaErrorInvalidValue;
  const TcGemm& g = gs[0];
  const bool tf32 = g.ab_dtype == BG_F32;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (n_prob > 1 && g.M > 128 && g.N > 128 && g_tc_pair_mode != 0) {
    bool launched = false;
    const int tn = g_tc_pair_width ? g_tc_pair_width : pair_tile_width(g.M, g.N, sms / 2, tf32, n_prob);
    {
      cudaError_t e = tf32 ? launch_pair_width<true>(tn, gs, n_prob, status, s, &launched) : launch_pair_width<false>(tn, gs, n_prob, status, s, &launched);
      if (e != cudaSuccess || launched) return e;
    }
  }
  for (int i = 0; i < n_prob; ++i) {
    cudaError_t e = launch_gemm_tc(gs[i], status, s);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_gemm_tc(const TcGemm& g, int* status, cudaStream_t s) {
  const bool tf32 = g.ab_dtype == BG_F32;
  const int64_t tiles256 = ((g.M + 255) / 256) * ((g.N + 255) / 256);
  const bool pair_ok = g.M > 128 && g.N > 128;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (pair_ok && (g_tc_pair_mode == 2 || (g_tc_pair_mode == 1 && tiles256 >= 64))) {
    bool launched = false;
    const int tn = g_tc_pair_width ? g_tc_pair_width : pair_tile_width(g.M, g.N, sms / 2, tf32);
    cudaError_t e = tf32 ? launch_pair_width<true>(tn, &g, 1, status, s, &launched) : launch_pair_width<false>(tn, &g, 1, status, s, &launched);
    if (e != cudaSuccess || launched) return e;
  }
  // 128 x 256 tiles halve the B traffic per flop; 128 x 128 tiles when the wide ones would leave SMs idle
  const int64_t wide_tiles = ((g.M + BM - 1) / BM) * ((g.N + 255) / 256);
  const bool wide_tile = g.N > 128 && wide_tiles >= sms;
  if (tf32) return wide_tile ? launch_variant<256, true>(g, status, s) : launch_variant<128, true>(g, status, s);
  return wide_tile ? launch_variant<256, false>(g, status, s) : launch_variant<128, false>(g, status, s);
}

cudaError_t launch_convert16(const void* src, int src_dtype, void* dst, int64_t n, int dtype16, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  // vector path needs 32-byte aligned source and 16-byte aligned destination; slots and handles are 256-byte aligned,
  // view offsets inside them need not be
  if ((reinterpret_cast<uintptr_t>(src) & 31) || (reinterpret_cast<uintptr_t>(dst) & 15)) return cudaErrorInvalidValue;
  int64_t grid = (n / 8 + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) grid = 1;
  if (src_dtype == BG_F64)
    convert16_kernel<double><<<(unsigned)grid, 256, 0, s>>>(reinterpret_cast<const double*>(src), dst, n, dtype16 == BG_BF16 ? 1 : 0);
  else
    convert16_kernel<float><<<(unsigned)grid, 256, 0, s>>>(reinterpret_cast<const float*>(src), dst, n, dtype16 == BG_BF16 ? 1 : 0);
  return cudaGetLastError();
}

// `lo` (n fp32 slots) receives, for rows of k elements that can travel as bf16, the bf16 plane and then the bf16 residual
// plane; otherwise the fp32 residual plane.
cudaError_t launch_tf32_split(const void* src, int src_dtype, float* hi, float* lo, int64_t n, int64_t k, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (!split_is_mixed(k)) {
    int64_t grid = (n + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    tf32_split_legacy_kernel<<<(unsigned)grid, 256, 0, s>>>(src, src_dtype, hi, lo, n);
    return cudaGetLastError();
  }
  __nv_bfloat16* x16 = reinterpret_cast<__nv_bfloat16*>(lo);
  __nv_bfloat16* lo16 = x16 + n;
  const bool vec = (src_dtype == BG_F32 || src_dtype == BG_F64) && n % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(hi)) & 15) == 0 &&
                   ((reinterpret_cast<uintptr_t>(x16) | reinterpret_cast<uintptr_t>(lo16)) & 7) == 0;
  if (vec) {
    int64_t grid = (n / 4 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    if (src_dtype == BG_F64)
      tf32_split4_kernel<double><<<(unsigned)grid, 256, 0, s>>>(reinterpret_cast<const double*>(src), reinterpret_cast<float4*>(hi),
                                                                reinterpret_cast<uint2*>(x16), reinterpret_cast<uint2*>(lo16), n / 4);
    else
      tf32_split4_kernel<float><<<(unsigned)grid, 256, 0, s>>>(reinterpret_cast<const float*>(src), reinterpret_cast<float4*>(hi),
                                                               reinterpret_cast<uint2*>(x16), reinterpret_cast<uint2*>(lo16), n / 4);
    return cudaGetLastError();
  }
  int64_t grid = (n + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  tf32_split_kernel<<<(unsigned)grid, 256, 0, s>>>(src, src_dtype, hi, x16, lo16, n);
  return cudaGetLastError();
}

// One CTA waits, with the bounded wait every tensor-core kernel uses, on a barrier that nothing ever arrives on, and
// reports the give-up through the status word exactly as those kernels do: the host-visible half of the protocol
// (status word -> BG_ERR_DEVICE_TIMEOUT, context usable afterwards) can be exercised without a fault.
__global__ void wait_timeout_selftest_kernel(long long limit_cycles, int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) tc::mbar_wait(&bar, 0, &abort_flag, limit_cycles);
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) atomicExch(status, BG_ERR_DEVICE_TIMEOUT);
}

cudaError_t launch_wait_timeout_selftest(long long limit_cycles, int* status, cudaStream_t s) {
  wait_timeout_selftest_kernel<<<1, 32, 0, s>>>(limit_cycles, status);
  return cudaGetLastError();
}

}  // namespace bg
