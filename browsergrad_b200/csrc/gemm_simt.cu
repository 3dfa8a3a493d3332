// SIMT GEMM for the operand types and shapes the tensor-core kernels do not take:
// fp64 (DFMA), exact int64, tiny or unaligned problems, arbitrary operand strides and
// broadcast batch dimensions.  64x64 output tile per CTA, 16-deep k slabs staged in shared
// memory, 4x4 outputs per thread.  fp16/bf16 inputs accumulate in fp32 as the reference's
// matmul does (packages/browsergrad-jit/src/python/_realize.py:395-410).
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace bg {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T> __device__ __forceinline__ T load_elem(const void* p, int dt, int64_t i);
template <> __device__ __forceinline__ float load_elem<float>(const void* p, int dt, int64_t i) {
  switch (dt) {
    case BG_F32: return reinterpret_cast<const float*>(p)[i];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case BG_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case BG_F64: return (float)reinterpret_cast<const double*>(p)[i];
    default: return 0.f;
  }
}
template <> __device__ __forceinline__ double load_elem<double>(const void* p, int dt, int64_t i) {
  switch (dt) {
    case BG_F64: return reinterpret_cast<const double*>(p)[i];
    case BG_F32: return reinterpret_cast<const float*>(p)[i];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case BG_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case BG_I64: return (double)reinterpret_cast<const long long*>(p)[i];
    case BG_I32: return (double)reinterpret_cast<const int*>(p)[i];
    default: return 0.0;
  }
}
template <> __device__ __forceinline__ long long load_elem<long long>(const void* p, int dt, int64_t i) {
  switch (dt) {
    case BG_I64: case BG_U64: return reinterpret_cast<const long long*>(p)[i];
    case BG_I32: return reinterpret_cast<const int*>(p)[i];
    case BG_U32: return reinterpret_cast<const unsigned*>(p)[i];
    case BG_I16: return reinterpret_cast<const short*>(p)[i];
    case BG_U16: return reinterpret_cast<const unsigned short*>(p)[i];
    case BG_I8: return reinterpret_cast<const signed char*>(p)[i];
    default: return reinterpret_cast<const unsigned char*>(p)[i];
  }
}

template <typename T> __device__ __forceinline__ void store_elem(void* p, int dt, int64_t i, T v);
template <> __device__ __forceinline__ void store_elem<float>(void* p, int dt, int64_t i, float v) {
  switch (dt) {
    case BG_F32: reinterpret_cast<float*>(p)[i] = v; break;
    case BG_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case BG_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    default: reinterpret_cast<double*>(p)[i] = v; break;
  }
}
template <> __device__ __forceinline__ void store_elem<double>(void* p, int dt, int64_t i, double v) {
  if (dt == BG_F64) reinterpret_cast<double*>(p)[i] = v;
  else reinterpret_cast<float*>(p)[i] = (float)v;
}
template <> __device__ __forceinline__ void store_elem<long long>(void* p, int dt, int64_t i, long long v) {
  switch (dt) {
    case BG_I64: case BG_U64: reinterpret_cast<long long*>(p)[i] = v; break;
    case BG_I32: case BG_U32: reinterpret_cast<int*>(p)[i] = (int)v; break;
    case BG_I16: case BG_U16: reinterpret_cast<short*>(p)[i] = (short)v; break;
    default: reinterpret_cast<signed char*>(p)[i] = (signed char)v; break;
  }
}

template <typename T> __device__ __forceinline__ T mad(T a, T b, T c) { return a * b + c; }
template <> __device__ __forceinline__ float mad<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double mad<double>(double a, double b, double c) { return fma(a, b, c); }
template <> __device__ __forceinline__ long long mad<long long>(long long a, long long b, long long c) {
  return (long long)((unsigned long long)a * (unsigned long long)b + (unsigned long long)c);
}

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const __grid_constant__ GemmProblem p) {
  __shared__ T As[TK][TM + 1];
  __shared__ T Bs[TK][TN + 1];
  // batch offsets
  int64_t bz = blockIdx.z, a_off = 0, b_off = 0;
  for (int d = p.n_batch_dims - 1; d >= 0; --d) {
    int64_t q = bz / p.batch_shape[d];
    int64_t c = bz - q * p.batch_shape[d];
    bz = q;
    a_off += c * p.a.batch_stride[d];
    b_off += c * p.b.batch_stride[d];
  }
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = T(0);
  for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      // pick the loop order that walks the operand's unit stride fastest
      int mm, kk;
      if (p.a.col_stride == 1) { kk = i % TK; mm = i / TK; } else { mm = i % TM; kk = i / TM; }
      int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < p.m && k < p.k) ? load_elem<T>(p.a.ptr, p.a.dtype, a_off + m * p.a.row_stride + k * p.a.col_stride) : T(0);
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      int nn, kk;
      if (p.b.col_stride == 1) { nn = i % TN; kk = i / TN; } else { kk = i % TK; nn = i / TK; }
      int64_t n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < p.n && k < p.k) ? load_elem<T>(p.b.ptr, p.b.dtype, b_off + k * p.b.row_stride + n * p.b.col_stride) : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = mad<T>(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  const int64_t c_off = (int64_t)blockIdx.z * p.m * p.n;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < p.n) store_elem<T>(p.c, p.c_dtype, c_off + m * p.n + n, acc[i][j]);
    }
  }
}

// ------------------------------------------------------------------------------------
// Small fp32 problems: split-K over many CTAs, bias and ReLU folded
// ------------------------------------------------------------------------------------
// A 2-D fp32 product too small for the tensor-core kernels (a few MFLOP) is latency: the 64x64 tiling above gives it
// one or two CTAs that walk all of K.  Here a CTA owns a 32x32 output tile and one slice of K, so a [64,784].[784,128]
// product runs on 128 CTAs of 49 k each.  Every CTA writes its partial tile; the CTA that arrives last at the tile's
// counter adds the partials in slice order (the same order whichever CTA it is), applies bias / ReLU and stores.  The
// counters live in the context, start at zero and are set back to zero by that last CTA.
constexpr int SM_T = 32;          // tile edge
constexpr int SM_KC = 64;         // largest K slice held in shared memory

__global__ void __launch_bounds__(256) gemm_small_kernel(const __grid_constant__ GemmProblem p, const float* __restrict__ bias, int act,
                                                         float* __restrict__ partials, int* __restrict__ counters, int kc) {
  __shared__ float As[SM_KC][SM_T + 1];
  __shared__ float Bs[SM_KC][SM_T + 1];
  __shared__ int s_last;
  grid_dependency_wait();
  grid_launch_dependents();
  const int splits = gridDim.z;
  const int64_t m0 = (int64_t)blockIdx.y * SM_T, n0 = (int64_t)blockIdx.x * SM_T;
  const int64_t k0 = (int64_t)blockIdx.z * kc;
  const int64_t k1 = k0 + kc < p.k ? k0 + kc : p.k;
  const int klen = (int)(k1 - k0);
  const float* A = reinterpret_cast<const float*>(p.a.ptr);
  const float* B = reinterpret_cast<const float*>(p.b.ptr);
  for (int i = threadIdx.x; i < SM_T * klen; i += 256) {
    int mm, kk;
    if (p.a.col_stride == 1) { kk = i % klen; mm = i / klen; } else { mm = i % SM_T; kk = i / SM_T; }
    const int64_t m = m0 + mm;
    As[kk][mm] = m < p.m ? A[m * p.a.row_stride + (k0 + kk) * p.a.col_stride] : 0.f;
  }
  for (int i = threadIdx.x; i < SM_T * klen; i += 256) {
    int nn, kk;
    if (p.b.col_stride == 1) { nn = i % SM_T; kk = i / SM_T; } else { kk = i % klen; nn = i / klen; }
    const int64_t n = n0 + nn;
    Bs[kk][nn] = n < p.n ? B[(k0 + kk) * p.b.row_stride + n * p.b.col_stride] : 0.f;
  }
  __syncthreads();
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll 4
  for (int kk = 0; kk < klen; ++kk) {
    const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1], b0 = Bs[kk][tx * 2], b1 = Bs[kk][tx * 2 + 1];
    acc[0][0] = fmaf(a0, b0, acc[0][0]);
    acc[0][1] = fmaf(a0, b1, acc[0][1]);
    acc[1][0] = fmaf(a1, b0, acc[1][0]);
    acc[1][1] = fmaf(a1, b1, acc[1][1]);
  }
  float* C = reinterpret_cast<float*>(p.c);
  auto finish = [&](int i, int j, float v) {
    const int64_t m = m0 + ty * 2 + i, n = n0 + tx * 2 + j;
    if (m >= p.m || n >= p.n) return;
    if (bias) v = __fadd_rn(v, bias[n]);
    if (act == TC_ACT_RELU) v = v > 0.f ? v : 0.f;
    C[m * p.n + n] = v;
  };
  if (splits == 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) finish(i, j, acc[i][j]);
    return;
  }
  const int tile = blockIdx.y * gridDim.x + blockIdx.x;
  const int n_tiles = gridDim.x * gridDim.y;
  // partials[slice][tile][32 x 32]
  float* mine = partials + ((int64_t)blockIdx.z * n_tiles + tile) * (SM_T * SM_T);
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) mine[(ty * 2 + i) * SM_T + tx * 2 + j] = acc[i][j];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&counters[tile], 1) == splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float v = 0.f;
      const float* q = partials + (int64_t)tile * (SM_T * SM_T) + (ty * 2 + i) * SM_T + tx * 2 + j;
      const int64_t zs = (int64_t)n_tiles * (SM_T * SM_T);
      // eight loads in flight, added in slice order
      for (int z0 = 0; z0 < splits; z0 += 8) {
        float t[8];
#pragma unroll
        for (int z = 0; z < 8; ++z) t[z] = z0 + z < splits ? __ldcg(q + (z0 + z) * zs) : 0.f;
#pragma unroll
        for (int z = 0; z < 8; ++z)
          if (z0 + z < splits) v = __fadd_rn(v, t[z]);
      }
      finish(i, j, v);
    }
  if (threadIdx.x == 0) counters[tile] = 0;
}

}  // namespace

bool gemm_small_plan(const GemmProblem& p, int sm_count, int* splits, int64_t* partial_bytes) {
  if (p.n_batch_dims != 0 || p.c_dtype != BG_F32 || p.a.dtype != BG_F32 || p.b.dtype != BG_F32) return false;
  if (p.m < 1 || p.n < 1 || p.k < 32) return false;
  const int64_t tiles = ((p.m + SM_T - 1) / SM_T) * ((p.n + SM_T - 1) / SM_T);
  if (tiles > 1024 || tiles > 2 * (int64_t)sm_count) return false;   // enough tiles to fill the GPU: the 64x64 kernel does
  int64_t want = (2 * (int64_t)sm_count + tiles - 1) / tiles;        // about two CTAs per SM in all
  const int64_t most = (p.k + 31) / 32;                              // slices of at least 32 k
  if (want > most) want = most;
  const int64_t least = (p.k + SM_KC - 1) / SM_KC;                   // a slice has to fit the shared-memory slab
  if (want < least) want = least;
  if (want > 65535) return false;
  int64_t kc = (p.k + want - 1) / want;
  want = (p.k + kc - 1) / kc;
  if (kc > SM_KC) return false;
  *splits = (int)want;
  *partial_bytes = want > 1 ? want * tiles * SM_T * SM_T * 4 : 0;
  if (*partial_bytes > ((int64_t)64 << 20)) return false;
  return true;
}

cudaError_t launch_gemm_small(const GemmProblem& p, const void* bias, int act, void* partials, int* counters, int splits, cudaStream_t s) {
  const int64_t kc = (p.k + splits - 1) / splits;
  dim3 grid((unsigned)((p.n + SM_T - 1) / SM_T), (unsigned)((p.m + SM_T - 1) / SM_T), (unsigned)splits);
  return launch_dependent(gemm_small_kernel, grid, dim3(256), 0, s, p, reinterpret_cast<const float*>(bias), act,
                          reinterpret_cast<float*>(partials), counters, (int)kc);
}

cudaError_t launch_gemm_simt(const GemmProblem& p, cudaStream_t s) {
  int64_t nb = 1;
  for (int d = 0; d < p.n_batch_dims; ++d) nb *= p.batch_shape[d];
  if (p.m == 0 || p.n == 0 || nb == 0) return cudaSuccess;
  if (nb > 65535 || (p.m + TM - 1) / TM > 65535) return cudaErrorInvalidConfiguration;
  dim3 grid((unsigned)((p.n + TN - 1) / TN), (unsigned)((p.m + TM - 1) / TM), (unsigned)nb);
  if (p.c_dtype == BG_F64) gemm_simt_kernel<double><<<grid, 256, 0, s>>>(p);
  else if (dtype_is_float(p.c_dtype)) gemm_simt_kernel<float><<<grid, 256, 0, s>>>(p);
  else gemm_simt_kernel<long long><<<grid, 256, 0, s>>>(p);
  return cudaGetLastError();
}

}  // namespace bg
