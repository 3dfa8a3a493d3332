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

}  // namespace

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
