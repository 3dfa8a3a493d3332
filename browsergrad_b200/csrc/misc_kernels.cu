// Data-movement and small-op kernels: strided copy (permute / broadcast materialisation), gather,
// generic [outer, R, inner] reductions and softmax for axes other than the last, cross entropy.
// They are HBM-bound byte/index work: one element per thread with coalesced stores, grid sized
// from the element count.
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

namespace bg {

namespace {

struct CopyParams {
  const char* in;
  char* out;
  int32_t esize, rank;
  int64_t numel;
  int64_t shape[kMaxRank];
  int64_t stride[kMaxRank];
};

template <typename T>
__global__ void strided_copy_kernel(const __grid_constant__ CopyParams p) {
  const T* in = reinterpret_cast<const T*>(p.in);
  T* out = reinterpret_cast<T*>(p.out);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < p.numel; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, off = 0;
#pragma unroll 1
    for (int d = p.rank - 1; d >= 0; --d) {
      int64_t q = rem / p.shape[d];
      off += (rem - q * p.shape[d]) * p.stride[d];
      rem = q;
    }
    out[i] = in[off];
  }
}

// Tiled transpose of the two fastest-varying axes when the innermost output axis reads with a
// large stride: [batch.., A, B] view whose input has unit stride along A.
template <typename T>
__global__ void transpose_tile_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t A, int64_t B,
                                      int64_t in_stride_b, int64_t in_batch_stride, int64_t n_batch_inner,
                                      const __grid_constant__ CopyParams batch) {
  __shared__ T tile[32][33];
  const int64_t bz = blockIdx.z;
  // decompose batch index over the leading dims described in `batch`
  int64_t rem = bz, boff = 0;
  for (int d = batch.rank - 1; d >= 0; --d) {
    int64_t q = rem / batch.shape[d];
    boff += (rem - q * batch.shape[d]) * batch.stride[d];
    rem = q;
  }
  const int64_t a0 = (int64_t)blockIdx.y * 32, b0 = (int64_t)blockIdx.x * 32;
  // read: unit stride along A
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int64_t b = b0 + j, a = a0 + threadIdx.x;
    if (a < A && b < B) tile[j][threadIdx.x] = in[boff + b * in_stride_b + a];
  }
  __syncthreads();
  // write: out[batch, a, b], unit stride along B
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int64_t a = a0 + j, b = b0 + threadIdx.x;
    if (a < A && b < B) out[bz * A * B + a * B + b] = tile[threadIdx.x][j];
  }
  (void)in_batch_stride; (void)n_batch_inner;
}

template <typename T> __device__ __forceinline__ double as_double(T v) { return (double)v; }

__device__ __forceinline__ double load_as_double(const void* p, int dt, int64_t i) {
  switch (dt) {
    case BG_F32: return reinterpret_cast<const float*>(p)[i];
    case BG_F64: return reinterpret_cast<const double*>(p)[i];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case BG_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    default: return 0.0;
  }
}
__device__ __forceinline__ long long load_as_i64(const void* p, int dt, int64_t i) {
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
__device__ __forceinline__ void store_from(void* p, int dt, int64_t i, double fv, long long iv, bool is_int) {
  switch (dt) {
    case BG_F32: reinterpret_cast<float*>(p)[i] = is_int ? (float)iv : (float)fv; break;
    case BG_F64: reinterpret_cast<double*>(p)[i] = is_int ? (double)iv : fv; break;
    case BG_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(is_int ? (float)iv : (float)fv); break;
    case BG_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(is_int ? (float)iv : (float)fv); break;
    case BG_BOOL: reinterpret_cast<unsigned char*>(p)[i] = is_int ? (iv != 0) : (fv != 0.0); break;
    case BG_I64: case BG_U64: reinterpret_cast<long long*>(p)[i] = is_int ? iv : (long long)fv; break;
    case BG_I32: case BG_U32: reinterpret_cast<int*>(p)[i] = (int)(is_int ? iv : (long long)fv); break;
    case BG_I16: case BG_U16: reinterpret_cast<short*>(p)[i] = (short)(is_int ? iv : (long long)fv); break;
    default: reinterpret_cast<signed char*>(p)[i] = (signed char)(is_int ? iv : (long long)fv); break;
  }
}

// One thread per (outer, inner) output; loops over R with stride `inner` (coalesced across inner).
// ACC = float / double / long long.
template <typename ACC>
__global__ void reduce_generic_kernel(const void* in, void* out, int in_dt, int out_dt, int op, int64_t outer,
                                      int64_t R, int64_t inner) {
  constexpr bool kInt = sizeof(ACC) == 8 && (ACC(1) / ACC(2) == ACC(0));
  const int64_t n = outer * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = t / inner, i = t - o * inner;
    const int64_t base = o * R * inner + i;
    ACC acc = ACC(0);
    long long best = -1;
    bool nan = false;
    for (int64_t r = 0; r < R; ++r) {
      ACC v;
      if (kInt) v = (ACC)load_as_i64(in, in_dt, base + r * inner);
      else v = (ACC)load_as_double(in, in_dt, base + r * inner);
      switch (op) {
        case BG_RED_SUM: case BG_RED_MEAN: acc += v; break;
        case BG_RED_PROD: acc = r == 0 ? v : acc * v; break;
        case BG_RED_MAX: if (v != v) nan = true; acc = (r == 0 || v > acc) ? v : acc; break;
        case BG_RED_MIN: if (v != v) nan = true; acc = (r == 0 || v < acc) ? v : acc; break;
        case BG_RED_ARGMAX: case BG_RED_ARGMIN: {
          const bool vn = v != v, an = acc != acc;
          bool take;
          if (best < 0) take = true;
          else if (an) take = false;
          else if (vn) take = true;
          else take = op == BG_RED_ARGMAX ? v > acc : v < acc;
          if (take) { acc = v; best = r; }
          break;
        }
        case BG_RED_ANY: acc = (acc != ACC(0)) || (v != ACC(0)) ? ACC(1) : ACC(0); break;
        default: acc = (r == 0 ? true : acc != ACC(0)) && (v != ACC(0)) ? ACC(1) : ACC(0); break;
      }
    }
    if ((op == BG_RED_ALL || op == BG_RED_PROD) && R == 0) acc = ACC(1);
    if (op == BG_RED_ARGMAX || op == BG_RED_ARGMIN) {
      store_from(out, out_dt, t, 0.0, best < 0 ? 0 : best, true);
    } else if (op == BG_RED_MEAN) {
      if (kInt) store_from(out, out_dt, t, (double)acc / (double)R, 0, false);
      else store_from(out, out_dt, t, (double)(acc / (ACC)R), 0, false);
    } else {
      double fv = (double)acc;
      if (nan && !kInt) fv = CUDART_NAN;
      store_from(out, out_dt, t, fv, (long long)acc, kInt);
    }
  }
}

template <typename T>
__global__ void softmax_generic_kernel(const T* in, T* out, int64_t outer, int64_t R, int64_t inner) {
  const int64_t n = outer * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = t / inner, i = t - o * inner;
    const int64_t base = o * R * inner + i;
    T m = in[base];
    bool nan = m != m;
    for (int64_t r = 1; r < R; ++r) {
      T v = in[base + r * inner];
      if (v != v) nan = true;
      m = v > m ? v : m;
    }
    if (nan) m = (T)CUDART_NAN;
    T sum = T(0);
    for (int64_t r = 0; r < R; ++r) {
      T e = sizeof(T) == 4 ? (T)expf((float)(in[base + r * inner] - m)) : (T)exp((double)(in[base + r * inner] - m));
      out[base + r * inner] = e;
      sum += e;
    }
    for (int64_t r = 0; r < R; ++r) out[base + r * inner] = out[base + r * inner] / sum;
  }
}

struct GatherParams {
  const char* x;
  const int64_t* idx;
  char* out;
  int32_t esize, rank, dim;
  int64_t numel;
  int64_t x_shape[kMaxRank];
  int64_t idx_shape[kMaxRank];
  int* status;
};

template <typename T>
__global__ void gather_kernel(const __grid_constant__ GatherParams p) {
  const T* x = reinterpret_cast<const T*>(p.x);
  T* out = reinterpret_cast<T*>(p.out);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < p.numel; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, off = 0, mul = 1;
    const int64_t g = p.idx[i];
    bool bad = g < 0 || g >= p.x_shape[p.dim];
#pragma unroll 1
    for (int d = p.rank - 1; d >= 0; --d) {
      int64_t q = rem / p.idx_shape[d];
      int64_t c = rem - q * p.idx_shape[d];
      rem = q;
      if (d == p.dim) c = bad ? 0 : g;
      off += c * mul;
      mul *= p.x_shape[d];
    }
    if (bad) { atomicExch(p.status, BG_ERR_INDEX_RANGE); continue; }
    out[i] = x[off];
  }
}

// per-position cross entropy: -(log_softmax(logits)[target]) over the class axis of [outer, C, inner]
template <typename T>
__global__ void ce_rows_kernel(const T* logits, const int64_t* targets, T* per_pos, int64_t outer, int64_t C,
                               int64_t inner, int64_t ignore_index, int* status) {
  const int64_t n = outer * inner;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = t / inner, i = t - o * inner;
    const int64_t base = o * C * inner + i;
    const int64_t tg = targets[t];
    if (tg == ignore_index) { per_pos[t] = T(0); continue; }
    if (tg < 0 || tg >= C) { atomicExch(status, BG_ERR_INDEX_RANGE); per_pos[t] = T(0); continue; }
    T m = logits[base];
    for (int64_t c = 1; c < C; ++c) { T v = logits[base + c * inner]; m = v > m ? v : m; }
    T sum = T(0);
    for (int64_t c = 0; c < C; ++c) {
      T sh = logits[base + c * inner] - m;
      sum += sizeof(T) == 4 ? (T)expf((float)sh) : (T)exp((double)sh);
    }
    T lse = sizeof(T) == 4 ? (T)logf((float)sum) : (T)log((double)sum);
    T lp = (logits[base + tg * inner] - m) - lse;
    per_pos[t] = -lp;
  }
}

// Deterministic single-CTA reduction of per-position losses (sum, count of valid targets).
template <typename T>
__global__ void ce_reduce_kernel(const T* per_pos, const int64_t* targets, T* out, int64_t n, int reduction,
                                 int64_t ignore_index) {
  __shared__ double ssum[256];
  __shared__ long long scnt[256];
  double s = 0.0;
  long long c = 0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    s += (double)per_pos[i];
    c += targets[i] != ignore_index;
  }
  ssum[threadIdx.x] = s;
  scnt[threadIdx.x] = c;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) { ssum[threadIdx.x] += ssum[threadIdx.x + o]; scnt[threadIdx.x] += scnt[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    T num = (T)ssum[0];
    out[0] = reduction == 2 ? num : (T)(num / (T)scnt[0]);
  }
}

inline unsigned grid_for(int64_t n, int block) {
  int64_t g = (n + block - 1) / block;
  if (g < 1) g = 1;
  if (g > 148 * 32) g = 148 * 32;
  return (unsigned)g;
}

}  // namespace

cudaError_t launch_strided_copy(const StridedView& in, void* out, int64_t numel, cudaStream_t s) {
  if (numel == 0) return cudaSuccess;
  const int es = dtype_size(in.dtype);
  // Fast path: the output's last axis reads with a non-unit stride while the second-to-last
  // output axis is the input's unit-stride axis -> shared-memory tile transpose.
  if (in.rank >= 2 && in.stride[in.rank - 2] == 1 && in.stride[in.rank - 1] > 1 && in.shape[in.rank - 1] >= 16 &&
      in.shape[in.rank - 2] >= 16) {
    CopyParams batch{};
    batch.rank = in.rank - 2;
    int64_t nb = 1;
    for (int d = 0; d < batch.rank; ++d) { batch.shape[d] = in.shape[d]; batch.stride[d] = in.stride[d]; nb *= in.shape[d]; }
    const int64_t A = in.shape[in.rank - 2], B = in.shape[in.rank - 1];
    if (nb <= 65535 && (A + 31) / 32 <= 65535) {
      dim3 grid((unsigned)((B + 31) / 32), (unsigned)((A + 31) / 32), (unsigned)nb), block(32, 8);
      switch (es) {
        case 1: transpose_tile_kernel<uint8_t><<<grid, block, 0, s>>>((const uint8_t*)in.ptr, (uint8_t*)out, A, B, in.stride[in.rank - 1], 0, 0, batch); break;
        case 2: transpose_tile_kernel<uint16_t><<<grid, block, 0, s>>>((const uint16_t*)in.ptr, (uint16_t*)out, A, B, in.stride[in.rank - 1], 0, 0, batch); break;
        case 4: transpose_tile_kernel<uint32_t><<<grid, block, 0, s>>>((const uint32_t*)in.ptr, (uint32_t*)out, A, B, in.stride[in.rank - 1], 0, 0, batch); break;
        default: transpose_tile_kernel<uint64_t><<<grid, block, 0, s>>>((const uint64_t*)in.ptr, (uint64_t*)out, A, B, in.stride[in.rank - 1], 0, 0, batch); break;
      }
      return cudaGetLastError();
    }
  }
  CopyParams p{};
  p.in = reinterpret_cast<const char*>(in.ptr);
  p.out = reinterpret_cast<char*>(out);
  p.esize = es;
  p.rank = in.rank;
  p.numel = numel;
  for (int d = 0; d < in.rank; ++d) { p.shape[d] = in.shape[d]; p.stride[d] = in.stride[d]; }
  const unsigned g = grid_for(numel, 256);
  switch (es) {
    case 1: strided_copy_kernel<uint8_t><<<g, 256, 0, s>>>(p); break;
    case 2: strided_copy_kernel<uint16_t><<<g, 256, 0, s>>>(p); break;
    case 4: strided_copy_kernel<uint32_t><<<g, 256, 0, s>>>(p); break;
    default: strided_copy_kernel<uint64_t><<<g, 256, 0, s>>>(p); break;
  }
  return cudaGetLastError();
}

cudaError_t launch_reduce_generic(const void* in, void* out, int in_dtype, int out_dtype, int red_op, int64_t outer,
                                  int64_t R, int64_t inner, cudaStream_t s) {
  const int64_t n = outer * inner;
  if (n == 0) return cudaSuccess;
  const unsigned g = grid_for(n, 128);
  if (in_dtype == BG_F64) reduce_generic_kernel<double><<<g, 128, 0, s>>>(in, out, in_dtype, out_dtype, red_op, outer, R, inner);
  else if (dtype_is_float(in_dtype)) reduce_generic_kernel<float><<<g, 128, 0, s>>>(in, out, in_dtype, out_dtype, red_op, outer, R, inner);
  else reduce_generic_kernel<long long><<<g, 128, 0, s>>>(in, out, in_dtype, out_dtype, red_op, outer, R, inner);
  return cudaGetLastError();
}

cudaError_t launch_softmax_generic(const void* in, void* out, int dtype, int64_t outer, int64_t R, int64_t inner,
                                   cudaStream_t s) {
  const int64_t n = outer * inner;
  if (n == 0 || R == 0) return cudaSuccess;
  const unsigned g = grid_for(n, 128);
  if (dtype == BG_F64) softmax_generic_kernel<double><<<g, 128, 0, s>>>((const double*)in, (double*)out, outer, R, inner);
  else if (dtype == BG_F32) softmax_generic_kernel<float><<<g, 128, 0, s>>>((const float*)in, (float*)out, outer, R, inner);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_gather(const void* x, const int64_t* idx, void* out, int esize, int rank, const int64_t* x_shape,
                          const int64_t* idx_shape, int dim, int* status, cudaStream_t s) {
  GatherParams p{};
  p.x = reinterpret_cast<const char*>(x);
  p.idx = idx;
  p.out = reinterpret_cast<char*>(out);
  p.esize = esize;
  p.rank = rank;
  p.dim = dim;
  p.status = status;
  p.numel = 1;
  for (int d = 0; d < rank; ++d) { p.x_shape[d] = x_shape[d]; p.idx_shape[d] = idx_shape[d]; p.numel *= idx_shape[d]; }
  if (p.numel == 0) return cudaSuccess;
  const unsigned g = grid_for(p.numel, 256);
  switch (esize) {
    case 1: gather_kernel<uint8_t><<<g, 256, 0, s>>>(p); break;
    case 2: gather_kernel<uint16_t><<<g, 256, 0, s>>>(p); break;
    case 4: gather_kernel<uint32_t><<<g, 256, 0, s>>>(p); break;
    default: gather_kernel<uint64_t><<<g, 256, 0, s>>>(p); break;
  }
  return cudaGetLastError();
}

cudaError_t launch_ce_rows(const void* logits, const int64_t* targets, void* per_pos, int dtype, int64_t outer,
                           int64_t C, int64_t inner, int64_t ignore_index, int* status, cudaStream_t s) {
  const int64_t n = outer * inner;
  if (n == 0) return cudaSuccess;
  const unsigned g = grid_for(n, 128);
  if (dtype == BG_F64) ce_rows_kernel<double><<<g, 128, 0, s>>>((const double*)logits, targets, (double*)per_pos, outer, C, inner, ignore_index, status);
  else ce_rows_kernel<float><<<g, 128, 0, s>>>((const float*)logits, targets, (float*)per_pos, outer, C, inner, ignore_index, status);
  return cudaGetLastError();
}

cudaError_t launch_ce_reduce(const void* per_pos, const int64_t* targets, void* out, int dtype, int64_t n,
                             int reduction, int64_t ignore_index, cudaStream_t s) {
  if (dtype == BG_F64) ce_reduce_kernel<double><<<1, 256, 0, s>>>((const double*)per_pos, targets, (double*)out, n, reduction, ignore_index);
  else ce_reduce_kernel<float><<<1, 256, 0, s>>>((const float*)per_pos, targets, (float*)out, n, reduction, ignore_index);
  return cudaGetLastError();
}

}  // namespace bg
