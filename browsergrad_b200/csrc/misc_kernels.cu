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

// Strided copy whose innermost axis has unit stride: whole 16-byte vectors of the rows move (a permutation of the
// leading axes, e.g. [ranks, M, n] -> [M, ranks, n]).  shape / stride describe the view in units of vectors for the last
// axis and of bytes for the strides; one index decomposition per vector instead of one per element.
__global__ void strided_copy_vec_kernel(const __grid_constant__ CopyParams p) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < p.numel; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, off = 0;
#pragma unroll 1
    for (int d = p.rank - 1; d >= 0; --d) {
      int64_t q = rem / p.shape[d];
      off += (rem - q * p.shape[d]) * p.stride[d];
      rem = q;
    }
    reinterpret_cast<uint4*>(p.out)[i] = __ldcs(reinterpret_cast<const uint4*>(p.in + off));
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

// Rows of a table picked by an index of the output's full shape (an embedding lookup as the graph states it: x[R, C],
// idx[N, C], dim 0, 4-byte elements, C a multiple of 4): a thread takes four neighbouring elements of one output row,
// reads their four indices with two 16-byte loads and, when they name the same table row (they do when every output
// row repeats its token id), moves the values with one 16-byte load and store; otherwise element by element.
__global__ void gather_rows4_kernel(const uint32_t* __restrict__ x, const int64_t* __restrict__ idx, uint32_t* __restrict__ out,
                                    long long n4, int cols, long long x_rows, int* status) {
  const int c4 = cols >> 2;
  grid_dependency_wait();
  grid_launch_dependents();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % c4) * 4;
    const longlong2 a = __ldg(reinterpret_cast<const longlong2*>(idx) + 2 * i), b = __ldg(reinterpret_cast<const longlong2*>(idx) + 2 * i + 1);
    const long long g[4] = {a.x, a.y, b.x, b.y};
    bool bad = false;
#pragma unroll
    for (int e = 0; e < 4; ++e) bad |= g[e] < 0 || g[e] >= x_rows;
    if (bad) {
      // as the element-wise kernel: elements with a bad index are left unwritten and the status word says so
      atomicExch(status, BG_ERR_INDEX_RANGE);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (g[e] >= 0 && g[e] < x_rows) out[4 * i + e] = x[g[e] * cols + col + e];
      continue;
    }
    if (g[0] == g[1] && g[0] == g[2] && g[0] == g[3]) {
      reinterpret_cast<uint4*>(out)[i] = __ldg(reinterpret_cast<const uint4*>(x + g[0] * cols + col));
    } else {
      uint4 v;
      v.x = x[g[0] * cols + col]; v.y = x[g[1] * cols + col + 1]; v.z = x[g[2] * cols + col + 2]; v.w = x[g[3] * cols + col + 3];
      reinterpret_cast<uint4*>(out)[i] = v;
    }
  }
}

// ---- cross entropy (execute_cross_entropy_arrays, _framework_contracts.py:3756-3835) ---------------------------
// Per position, over the class axis of logits [outer, C, inner], in the logits' own float type T:
//   M = max_c x_c, S = sum_c exp(x_c - M), lse = log S, logp_c = (x_c - M) - lse                      (:3644-3664)
//   class-index targets:  loss = -logp_t * w_t; with label smoothing eps the loss becomes
//                         loss * (1 - eps) + (-sum_c logp_c w_c) * (eps / C); an ignored target gives 0    (:3801-3824)
//   probability targets:  loss = -sum_c logp_c * (p_c (1 - eps) + eps / C) * w_c                            (:3776-3799)
// Both class sums have the form sum_c q_c logp_c = T1 - lse * T2 with T1 = sum_c q_c (x_c - M), T2 = sum_c q_c, so one
// pass over the classes after the maximum yields S, T1 and T2 together.  w is all ones without class weights.
template <typename T>
struct CeRowArgs {
  const T* logits;
  const int64_t* idx;     // class-index targets, or null
  const T* prob;          // probability targets (same shape as logits), or null
  const T* weight;        // [C] or null
  T* per_pos;             // [outer * inner]
  T* sel_w;               // [outer * inner] weight of each position's target (0 when ignored), or null
  int64_t outer, C, inner, ignore_index;
  T smoothing;            // eps
  int* status;
};

template <typename T> __device__ __forceinline__ T ce_exp(T x);
template <> __device__ __forceinline__ float ce_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double ce_exp<double>(double x) { return exp(x); }
// exp of a non-positive shifted logit inside the long-row sum: fp32 rows use the hardware exp2 unit (the argument is
// bounded below by the row's range, so its rounding stays near 1e-6 relative on terms that matter); fp64 rows keep exp().
template <typename T> __device__ __forceinline__ T ce_exp_term(T x);
template <> __device__ __forceinline__ float ce_exp_term<float>(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}
template <> __device__ __forceinline__ double ce_exp_term<double>(double x) { return exp(x); }
template <typename T> __device__ __forceinline__ T ce_log(T x);
template <> __device__ __forceinline__ float ce_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double ce_log<double>(double x) { return log(x); }
template <typename T> __device__ __forceinline__ T ce_neg_inf();
template <> __device__ __forceinline__ float ce_neg_inf<float>() { return -CUDART_INF_F; }
template <> __device__ __forceinline__ double ce_neg_inf<double>() { return -CUDART_INF; }

// The loss of one position from its reduced statistics; x_t is the target's logit (index targets).
template <typename T>
__device__ __forceinline__ void ce_finish(const CeRowArgs<T>& a, int64_t pos, T M, T S, T T1, T T2, bool need_sums) {
  const T lse = ce_log<T>(S);
  const T eps = a.smoothing;
  if (a.prob) {
    a.per_pos[pos] = -(T1 - lse * T2);
    return;
  }
  const int64_t tg = a.idx[pos];
  if (tg == a.ignore_index) {
    a.per_pos[pos] = T(0);
    if (a.sel_w) a.sel_w[pos] = T(0);
    return;
  }
  if (tg < 0 || tg >= a.C) {
    atomicExch(a.status, BG_ERR_INDEX_RANGE);
    a.per_pos[pos] = T(0);
    if (a.sel_w) a.sel_w[pos] = T(0);
    return;
  }
  const int64_t o = pos / a.inner, i = pos - o * a.inner;
  const T xt = a.logits[(o * a.C + tg) * a.inner + i];
  const T wt = a.weight ? a.weight[tg] : T(1);
  T loss = -((xt - M) - lse);
  if (a.weight) loss *= wt;
  if (need_sums) loss = loss * (T(1) - eps) + (-(T1 - lse * T2)) * (eps / (T)a.C);
  a.per_pos[pos] = loss;
  if (a.sel_w) a.sel_w[pos] = wt;
}

template <typename T, int VEC> __device__ __forceinline__ void ce_load_vec(const T* p, T* out);
template <> __device__ __forceinline__ void ce_load_vec<float, 4>(const float* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> __device__ __forceinline__ void ce_load_vec<double, 2>(const double* p, double* out) {
  const double2 v = *reinterpret_cast<const double2*>(p);
  out[0] = v.x; out[1] = v.y;
}

// One thread per position; the class axis is `inner` elements apart, so neighbouring threads read neighbouring
// addresses when inner > 1.  Used for spatial logits and for short class axes.
template <typename T>
__device__ __forceinline__ void ce_one_position(const CeRowArgs<T>& a, int64_t t, bool need_sums) {
  const int64_t o = t / a.inner, i = t - o * a.inner;
  const int64_t base = o * a.C * a.inner + i;
  if (!a.prob && a.idx[t] == a.ignore_index) { ce_finish<T>(a, t, T(0), T(1), T(0), T(0), false); return; }
  T M = a.logits[base];
  for (int64_t c = 1; c < a.C; ++c) { const T v = a.logits[base + c * a.inner]; M = v > M ? v : M; }
  T S = T(0), T1 = T(0), T2 = T(0);
  for (int64_t c = 0; c < a.C; ++c) {
    const T sh = a.logits[base + c * a.inner] - M;
    S += ce_exp<T>(sh);
    if (need_sums) {
      T q = a.weight ? a.weight[c] : T(1);
      if (a.prob) q *= a.prob[base + c * a.inner] * (T(1) - a.smoothing) + a.smoothing / (T)a.C;
      T1 += q * sh;
      T2 += q;
    }
  }
  ce_finish<T>(a, t, M, S, T1, T2, need_sums);
}

template <typename T>
__global__ void ce_pos_kernel(const CeRowArgs<T> a) {
  const int64_t n = a.outer * a.inner;
  const bool need_sums = a.prob != nullptr || a.smoothing != T(0);
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x)
    ce_one_position<T>(a, t, need_sums);
}

// One CTA per position for class axes that are contiguous (inner == 1) and long: every thread walks the row in
// 16-byte vectors (coalesced), keeping a running maximum that is raised once per group of vectors, and the partial
// (M, S, T1, T2) of all threads are combined through shared memory.  The row is read from DRAM once; the statistics
// are rescaled, never the data.
// SUMS: 0 none (index targets, no smoothing); 1 label smoothing with neither probability targets nor class weights (the
// per-class factor is one: no second or third operand stream); 2 the general weighted sums.
template <typename T, int VEC, int SUMS>
__global__ void __launch_bounds__(256) ce_row_kernel(const CeRowArgs<T> a, int vec_ok) {
  constexpr int kGroup = (sizeof(T) == 4 && SUMS < 2) ? 8 : 4;   // vectors per thread in flight between maximum updates
  const int64_t row = blockIdx.x;
  const T* x = a.logits + row * a.C;
  const T* pr = (SUMS == 2 && a.prob) ? a.prob + row * a.C : nullptr;
  constexpr bool need_sums = SUMS != 0;           // probability targets or label smoothing: the weighted sums T1, T2
  const T eps = a.smoothing, unif = a.smoothing / (T)a.C;
  __shared__ T sh_m[8], sh_s[8], sh_t1[8], sh_t2[8];
  const bool skip = !a.prob && a.idx[row] == a.ignore_index;      // the whole CTA agrees
  T M = ce_neg_inf<T>(), S = T(0), T1 = T(0), T2 = T(0);           // T1 is kept relative to the running M
  if (!skip) {
    const bool use_w = SUMS == 2 && a.weight != nullptr;
    // raise the reference maximum to gm: S scales by exp(M - gm), T1 (kept relative to M) shifts by (M - gm) * T2
    auto raise = [&](T gm) {
      if (gm > M) {
        if (M != ce_neg_inf<T>()) { S *= ce_exp<T>(M - gm); T1 += (M - gm) * T2; }
        M = gm;
      }
    };
    auto add = [&](T xv, T pv, T wv) {
      const T shv = xv - M;
      S += ce_exp_term<T>(shv);
      if (need_sums) {
        T q = wv;
        if (pr) q *= pv * (T(1) - eps) + unif;
        T1 += q * shv;
        T2 += q;
      }
    };
    int64_t scalar_from = 0;
    if (vec_ok) {
      const int64_t n_vec = a.C / VEC;
      scalar_from = n_vec * VEC;
      for (int64_t v0 = threadIdx.x; v0 < n_vec; v0 += (int64_t)blockDim.x * kGroup) {
        T v[kGroup][VEC], pv[kGroup][VEC], wv[kGroup][VEC];
        T gm = ce_neg_inf<T>();
#pragma unroll
        for (int k = 0; k < kGroup; ++k) {
          const int64_t vi = v0 + (int64_t)k * blockDim.x;
          const bool live = vi < n_vec;
          ce_load_vec<T, VEC>(x + (live ? vi : 0) * VEC, v[k]);
          if (pr) ce_load_vec<T, VEC>(pr + (live ? vi : 0) * VEC, pv[k]);
          if (use_w) ce_load_vec<T, VEC>(a.weight + (live ? vi : 0) * VEC, wv[k]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            if (!live) v[k][e] = ce_neg_inf<T>();        // exp(-inf - M) = 0; the sums skip dead vectors below
            gm = v[k][e] > gm ? v[k][e] : gm;
          }
        }
        raise(gm);
#pragma unroll
        for (int k = 0; k < kGroup; ++k) {
          if (v0 + (int64_t)k * blockDim.x >= n_vec) continue;
#pragma unroll
          for (int e = 0; e < VEC; ++e) add(v[k][e], pr ? pv[k][e] : T(0), use_w ? wv[k][e] : T(1));
        }
      }
    }
    for (int64_t c = scalar_from + threadIdx.x; c < a.C; c += blockDim.x) {
      const T xv = x[c];
      raise(xv);
      add(xv, pr ? pr[c] : T(0), use_w ? a.weight[c] : T(1));
    }
    // combine within the warp, then across warps: (M, S, T1, T2) pairs merge by rescaling the smaller maximum's side
    auto merge = [&](T m2, T s2, T t12, T t22) {
      const T mm = m2 > M ? m2 : M;
      if (mm == ce_neg_inf<T>()) return;
      const T f1 = M == ce_neg_inf<T>() ? T(0) : ce_exp<T>(M - mm), f2 = m2 == ce_neg_inf<T>() ? T(0) : ce_exp<T>(m2 - mm);
      const T d1 = M == ce_neg_inf<T>() ? T(0) : (M - mm) * T2, d2 = m2 == ce_neg_inf<T>() ? T(0) : (m2 - mm) * t22;
      S = S * f1 + s2 * f2;
      T1 = (T1 + d1) + (t12 + d2);
      T2 += t22;
      M = mm;
    };
    for (int o = 16; o > 0; o >>= 1)
      merge(__shfl_xor_sync(0xffffffffu, M, o), __shfl_xor_sync(0xffffffffu, S, o), __shfl_xor_sync(0xffffffffu, T1, o),
            __shfl_xor_sync(0xffffffffu, T2, o));
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  if (lane == 0) { sh_m[warp] = M; sh_s[warp] = S; sh_t1[warp] = T1; sh_t2[warp] = T2; }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (skip) { ce_finish<T>(a, row, T(0), T(1), T(0), T(0), false); return; }
    T m = sh_m[0], s = sh_s[0], t1 = sh_t1[0], t2 = sh_t2[0];
    for (int w = 1; w < n_warps; ++w) {
      const T m2 = sh_m[w], mm = m2 > m ? m2 : m;
      if (mm == ce_neg_inf<T>()) continue;
      const T f1 = m == ce_neg_inf<T>() ? T(0) : ce_exp<T>(m - mm), f2 = m2 == ce_neg_inf<T>() ? T(0) : ce_exp<T>(m2 - mm);
      const T d1 = m == ce_neg_inf<T>() ? T(0) : (m - mm) * t2, d2 = m2 == ce_neg_inf<T>() ? T(0) : (m2 - mm) * sh_t2[w];
      s = s * f1 + sh_s[w] * f2;
      t1 = (t1 + d1) + (sh_t1[w] + d2);
      t2 += sh_t2[w];
      m = mm;
    }
    ce_finish<T>(a, row, m, s, t1, t2, need_sums);
  }
}

// Deterministic reduction of the per-position losses: sum, or mean over the valid targets (their count, their summed
// class weights when weights are given, or `fixed_count` positions for probability targets).  256 partial sums in
// double, combined in a fixed order.
template <typename T>
__global__ void ce_reduce_kernel(const T* per_pos, const int64_t* targets, const T* sel_w, T* out, int64_t n, int reduction,
                                 int64_t ignore_index, double fixed_count) {
  __shared__ double ssum[256];
  __shared__ double sden[256];
  double s = 0.0, c = 0.0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    s += (double)per_pos[i];
    if (sel_w) c += (double)sel_w[i];
    else if (targets) c += targets[i] != ignore_index ? 1.0 : 0.0;
  }
  ssum[threadIdx.x] = s;
  sden[threadIdx.x] = c;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) { ssum[threadIdx.x] += ssum[threadIdx.x + o]; sden[threadIdx.x] += sden[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const T num = (T)ssum[0];
    const T den = (sel_w || targets) ? (T)sden[0] : (T)fixed_count;
    out[0] = reduction == 2 ? num : (T)(num / den);
  }
}

// Up to 256 positions with a short class axis (a classifier head on one small batch): the per-position losses and
// their reduction in one launch of one CTA -- thread t takes position t, then the CTA reduces exactly as
// ce_reduce_kernel does (each of its 256 partial sums holds at most one position here), so the bits are the same.
template <typename T>
__global__ void __launch_bounds__(256) ce_small_kernel(const CeRowArgs<T> a, const int64_t* targets, T* out, int reduction, double fixed_count) {
  __shared__ double ssum[256];
  __shared__ double sden[256];
  grid_dependency_wait();
  grid_launch_dependents();
  const int64_t n = a.outer * a.inner;
  const bool need_sums = a.prob != nullptr || a.smoothing != T(0);
  double s = 0.0, c = 0.0;
  if ((int64_t)threadIdx.x < n) {
    ce_one_position<T>(a, threadIdx.x, need_sums);
    // the thread reads back what it has just written itself
    s = (double)a.per_pos[threadIdx.x];
    if (a.sel_w) c = (double)a.sel_w[threadIdx.x];
    else if (targets) c = targets[threadIdx.x] != a.ignore_index ? 1.0 : 0.0;
  }
  ssum[threadIdx.x] = s;
  sden[threadIdx.x] = c;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) { ssum[threadIdx.x] += ssum[threadIdx.x + o]; sden[threadIdx.x] += sden[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const T num = (T)ssum[0];
    const T den = (a.sel_w || targets) ? (T)sden[0] : (T)fixed_count;
    out[0] = reduction == 2 ? num : (T)(num / den);
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
  // rows of whole 16-byte vectors, every row starting on a 16-byte boundary
  if (in.rank >= 2 && in.stride[in.rank - 1] == 1 && (in.shape[in.rank - 1] * es) % 16 == 0 &&
      ((reinterpret_cast<uintptr_t>(in.ptr) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    bool ok = true;
    for (int d = 0; d + 1 < in.rank; ++d) ok = ok && in.stride[d] >= 0 && (in.stride[d] * es) % 16 == 0;
    if (ok) {
      CopyParams v{};
      v.in = reinterpret_cast<const char*>(in.ptr);
      v.out = reinterpret_cast<char*>(out);
      v.esize = 16;
      v.rank = in.rank;
      v.numel = numel * es / 16;
      for (int d = 0; d + 1 < in.rank; ++d) { v.shape[d] = in.shape[d]; v.stride[d] = in.stride[d] * es; }
      v.shape[in.rank - 1] = in.shape[in.rank - 1] * es / 16;
      v.stride[in.rank - 1] = 16;
      strided_copy_vec_kernel<<<grid_for(v.numel, 256), 256, 0, s>>>(v);
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
  if (esize == 4 && rank == 2 && dim == 0 && idx_shape[1] == x_shape[1] && x_shape[1] % 4 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(idx) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    const long long n4 = p.numel / 4;
    return launch_dependent(gather_rows4_kernel, dim3(grid_for(n4, 256)), dim3(256), 0, s, reinterpret_cast<const uint32_t*>(x), idx,
                            reinterpret_cast<uint32_t*>(out), n4, (int)x_shape[1], (long long)x_shape[0], status);
  }
  const unsigned g = grid_for(p.numel, 256);
  switch (esize) {
    case 1: gather_kernel<uint8_t><<<g, 256, 0, s>>>(p); break;
    case 2: gather_kernel<uint16_t><<<g, 256, 0, s>>>(p); break;
    case 4: gather_kernel<uint32_t><<<g, 256, 0, s>>>(p); break;
    default: gather_kernel<uint64_t><<<g, 256, 0, s>>>(p); break;
  }
  return cudaGetLastError();
}

namespace {
template <typename T>
CeRowArgs<T> ce_args(const CeProblem& c) {
  CeRowArgs<T> a{};
  a.logits = reinterpret_cast<const T*>(c.logits);
  a.idx = c.prob_targets ? nullptr : reinterpret_cast<const int64_t*>(c.targets);
  a.prob = c.prob_targets ? reinterpret_cast<const T*>(c.targets) : nullptr;
  a.weight = reinterpret_cast<const T*>(c.weight);
  a.per_pos = reinterpret_cast<T*>(c.per_pos);
  a.sel_w = reinterpret_cast<T*>(c.sel_w);
  a.outer = c.outer; a.C = c.C; a.inner = c.inner; a.ignore_index = c.ignore_index;
  a.smoothing = (T)c.label_smoothing;
  a.status = c.status;
  return a;
}
// long contiguous class axes take the CTA-per-row kernel, everything else a thread per position
bool ce_row_path(const CeProblem& c) { return c.inner == 1 && c.C >= 512 && c.outer * c.inner <= 0x7fffffff; }

template <typename T>
cudaError_t ce_rows_typed(const CeProblem& c, cudaStream_t s) {
  CeRowArgs<T> a = ce_args<T>(c);
  const int64_t n = c.outer * c.inner;
  if (ce_row_path(c)) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool aligned = (reinterpret_cast<uintptr_t>(c.logits) & 15) == 0 && c.C % VEC == 0 &&
                         (!c.prob_targets || (reinterpret_cast<uintptr_t>(c.targets) & 15) == 0) &&
                         (!c.weight || (reinterpret_cast<uintptr_t>(c.weight) & 15) == 0);
    const int threads = c.C >= 4096 ? 256 : 128;
    if (a.prob != nullptr || (a.smoothing != T(0) && a.weight != nullptr)) ce_row_kernel<T, VEC, 2><<<(unsigned)n, threads, 0, s>>>(a, aligned ? 1 : 0);
    else if (a.smoothing != T(0)) ce_row_kernel<T, VEC, 1><<<(unsigned)n, threads, 0, s>>>(a, aligned ? 1 : 0);
    else ce_row_kernel<T, VEC, 0><<<(unsigned)n, threads, 0, s>>>(a, aligned ? 1 : 0);
  } else {
    ce_pos_kernel<T><<<grid_for(n, 128), 128, 0, s>>>(a);
  }
  return cudaGetLastError();
}
}  // namespace

cudaError_t launch_ce_rows(const CeProblem& c, cudaStream_t s) {
  if (c.outer * c.inner == 0) return cudaSuccess;
  return c.dtype == BG_F64 ? ce_rows_typed<double>(c, s) : ce_rows_typed<float>(c, s);
}

bool ce_small_usable(const CeProblem& c) { const int64_t n = c.outer * c.inner; return n > 0 && n <= 256 && !ce_row_path(c); }

cudaError_t launch_ce_small(const CeProblem& c, void* out, int reduction, double fixed_count, cudaStream_t s) {
  const int64_t* targets = c.prob_targets ? nullptr : reinterpret_cast<const int64_t*>(c.targets);
  if (c.dtype == BG_F64)
    return launch_dependent(ce_small_kernel<double>, dim3(1), dim3(256), 0, s, ce_args<double>(c), targets, reinterpret_cast<double*>(out), reduction,
                            fixed_count);
  return launch_dependent(ce_small_kernel<float>, dim3(1), dim3(256), 0, s, ce_args<float>(c), targets, reinterpret_cast<float*>(out), reduction,
                          fixed_count);
}

cudaError_t launch_ce_reduce(const void* per_pos, const int64_t* targets, const void* sel_w, void* out, int dtype, int64_t n,
                             int reduction, int64_t ignore_index, double fixed_count, cudaStream_t s) {
  if (dtype == BG_F64)
    ce_reduce_kernel<double><<<1, 256, 0, s>>>((const double*)per_pos, targets, (const double*)sel_w, (double*)out, n, reduction,
                                                ignore_index, fixed_count);
  else
    ce_reduce_kernel<float><<<1, 256, 0, s>>>((const float*)per_pos, targets, (const float*)sel_w, (float*)out, n, reduction,
                                               ignore_index, fixed_count);
  return cudaGetLastError();
}

}  // namespace bg
