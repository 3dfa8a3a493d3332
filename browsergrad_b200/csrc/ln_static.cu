// Specialised kernel for the layer-norm rows of a pre-LayerNorm decoder:
//
//   h[r, :]   = t0[r, :] + t1[r, :] + ...          (1 to 4 terms: dense [rows, cols] tensors or
//                                                   [cols] vectors repeated on every row)
//   out[r, :] = (f32(h) - mean) / sqrt(var + eps) * w + b
//
// h is optionally stored (it is the residual stream the next block adds to).  The terms are fp32 or
// fp64 -- in an fp32 sum also f16 / bf16, widened exactly (the 16-bit output of an autocast Linear) -- and are
// added in the sum type T, left to right, exactly as the generic interpreter does;
// the statistics are fp32 over f32(h), the reference's rule for LAYER_NORM
// (packages/browsergrad-jit/src/python/_realize.py:1384-1402 casts the row to float32 first).
//
// One CTA owns one row at a time and a thread four of its values, so a row is read from HBM once and written once.
// (A warp per row, each lane holding cols / 32 values, ran at 0.6 of the copy bandwidth: each load sits behind the
// type switch of its term, so a lane waited out some thirty memory round trips one after another, with too few warps
// resident to hide them.)
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace bg {
namespace {


template <typename T> struct Vec4 { T v[4]; };

template <typename T>
__device__ __forceinline__ Vec4<T> load4(const void* base, int dtype, int64_t elem) {
  Vec4<T> r;
  if (dtype == BG_F64) {
    const double2 a = __ldg(reinterpret_cast<const double2*>(reinterpret_cast<const double*>(base) + elem));
    const double2 b = __ldg(reinterpret_cast<const double2*>(reinterpret_cast<const double*>(base) + elem) + 1);
    r.v[0] = (T)a.x; r.v[1] = (T)a.y; r.v[2] = (T)b.x; r.v[3] = (T)b.y;
  } else if (dtype == BG_F16) {
    const uint2 a = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(base) + elem));
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&a.x)), hi = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
    r.v[0] = (T)lo.x; r.v[1] = (T)lo.y; r.v[2] = (T)hi.x; r.v[3] = (T)hi.y;
  } else if (dtype == BG_BF16) {
    const uint2 a = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem));
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    r.v[0] = (T)lo.x; r.v[1] = (T)lo.y; r.v[2] = (T)hi.x; r.v[3] = (T)hi.y;
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem));
    r.v[0] = (T)a.x; r.v[1] = (T)a.y; r.v[2] = (T)a.z; r.v[3] = (T)a.w;
  }
  return r;
}

__device__ __forceinline__ void store4(void* base, int dtype, int64_t elem, const float* y) {
  if (dtype == BG_F64) {
    double2* q = reinterpret_cast<double2*>(reinterpret_cast<double*>(base) + elem);
    q[0] = make_double2((double)y[0], (double)y[1]);
    q[1] = make_double2((double)y[2], (double)y[3]);
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + elem) = make_float4(y[0], y[1], y[2], y[3]);
  }
}

// The planes launch_tf32_split makes of the row (tf32(y); bf16(y); bf16(y - tf32(y))), for an output that only feeds
// split products as their A operand.
__device__ __forceinline__ void store4_planes(float* hi, __nv_bfloat16* x16, __nv_bfloat16* lo16, int64_t elem, const float* y) {
  uint32_t h[4];
  float l[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h[e]) : "f"(y[e]));
    l[e] = __fadd_rn(y[e], -__uint_as_float(h[e]));
  }
  *reinterpret_cast<uint4*>(hi + elem) = make_uint4(h[0], h[1], h[2], h[3]);
  __nv_bfloat162 a0 = __floats2bfloat162_rn(y[0], y[1]), a1 = __floats2bfloat162_rn(y[2], y[3]);
  __nv_bfloat162 l0 = __floats2bfloat162_rn(l[0], l[1]), l1 = __floats2bfloat162_rn(l[2], l[3]);
  *reinterpret_cast<uint2*>(x16 + elem) = make_uint2(*reinterpret_cast<uint32_t*>(&a0), *reinterpret_cast<uint32_t*>(&a1));
  *reinterpret_cast<uint2*>(lo16 + elem) = make_uint2(*reinterpret_cast<uint32_t*>(&l0), *reinterpret_cast<uint32_t*>(&l1));
}

// Four fp32 or 16-bit values of a term as raw bytes: the type switch holds nothing but the loads themselves
// (predicated loads, no use of the data), so the loads of several terms are in flight together; load4 converts inside
// the switch, which makes a thread wait for each load before it issues the next.
__device__ __forceinline__ uint4 load_raw4(const void* base, int dtype, int64_t elem) {
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (dtype == BG_F32) {
    r = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + elem));
  } else {
    const uint2 h = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + elem));
    r.x = h.x;
    r.y = h.y;
  }
  return r;
}
__device__ __forceinline__ Vec4<float> convert_raw4(const uint4& r, int dtype) {
  Vec4<float> o;
  if (dtype == BG_F32) {
    o.v[0] = __uint_as_float(r.x); o.v[1] = __uint_as_float(r.y); o.v[2] = __uint_as_float(r.z); o.v[3] = __uint_as_float(r.w);
  } else if (dtype == BG_F16) {
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&r.x)), hi = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    o.v[0] = lo.x; o.v[1] = lo.y; o.v[2] = hi.x; o.v[3] = hi.y;
  } else {
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    o.v[0] = lo.x; o.v[1] = lo.y; o.v[2] = hi.x; o.v[3] = hi.y;
  }
  return o;
}

// The value an fp32 / fp64 store followed by a CAST to the 16-bit type would give: y is an fp32 number.
__device__ __forceinline__ void store4_16(void* base, int dtype16, int64_t elem, const float* y) {
  uint2 w;
  if (dtype16 == BG_BF16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
    w = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  } else {
    __half2 lo = __floats2half2_rn(y[0], y[1]), hi = __floats2half2_rn(y[2], y[3]);
    w = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
  *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + elem) = w;
}

__device__ __forceinline__ void store4_sum(float* base, int64_t elem, const float* h) {
  *reinterpret_cast<float4*>(base + elem) = make_float4(h[0], h[1], h[2], h[3]);
}
__device__ __forceinline__ void store4_sum(double* base, int64_t elem, const double* h) {
  double2* q = reinterpret_cast<double2*>(base + elem);
  q[0] = make_double2(h[0], h[1]);
  q[1] = make_double2(h[2], h[3]);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// G = float4 groups a lane may hold (cols <= 128 * G)
// OUT: 0 the rows in out_dtype, 1 split-product operand planes, 2 the rows rounded to f16 / bf16 (out16_dtype)
// One CTA per row, one float4 group per thread (cols / 4 threads, rounded up to whole warps): a thread holds four
// values, so some sixty warps are resident per SM and the loads of a row -- each behind the type switch of its term --
// overlap across warps instead of queueing up in one lane.  The two statistics are reduced by shuffles inside a warp
// and through shared memory across the warps (every thread adds the warps' partial sums in the same order, so all agree
// on the bits); two scratch rows alternate, so a row costs two barriers.  gamma and beta are read once per CTA.
template <typename T, int OUT>
__global__ void __launch_bounds__(256) static_ln_cta_kernel(const __grid_constant__ LnArgs a) {
  __shared__ float red_sum[2][8], red_sq[2][8];
  grid_dependency_wait();
  grid_launch_dependents();
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int c4 = (int)(a.cols >> 2);
  const int grp = threadIdx.x;
  const bool on = grp < c4;
  Vec4<float> w, b;
#pragma unroll
  for (int e = 0; e < 4; ++e) { w.v[e] = 0.f; b.v[e] = 0.f; }
  if (on) {
    w = load4<float>(a.w, a.w_dtype, (int64_t)grp * 4);
    b = load4<float>(a.b, a.b_dtype, (int64_t)grp * 4);
  }
  int flip = 0;
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x, flip ^= 1) {
    const int64_t at = row * a.cols + (int64_t)grp * 4;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (on) {
      T h[4];
      if constexpr (sizeof(T) == 4) {
        // fp32 sums move few bytes per load (a 16-bit or fp32 term): all terms' loads are issued before the first use
        uint4 raw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < a.n_terms) raw[k] = load_raw4(a.term[k], a.term_dtype[k], a.term_rowvec[k] ? (int64_t)grp * 4 : at);
        {
          const Vec4<float> t = convert_raw4(raw[0], a.term_dtype[0]);
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = t.v[e];
        }
#pragma unroll
        for (int k = 1; k < 4; ++k)
          if (k < a.n_terms) {
            const Vec4<float> t = convert_raw4(raw[k], a.term_dtype[k]);
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = h[e] + t.v[e];
          }
      } else {
        // fp64 sums: one term at a time keeps the thread at 40 registers (48 warps per SM), which is what fills HBM here
        {
          const Vec4<T> t = load4<T>(a.term[0], a.term_dtype[0], a.term_rowvec[0] ? (int64_t)grp * 4 : at);
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = t.v[e];
        }
#pragma unroll 1
        for (int k = 1; k < a.n_terms; ++k) {
          const Vec4<T> t = load4<T>(a.term[k], a.term_dtype[k], a.term_rowvec[k] ? (int64_t)grp * 4 : at);
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = h[e] + t.v[e];
        }
      }
      if (a.sum_out) store4_sum(reinterpret_cast<T*>(a.sum_out), at, h);
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = (float)h[e];
    }
    float s = warp_sum((x[0] + x[1]) + (x[2] + x[3]));
    if (lane == 0) red_sum[flip][wid] = s;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += red_sum[flip][i];
    const float mean = tot / (float)a.cols;
    float c[4], sq = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      c[e] = on ? __fadd_rn(x[e], -mean) : 0.f;
      sq += __fmul_rn(c[e], c[e]);
    }
    sq = warp_sum(sq);
    if (lane == 0) red_sq[flip][wid] = sq;
    __syncthreads();
    float tsq = 0.f;
    for (int i = 0; i < nw; ++i) tsq += red_sq[flip][i];
    const float inv = 1.0f / sqrtf(tsq / (float)a.cols + a.eps);
    if (on) {
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = __fadd_rn(__fmul_rn(__fmul_rn(c[e], inv), w.v[e]), b.v[e]);
      if constexpr (OUT == 1) {
        __nv_bfloat16* x16 = reinterpret_cast<__nv_bfloat16*>(a.planes_lo);
        store4_planes(reinterpret_cast<float*>(a.planes_hi), x16, x16 + a.rows * a.cols, at, y);
      } else if constexpr (OUT == 2) {
        store4_16(a.out16, a.out16_dtype, at, y);
      } else {
        store4(a.out, a.out_dtype, at, y);
      }
    }
  }
}

template <typename T, int OUT>
cudaError_t launch_t(const LnArgs& a, cudaStream_t s, int sm_count) {
  const int c4 = (int)(a.cols >> 2);
  const int threads = ((c4 + 31) / 32) * 32;
  // persistent CTAs, as many as are resident by their registers (40 per thread for fp64 sums, 56 for fp32 sums)
  int per_sm = (sizeof(T) == 8 ? 1536 : 1152) / threads;
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 16) per_sm = 16;
  int64_t grid = (int64_t)sm_count * per_sm;
  if (grid > a.rows) grid = a.rows;
  return launch_dependent(static_ln_cta_kernel<T, OUT>, dim3((unsigned)grid), dim3((unsigned)threads), 0, s, a);
}

}  // namespace

bool static_ln_shape_ok(int64_t rows, int64_t cols) { return rows > 0 && cols >= 4 && cols % 4 == 0 && cols <= 1024; }

cudaError_t launch_static_ln(const LnArgs& a, cudaStream_t s, int sm_count) {
  if (!static_ln_shape_ok(a.rows, a.cols) || a.n_terms < 1 || a.n_terms > 4) return cudaErrorInvalidValue;
  for (int k = 0; k < a.n_terms; ++k)
    if (!a.wide && a.term_dtype[k] == BG_F64) return cudaErrorInvalidValue;      // an fp32 sum has no fp64 term
  if (a.planes_hi) return a.wide ? launch_t<double, 1>(a, s, sm_count) : launch_t<float, 1>(a, s, sm_count);
  if (a.out16) return a.wide ? launch_t<double, 2>(a, s, sm_count) : launch_t<float, 2>(a, s, sm_count);
  return a.wide ? launch_t<double, 0>(a, s, sm_count) : launch_t<float, 0>(a, s, sm_count);
}

}  // namespace bg
