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
// One warp owns one row: a lane keeps cols/32 values in registers, so a row is read from HBM once
// and written once, the two reductions are shuffles, and no block-wide barrier is needed.  All
// loads of one term's row share are independent, so many are in flight per lane.
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace bg {
namespace {

constexpr int kLnThreads = 256;

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
template <typename T, int G, int OUT>
__global__ void __launch_bounds__(kLnThreads) static_ln_kernel(const __grid_constant__ LnArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kLnThreads + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * kLnThreads) >> 5;
  const int c4 = (int)(a.cols >> 2);
  for (int64_t row = warp; row < a.rows; row += n_warps) {
    const int64_t rbase = row * a.cols;
    T h[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int grp = g * 32 + lane;
      if (grp < c4) {
        const Vec4<T> t = load4<T>(a.term[0], a.term_dtype[0], (a.term_rowvec[0] ? 0 : rbase) + (int64_t)grp * 4);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[g][e] = t.v[e];
      }
    }
#pragma unroll
    for (int k = 1; k < 4; ++k) {
      if (k < a.n_terms) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const int grp = g * 32 + lane;
          if (grp < c4) {
            const Vec4<T> t = load4<T>(a.term[k], a.term_dtype[k], (a.term_rowvec[k] ? 0 : rbase) + (int64_t)grp * 4);
#pragma unroll
            for (int e = 0; e < 4; ++e) h[g][e] = h[g][e] + t.v[e];
          }
        }
      }
    }
    float x[G][4];
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int grp = g * 32 + lane;
      if (grp < c4) {
        if (a.sum_out) store4_sum(reinterpret_cast<T*>(a.sum_out), rbase + (int64_t)grp * 4, h[g]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          x[g][e] = (float)h[g][e];
          sum += x[g][e];
        }
      }
    }
    const float mean = warp_sum(sum) / (float)a.cols;
    float sq = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (g * 32 + lane < c4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float c = __fadd_rn(x[g][e], -mean);
          sq += __fmul_rn(c, c);
        }
      }
    }
    const float var = warp_sum(sq) / (float)a.cols;
    const float inv = 1.0f / sqrtf(var + a.eps);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int grp = g * 32 + lane;
      if (grp < c4) {
        const Vec4<float> w = load4<float>(a.w, a.w_dtype, (int64_t)grp * 4);
        const Vec4<float> b = load4<float>(a.b, a.b_dtype, (int64_t)grp * 4);
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float xh = __fmul_rn(__fadd_rn(x[g][e], -mean), inv);
          y[e] = __fadd_rn(__fmul_rn(xh, w.v[e]), b.v[e]);
        }
        if constexpr (OUT == 1) {
          __nv_bfloat16* x16 = reinterpret_cast<__nv_bfloat16*>(a.planes_lo);
          store4_planes(reinterpret_cast<float*>(a.planes_hi), x16, x16 + a.rows * a.cols, rbase + (int64_t)grp * 4, y);
        } else if constexpr (OUT == 2) {
          // the value an fp32 / fp64 store followed by a CAST to the 16-bit type would give: y is an fp32 number
          uint2 w;
          if (a.out16_dtype == BG_BF16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
            w = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          } else {
            __half2 lo = __floats2half2_rn(y[0], y[1]), hi = __floats2half2_rn(y[2], y[3]);
            w = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          }
          *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.out16) + rbase + (int64_t)grp * 4) = w;
        } else {
          store4(a.out, a.out_dtype, rbase + (int64_t)grp * 4, y);
        }
      }
    }
  }
}

template <typename T, int OUT>
cudaError_t launch_t(const LnArgs& a, cudaStream_t s, int sm_count) {
  const int c4 = (int)(a.cols >> 2);
  const int groups = (c4 + 31) / 32;
  const int64_t warps_per_cta = kLnThreads / 32;
  int64_t grid = (a.rows + warps_per_cta - 1) / warps_per_cta;
  const int64_t cap = (int64_t)sm_count * 8;
  if (grid > cap) grid = cap;
  if (groups <= 2) static_ln_kernel<T, 2, OUT><<<(unsigned)grid, kLnThreads, 0, s>>>(a);
  else if (groups <= 4) static_ln_kernel<T, 4, OUT><<<(unsigned)grid, kLnThreads, 0, s>>>(a);
  else if (groups <= 6) static_ln_kernel<T, 6, OUT><<<(unsigned)grid, kLnThreads, 0, s>>>(a);
  else static_ln_kernel<T, 8, OUT><<<(unsigned)grid, kLnThreads, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace

bool static_ln_shape_ok(int64_t rows, int64_t cols) { return rows > 0 && cols >= 4 && cols % 4 == 0 && cols <= 1024; }

cudaError_t launch_static_ln(const LnArgs& a, cudaStream_t s, int sm_count) {
  if (!static_ln_shape_ok(a.rows, a.cols) || a.n_terms < 1 || a.n_terms > 4) return cudaErrorInvalidValue;
  if (a.planes_hi) return a.wide ? launch_t<double, 1>(a, s, sm_count) : launch_t<float, 1>(a, s, sm_count);
  if (a.out16) return a.wide ? launch_t<double, 2>(a, s, sm_count) : launch_t<float, 2>(a, s, sm_count);
  return a.wide ? launch_t<double, 0>(a, s, sm_count) : launch_t<float, 0>(a, s, sm_count);
}

}  // namespace bg
