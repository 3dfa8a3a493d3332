// Specialised kernels for the dominant fused fp32 patterns.
//
// The plan compiler lowers every fusion group to an EwProgram for the generic interpreter
// (ew_kernel.cu).  When a group is all-fp32 over dense, vector-aligned operands and its
// expression matches one of the patterns below, the same group runs here instead: the
// expression is a compile-time functor, values stay in real registers, and the kernel is a pure
// HBM stream - 128-bit coalesced loads with several independent loads in flight per thread,
// grid sized as a multiple of the SM count.
//
//   flat     out[i] = f(in0[i], ..)                     grid-stride over 4096-element tiles
//   rowsum   out[r] = sum_c f(in0[r,c], ..)             one warp per row, shuffle reduction
//   softmax  out[r,:] = softmax_c f(in0[r,c], ..)       one CTA per row, row held in registers
//
// The expression itself uses the same rounding as the interpreter (separate multiply and add, expf);
// the softmax tail uses the hardware exp2 unit and one reciprocal per row, which agrees with the
// generic path to ~1e-6 relative.
#include "common.h"

#include <math_constants.h>

namespace bg {
namespace {

__device__ __forceinline__ float fadd_(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fmul_(float a, float b) { return __fmul_rn(a, b); }

__device__ __forceinline__ float ex2_approx_(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// relu(a*b + c) * exp(-d)
struct PatChain {
  static constexpr int NIN = 4;
  __device__ static __forceinline__ float f(const float* x) {
    float t = fadd_(fmul_(x[0], x[1]), x[2]);
    t = t > 0.f ? t : 0.f;
    return fmul_(t, expf(-x[3]));
  }
};
// a single dense operand (softmax / row sum of a stored tensor)
struct PatIdent {
  static constexpr int NIN = 1;
  __device__ static __forceinline__ float f(const float* x) { return x[0]; }
};
// a + b (residual add)
struct PatAdd {
  static constexpr int NIN = 2;
  __device__ static __forceinline__ float f(const float* x) { return fadd_(x[0], x[1]); }
};
// a * b
struct PatMul {
  static constexpr int NIN = 2;
  __device__ static __forceinline__ float f(const float* x) { return fmul_(x[0], x[1]); }
};

template <class P>
__device__ __forceinline__ void eval4(const float4* v, float* r) {
  float x[P::NIN];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
#pragma unroll
    for (int k = 0; k < P::NIN; ++k) x[k] = reinterpret_cast<const float*>(&v[k])[e];
    r[e] = P::f(x);
  }
}

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <class P>
__global__ void __launch_bounds__(kThreads) static_flat_kernel(const __grid_constant__ StaticArgs a) {
  const int64_t n4 = a.numel >> 2;  // whole float4 groups
  const int64_t tile = (int64_t)kThreads * kUnroll;
  for (int64_t base = (int64_t)blockIdx.x * tile; base < n4; base += (int64_t)gridDim.x * tile) {
    float4 v[kUnroll][P::NIN];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + (int64_t)u * kThreads + threadIdx.x;
      if (i < n4) {
#pragma unroll
        for (int k = 0; k < P::NIN; ++k) v[u][k] = __ldcs(reinterpret_cast<const float4*>(a.in[k]) + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + (int64_t)u * kThreads + threadIdx.x;
      if (i < n4) {
        float r[4];
        eval4<P>(v[u], r);
        __stcs(reinterpret_cast<float4*>(a.out) + i, make_float4(r[0], r[1], r[2], r[3]));
      }
    }
  }
  // ragged end (numel not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (a.numel & 3)) {
    const int64_t i = (n4 << 2) + threadIdx.x;
    float x[P::NIN];
#pragma unroll
    for (int k = 0; k < P::NIN; ++k) x[k] = a.in[k][i];
    a.out[i] = P::f(x);
  }
}

// One warp per row; cols % 4 == 0.
template <class P>
__global__ void __launch_bounds__(kThreads) static_rowsum_kernel(const __grid_constant__ StaticArgs a, int mean) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int64_t c4 = a.cols >> 2;
  for (int64_t row = warp; row < a.rows; row += n_warps) {
    const int64_t rbase = row * c4;
    float acc[kUnroll] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t c = lane; c < c4; c += 32 * kUnroll) {
      float4 v[kUnroll][P::NIN];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t cc = c + 32 * u;
        if (cc < c4) {
#pragma unroll
          for (int k = 0; k < P::NIN; ++k) v[u][k] = __ldcs(reinterpret_cast<const float4*>(a.in[k]) + rbase + cc);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (c + 32 * u < c4) {
          float r[4];
          eval4<P>(v[u], r);
          acc[u] += (r[0] + r[1]) + (r[2] + r[3]);
        }
      }
    }
    float s = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) a.out[row] = mean ? s / (float)a.cols : s;
  }
}

// One CTA per row, N float4 per thread (cols <= 1024 * N), cols % 4 == 0.
template <class P, int N>
__global__ void __launch_bounds__(kThreads) static_softmax_kernel(const __grid_constant__ StaticArgs a) {
  __shared__ float red[2][kThreads / 32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t c4 = a.cols >> 2;
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const int64_t rbase = row * c4;
    float4 v[N][P::NIN];
#pragma unroll
    for (int u = 0; u < N; ++u) {
      const int64_t cc = (int64_t)u * kThreads + threadIdx.x;
      if (cc < c4) {
#pragma unroll
        for (int k = 0; k < P::NIN; ++k) v[u][k] = __ldcs(reinterpret_cast<const float4*>(a.in[k]) + rbase + cc);
      }
    }
    float y[N][4];
    float m = -CUDART_INF_F;
    bool nan = false;
#pragma unroll
    for (int u = 0; u < N; ++u) {
      if ((int64_t)u * kThreads + threadIdx.x < c4) {
        eval4<P>(v[u], y[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          nan |= y[u][e] != y[u][e];
          m = y[u][e] > m ? y[u][e] : m;
        }
      }
    }
    if (nan) m = CUDART_NAN_F;   // NaN propagates through the max like NumPy's
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float t = __shfl_xor_sync(0xffffffffu, m, o);
      m = (t != t || m != m) ? CUDART_NAN_F : (t > m ? t : m);
    }
    if (lane == 0) red[0][w] = m;
    __syncthreads();
    float mm = red[0][lane & 7];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      float t = __shfl_xor_sync(0xffffffffu, mm, o);
      mm = (t != t || mm != mm) ? CUDART_NAN_F : (t > mm ? t : mm);
    }
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < N; ++u) {
      if ((int64_t)u * kThreads + threadIdx.x < c4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // exp(y - m) as 2^((y - m) * log2 e) on the hardware exp2 unit: |y - m| is bounded by the row's
          // range, so the argument rounding stays near 1e-6 relative
          y[u][e] = ex2_approx_(fmul_(fadd_(y[u][e], -mm), 1.4426950408889634f));
          s += y[u][e];
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[1][w] = s;
    __syncthreads();
    float ss = red[1][lane & 7];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = __fdiv_rn(1.0f, ss);   // one IEEE divide per row, then one multiply per element
#pragma unroll
    for (int u = 0; u < N; ++u) {
      const int64_t cc = (int64_t)u * kThreads + threadIdx.x;
      if (cc < c4)
        __stcs(reinterpret_cast<float4*>(a.out) + rbase + cc,
               make_float4(fmul_(y[u][0], inv), fmul_(y[u][1], inv), fmul_(y[u][2], inv), fmul_(y[u][3], inv)));
    }
    // no trailing barrier: red[0] of the next row is written before its first barrier, which no
    // warp passes until every warp has finished reading red[0] and red[1] of this row
  }
}

struct PatternEntry {
  const char* sig;
  int id;
};
const PatternEntry kPatterns[] = {
    {"mul(relu(add(mul(i0,i1),i2)),expneg(i3))", 0},
    {"i0", 1},
    {"add(i0,i1)", 2},
    {"mul(i0,i1)", 3},
};

template <class P>
cudaError_t launch_pattern(int kind, const StaticArgs& a, int arg, cudaStream_t s, int sm_count) {
  if (kind == SK_FLAT) {
    const int64_t tiles = ((a.numel >> 2) + kThreads * kUnroll - 1) / (kThreads * kUnroll);
    int64_t grid = (int64_t)sm_count * 8;
    if (grid > tiles) grid = tiles > 0 ? tiles : 1;
    static_flat_kernel<P><<<(unsigned)grid, kThreads, 0, s>>>(a);
  } else if (kind == SK_ROWSUM) {
    int64_t grid = (a.rows + 7) / 8;
    const int64_t cap = (int64_t)sm_count * 8;
    if (grid > cap) grid = cap;
    static_rowsum_kernel<P><<<(unsigned)grid, kThreads, 0, s>>>(a, arg);
  } else {
    int64_t grid = a.rows;
    const int64_t cap = (int64_t)sm_count * 8;
    if (grid > cap) grid = cap;
    const int64_t n = (a.cols + 1023) / 1024;
    if (n <= 1) static_softmax_kernel<P, 1><<<(unsigned)grid, kThreads, 0, s>>>(a);
    else if (n <= 2) static_softmax_kernel<P, 2><<<(unsigned)grid, kThreads, 0, s>>>(a);
    else if (n <= 4) static_softmax_kernel<P, 4><<<(unsigned)grid, kThreads, 0, s>>>(a);
    else static_softmax_kernel<P, 8><<<(unsigned)grid, kThreads, 0, s>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace

int static_pattern_id(const std::string& sig, int* n_inputs) {
  static const int nin[] = {PatChain::NIN, PatIdent::NIN, PatAdd::NIN, PatMul::NIN};
  for (const auto& p : kPatterns)
    if (sig == p.sig) {
      if (n_inputs) *n_inputs = nin[p.id];
      return p.id;
    }
  return -1;
}

bool static_shape_ok(int kind, int64_t rows, int64_t cols, int64_t numel, int sm_count) {
  if (numel <= 0) return false;
  if (kind == SK_FLAT) return true;
  if (cols % 4 != 0 || cols <= 0) return false;
  if (kind == SK_ROWSUM) return rows >= (int64_t)sm_count * 8 && cols >= 128;   // enough rows to give every warp one
  return cols <= 8192 && rows >= sm_count;
}

cudaError_t launch_static(int pattern, int kind, const StaticArgs& a, int arg, cudaStream_t s, int sm_count) {
  switch (pattern) {
    case 0: return launch_pattern<PatChain>(kind, a, arg, s, sm_count);
    case 1: return launch_pattern<PatIdent>(kind, a, arg, s, sm_count);
    case 2: return launch_pattern<PatAdd>(kind, a, arg, s, sm_count);
    case 3: return launch_pattern<PatMul>(kind, a, arg, s, sm_count);
  }
  return cudaErrorInvalidValue;
}

}  // namespace bg
