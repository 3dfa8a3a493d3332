// Generic fused elementwise / row-reduction kernel for sm_100a.
//
// A fusion group arrives as an EwProgram: a short register program (LOAD, arithmetic, CMP,
// WHERE, CVT, STORE ...) passed as a __grid_constant__ parameter, so every thread fetches the
// same instruction from the constant bank and the opcode switch is warp-uniform.  The virtual
// registers live in shared memory, one 16-byte slot per thread per plane
// (plane = register x chunk [x half for 64-bit classes]); consecutive threads own consecutive
// slots, so every LDS.128/STS.128 is conflict free and dynamic register numbers cost nothing.
// Each thread handles 4 consecutive elements per chunk: contiguous operands move with one
// 128-bit coalesced load/store per thread (512 B per warp), strided/broadcast operands fall
// back to per-lane addressing.
//
// Two kernels share the interpreter:
//   ew_kernel   - flat iteration space, grid-stride over tiles of U chunks;
//   row_kernel  - one CTA per row of [rows, cols]; after the program has produced the row in a
//                 register, a tail (reduce / softmax / layer norm) finishes it on chip with
//                 warp shuffles, so the row is read from HBM once and written once.
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <map>
#include <mutex>
#include <tuple>

namespace bg {

// CTAs per SM the flat kernel is compiled for (caps its registers per thread at 65536 / (256 * this)).
#ifndef BG_EW_MIN_CTAS
#define BG_EW_MIN_CTAS 3
#endif

constexpr int kBlock = 256;
constexpr int kVec = 4;
constexpr int kChunk = kBlock * kVec;  // 1024 elements

// ------------------------------------------------------------------------------------
// Register file access
// ------------------------------------------------------------------------------------
struct RegFile {
  char* tbase;       // shared-memory base of this thread's slots
  int U;             // chunks per pass
  uint32_t rstride;  // bytes between registers
  uint32_t ustride;  // bytes between chunks of one register
  __device__ __forceinline__ RegFile(char* base, int U_, int planes)
      : tbase(base + threadIdx.x * 16), U(U_), rstride((uint32_t)U_ * planes * (kBlock * 16)),
        ustride((uint32_t)planes * (kBlock * 16)) {}
  // The same register file seen from chunk u0 on, n chunks long.
  __device__ __forceinline__ RegFile group(int u0, int n) const {
    RegFile g = *this;
    g.tbase += (uint32_t)u0 * ustride;
    g.U = n;
    return g;
  }
  __device__ __forceinline__ char* slot(int r, int u, int h) const {
    return tbase + (uint32_t)r * rstride + (uint32_t)u * ustride + (uint32_t)h * (kBlock * 16);
  }
};

// Position of a pass: chunk u starts at linear index idx0 + u * kChunk (lane 0 of this thread);
// elements at or beyond `end` (tensor end, or row end in row mode) do not exist.
struct Pos {
  int64_t idx0;
  int64_t end;
  __device__ __forceinline__ int64_t idx(int u) const { return idx0 + (int64_t)u * kChunk; }
  __device__ __forceinline__ int nvalid(int u) const {
    int64_t left = end - idx(u);
    return left >= 4 ? 4 : (left > 0 ? (int)left : 0);
  }
};

template <typename T> struct V4 { T v[4]; };

template <typename T> __device__ __forceinline__ V4<T> rget(const RegFile& rf, int r, int u);
template <typename T> __device__ __forceinline__ void rput(const RegFile& rf, int r, int u, const V4<T>& x);

template <> __device__ __forceinline__ V4<float> rget<float>(const RegFile& rf, int r, int u) {
  float4 t = *reinterpret_cast<const float4*>(rf.slot(r, u, 0));
  return {{t.x, t.y, t.z, t.w}};
}
template <> __device__ __forceinline__ void rput<float>(const RegFile& rf, int r, int u, const V4<float>& x) {
  *reinterpret_cast<float4*>(rf.slot(r, u, 0)) = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
}
template <> __device__ __forceinline__ V4<uint32_t> rget<uint32_t>(const RegFile& rf, int r, int u) {
  uint4 t = *reinterpret_cast<const uint4*>(rf.slot(r, u, 0));
  return {{t.x, t.y, t.z, t.w}};
}
template <> __device__ __forceinline__ void rput<uint32_t>(const RegFile& rf, int r, int u, const V4<uint32_t>& x) {
  *reinterpret_cast<uint4*>(rf.slot(r, u, 0)) = make_uint4(x.v[0], x.v[1], x.v[2], x.v[3]);
}
template <> __device__ __forceinline__ V4<double> rget<double>(const RegFile& rf, int r, int u) {
  double2 a = *reinterpret_cast<const double2*>(rf.slot(r, u, 0));
  double2 b = *reinterpret_cast<const double2*>(rf.slot(r, u, 1));
  return {{a.x, a.y, b.x, b.y}};
}
template <> __device__ __forceinline__ void rput<double>(const RegFile& rf, int r, int u, const V4<double>& x) {
  *reinterpret_cast<double2*>(rf.slot(r, u, 0)) = make_double2(x.v[0], x.v[1]);
  *reinterpret_cast<double2*>(rf.slot(r, u, 1)) = make_double2(x.v[2], x.v[3]);
}
template <> __device__ __forceinline__ V4<long long> rget<long long>(const RegFile& rf, int r, int u) {
  longlong2 a = *reinterpret_cast<const longlong2*>(rf.slot(r, u, 0));
  longlong2 b = *reinterpret_cast<const longlong2*>(rf.slot(r, u, 1));
  return {{a.x, a.y, b.x, b.y}};
}
template <> __device__ __forceinline__ void rput<long long>(const RegFile& rf, int r, int u, const V4<long long>& x) {
  *reinterpret_cast<longlong2*>(rf.slot(r, u, 0)) = make_longlong2(x.v[0], x.v[1]);
  *reinterpret_cast<longlong2*>(rf.slot(r, u, 1)) = make_longlong2(x.v[2], x.v[3]);
}

// ------------------------------------------------------------------------------------
// Scalar element access with dtype conversion to the natural register class
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float ld_f32class(const void* p, int dt, int64_t i) {
  switch (dt) {
    case BG_F32: return reinterpret_cast<const float*>(p)[i];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    default: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
}
__device__ __forceinline__ long long ld_i64class(const void* p, int dt, int64_t i) {
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
__device__ __forceinline__ void st_f32class(void* p, int dt, int64_t i, float x) {
  switch (dt) {
    case BG_F32: reinterpret_cast<float*>(p)[i] = x; break;
    case BG_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(x); break;
    default: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x); break;
  }
}
__device__ __forceinline__ void st_i64class(void* p, int dt, int64_t i, long long x) {
  switch (dt) {
    case BG_I64: case BG_U64: reinterpret_cast<long long*>(p)[i] = x; break;
    case BG_I32: case BG_U32: reinterpret_cast<int*>(p)[i] = (int)x; break;
    case BG_I16: case BG_U16: reinterpret_cast<short*>(p)[i] = (short)x; break;
    default: reinterpret_cast<signed char*>(p)[i] = (signed char)x; break;
  }
}

__device__ __forceinline__ float narrow_f32(float x, int dt) {
  if (dt == BG_F16) return __half2float(__float2half_rn(x));
  if (dt == BG_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  return x;
}
__device__ __forceinline__ long long narrow_i64(long long x, int dt) {
  switch (dt) {
    case BG_I32: return (int)x;
    case BG_U32: return (unsigned)x;
    case BG_I16: return (short)x;
    case BG_U16: return (unsigned short)x;
    case BG_I8: return (signed char)x;
    case BG_U8: return (unsigned char)x;
    case BG_BOOL: return x != 0;
    default: return x;
  }
}

// ------------------------------------------------------------------------------------
// Per-chunk iteration state
// ------------------------------------------------------------------------------------
struct ChunkPos {
  int64_t idx;   // linear index of lane 0 in the iteration space
  int nvalid;    // 0..4 lanes inside the tensor (row mode: inside the row)
};

// Offsets of the 4 lanes of a strided operand.
__device__ __noinline__ void strided_offsets(const EwProgram& p, const EwOperand& o, int64_t idx, int nvalid,
                                             int64_t off[4]) {
  const int nd = p.ndim;
  const int64_t last = p.shape[nd - 1];
  if ((last & 3) == 0) {
    int64_t rem = idx, base = 0;
#pragma unroll 1
    for (int d = nd - 1; d >= 0; --d) {
      int64_t s = p.shape[d];
      int64_t q = rem / s;
      base += (rem - q * s) * o.stride[d];
      rem = q;
    }
    const int64_t si = o.stride[nd - 1];
#pragma unroll
    for (int e = 0; e < 4; ++e) off[e] = base + e * si;
  } else {
#pragma unroll 1
    for (int e = 0; e < 4; ++e) {
      int64_t rem = idx + (e < nvalid ? e : 0), base = 0;
#pragma unroll 1
      for (int d = nd - 1; d >= 0; --d) {
        int64_t s = p.shape[d];
        int64_t q = rem / s;
        base += (rem - q * s) * o.stride[d];
        rem = q;
      }
      off[e] = base;
    }
  }
}

// General load of one chunk: any dtype, any addressing mode, partial chunks.
__device__ __noinline__ void load_chunk(const EwProgram& p, const EwInstr ins, const RegFile rf, int u, ChunkPos cp) {
  if (cp.nvalid == 0) return;
  const EwOperand& o = p.inputs[ins.aux];
  int64_t off[4];
  bool vec = false;
  if (o.mode == A_CONTIG) {
#pragma unroll
    for (int e = 0; e < 4; ++e) off[e] = cp.idx + (e < cp.nvalid ? e : 0);
    vec = o.vec_ok && cp.nvalid == 4;
  } else if (o.mode == A_SCALAR) {
#pragma unroll
    for (int e = 0; e < 4; ++e) off[e] = 0;
  } else {
    strided_offsets(p, o, cp.idx, cp.nvalid, off);
    vec = o.vec_ok && cp.nvalid == 4 && o.stride[p.ndim - 1] == 1 && (p.shape[p.ndim - 1] & 3) == 0;
  }
  const int dt = o.dtype;
  if (dt == BG_F32 || dt == BG_F16 || dt == BG_BF16) {
    V4<float> r;
    if (vec && dt == BG_F32) {
      float4 t = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(o.ptr) + off[0]));
      r = {{t.x, t.y, t.z, t.w}};
    } else if (vec && dt == BG_F16) {
      uint2 t = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(o.ptr) + off[0]));
      __half2 h0 = *reinterpret_cast<__half2*>(&t.x), h1 = *reinterpret_cast<__half2*>(&t.y);
      float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
      r = {{f0.x, f0.y, f1.x, f1.y}};
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) r.v[e] = ld_f32class(o.ptr, dt, off[e]);
    }
    rput<float>(rf, ins.dst, u, r);
  } else if (dt == BG_F64) {
    V4<double> r;
    const double* q = reinterpret_cast<const double*>(o.ptr);
    if (vec) {
      double2 a = __ldg(reinterpret_cast<const double2*>(q + off[0]));
      double2 b = __ldg(reinterpret_cast<const double2*>(q + off[0] + 2));
      r = {{a.x, a.y, b.x, b.y}};
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) r.v[e] = q[off[e]];
    }
    rput<double>(rf, ins.dst, u, r);
  } else if (dt == BG_BOOL) {
    V4<uint32_t> r;
    const unsigned char* q = reinterpret_cast<const unsigned char*>(o.ptr);
    if (vec) {
      uint32_t t = __ldg(reinterpret_cast<const uint32_t*>(q + off[0]));
      r = {{(t & 0xffu) != 0, ((t >> 8) & 0xffu) != 0, ((t >> 16) & 0xffu) != 0, (t >> 24) != 0}};
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) r.v[e] = q[off[e]] != 0;
    }
    rput<uint32_t>(rf, ins.dst, u, r);
  } else {
    V4<long long> r;
    if (vec && (dt == BG_I64 || dt == BG_U64)) {
      const long long* q = reinterpret_cast<const long long*>(o.ptr);
      longlong2 a = __ldg(reinterpret_cast<const longlong2*>(q + off[0]));
      longlong2 b = __ldg(reinterpret_cast<const longlong2*>(q + off[0] + 2));
      r = {{a.x, a.y, b.x, b.y}};
    } else if (vec && dt == BG_I32) {
      int4 t = __ldg(reinterpret_cast<const int4*>(reinterpret_cast<const int*>(o.ptr) + off[0]));
      r = {{t.x, t.y, t.z, t.w}};
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) r.v[e] = ld_i64class(o.ptr, dt, off[e]);
    }
    rput<long long>(rf, ins.dst, u, r);
  }
}

// General store of one chunk.
__device__ __noinline__ void store_chunk(const EwProgram& p, const EwInstr ins, const RegFile rf, int u, ChunkPos cp) {
  if (cp.nvalid <= 0) return;
  const EwOutput& o = p.outputs[ins.aux];
  const int dt = o.dtype;
  const bool vec = o.vec_ok && cp.nvalid == 4;
  const int64_t i0 = cp.idx;
  if (ins.type == T_F32) {
    V4<float> r = rget<float>(rf, ins.a, u);
    if (vec && dt == BG_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(o.ptr) + i0) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    } else if (vec && dt == BG_F16) {
      __half2 h0 = __floats2half2_rn(r.v[0], r.v[1]), h1 = __floats2half2_rn(r.v[2], r.v[3]);
      uint2 t;
      t.x = *reinterpret_cast<uint32_t*>(&h0);
      t.y = *reinterpret_cast<uint32_t*>(&h1);
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(o.ptr) + i0) = t;
    } else if (vec && dt == BG_BF16) {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(r.v[0], r.v[1]), h1 = __floats2bfloat162_rn(r.v[2], r.v[3]);
      uint2 t;
      t.x = *reinterpret_cast<uint32_t*>(&h0);
      t.y = *reinterpret_cast<uint32_t*>(&h1);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(o.ptr) + i0) = t;
    } else {
      for (int e = 0; e < cp.nvalid; ++e) st_f32class(o.ptr, dt, i0 + e, r.v[e]);
    }
  } else if (ins.type == T_F64) {
    V4<double> r = rget<double>(rf, ins.a, u);
    double* q = reinterpret_cast<double*>(o.ptr);
    if (vec) {
      *reinterpret_cast<double2*>(q + i0) = make_double2(r.v[0], r.v[1]);
      *reinterpret_cast<double2*>(q + i0 + 2) = make_double2(r.v[2], r.v[3]);
    } else {
      for (int e = 0; e < cp.nvalid; ++e) q[i0 + e] = r.v[e];
    }
  } else if (ins.type == T_B) {
    V4<uint32_t> r = rget<uint32_t>(rf, ins.a, u);
    unsigned char* q = reinterpret_cast<unsigned char*>(o.ptr);
    if (vec) {
      *reinterpret_cast<uint32_t*>(q + i0) = (r.v[0] & 1u) | ((r.v[1] & 1u) << 8) | ((r.v[2] & 1u) << 16) | ((r.v[3] & 1u) << 24);
    } else {
      for (int e = 0; e < cp.nvalid; ++e) q[i0 + e] = (unsigned char)(r.v[e] != 0);
    }
  } else {
    V4<long long> r = rget<long long>(rf, ins.a, u);
    if (vec && (dt == BG_I64 || dt == BG_U64)) {
      long long* q = reinterpret_cast<long long*>(o.ptr);
      *reinterpret_cast<longlong2*>(q + i0) = make_longlong2(r.v[0], r.v[1]);
      *reinterpret_cast<longlong2*>(q + i0 + 2) = make_longlong2(r.v[2], r.v[3]);
    } else if (vec && (dt == BG_I32 || dt == BG_U32)) {
      *reinterpret_cast<int4*>(reinterpret_cast<int*>(o.ptr) + i0) = make_int4((int)r.v[0], (int)r.v[1], (int)r.v[2], (int)r.v[3]);
    } else {
      for (int e = 0; e < cp.nvalid; ++e) st_i64class(o.ptr, dt, i0 + e, r.v[e]);
    }
  }
}

template <typename T> __device__ __forceinline__ bool cmp_op(T a, T b, int op) {
  switch (op) {
    case BG_CMP_EQ: return a == b;
    case BG_CMP_NE: return a != b;
    case BG_CMP_LT: return a < b;
    case BG_CMP_LE: return a <= b;
    case BG_CMP_GT: return a > b;
    default: return a >= b;
  }
}

template <typename T> __device__ __forceinline__ T f_exp(T x);
template <> __device__ __forceinline__ float f_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double f_exp<double>(double x) { return exp(x); }
template <typename T> __device__ __forceinline__ T f_log(T x);
template <> __device__ __forceinline__ float f_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double f_log<double>(double x) { return log(x); }
template <typename T> __device__ __forceinline__ T f_sin(T x);
template <> __device__ __forceinline__ float f_sin<float>(float x) { return sinf(x); }
template <> __device__ __forceinline__ double f_sin<double>(double x) { return sin(x); }
template <typename T> __device__ __forceinline__ T f_cos(T x);
template <> __device__ __forceinline__ float f_cos<float>(float x) { return cosf(x); }
template <> __device__ __forceinline__ double f_cos<double>(double x) { return cos(x); }

// Arithmetic on floating classes.  Explicit __f*_rn / __d*_rn keep the compiler from contracting
// a MUL followed by an ADD into an FMA: NumPy rounds after each ufunc.
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double fadd(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double fmul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double fdiv(double a, double b) { return __ddiv_rn(a, b); }

// The opcode switch sits outside the chunk loop: one decode per instruction per pass, then the
// same operation over all U chunks (unrolled when UT > 0).
#define BG_FOR_U _Pragma("unroll 4") for (int u = 0; u < nU; ++u)
#define BG_UNARY(T, EXPR)                                   \
  BG_FOR_U {                                                \
    V4<T> a = rget<T>(rf, ins.a, u), r;                     \
    _Pragma("unroll") for (int e = 0; e < 4; ++e) { const T x = a.v[e]; r.v[e] = (EXPR); } \
    rput<T>(rf, ins.dst, u, r);                             \
  }
#define BG_BINARY(T, EXPR)                                  \
  BG_FOR_U {                                                \
    V4<T> a = rget<T>(rf, ins.a, u), b = rget<T>(rf, ins.b, u), r; \
    _Pragma("unroll") for (int e = 0; e < 4; ++e) { const T x = a.v[e]; const T y = b.v[e]; r.v[e] = (EXPR); } \
    rput<T>(rf, ins.dst, u, r);                             \
  }

// ------------------------------------------------------------------------------------
// fp32 fast path
// ------------------------------------------------------------------------------------
// fp32 arithmetic, compares, selects and dense copies work on the UT chunks of a pass at once, with
// their operands in real registers.  An operand field names a shared-memory register, input k of the
// program (read straight from global memory), a constant, or the accumulator: the registers the
// previous instruction left its result in.  A result field names a shared-memory register, output k
// (written straight to global memory) or the accumulator alone.  Lanes beyond the end of the tensor
// or row read zero and are not stored; what is computed on them is never seen.
template <int UT>
__device__ __forceinline__ void fast_fetch(const EwProgram& p, const RegFile& rf, const Pos& pos, bool full, int r,
                                           float4 (&x)[UT]) {
  if (r & kEwDirect) {
    if ((r & kEwConst) == kEwConst) {
      const float f = (float)__longlong_as_double(p.consts[r & 0x3f]);
#pragma unroll
      for (int u = 0; u < UT; ++u) x[u] = make_float4(f, f, f, f);
      return;
    }
    const float* src = reinterpret_cast<const float*>(p.inputs[r & 0x3f].ptr) + pos.idx0;
    if (full) {
#pragma unroll
      for (int u = 0; u < UT; ++u) x[u] = __ldg(reinterpret_cast<const float4*>(src) + u * (kChunk / 4));
    } else {
#pragma unroll
      for (int u = 0; u < UT; ++u) {
        const int nv = pos.nvalid(u);
        const float* q = src + u * kChunk;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (nv == 4) {
          t = __ldg(reinterpret_cast<const float4*>(q));
        } else if (nv > 0) {
          t.x = q[0];
          if (nv > 1) t.y = q[1];
          if (nv > 2) t.z = q[2];
        }
        x[u] = t;
      }
    }
    return;
  }
  const char* s = rf.tbase + (uint32_t)r * rf.rstride;
#pragma unroll
  for (int u = 0; u < UT; ++u) x[u] = *reinterpret_cast<const float4*>(s + u * rf.ustride);
}

template <int UT>
__device__ __forceinline__ void fast_put(const EwProgram& p, const RegFile& rf, const Pos& pos, bool full, int r,
                                         const float4 (&x)[UT]) {
  if (r == kEwAcc) return;
  if (r & kEwDirect) {
    if (p.outputs[r & 0x3f].dtype == BG_F64) {
      // an fp32 value stored into a float64 output
      double* dst = reinterpret_cast<double*>(p.outputs[r & 0x3f].ptr) + pos.idx0;
#pragma unroll
      for (int u = 0; u < UT; ++u) {
        const int nv = full ? 4 : pos.nvalid(u);
        double* q = dst + u * kChunk;
        if (nv == 4) {
          reinterpret_cast<double2*>(q)[0] = make_double2((double)x[u].x, (double)x[u].y);
          reinterpret_cast<double2*>(q)[1] = make_double2((double)x[u].z, (double)x[u].w);
        } else if (nv > 0) {
          q[0] = (double)x[u].x;
          if (nv > 1) q[1] = (double)x[u].y;
          if (nv > 2) q[2] = (double)x[u].z;
        }
      }
      return;
    }
    float* dst = reinterpret_cast<float*>(p.outputs[r & 0x3f].ptr) + pos.idx0;
    if (full) {
#pragma unroll
      for (int u = 0; u < UT; ++u) reinterpret_cast<float4*>(dst)[u * (kChunk / 4)] = x[u];
    } else {
#pragma unroll
      for (int u = 0; u < UT; ++u) {
        const int nv = pos.nvalid(u);
        float* q = dst + u * kChunk;
        if (nv == 4) {
          *reinterpret_cast<float4*>(q) = x[u];
        } else if (nv > 0) {
          q[0] = x[u].x;
          if (nv > 1) q[1] = x[u].y;
          if (nv > 2) q[2] = x[u].z;
        }
      }
    }
    return;
  }
  char* d = rf.tbase + (uint32_t)r * rf.rstride;
#pragma unroll
  for (int u = 0; u < UT; ++u) *reinterpret_cast<float4*>(d + u * rf.ustride) = x[u];
}

// f over every element of the pass.
template <int UT, typename F>
__device__ __forceinline__ void map1(float4 (&a)[UT], F f) {
#pragma unroll
  for (int u = 0; u < UT; ++u) a[u] = make_float4(f(a[u].x), f(a[u].y), f(a[u].z), f(a[u].w));
}
template <int UT, typename F>
__device__ __forceinline__ void map2(float4 (&a)[UT], const float4 (&b)[UT], F f) {
#pragma unroll
  for (int u = 0; u < UT; ++u) a[u] = make_float4(f(a[u].x, b[u].x), f(a[u].y, b[u].y), f(a[u].z, b[u].z), f(a[u].w, b[u].w));
}
// Bulky bodies exist once, out of line, and are called per chunk.
__device__ __noinline__ float4 div4(float4 a, float4 b) { return make_float4(fdiv(a.x, b.x), fdiv(a.y, b.y), fdiv(a.z, b.z), fdiv(a.w, b.w)); }
__device__ __noinline__ float4 log4(float4 a) { return make_float4(logf(a.x), logf(a.y), logf(a.z), logf(a.w)); }
__device__ __noinline__ float4 sin4(float4 a) { return make_float4(sinf(a.x), sinf(a.y), sinf(a.z), sinf(a.w)); }
__device__ __noinline__ float4 cos4(float4 a) { return make_float4(cosf(a.x), cosf(a.y), cosf(a.z), cosf(a.w)); }
// tanh GELU of an fp32 value: with u = k (x + 0.044715 x^3), 0.5 x (1 + tanh u) = x / (1 + e^(-2u)).  One
// exponential and no cancellation for negative x.  Where the float64 form overflows (|u| beyond the largest argument
// of exp, 709.78) it yields inf / inf = NaN, and so does this.
__device__ __forceinline__ float gelu1(float x) {
  float t = fmul(0.044715f, x);
  t = fmul(t, x);
  t = fmul(t, x);
  const float u = fmul(0.7978845608028654f, fadd(x, t));
  const float e = expf(fmul(-2.0f, u));
  const float g = __fdividef(x, fadd(1.0f, e));
  return fabsf(u) > 709.782712893384f ? CUDART_NAN_F : g;
}
__device__ __forceinline__ float sign1(float x) { return x != x ? x : (float)((x > 0) - (x < 0)); }
__device__ __noinline__ float4 sign4(float4 a) { return make_float4(sign1(a.x), sign1(a.y), sign1(a.z), sign1(a.w)); }

template <int UT, typename F>
__device__ __forceinline__ void cmp_put(const RegFile& rf, int dst, const float4 (&a)[UT], const float4 (&b)[UT], F f) {
  char* d = rf.tbase + (uint32_t)dst * rf.rstride;
#pragma unroll
  for (int u = 0; u < UT; ++u)
    *reinterpret_cast<uint4*>(d + u * rf.ustride) =
        make_uint4(f(a[u].x, b[u].x), f(a[u].y, b[u].y), f(a[u].z, b[u].z), f(a[u].w, b[u].w));
}

// Opcodes the fast path executes when the instruction's class is fp32.
constexpr uint32_t kFastOps = (1u << E_ADD) | (1u << E_MUL) | (1u << E_DIV) | (1u << E_NEG) | (1u << E_EXP) | (1u << E_LOG) |
                              (1u << E_ABS) | (1u << E_SIGN) | (1u << E_SIN) | (1u << E_COS) | (1u << E_CMP) | (1u << E_WHERE) |
                              (1u << E_SUB) | (1u << E_RELU) | (1u << E_EXPNEG) | (1u << E_COPY) | (1u << E_GELU);
constexpr uint32_t kTwoOperandOps = (1u << E_ADD) | (1u << E_MUL) | (1u << E_DIV) | (1u << E_SUB) | (1u << E_CMP) | (1u << E_WHERE);
static_assert(E_OPCOUNT <= 32, "opcode masks are 32 bits wide");

template <int UT>
__device__ __forceinline__ void fast_instr(const EwProgram& p, const EwInstr ins, const RegFile& rf, const Pos& pos, bool full,
                                           float4 (&acc)[UT]) {
  const int op = ins.op;
  const int ra = op == E_WHERE ? ins.b : ins.a;
  if (ra != kEwAcc) fast_fetch<UT>(p, rf, pos, full, ra, acc);
  if ((kTwoOperandOps >> op) & 1u) {
    float4 b[UT];
    fast_fetch<UT>(p, rf, pos, full, op == E_WHERE ? ins.c : ins.b, b);
    switch (op) {
      case E_ADD: map2<UT>(acc, b, [](float x, float y) { return fadd(x, y); }); break;
      case E_SUB: map2<UT>(acc, b, [](float x, float y) { return fadd(x, -y); }); break;
      case E_MUL: map2<UT>(acc, b, [](float x, float y) { return fmul(x, y); }); break;
      case E_DIV:
#pragma unroll
        for (int u = 0; u < UT; ++u) acc[u] = div4(acc[u], b[u]);
        break;
      case E_WHERE: {
        const char* c = rf.tbase + (uint32_t)ins.a * rf.rstride;
#pragma unroll
        for (int u = 0; u < UT; ++u) {
          const uint4 m = *reinterpret_cast<const uint4*>(c + u * rf.ustride);
          acc[u] = make_float4(m.x ? acc[u].x : b[u].x, m.y ? acc[u].y : b[u].y, m.z ? acc[u].z : b[u].z, m.w ? acc[u].w : b[u].w);
        }
        break;
      }
      default:   // E_CMP: the result is a predicate register in shared memory; the accumulator keeps operand a
        switch (ins.aux) {
          case BG_CMP_EQ: cmp_put<UT>(rf, ins.dst, acc, b, [](float x, float y) { return (uint32_t)(x == y); }); break;
          case BG_CMP_NE: cmp_put<UT>(rf, ins.dst, acc, b, [](float x, float y) { return (uint32_t)(x != y); }); break;
          case BG_CMP_LT: cmp_put<UT>(rf, ins.dst, acc, b, [](float x, float y) { return (uint32_t)(x < y); }); break;
          case BG_CMP_LE: cmp_put<UT>(rf, ins.dst, acc, b, [](float x, float y) { return (uint32_t)(x <= y); }); break;
          case BG_CMP_GT: cmp_put<UT>(rf, ins.dst, acc, b, [](float x, float y) { return (uint32_t)(x > y); }); break;
          default: cmp_put<UT>(rf, ins.dst, acc, b, [](float x, float y) { return (uint32_t)(x >= y); }); break;
        }
        return;
    }
  } else {
#define BG_CALL4(FN) _Pragma("unroll") for (int u = 0; u < UT; ++u) acc[u] = FN(acc[u])
    switch (op) {
      case E_NEG: map1<UT>(acc, [](float x) { return -x; }); break;
      case E_RELU: map1<UT>(acc, [](float x) { return x > 0.f ? x : 0.f; }); break;
      case E_EXPNEG:
        map1<UT>(acc, [](float x) { return -x; });
        // fall through
      case E_EXP: map1<UT>(acc, [](float x) { return expf(x); }); break;
      case E_GELU: map1<UT>(acc, [](float x) { return gelu1(x); }); break;
      case E_LOG: BG_CALL4(log4); break;
      case E_ABS: map1<UT>(acc, [](float x) { return x < 0 ? -x : (x == 0 ? 0.f : x); }); break;
      case E_SIGN: BG_CALL4(sign4); break;
      case E_SIN: BG_CALL4(sin4); break;
      case E_COS: BG_CALL4(cos4); break;
      default: break;   // E_COPY
    }
#undef BG_CALL4
  }
  fast_put<UT>(p, rf, pos, full, ins.dst, acc);
}

template <int UT, typename T>
__device__ __forceinline__ void float_instr(const EwInstr ins, const RegFile& rf) {
  const int nU = UT > 0 ? UT : rf.U;
  switch (ins.op) {
    case E_ADD: BG_BINARY(T, fadd(x, y)) break;
    case E_MUL: BG_BINARY(T, fmul(x, y)) break;
    case E_DIV: BG_BINARY(T, fdiv(x, y)) break;
    case E_NEG: BG_UNARY(T, -x) break;
    case E_EXP: BG_UNARY(T, f_exp<T>(x)) break;
    case E_LOG: BG_UNARY(T, f_log<T>(x)) break;
    case E_ABS: BG_UNARY(T, x < 0 ? -x : (x == 0 ? T(0) : x)) break;
    case E_SIGN: BG_UNARY(T, x != x ? x : T((x > 0) - (x < 0))) break;
    case E_SIN: BG_UNARY(T, f_sin<T>(x)) break;
    default: BG_UNARY(T, f_cos<T>(x)) break;
  }
}

template <int UT>
__device__ __forceinline__ void int_instr(const EwInstr ins, const RegFile& rf) {
  const int nU = UT > 0 ? UT : rf.U;
  typedef long long T;
  typedef unsigned long long UL;
  switch (ins.op) {
    case E_ADD: BG_BINARY(T, (T)((UL)x + (UL)y)) break;
    case E_MUL: BG_BINARY(T, (T)((UL)x * (UL)y)) break;
    case E_DIV: BG_BINARY(T, (T)((double)x / (double)y)) break;
    case E_NEG: BG_UNARY(T, (T)(0ull - (UL)x)) break;
    case E_ABS: BG_UNARY(T, x < 0 ? (T)(0ull - (UL)x) : x) break;
    default: BG_UNARY(T, (T)((x > 0) - (x < 0))) break;
  }
}

template <int UT, typename T>
__device__ __forceinline__ void where_instr(const EwInstr ins, const RegFile& rf) {
  const int nU = UT > 0 ? UT : rf.U;
  BG_FOR_U {
    V4<uint32_t> c = rget<uint32_t>(rf, ins.a, u);
    V4<T> x = rget<T>(rf, ins.b, u), y = rget<T>(rf, ins.c, u), r;
#pragma unroll
    for (int e = 0; e < 4; ++e) r.v[e] = c.v[e] ? x.v[e] : y.v[e];
    rput<T>(rf, ins.dst, u, r);
  }
}

template <int UT, typename T>
__device__ __forceinline__ void cmp_instr(const EwInstr ins, const RegFile& rf) {
  const int nU = UT > 0 ? UT : rf.U;
  BG_FOR_U {
    V4<T> a = rget<T>(rf, ins.a, u), b = rget<T>(rf, ins.b, u);
    V4<uint32_t> r;
#pragma unroll
    for (int e = 0; e < 4; ++e) r.v[e] = cmp_op<T>(a.v[e], b.v[e], ins.aux);
    rput<uint32_t>(rf, ins.dst, u, r);
  }
}

template <typename S, typename D> __device__ __forceinline__ D cvt1(S x) { return (D)x; }
template <> __device__ __forceinline__ uint32_t cvt1<float, uint32_t>(float x) { return x != 0.0f; }
template <> __device__ __forceinline__ uint32_t cvt1<double, uint32_t>(double x) { return x != 0.0; }
template <> __device__ __forceinline__ uint32_t cvt1<long long, uint32_t>(long long x) { return x != 0; }
template <> __device__ __forceinline__ float cvt1<double, float>(double x) { return __double2float_rn(x); }
template <> __device__ __forceinline__ float cvt1<long long, float>(long long x) { return __ll2float_rn(x); }
template <> __device__ __forceinline__ double cvt1<long long, double>(long long x) { return __ll2double_rn(x); }
template <> __device__ __forceinline__ long long cvt1<float, long long>(float x) { return __float2ll_rz(x); }
template <> __device__ __forceinline__ long long cvt1<double, long long>(double x) { return __double2ll_rz(x); }

template <typename S, typename D>
__device__ __forceinline__ void cvt_instr(const EwInstr ins, const RegFile& rf) {
  const int nU = rf.U;
#pragma unroll 1
  for (int u = 0; u < nU; ++u) {
    V4<S> a = rget<S>(rf, ins.a, u);
    V4<D> r;
#pragma unroll
    for (int e = 0; e < 4; ++e) r.v[e] = cvt1<S, D>(a.v[e]);
    rput<D>(rf, ins.dst, u, r);
  }
}

template <typename S> __device__ __forceinline__ void cvt_from(const EwInstr ins, const RegFile& rf) {
  switch (ins.type) {
    case T_F32: cvt_instr<S, float>(ins, rf); break;
    case T_F64: cvt_instr<S, double>(ins, rf); break;
    case T_I64: cvt_instr<S, long long>(ins, rf); break;
    default: cvt_instr<S, uint32_t>(ins, rf); break;
  }
}

// Everything outside the fp32 fast path, out of line and shared by every kernel: loads and stores of any
// dtype and addressing mode, constants, conversions, 64-bit and boolean arithmetic.
__device__ __noinline__ void slow_instr(const EwProgram& p, const EwInstr ins, const RegFile rf, const Pos pos) {
  const int nU = rf.U;
  switch (ins.op) {
    case E_LOAD:
#pragma unroll 1
      for (int u = 0; u < nU; ++u) load_chunk(p, ins, rf, u, ChunkPos{pos.idx(u), pos.nvalid(u)});
      break;
    case E_STORE:
#pragma unroll 1
      for (int u = 0; u < nU; ++u) store_chunk(p, ins, rf, u, ChunkPos{pos.idx(u), pos.nvalid(u)});
      break;
    case E_CONST: {
      const int64_t bits = p.consts[ins.aux];
#pragma unroll 1
      for (int u = 0; u < nU; ++u) {
        if (ins.type == T_F32) {
          float f = (float)__longlong_as_double(bits);
          rput<float>(rf, ins.dst, u, {{f, f, f, f}});
        } else if (ins.type == T_F64) {
          double d = __longlong_as_double(bits);
          rput<double>(rf, ins.dst, u, {{d, d, d, d}});
        } else if (ins.type == T_I64) {
          rput<long long>(rf, ins.dst, u, {{bits, bits, bits, bits}});
        } else {
          uint32_t b = bits != 0;
          rput<uint32_t>(rf, ins.dst, u, {{b, b, b, b}});
        }
      }
      break;
    }
    case E_ISNAN:
#pragma unroll 1
      for (int u = 0; u < nU; ++u) {
        V4<uint32_t> r;
        if (ins.type == T_F32) {
          V4<float> a = rget<float>(rf, ins.a, u);
#pragma unroll
          for (int e = 0; e < 4; ++e) r.v[e] = a.v[e] != a.v[e];
        } else if (ins.type == T_F64) {
          V4<double> a = rget<double>(rf, ins.a, u);
#pragma unroll
          for (int e = 0; e < 4; ++e) r.v[e] = a.v[e] != a.v[e];
        } else {
          r = {{0, 0, 0, 0}};
        }
        rput<uint32_t>(rf, ins.dst, u, r);
      }
      break;
    case E_CVT:
      switch (ins.aux & 0xF) {
        case T_F32: cvt_from<float>(ins, rf); break;
        case T_F64: cvt_from<double>(ins, rf); break;
        case T_I64: cvt_from<long long>(ins, rf); break;
        default: cvt_from<uint32_t>(ins, rf); break;
      }
      break;
    case E_NARROW:
#pragma unroll 1
      for (int u = 0; u < nU; ++u) {
        if (ins.type == T_F32) {
          V4<float> a = rget<float>(rf, ins.a, u);
#pragma unroll
          for (int e = 0; e < 4; ++e) a.v[e] = narrow_f32(a.v[e], ins.aux);
          rput<float>(rf, ins.dst, u, a);
        } else if (ins.type == T_I64) {
          V4<long long> a = rget<long long>(rf, ins.a, u);
#pragma unroll
          for (int e = 0; e < 4; ++e) a.v[e] = narrow_i64(a.v[e], ins.aux);
          rput<long long>(rf, ins.dst, u, a);
        }
      }
      break;
    case E_AND: case E_OR:
#pragma unroll 1
      for (int u = 0; u < nU; ++u) {
        V4<uint32_t> a = rget<uint32_t>(rf, ins.a, u), b = rget<uint32_t>(rf, ins.b, u);
#pragma unroll
        for (int e = 0; e < 4; ++e) a.v[e] = ins.op == E_AND ? (a.v[e] & b.v[e]) : (a.v[e] | b.v[e]);
        rput<uint32_t>(rf, ins.dst, u, a);
      }
      break;
    case E_CMP:
      if (ins.type == T_F64) cmp_instr<0, double>(ins, rf);
      else if (ins.type == T_I64) cmp_instr<0, long long>(ins, rf);
      else cmp_instr<0, uint32_t>(ins, rf);
      break;
    case E_WHERE:
      if (ins.type == T_F64) where_instr<0, double>(ins, rf);
      else if (ins.type == T_I64) where_instr<0, long long>(ins, rf);
      else where_instr<0, uint32_t>(ins, rf);
      break;
    default:
      if (ins.type == T_F64) float_instr<0, double>(ins, rf);
      else int_instr<0>(ins, rf);
      break;
  }
}

// The program over the UT chunks of one pass.
// `acc` is the accumulator; the caller may read the last instruction's result from it.
template <int UT>
__device__ __forceinline__ void run_program(const EwProgram& p, const RegFile& rf, const Pos& pos, float4 (&acc)[UT]) {
#pragma unroll
  for (int u = 0; u < UT; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool full = pos.end - pos.idx(UT - 1) >= 4;   // every chunk of this thread is complete
#pragma unroll 1
  for (int i = 0; i < p.n_instr; ++i) {
    const EwInstr ins = p.instr[i];
    if (ins.type == T_F32 && ((kFastOps >> ins.op) & 1u)) {
      fast_instr<UT>(p, ins, rf, pos, full, acc);
    } else {
      slow_instr(p, ins, rf, pos);
      // nothing reads the accumulator across an instruction of the slow path: it need not survive the call
#pragma unroll
      for (int u = 0; u < UT; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// ------------------------------------------------------------------------------------
// Flat elementwise kernel
// ------------------------------------------------------------------------------------
template <int UT>
__global__ void __launch_bounds__(kBlock, BG_EW_MIN_CTAS) ew_kernel(const __grid_constant__ EwProgram p, int U, int64_t n_tiles) {
  extern __shared__ __align__(16) char smem[];
  const RegFile rf(smem, U, p.wide ? 2 : 1);
  const int64_t tile_elems = (int64_t)U * kChunk;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const Pos pos{tile * tile_elems + (int64_t)threadIdx.x * kVec, p.numel};
    float4 acc[UT];
    run_program<UT>(p, rf, pos, acc);
  }
}

// Shared-memory opt-in and carve-out for a launch with `smem` dynamic bytes; *ctas_per_sm receives how many
// CTAs of it one SM holds, which sizes the grid of the persistent loops.
static cudaError_t prepare_kernel(const void* kern, size_t smem, int* ctas_per_sm) {
  // remembered per (device, kernel, size): the attribute and occupancy calls cost microseconds each
  static std::mutex mu;
  static std::map<std::tuple<int, const void*, size_t>, int> known;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const auto key = std::make_tuple(dev, kern, smem);
  std::lock_guard<std::mutex> lock(mu);
  auto it = known.find(key);
  if (it != known.end()) { *ctas_per_sm = it->second; return cudaSuccess; }
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  int n = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kBlock, smem);
  if (e != cudaSuccess) return e;
  *ctas_per_sm = n < 1 ? 1 : n;
  known[key] = *ctas_per_sm;
  return cudaSuccess;
}

cudaError_t launch_elementwise(const EwProgram& p, cudaStream_t s, int sm_count) {
  if (p.numel == 0) return cudaSuccess;
  const int planes = p.wide ? 2 : 1;
  const size_t per_chunk = (size_t)p.n_regs * planes * kBlock * 16;
  int U = 4;
  while (U > 1 && (per_chunk * U > 64 * 1024 || p.numel < (int64_t)kChunk * U * sm_count)) U >>= 1;
  const size_t smem = per_chunk * U;
  if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
  auto kern = U == 4 ? ew_kernel<4> : (U == 2 ? ew_kernel<2> : ew_kernel<1>);
  const int64_t tile_elems = (int64_t)U * kChunk;
  const int64_t n_tiles = (p.numel + tile_elems - 1) / tile_elems;
  int ctas_per_sm = 1;
  cudaError_t e = prepare_kernel(reinterpret_cast<const void*>(kern), smem, &ctas_per_sm);
  if (e != cudaSuccess) return e;
  int64_t grid = (int64_t)sm_count * ctas_per_sm;
  if (grid > n_tiles) grid = n_tiles;
  kern<<<(unsigned)grid, kBlock, smem, s>>>(p, U, n_tiles);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------
// Row kernel: program + on-chip tail over the last axis
// ------------------------------------------------------------------------------------
// Reduction over the CTA with one barrier.  Warp results go to one of two scratch buffers, `flip` says which and
// alternates from call to call: a buffer is written again only after the barrier of the call in between, which
// every thread passes after it has read the buffer.  Lane l of every warp combines buffer entries l & 7 by the same
// butterfly, so all threads hold the same bits.
template <typename T, typename F>
__device__ __forceinline__ T block_reduce(T v, F f, char* scratch, int& flip) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T other = __shfl_xor_sync(0xffffffffu, v, o);
    v = f(v, other);
  }
  T* s = reinterpret_cast<T*>(scratch + 256 + flip * 64);
  flip ^= 1;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) s[w] = v;
  __syncthreads();
  T r = s[l & (kBlock / 32 - 1)];
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    T other = __shfl_xor_sync(0xffffffffu, r, o);
    r = f(r, other);
  }
  return r;
}

template <typename T> __device__ __forceinline__ T lowest();
template <> __device__ __forceinline__ float lowest<float>() { return -CUDART_INF_F; }
template <> __device__ __forceinline__ double lowest<double>() { return -CUDART_INF; }
template <> __device__ __forceinline__ long long lowest<long long>() { return (long long)0x8000000000000000ull; }
template <typename T> __device__ __forceinline__ T highest();
template <> __device__ __forceinline__ float highest<float>() { return CUDART_INF_F; }
template <> __device__ __forceinline__ double highest<double>() { return CUDART_INF; }
template <> __device__ __forceinline__ long long highest<long long>() { return 0x7fffffffffffffffll; }

template <typename T>
__device__ __forceinline__ bool arg_better(T v, long long i, T bv, long long bi, bool want_max) {
  // First occurrence wins; a NaN beats every number (NumPy argmax/argmin propagate the first NaN).
  const bool vn = v != v, bn = bv != bv;
  if (bi < 0) return true;
  if (vn || bn) {
    if (vn && bn) return i < bi;
    return vn;
  }
  if (v == bv) return i < bi;
  return want_max ? v > bv : v < bv;
}

template <typename T>
__device__ __forceinline__ void block_argreduce(T& v, long long& i, bool want_max, char* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T ov = __shfl_xor_sync(0xffffffffu, v, o);
    long long oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (oi >= 0 && arg_better<T>(ov, oi, v, i, want_max)) { v = ov; i = oi; }
  }
  T* sv = reinterpret_cast<T*>(scratch);
  long long* si = reinterpret_cast<long long*>(scratch + 64);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) { sv[w] = v; si[w] = i; }
  __syncthreads();
  if (l < kBlock / 32) { v = sv[l]; i = si[l]; } else { i = -1; }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    T ov = __shfl_xor_sync(0xffffffffu, v, o);
    long long oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (oi >= 0 && arg_better<T>(ov, oi, v, i, want_max)) { v = ov; i = oi; }
  }
  v = __shfl_sync(0xffffffffu, v, 0);
  i = __shfl_sync(0xffffffffu, i, 0);
}

__device__ __forceinline__ void store_scalar(void* ptr, int dt, int64_t i, double fv, long long iv, bool is_int) {
  switch (dt) {
    case BG_F32: reinterpret_cast<float*>(ptr)[i] = is_int ? (float)iv : (float)fv; break;
    case BG_F64: reinterpret_cast<double*>(ptr)[i] = is_int ? (double)iv : fv; break;
    case BG_F16: reinterpret_cast<__half*>(ptr)[i] = __float2half_rn(is_int ? (float)iv : (float)fv); break;
    case BG_BF16: reinterpret_cast<__nv_bfloat16*>(ptr)[i] = __float2bfloat16_rn(is_int ? (float)iv : (float)fv); break;
    case BG_BOOL: reinterpret_cast<unsigned char*>(ptr)[i] = is_int ? (iv != 0) : (fv != 0.0); break;
    default: st_i64class(ptr, dt, i, is_int ? iv : (long long)fv); break;
  }
}

// The program over chunks [c_begin, c_end) of a row that starts at linear index row_base and ends before
// row_end: groups of four chunks, then single chunks.  With `resident` chunk c uses slot c of the register
// file (the whole row stays on chip); otherwise chunk c uses slot c - c_begin.
// `last` receives the accumulator of the last group (all four entries after a group of four, entry 0 after a single chunk).
__device__ __forceinline__ void run_row_chunks(const EwProgram& p, const RegFile& rf, int64_t row_base, int64_t row_end, int c_begin,
                                               int c_end, bool resident, float4 (&last)[4]) {
  int c = c_begin;
  for (; c + 4 <= c_end; c += 4) {
    const Pos pos{row_base + (int64_t)c * kChunk + (int64_t)threadIdx.x * kVec, row_end};
    run_program<4>(p, rf.group(resident ? c : c - c_begin, 4), pos, last);
  }
  for (; c < c_end; ++c) {
    const Pos pos{row_base + (int64_t)c * kChunk + (int64_t)threadIdx.x * kVec, row_end};
    float4 one[1];
    run_program<1>(p, rf.group(resident ? c : c - c_begin, 1), pos, one);
    last[0] = one[0];
  }
}

// Reduction over one row with values of class T arriving pass by pass (up to four chunks per pass).
template <typename T>
__device__ __forceinline__ void row_reduce(const EwProgram& p, const RegFile& rf, int64_t row, int64_t n_chunks,
                                           char* scratch, int& flip) {
  const int op = p.tail_arg;
  const bool is_arg = op == BG_RED_ARGMAX || op == BG_RED_ARGMIN;
  T acc = T(0);
  long long best_i = -1;
  if (op == BG_RED_MAX) acc = lowest<T>();
  if (op == BG_RED_MIN) acc = highest<T>();
  if (op == BG_RED_PROD) acc = T(1);
  bool any_nan = false;
  const int64_t row_base = row * p.cols;
  const int64_t row_end = row_base + p.cols;
  const int step = rf.U >= 4 ? 4 : 1;
  for (int64_t c0 = 0; c0 < n_chunks; c0 += step) {
    const int nU = n_chunks - c0 >= step ? step : (int)(n_chunks - c0);
    const int64_t col0 = c0 * kChunk + (int64_t)threadIdx.x * kVec;
    const Pos pos{row_base + col0, row_end};
    float4 last[4];
    run_row_chunks(p, rf, row_base, row_end, (int)c0, (int)c0 + nU, false, last);
    if (op == BG_RED_SUM || op == BG_RED_MEAN) {
      if (nU == 4 && pos.end - pos.idx(3) >= 4) {
        if (sizeof(T) == 4 && p.tail_acc) {
#pragma unroll
          for (int u = 0; u < 4; ++u) acc += (T)((last[u].x + last[u].y) + (last[u].z + last[u].w));
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            V4<T> x = rget<T>(rf, p.tail_reg, u);
            acc += (x.v[0] + x.v[1]) + (x.v[2] + x.v[3]);
          }
        }
        continue;
      }
    }
#pragma unroll 1
    for (int u = 0; u < nU; ++u) {
      const int nv = pos.nvalid(u);
      if (nv == 0) continue;
      const int64_t col = col0 + (int64_t)u * kChunk;
      V4<T> x = rget<T>(rf, p.tail_reg, u);
      for (int e = 0; e < nv; ++e) {
        const T v = x.v[e];
        if (op == BG_RED_SUM || op == BG_RED_MEAN) { acc += v; continue; }
        if (op == BG_RED_PROD) { acc *= v; continue; }
        if (is_arg) {
          if (arg_better<T>(v, col + e, acc, best_i, op == BG_RED_ARGMAX)) { acc = v; best_i = col + e; }
        } else {
          if (v != v) any_nan = true;
          if (op == BG_RED_MAX) acc = v > acc ? v : acc;
          else acc = v < acc ? v : acc;
        }
      }
    }
  }
  constexpr bool kIsInt = sizeof(T) == 8 && (T(1) / T(2) == T(0));
  if (is_arg) {
    block_argreduce<T>(acc, best_i, op == BG_RED_ARGMAX, scratch);
    if (threadIdx.x == 0) store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, 0.0, best_i, true);
    return;
  }
  if (op == BG_RED_SUM || op == BG_RED_MEAN) {
    acc = block_reduce<T>(acc, [](T a, T b) { return a + b; }, scratch, flip);
    if (threadIdx.x == 0) {
      if (op == BG_RED_MEAN) {
        if (kIsInt) store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, (double)acc / (double)p.cols, 0, false);
        else store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, (double)(acc / (T)p.cols), 0, false);
      } else {
        store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, (double)acc, (long long)acc, kIsInt);
      }
    }
    return;
  }
  if (op == BG_RED_PROD) {
    acc = block_reduce<T>(acc, [](T a, T b) { return a * b; }, scratch, flip);
    if (threadIdx.x == 0) store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, (double)acc, (long long)acc, kIsInt);
    return;
  }
  const bool want_max = op == BG_RED_MAX;
  acc = block_reduce<T>(acc, [want_max](T a, T b) { return want_max ? (a > b ? a : b) : (a < b ? a : b); }, scratch, flip);
  int nan_any = __syncthreads_or(any_nan ? 1 : 0);
  if (threadIdx.x == 0) {
    double fv = (double)acc;
    if (nan_any && !kIsInt) fv = CUDART_NAN;
    store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, fv, (long long)acc, kIsInt);
  }
}

__device__ __forceinline__ void row_reduce_bool(const EwProgram& p, const RegFile& rf, int64_t row, int64_t n_chunks) {
  const int step = rf.U >= 4 ? 4 : 1;
  const bool is_any = p.tail_arg == BG_RED_ANY;
  int local = is_any ? 0 : 1;
  const int64_t row_base = row * p.cols;
  const int64_t row_end = row_base + p.cols;
  for (int64_t c0 = 0; c0 < n_chunks; c0 += step) {
    const int nU = n_chunks - c0 >= step ? step : (int)(n_chunks - c0);
    const Pos pos{row_base + c0 * kChunk + (int64_t)threadIdx.x * kVec, row_end};
    float4 last[4];
    run_row_chunks(p, rf, row_base, row_end, (int)c0, (int)c0 + nU, false, last);
#pragma unroll 1
    for (int u = 0; u < nU; ++u) {
      const int nv = pos.nvalid(u);
      V4<uint32_t> x = rget<uint32_t>(rf, p.tail_reg, u);
      for (int e = 0; e < nv; ++e) {
        if (is_any) local |= (x.v[e] != 0);
        else local &= (x.v[e] != 0);
      }
    }
  }
  int r = is_any ? __syncthreads_or(local) : __syncthreads_and(local);
  if (threadIdx.x == 0) store_scalar(p.outputs[p.tail_out].ptr, p.tail_out_dtype, row, 0.0, r != 0, true);
}

// exp(x - m) and the division by the row sum of the fp32 softmax tails, as the specialised softmax kernel does them:
// 2^((x - m) * log2 e) on the hardware exp2 unit (x - m <= 0 is bounded by the row's range, so the rounding of the
// argument stays near 1e-6 relative), one IEEE reciprocal per row and one multiply per element.  fp64 rows keep
// exp() and a true division.
template <typename T> __device__ __forceinline__ T softmax_exp(T x, T m);
template <> __device__ __forceinline__ float softmax_exp<float>(float x, float m) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmul(fadd(x, -m), 1.4426950408889634f)));
  return y;
}
template <> __device__ __forceinline__ double softmax_exp<double>(double x, double m) { return exp(fadd(x, -m)); }
template <typename T> __device__ __forceinline__ T softmax_scale(T sum);
template <> __device__ __forceinline__ float softmax_scale<float>(float sum) { return __fdiv_rn(1.0f, sum); }
template <> __device__ __forceinline__ double softmax_scale<double>(double sum) { return sum; }
template <typename T> __device__ __forceinline__ T softmax_norm(T e, T scale);
template <> __device__ __forceinline__ float softmax_norm<float>(float e, float scale) { return fmul(e, scale); }
template <> __device__ __forceinline__ double softmax_norm<double>(double e, double scale) { return fdiv(e, scale); }

// Softmax of a row of N complete fp32 chunks with the row in real registers: same operations in the same order as
// the general tail below.  A NaN in the row needs no test of its own: the maximum skips it, its exponential is NaN,
// so is the sum, and every quotient by that sum.
template <int N>
__device__ __forceinline__ void softmax_in_registers(const RegFile& rf, int r, bool in_acc, const float4 (&last)[4], float* dst,
                                                     char* scratch, int& flip) {
  float4 x[N];
  if (in_acc) {
#pragma unroll
    for (int u = 0; u < N; ++u) x[u] = last[u];
  } else {
#pragma unroll
    for (int u = 0; u < N; ++u) x[u] = *reinterpret_cast<const float4*>(rf.slot(r, u, 0));
  }
  float m = -CUDART_INF_F;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    m = x[u].x > m ? x[u].x : m;
    m = x[u].y > m ? x[u].y : m;
    m = x[u].z > m ? x[u].z : m;
    m = x[u].w > m ? x[u].w : m;
  }
  m = block_reduce<float>(m, [](float a, float b) { return a > b ? a : b; }, scratch, flip);
  float sum = 0.f;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    x[u] = make_float4(softmax_exp<float>(x[u].x, m), softmax_exp<float>(x[u].y, m), softmax_exp<float>(x[u].z, m),
                       softmax_exp<float>(x[u].w, m));
    sum += x[u].x;
    sum += x[u].y;
    sum += x[u].z;
    sum += x[u].w;
  }
  sum = block_reduce<float>(sum, [](float a, float b) { return a + b; }, scratch, flip);
  const float inv = softmax_scale<float>(sum);
#pragma unroll
  for (int u = 0; u < N; ++u)
    reinterpret_cast<float4*>(dst)[u * (kChunk / 4)] = make_float4(fmul(x[u].x, inv), fmul(x[u].y, inv), fmul(x[u].z, inv), fmul(x[u].w, inv));
}

// softmax / layer norm: the whole row stays in the register file (n_chunks <= U).
template <typename T, bool SOFTMAX>
__device__ __forceinline__ void row_resident_tail(const EwProgram& p, const RegFile& rf, int64_t row, char* scratch, int& flip) {
  const int nU = rf.U;
  const int64_t col0 = (int64_t)threadIdx.x * kVec;
  const Pos pos{row * p.cols + col0, (row + 1) * p.cols};
  float4 last[4];
  run_row_chunks(p, rf, row * p.cols, (row + 1) * p.cols, 0, nU, true, last);
  const int r = p.tail_reg;
  const EwOutput& out = p.outputs[p.tail_out];
  const bool full = pos.end - pos.idx(nU - 1) >= 4;   // every chunk of this thread is complete
  // (the test is the same for every thread of the CTA: the branch holds barriers)
  if (SOFTMAX && sizeof(T) == 4 && p.cols == (int64_t)nU * kChunk && out.vec_ok && out.dtype == BG_F32 &&
      (nU == 4 || nU == 2 || nU == 1)) {
    const bool in_acc = p.tail_acc && nU != 2;
    float* dst = reinterpret_cast<float*>(out.ptr) + pos.idx0;
    if (nU == 4) softmax_in_registers<4>(rf, r, in_acc, last, dst, scratch, flip);
    else if (nU == 2) softmax_in_registers<2>(rf, r, in_acc, last, dst, scratch, flip);
    else softmax_in_registers<1>(rf, r, in_acc, last, dst, scratch, flip);
    return;
  }
  if (SOFTMAX) {
    T m = lowest<T>();
    bool nan = false;
    BG_FOR_U {
      const int nv = full ? 4 : pos.nvalid(u);
      V4<T> x = rget<T>(rf, r, u);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < nv) {
          if (x.v[e] != x.v[e]) nan = true;
          m = x.v[e] > m ? x.v[e] : m;
        }
    }
    m = block_reduce<T>(m, [](T a, T b) { return a > b ? a : b; }, scratch, flip);
    if (__syncthreads_or(nan ? 1 : 0)) m = (T)CUDART_NAN;
    T sum = T(0);
    BG_FOR_U {
      const int nv = full ? 4 : pos.nvalid(u);
      if (nv > 0) {
        V4<T> x = rget<T>(rf, r, u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          x.v[e] = softmax_exp<T>(x.v[e], m);
          if (e < nv) sum += x.v[e];
        }
        rput<T>(rf, r, u, x);
      }
    }
    sum = block_reduce<T>(sum, [](T a, T b) { return a + b; }, scratch, flip);
    const T scale = softmax_scale<T>(sum);
    const EwInstr st{E_STORE, (uint8_t)p.tail_type, 0, (uint8_t)r, 0, 0, (uint16_t)p.tail_out};
    BG_FOR_U {
      const int nv = full ? 4 : pos.nvalid(u);
      if (nv > 0) {
        V4<T> x = rget<T>(rf, r, u);
#pragma unroll
        for (int e = 0; e < 4; ++e) x.v[e] = softmax_norm<T>(x.v[e], scale);
        if (sizeof(T) == 4 && nv == 4 && out.vec_ok && out.dtype == BG_F32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(out.ptr) + pos.idx(u)) =
              make_float4((float)x.v[0], (float)x.v[1], (float)x.v[2], (float)x.v[3]);
        } else {
          rput<T>(rf, r, u, x);
          store_chunk(p, st, rf, u, ChunkPos{pos.idx(u), nv});
        }
      }
    }
  } else {  // TAIL_LAYERNORM, fp32 statistics as in the reference (x.astype(float32))
    float sum = 0.f;
    BG_FOR_U {
      const int nv = full ? 4 : pos.nvalid(u);
      V4<T> x = rget<T>(rf, r, u);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < nv) sum += (float)x.v[e];
    }
    sum = block_reduce<float>(sum, [](float a, float b) { return a + b; }, scratch, flip);
    const float mean = sum / (float)p.cols;
    float sq = 0.f;
    BG_FOR_U {
      const int nv = full ? 4 : pos.nvalid(u);
      V4<T> x = rget<T>(rf, r, u);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < nv) {
          float c = __fadd_rn((float)x.v[e], -mean);
          sq += __fmul_rn(c, c);
        }
    }
    sq = block_reduce<float>(sq, [](float a, float b) { return a + b; }, scratch, flip);
    const float var = sq / (float)p.cols;
    const float inv = 1.0f / sqrtf(var + p.tail_eps);
    const EwOperand& w = p.inputs[p.tail_w];
    const EwOperand& b = p.inputs[p.tail_b];
    BG_FOR_U {
      const int nv = full ? 4 : pos.nvalid(u);
      if (nv > 0) {
        const int64_t col = col0 + (int64_t)u * kChunk;
        V4<T> x = rget<T>(rf, r, u);
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (e < nv) {
            float c = __fadd_rn((float)x.v[e], -mean);
            float xh = __fmul_rn(c, inv);
            float wv = w.dtype == BG_F64 ? (float)reinterpret_cast<const double*>(w.ptr)[col + e] : ld_f32class(w.ptr, w.dtype, col + e);
            float bv = b.dtype == BG_F64 ? (float)reinterpret_cast<const double*>(b.ptr)[col + e] : ld_f32class(b.ptr, b.dtype, col + e);
            y[e] = __fadd_rn(__fmul_rn(xh, wv), bv);
          }
        if (nv == 4 && out.vec_ok && out.dtype == BG_F32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(out.ptr) + pos.idx(u)) = make_float4(y[0], y[1], y[2], y[3]);
        } else if (nv == 4 && out.vec_ok && out.dtype == BG_F64) {
          double* q = reinterpret_cast<double*>(out.ptr) + pos.idx(u);
          *reinterpret_cast<double2*>(q) = make_double2((double)y[0], (double)y[1]);
          *reinterpret_cast<double2*>(q + 2) = make_double2((double)y[2], (double)y[3]);
        } else {
          for (int e = 0; e < nv; ++e) store_scalar(out.ptr, out.dtype, pos.idx(u) + e, (double)y[e], 0, false);
        }
      }
    }
  }
}

// One kernel per kind of tail, so that each carries only its own tail's registers.
enum RowKind {
  ROW_REDUCE_F32 = 0, ROW_REDUCE_F64, ROW_REDUCE_I64, ROW_REDUCE_BOOL,
  ROW_SOFTMAX_F32, ROW_SOFTMAX_F64, ROW_LAYERNORM_F32, ROW_LAYERNORM_F64
};

template <int KIND>
__global__ void __launch_bounds__(kBlock, BG_EW_MIN_CTAS) row_kernel(const __grid_constant__ EwProgram p, int U, int64_t n_chunks) {
  extern __shared__ __align__(16) char smem[];
  const int planes = p.wide ? 2 : 1;
  const RegFile rf(smem, U, planes);
  char* scratch = smem + (size_t)p.n_regs * U * planes * kBlock * 16;
  int flip = 0;   // which scratch buffer the next block reduction uses
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    if (KIND == ROW_REDUCE_F32) row_reduce<float>(p, rf, row, n_chunks, scratch, flip);
    else if (KIND == ROW_REDUCE_F64) row_reduce<double>(p, rf, row, n_chunks, scratch, flip);
    else if (KIND == ROW_REDUCE_I64) row_reduce<long long>(p, rf, row, n_chunks, scratch, flip);
    else if (KIND == ROW_REDUCE_BOOL) row_reduce_bool(p, rf, row, n_chunks);
    else if (KIND == ROW_SOFTMAX_F32) row_resident_tail<float, true>(p, rf, row, scratch, flip);
    else if (KIND == ROW_SOFTMAX_F64) row_resident_tail<double, true>(p, rf, row, scratch, flip);
    else if (KIND == ROW_LAYERNORM_F32) row_resident_tail<float, false>(p, rf, row, scratch, flip);
    else row_resident_tail<double, false>(p, rf, row, scratch, flip);
  }
}

int rowwise_max_chunks(int n_regs, int wide) {
  const size_t per_chunk = (size_t)(n_regs > 0 ? n_regs : 1) * (wide ? 2 : 1) * kBlock * 16;
  return (int)((200 * 1024 - 512) / per_chunk);
}

cudaError_t launch_rowwise(const EwProgram& p, cudaStream_t s, int sm_count, int* /*status_flag*/) {
  if (p.rows == 0) return cudaSuccess;
  const int planes = p.wide ? 2 : 1;
  const size_t per_chunk = (size_t)p.n_regs * planes * kBlock * 16;
  const int64_t n_chunks = (p.cols + kChunk - 1) / kChunk;
  int U;
  if (p.tail == TAIL_REDUCE) {
    // passes of four chunks where the row and the register file allow, else of one
    U = (n_chunks >= 4 && per_chunk * 4 <= 64 * 1024) ? 4 : 1;
  } else {
    U = (int)n_chunks;
  }
  if (U < 1) U = 1;
  const size_t smem = per_chunk * U + 512;
  if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
  void (*kern)(EwProgram, int, int64_t);
  if (p.tail == TAIL_REDUCE) {
    kern = p.tail_type == T_F32 ? row_kernel<ROW_REDUCE_F32>
         : p.tail_type == T_F64 ? row_kernel<ROW_REDUCE_F64>
         : p.tail_type == T_I64 ? row_kernel<ROW_REDUCE_I64> : row_kernel<ROW_REDUCE_BOOL>;
  } else {
    const bool wide_row = p.tail_type == T_F64;
    if (p.tail == TAIL_SOFTMAX) kern = wide_row ? row_kernel<ROW_SOFTMAX_F64> : row_kernel<ROW_SOFTMAX_F32>;
    else kern = wide_row ? row_kernel<ROW_LAYERNORM_F64> : row_kernel<ROW_LAYERNORM_F32>;
  }
  int ctas_per_sm = 1;
  cudaError_t e = prepare_kernel(reinterpret_cast<const void*>(kern), smem, &ctas_per_sm);
  if (e != cudaSuccess) return e;
  int64_t grid = (int64_t)sm_count * ctas_per_sm;
  if (grid > p.rows) grid = p.rows;
  kern<<<(unsigned)grid, kBlock, smem, s>>>(p, U, n_chunks);
  return cudaGetLastError();
}

}  // namespace bg
