// Data-movement kernels: TRIL / TRIU, FLIP, CONCAT blocks and CUMSUM.  Each reads a strided view (so a
// permuted or broadcast operand needs no dense copy first) and writes a dense row-major tensor.
// The work is bytes in, bytes out: one thread per output element, consecutive threads on consecutive
// output addresses; values are moved as 1 / 2 / 4 / 8-byte words, bit-exact.
// Reference semantics: np.tril / np.triu, np.flip, np.concatenate with a cast to the result dtype,
// np.cumsum(dtype = result dtype) (packages/browsergrad-jit/src/python/_realize.py:268-327).
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

namespace bg {
namespace {

struct ViewArg {
  const void* ptr;
  int rank;
  int64_t shape[kMaxRank];
  int64_t stride[kMaxRank];
};

ViewArg to_arg(const StridedView& v) {
  ViewArg a{};
  a.ptr = v.ptr;
  a.rank = v.rank;
  for (int d = 0; d < v.rank; ++d) { a.shape[d] = v.shape[d]; a.stride[d] = v.stride[d]; }
  return a;
}

unsigned grid_for(int64_t n) {
  int64_t g = (n + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  return (unsigned)(g < 1 ? 1 : g);
}

// mode 0: tri (p0 = upper, p1 = diagonal); mode 1: flip (p0 = axis)
template <typename W>
__global__ void index_map_kernel(ViewArg in, W* __restrict__ out, int64_t numel, int mode, int64_t p0, int64_t p1) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < numel; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, off = 0, row = 0, col = 0;
    for (int d = in.rank - 1; d >= 0; --d) {
      int64_t c = rem % in.shape[d];
      rem /= in.shape[d];
      if (d == in.rank - 1) col = c;
      if (d == in.rank - 2) row = c;
      if (mode == 1 && d == (int)p0) c = in.shape[d] - 1 - c;
      off += c * in.stride[d];
    }
    bool keep = true;
    if (mode == 0) keep = p0 ? (col - row >= p1) : (col - row <= p1);
    out[i] = keep ? reinterpret_cast<const W*>(in.ptr)[off] : W(0);
  }
}

template <typename W>
cudaError_t launch_index_map(const StridedView& in, void* out, int64_t numel, int mode, int64_t p0, int64_t p1, cudaStream_t s) {
  if (numel == 0) return cudaSuccess;
  index_map_kernel<W><<<grid_for(numel), 256, 0, s>>>(to_arg(in), reinterpret_cast<W*>(out), numel, mode, p0, p1);
  return cudaGetLastError();
}

cudaError_t dispatch_index_map(const StridedView& in, void* out, int64_t numel, int mode, int64_t p0, int64_t p1, cudaStream_t s) {
  switch (dtype_size(in.dtype)) {
    case 1: return launch_index_map<uint8_t>(in, out, numel, mode, p0, p1, s);
    case 2: return launch_index_map<uint16_t>(in, out, numel, mode, p0, p1, s);
    case 4: return launch_index_map<uint32_t>(in, out, numel, mode, p0, p1, s);
    default: return launch_index_map<unsigned long long>(in, out, numel, mode, p0, p1, s);
  }
}

// value conversion for CONCAT (inputs of mixed dtype are cast to the result dtype, as np.asarray(dtype=) does)
// and for CUMSUM (accumulation in the result dtype)
__device__ __forceinline__ double load_as_double(const void* p, int dt, int64_t i) {
  switch (dt) {
    case BG_F64: return reinterpret_cast<const double*>(p)[i];
    case BG_F32: return reinterpret_cast<const float*>(p)[i];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case BG_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case BG_I64: return (double)reinterpret_cast<const long long*>(p)[i];
    case BG_U64: return (double)reinterpret_cast<const unsigned long long*>(p)[i];
    case BG_I32: return reinterpret_cast<const int*>(p)[i];
    case BG_U32: return reinterpret_cast<const unsigned*>(p)[i];
    case BG_I16: return reinterpret_cast<const short*>(p)[i];
    case BG_U16: return reinterpret_cast<const unsigned short*>(p)[i];
    case BG_I8: return reinterpret_cast<const signed char*>(p)[i];
    default: return reinterpret_cast<const unsigned char*>(p)[i];   // u8, bool
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
    case BG_U8: case BG_BOOL: return reinterpret_cast<const unsigned char*>(p)[i];
    default: return (long long)load_as_double(p, dt, i);
  }
}
__device__ __forceinline__ bool is_int_dtype(int dt) {
  return dt == BG_I64 || dt == BG_U64 || dt == BG_I32 || dt == BG_U32 || dt == BG_I16 || dt == BG_U16 || dt == BG_I8 || dt == BG_U8 ||
         dt == BG_BOOL;
}
__device__ __forceinline__ void store_value(void* p, int dt, int64_t i, double f, long long n, bool from_int) {
  switch (dt) {
    case BG_F64: reinterpret_cast<double*>(p)[i] = from_int ? (double)n : f; break;
    case BG_F32: reinterpret_cast<float*>(p)[i] = from_int ? (float)n : (float)f; break;
    case BG_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(from_int ? (float)n : (float)f); break;
    case BG_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(from_int ? (float)n : (float)f); break;
    case BG_I64: case BG_U64: reinterpret_cast<long long*>(p)[i] = from_int ? n : (long long)f; break;
    case BG_I32: case BG_U32: reinterpret_cast<int*>(p)[i] = (int)(from_int ? n : (long long)f); break;
    case BG_I16: case BG_U16: reinterpret_cast<short*>(p)[i] = (short)(from_int ? n : (long long)f); break;
    case BG_BOOL: reinterpret_cast<unsigned char*>(p)[i] = from_int ? (n != 0) : (f != 0.0); break;
    default: reinterpret_cast<signed char*>(p)[i] = (signed char)(from_int ? n : (long long)f); break;
  }
}

struct PlaceArg {
  int64_t out_stride[kMaxRank];   // dense strides of the output
  int64_t base;                   // axis_offset * out_stride[axis]
  int fill;                       // 1: every element is the constant below (the source view gives the block's shape only)
  int fill_is_int;
  double fill_f;
  long long fill_n;
};

__global__ void place_kernel(ViewArg in, int in_dtype, void* out, int out_dtype, PlaceArg pa, int64_t numel) {
  const bool from_int = is_int_dtype(in_dtype);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < numel; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, src = 0, dst = pa.base;
    for (int d = in.rank - 1; d >= 0; --d) {
      const int64_t c = rem % in.shape[d];
      rem /= in.shape[d];
      src += c * in.stride[d];
      dst += c * pa.out_stride[d];
    }
    if (pa.fill) store_value(out, out_dtype, dst, pa.fill_f, pa.fill_n, pa.fill_is_int != 0);
    else if (from_int) store_value(out, out_dtype, dst, 0.0, load_as_i64(in.ptr, in_dtype, src), true);
    else store_value(out, out_dtype, dst, load_as_double(in.ptr, in_dtype, src), 0, false);
  }
}

// One thread per line along the scanned axis; consecutive threads take consecutive inner positions.
template <typename Acc>
__global__ void cumsum_kernel(ViewArg in, int in_dtype, void* out, int out_dtype, int axis, int reverse, int64_t lines, int64_t inner) {
  const int64_t len = in.shape[axis];
  for (int64_t line = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; line < lines; line += (int64_t)gridDim.x * blockDim.x) {
    // line enumerates (outer, inner) densely; recover the source offset of its first element
    const int64_t in_pos = line % inner, outer = line / inner;
    int64_t src0 = 0, rem = in_pos;
    for (int d = in.rank - 1; d > axis; --d) { src0 += (rem % in.shape[d]) * in.stride[d]; rem /= in.shape[d]; }
    rem = outer;
    for (int d = axis - 1; d >= 0; --d) { src0 += (rem % in.shape[d]) * in.stride[d]; rem /= in.shape[d]; }
    const int64_t dst0 = outer * len * inner + in_pos;
    Acc acc = Acc(0);
    for (int64_t k = 0; k < len; ++k) {
      const int64_t kk = reverse ? len - 1 - k : k;
      const int64_t so = src0 + kk * in.stride[axis], doff = dst0 + kk * inner;
      if (std::is_integral<Acc>::value) {
        acc += (Acc)load_as_i64(in.ptr, in_dtype, so);
        store_value(out, out_dtype, doff, 0.0, (long long)acc, true);
      } else {
        // the source is converted to the result dtype before it is added, as NumPy's dtype= argument does
        Acc x = (Acc)load_as_double(in.ptr, in_dtype, so);
        if (out_dtype == BG_F16) x = (Acc)__half2float(__float2half_rn((float)x));
        if (out_dtype == BG_BF16) x = (Acc)__bfloat162float(__float2bfloat16_rn((float)x));
        acc += x;
        if (out_dtype == BG_F16) acc = (Acc)__half2float(__float2half_rn((float)acc));
        if (out_dtype == BG_BF16) acc = (Acc)__bfloat162float(__float2bfloat16_rn((float)acc));
        store_value(out, out_dtype, doff, (double)acc, 0, false);
      }
    }
  }
}

}  // namespace

cudaError_t launch_tri(const StridedView& in, void* out, int64_t numel, int upper, int64_t diagonal, cudaStream_t s) {
  if (in.rank < 2) return cudaErrorInvalidValue;
  return dispatch_index_map(in, out, numel, 0, upper, diagonal, s);
}

cudaError_t launch_flip(const StridedView& in, void* out, int64_t numel, int axis, cudaStream_t s) {
  if (axis < 0 || axis >= in.rank) return cudaErrorInvalidValue;
  return dispatch_index_map(in, out, numel, 1, axis, 0, s);
}

cudaError_t launch_place(const StridedView& in, void* out, int out_dtype, const int64_t* out_shape, int axis, int64_t axis_offset,
                         cudaStream_t s, const PlaceFill* fill) {
  if (axis < 0 || axis >= in.rank) return cudaErrorInvalidValue;
  int64_t numel = 1;
  for (int d = 0; d < in.rank; ++d) numel *= in.shape[d];
  if (numel == 0) return cudaSuccess;
  PlaceArg pa{};
  int64_t st = 1;
  for (int d = in.rank - 1; d >= 0; --d) { pa.out_stride[d] = st; st *= out_shape[d]; }
  pa.base = axis_offset * pa.out_stride[axis];
  if (fill) { pa.fill = 1; pa.fill_is_int = fill->is_int; pa.fill_f = fill->f; pa.fill_n = fill->n; }
  place_kernel<<<grid_for(numel), 256, 0, s>>>(to_arg(in), in.dtype, out, out_dtype, pa, numel);
  return cudaGetLastError();
}

// One thread per index entry: its coordinates, with the entry's value in place of the coordinate along `dim`,
// name the destination in the dense output.  `claim` (one int per output element, zeroed) catches two entries
// that name one destination.
struct ScatterArg {
  int64_t idx_shape[kMaxRank];
  int64_t out_stride[kMaxRank];
  int64_t axis_extent;
  int rank, dim, esize;
  int src_is_const;
  unsigned long long const_bits;   // the scalar source in the output's representation
};

__global__ void scatter_kernel(const int64_t* idx, const char* src, char* out, int* claim, ScatterArg a, int64_t numel, int* status) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < numel; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t g = idx[i];
    if (g < 0 || g >= a.axis_extent) { atomicExch(status, BG_ERR_INDEX_RANGE); continue; }
    int64_t rem = i, dst = 0;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t c = rem % a.idx_shape[d];
      rem /= a.idx_shape[d];
      dst += (d == a.dim ? g : c) * a.out_stride[d];
    }
    if (atomicExch(&claim[dst], 1) != 0) { atomicExch(status, BG_ERR_INDEX_RANGE); continue; }
    switch (a.esize) {
      case 1: reinterpret_cast<uint8_t*>(out)[dst] = a.src_is_const ? (uint8_t)a.const_bits : reinterpret_cast<const uint8_t*>(src)[i]; break;
      case 2: reinterpret_cast<uint16_t*>(out)[dst] = a.src_is_const ? (uint16_t)a.const_bits : reinterpret_cast<const uint16_t*>(src)[i]; break;
      case 4: reinterpret_cast<uint32_t*>(out)[dst] = a.src_is_const ? (uint32_t)a.const_bits : reinterpret_cast<const uint32_t*>(src)[i]; break;
      default: reinterpret_cast<unsigned long long*>(out)[dst] = a.src_is_const ? a.const_bits : reinterpret_cast<const unsigned long long*>(src)[i]; break;
    }
  }
}

cudaError_t launch_scatter(const int64_t* idx, const void* src, void* out, int* claim, int esize, int rank, const int64_t* out_shape,
                           const int64_t* idx_shape, int dim, bool src_is_const, unsigned long long const_bits, int* status, cudaStream_t s) {
  if (dim < 0 || dim >= rank || rank > kMaxRank) return cudaErrorInvalidValue;
  ScatterArg a{};
  int64_t numel = 1, st = 1, out_numel = 1;
  for (int d = rank - 1; d >= 0; --d) { a.out_stride[d] = st; st *= out_shape[d]; }
  for (int d = 0; d < rank; ++d) { a.idx_shape[d] = idx_shape[d]; numel *= idx_shape[d]; out_numel *= out_shape[d]; }
  if (numel == 0 || out_numel == 0) return cudaSuccess;
  a.axis_extent = out_shape[dim];
  a.rank = rank; a.dim = dim; a.esize = esize;
  a.src_is_const = src_is_const ? 1 : 0;
  a.const_bits = const_bits;
  cudaError_t e = cudaMemsetAsync(claim, 0, (size_t)out_numel * sizeof(int), s);
  if (e != cudaSuccess) return e;
  scatter_kernel<<<grid_for(numel), 256, 0, s>>>(idx, reinterpret_cast<const char*>(src), reinterpret_cast<char*>(out), claim, a, numel, status);
  return cudaGetLastError();
}

cudaError_t launch_cumsum(const StridedView& in, void* out, int out_dtype, int axis, int reverse, cudaStream_t s) {
  if (axis < 0 || axis >= in.rank) return cudaErrorInvalidValue;
  int64_t lines = 1, inner = 1;
  for (int d = 0; d < in.rank; ++d)
    if (d != axis) lines *= in.shape[d];
  for (int d = axis + 1; d < in.rank; ++d) inner *= in.shape[d];
  if (lines == 0 || in.shape[axis] == 0) return cudaSuccess;
  const ViewArg a = to_arg(in);
  const unsigned grid = grid_for(lines);
  switch (out_dtype) {
    case BG_F64: cumsum_kernel<double><<<grid, 256, 0, s>>>(a, in.dtype, out, out_dtype, axis, reverse, lines, inner); break;
    case BG_F32: case BG_F16: case BG_BF16: cumsum_kernel<float><<<grid, 256, 0, s>>>(a, in.dtype, out, out_dtype, axis, reverse, lines, inner); break;
    default: cumsum_kernel<long long><<<grid, 256, 0, s>>>(a, in.dtype, out, out_dtype, axis, reverse, lines, inner); break;
  }
  return cudaGetLastError();
}

}  // namespace bg

// ---- stable ordering of lines (SORT_INDICES, TOPK_INDICES) ------------------------------------------
// One CTA sorts one line in shared memory with a bitonic network over (key, position) pairs.  Keys are the
// values mapped to unsigned integers whose order is NumPy's sort order: -0.0 and +0.0 compare equal, NaNs
// are the largest values and equal to each other; ties keep their original order because the position is
// the low word of the comparison.  A descending order complements the key, which puts NaNs first and still
// keeps ties in original order -- what the reference obtains by sorting the reversed line and flipping back.
namespace bg {
namespace {

__device__ __forceinline__ unsigned long long sort_key(const void* p, int dt, int64_t off) {
  switch (dt) {
    case BG_F64: {
      double v = reinterpret_cast<const double*>(p)[off];
      if (v != v) return ~0ull;
      if (v == 0.0) v = 0.0;
      unsigned long long b = (unsigned long long)__double_as_longlong(v);
      return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
    }
    case BG_F32: case BG_F16: case BG_BF16: {
      float v = dt == BG_F32 ? reinterpret_cast<const float*>(p)[off]
                : dt == BG_F16 ? __half2float(reinterpret_cast<const __half*>(p)[off])
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[off]);
      if (v != v) return ~0ull;
      if (v == 0.f) v = 0.f;
      unsigned b = __float_as_uint(v);
      b = (b >> 31) ? ~b : (b | 0x80000000u);
      return (unsigned long long)b << 32;
    }
    case BG_U64: return reinterpret_cast<const unsigned long long*>(p)[off];
    default: return (unsigned long long)load_as_i64(p, dt, off) ^ 0x8000000000000000ull;
  }
}

__global__ void __launch_bounds__(256) sort_lines_kernel(ViewArg in, int in_dtype, int64_t* out, int axis, int descending, int64_t keep,
                                                         int64_t inner, int n2) {
  extern __shared__ __align__(16) unsigned char sort_smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(sort_smem);
  unsigned* pos = reinterpret_cast<unsigned*>(keys + n2);
  const int64_t len = in.shape[axis];
  const int64_t line = blockIdx.x;
  const int64_t in_pos = line % inner, outer = line / inner;
  int64_t src0 = 0, rem = in_pos;
  for (int d = in.rank - 1; d > axis; --d) { src0 += (rem % in.shape[d]) * in.stride[d]; rem /= in.shape[d]; }
  rem = outer;
  for (int d = axis - 1; d >= 0; --d) { src0 += (rem % in.shape[d]) * in.stride[d]; rem /= in.shape[d]; }
  for (int i = threadIdx.x; i < n2; i += blockDim.x) {
    if (i < len) {
      const unsigned long long k = sort_key(in.ptr, in_dtype, src0 + i * in.stride[axis]);
      keys[i] = descending ? ~k : k;
      pos[i] = (unsigned)i;
    } else {
      keys[i] = ~0ull;             // padding sorts behind every element (its position word is the largest too)
      pos[i] = 0xffffffffu;
    }
  }
  __syncthreads();
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < n2 / 2; i += blockDim.x) {
        const int lo = 2 * i - (i & (stride - 1)), hi = lo + stride;
        const bool up = (lo & size) == 0;
        const unsigned long long ka = keys[lo], kb = keys[hi];
        const unsigned pa = pos[lo], pb = pos[hi];
        const bool a_after_b = ka > kb || (ka == kb && pa > pb);
        if (a_after_b == up) { keys[lo] = kb; keys[hi] = ka; pos[lo] = pb; pos[hi] = pa; }
      }
      __syncthreads();
    }
  }
  const int64_t dst0 = outer * keep * inner + in_pos;
  for (int64_t i = threadIdx.x; i < keep; i += blockDim.x) out[dst0 + i * inner] = (int64_t)pos[i];
}

}  // namespace

cudaError_t launch_sort_lines(const StridedView& in, int64_t* out, int axis, int descending, int64_t keep, cudaStream_t s) {
  if (axis < 0 || axis >= in.rank) return cudaErrorInvalidValue;
  const int64_t len = in.shape[axis];
  if (len > kSortMaxLine || keep > len) return cudaErrorInvalidValue;
  int64_t lines = 1, inner = 1;
  for (int d = 0; d < in.rank; ++d)
    if (d != axis) lines *= in.shape[d];
  for (int d = axis + 1; d < in.rank; ++d) inner *= in.shape[d];
  if (lines == 0 || len == 0 || keep == 0) return cudaSuccess;
  if (lines > 0x7fffffff) return cudaErrorInvalidValue;
  int n2 = 2;
  while (n2 < len) n2 <<= 1;
  const size_t smem = (size_t)n2 * 12;
  sort_lines_kernel<<<(unsigned)lines, 256, smem, s>>>(to_arg(in), in.dtype, out, axis, descending, keep, inner, n2);
  return cudaGetLastError();
}

}  // namespace bg
