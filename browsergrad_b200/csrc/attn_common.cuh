// Declarations shared by the fused attention kernels (attn_tc.cu, attn16_pair.cu): kernel parameters and
// the small PTX helpers both files use.
#pragma once
#include <cuda_bf16.h>

#include <cuda.h>
#include <stdint.h>

#include "tc_common.cuh"

namespace bg {
namespace attn {

using namespace tc;

constexpr int kHeadDim = 64;
constexpr int kQRows = 128;
constexpr int kAttnThreads = 320;   // producer warp, MMA warp, 2 x 4 softmax warps

__device__ __forceinline__ void tma_load_4d(const CUtensorMap* map, void* smem_dst, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// max of three in one instruction (sm_100 has the three-input form)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnParams {
  int B, H, Sq, Sk;
  float scale;                 // used when scale_buf is null or *scale_uniform != 0
  const float* scale_buf;      // [B,H,Sq,Sk] or null
  const int* scale_uniform;    // device flag: scale_buf holds one repeated value (then scale_buf[0] is used)
  const void* mask;            // additive fp32 or bool (1 = fill -inf), or null
  int mask_is_bool;
  long long mask_sb, mask_sh;  // element strides over batch / head (0 when broadcast); rows are Sk apart
  const unsigned char* tile_class;   // [ceil(Sq/128), ceil(Sk/BKV)]: 0 skip, 1 plain, 2 binary mixed, 3 biased; null = none computed
  const uint32_t* mask_bits;         // [Sq, mask_words] "masked" bits, valid where tile_class is
  int mask_words;
  void* out;                   // rows of 64 at b * out_sb + h * out_sh + row * out_ss elements
  long long out_sb, out_sh, out_ss;
  int out_dtype;
  int round_scores;            // dtype + 1: round S through f16 / bf16 before the softmax (autocast graphs)
  uint32_t idesc_qk, idesc_pv;
  float* planes_hi;            // 3xTF32 row kernel: store the result as split-product operand planes instead of `out`
  __nv_bfloat16* planes_16;    // bf16(x) plane; the bf16(x - tf32(x)) plane follows after planes_n elements
  long long planes_n;
  int* status;
  // query rows read by the kernel itself (pair kernel): 64 contiguous values per row, fp32 (rounded to the operand
  // type as the graph's CAST would) or already of the operand type, at b * q_sb + h * q_sh + row * q_ss elements
  const void* q_ptr;
  long long q_sb, q_sh, q_ss;
  int q_f32;
};

}  // namespace attn

// Two-query-tile 16-bit kernel (attn16_pair.cu).  `p` carries the query rows' address and strides; K tiles are
// [128 keys, 64] boxes of tm_k; tm_v gives [128 keys, 64] boxes of V (v_mn) or [64, 64 keys] boxes of V^T.  With
// kv_fp32 (needs v_mn and p_in_tmem) both maps describe fp32 tensors in boxes of [128 keys, 32 values] and the kernel
// rounds the tiles to the operand type itself.
bool attn16_pair_usable(int Sk, int out_dtype, const void* out, long long out_sb, long long out_sh, long long out_ss);
cudaError_t launch_attn16_pair(const attn::AttnParams& p, bool bf16, bool v_mn, bool p_in_tmem, bool kv_fp32, const CUtensorMap& tm_k,
                               const CUtensorMap& tm_v, cudaStream_t s);

// 3xTF32 kernel with one thread per query row and P / O in tensor memory (attn_tf32_row.cu).  maps: Q hi, Q lo
// ([128 rows, 32] boxes), K hi, K lo ([64 keys, 32] boxes), V^T hi, V^T lo ([64 rows, 32 keys] boxes).  With `raw`
// the Q hi and K hi maps describe the caller's own fp32 rows (same boxes), the lo maps of Q and K are not used and the
// kernel splits the values itself (one more K stage in shared memory, hence the flag in the usability check).
bool attn_tf32_row_usable(int Sk, int out_dtype, const void* out, long long out_sb, long long out_sh, long long out_ss, bool raw);
cudaError_t launch_attn_tf32_row(const attn::AttnParams& p, const CUtensorMap maps[6], bool raw, cudaStream_t s);

}  // namespace bg
