// Fused softmax attention forward for sm_100a (head dimension 64):
//   O[b,h,q,:] = softmax_k( scale * Q[b,h,q,:].K[b,h,k,:] (+ mask) ) . V[b,h,k,:]
// with the score tile kept on chip: S = Q K^T is produced by tcgen05.mma into tensor memory, the
// softmax warps read it with tcgen05.ld, keep the running max / sum per query row, write the
// probabilities P back to shared memory in the operand layout, and a second tcgen05.mma forms P V.
//
// One CTA owns 128 query rows of one (batch, head):
//   warp 0     TMA producer: Q once, then K tiles and V^T tiles into their rings
//   warp 1     MMA issuer (one thread): QK^T ahead of the softmax, P.V as soon as P is published
//   warps 2-9  softmax: two threads per query row (each half of the keys / output columns)
// Two kernels, one per operand encoding:
//   attn_tf32_fwd_kernel  3xTF32 for fp32-faithful results: Q, K, V^T pre-split into hi = tf32(x), lo = x - hi, P split
//                         on the fly, the cross products lo.hi, hi.lo, hi.hi in one accumulator; 64-key tiles, the
//                         previous tile's P.V folded into registers while the tensor core works on the current one;
//   attn16_fwd_kernel     f16 / bf16 operands: 128-key tiles, P.V accumulated in tensor memory with lazy rescaling,
//                         two CTAs per SM (described at the kernel).
// All operands are K-major tiles with 128-byte swizzle; V is consumed as V^T [D, keys], prepared by a
// transposing pre-pass that also performs the autocast casts.
// Masks: additive fp32 [B|1, H|1, Sq, Sk], or boolean "fill with -inf"; a per-(q tile, k tile)
// class (skip / plain / mixed) computed by a pre-pass lets fully masked tiles (the causal upper
// triangle) be skipped by every role alike.  No cluster multicast; every wait is clock-bounded; tensor-memory
// loads and stores are issued by whole warps.
#include "common.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "attn_common.cuh"
#include "tc_common.cuh"

namespace bg {
namespace {

using namespace tc;
using namespace attn;

struct AttnCfg {
  static constexpr int BKV = 64;                              // keys per tile
  // K and V^T tiles travel in rings of their own: K(t+1) can be fetched as soon as Q.K(t)^T has been issued,
  // V(t+1) once P.V(t) has completed.  With hi + lo planes of 4-byte elements there is room for one tile of each.
  static constexpr int NK = 1;
  static constexpr int NV = 1;
  static constexpr int NP = 1;                                // P buffers
  // planes: hi k-block 0, hi k-block 1, lo k-block 0, lo k-block 1 (a k-block is 32 floats = 128 bytes)
  static constexpr int QBytes = 4 * kQRows * 128;
  static constexpr int KBytes = 4 * BKV * 128;
  static constexpr int VBytes = 4 * kHeadDim * 128;           // V^T: 64 rows x (2 x 32) keys
  static constexpr int PBytes = 4 * kQRows * 128;
  static constexpr int SCols = BKV;
  static constexpr int TmemCols = 256;                        // 2 x S + 2 x PV
  static constexpr int SmemBytes = QBytes + NK * KBytes + NV * VBytes + NP * PBytes;   // 192 KB: one CTA per SM
};

__global__ void __launch_bounds__(kAttnThreads, 1)
attn_tf32_fwd_kernel(const __grid_constant__ CUtensorMap tmQ0, const __grid_constant__ CUtensorMap tmQ1,
                const __grid_constant__ CUtensorMap tmK0, const __grid_constant__ CUtensorMap tmK1,
                const __grid_constant__ CUtensorMap tmV0, const __grid_constant__ CUtensorMap tmV1,
                const __grid_constant__ AttnParams p) {
  using C = AttnCfg;
  constexpr int BKV = C::BKV;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;
  unsigned char* sK = sQ + C::QBytes;
  unsigned char* sV = sK + C::NK * C::KBytes;
  unsigned char* sP = sV + C::NV * C::VBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::NP * C::PBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + C::NK;
  uint64_t* v_full = k_empty + C::NK;
  uint64_t* v_empty = v_full + C::NV;
  uint64_t* s_full = v_empty + C::NV;     // [2]
  uint64_t* p_full = s_full + 2;          // [NP]
  uint64_t* pv_full = p_full + C::NP;     // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* pmax = reinterpret_cast<float*>(tmem_holder + 4);   // [2 buffers][2 halves][128 rows] tile maxima

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // query tiles are issued last-first: under a causal mask the late tiles carry the most key tiles
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_tile * kQRows;
  const int n_kv = (p.Sk + BKV - 1) / BKV;
  const unsigned char* cls = p.tile_class ? p.tile_class + (size_t)q_tile * n_kv : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < C::NV; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&pv_full[i], 1); }
    for (int i = 0; i < C::NP; ++i) mbar_init(&p_full[i], 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(C::TmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;                       // S buffers: columns [0, 2*BKV)
  const uint32_t tmem_pv = tmem_base + 2 * C::SCols;       // PV buffers: 2 x 64 columns

  if (warp == 0) {
    if (lane == 0) {
      // Q: loaded once
      mbar_expect_tx(q_full, C::QBytes);
      {
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(&tmQ0, sQ + kb * (kQRows * 128), q_full, kb * 32, q0, h, b);
          tma_load_4d(&tmQ1, sQ + 2 * (kQRows * 128) + kb * (kQRows * 128), q_full, kb * 32, q0, h, b);
        }
      }
      // K runs one tile ahead of V in issue order: its slot frees as soon as Q.K^T of the previous occupant is done
      auto next_tile = [&](int j) { while (j < n_kv && cls && cls[j] == 0) ++j; return j; };
      auto load_k = [&](int j, int t) -> bool {
        const int s = t % C::NK;
        if (!mbar_wait(&k_empty[s], ((uint32_t)(t / C::NK) & 1u) ^ 1u, abort_flag)) return false;
        unsigned char* st = sK + s * C::KBytes;
        const int k0 = j * BKV;
        mbar_expect_tx(&k_full[s], C::KBytes);
        {
          for (int kb = 0; kb < 2; ++kb) {
            tma_load_4d(&tmK0, st + kb * (BKV * 128), &k_full[s], kb * 32, k0, h, b);
            tma_load_4d(&tmK1, st + (2 + kb) * (BKV * 128), &k_full[s], kb * 32, k0, h, b);
          }
        }
        return true;
      };
      auto load_v = [&](int j, int t) -> bool {
        const int s = t % C::NV;
        if (!mbar_wait(&v_empty[s], ((uint32_t)(t / C::NV) & 1u) ^ 1u, abort_flag)) return false;
        unsigned char* st = sV + s * C::VBytes;
        const int k0 = j * BKV;
        mbar_expect_tx(&v_full[s], C::VBytes);
        {
          for (int kb = 0; kb < 2; ++kb) {
            tma_load_4d(&tmV0, st + kb * (kHeadDim * 128), &v_full[s], k0 + kb * 32, 0, h, b);
            tma_load_4d(&tmV1, st + (2 + kb) * (kHeadDim * 128), &v_full[s], k0 + kb * 32, 0, h, b);
          }
        }
        return true;
      };
      int jk = next_tile(0), jv = jk, tk = 0, tv = 0;
      bool okp = true;
      while (jv < n_kv && okp) {
        while (okp && jk < n_kv && tk <= tv + 1) {
          okp = load_k(jk, tk);
          ++tk;
          jk = next_tile(jk + 1);
        }
        if (okp) okp = load_v(jv, tv);
        ++tv;
        jv = next_tile(jv + 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // number of tiles that are processed, and the order: QK(0), QK(1), PV(0), QK(2), PV(1), ...
      int n_proc = 0;
      for (int j = 0; j < n_kv; ++j) n_proc += !(cls && cls[j] == 0);
      bool ok = n_proc == 0 || mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_qk = [&](int t) -> bool {   // t-th processed tile
        const int s = t % C::NK;
        if (!mbar_wait(&k_full[s], (uint32_t)(t / C::NK) & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * C::KBytes);
        const uint32_t d_s = tmem_s + (uint32_t)((t & 1) * C::SCols);
        {
          // passes lo.hi, hi.lo, hi.hi; each: 2 k-blocks x 4 k-steps of 8 floats
          uint32_t first = 1;
          for (int pass = 0; pass < 3; ++pass) {
            const uint32_t qa = q_addr + (pass == 0 ? 2 * (kQRows * 128) : 0);
            const uint32_t ka = k_addr + (pass == 1 ? 2 * (BKV * 128) : 0);
            for (int kb = 0; kb < 2; ++kb) {
              const uint64_t da = make_kmajor_sw128_desc(qa + kb * (kQRows * 128));
              const uint64_t db = make_kmajor_sw128_desc(ka + kb * (BKV * 128));
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                umma<true>(d_s, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), p.idesc_qk, first ? 0u : 1u);
                first = 0;
              }
            }
          }
        }
        umma_commit(&s_full[t & 1]);
        umma_commit(&k_empty[s]);
        return true;
      };
      auto issue_pv = [&](int t) -> bool {
        const int s = t % C::NV, pbuf = t % C::NP;
        if (!mbar_wait(&p_full[pbuf], (uint32_t)(t / C::NP) & 1u, abort_flag)) return false;
        if (!mbar_wait(&v_full[s], (uint32_t)(t / C::NV) & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP + pbuf * C::PBytes);
        const uint32_t v_addr = smem_u32(sV + s * C::VBytes);
        const uint32_t d_pv = tmem_pv + (uint32_t)((t & 1) * kHeadDim);
        {
          // passes lo.hi, hi.lo, hi.hi over the tile's two k-blocks of 32 keys
          uint32_t first = 1;
          for (int pass = 0; pass < 3; ++pass) {
            const uint32_t pa = p_addr + (pass == 0 ? 2 * (kQRows * 128) : 0);
            const uint32_t va = v_addr + (pass == 1 ? 2 * (kHeadDim * 128) : 0);
            for (int kb = 0; kb < 2; ++kb) {
              const uint64_t da = make_kmajor_sw128_desc(pa + kb * (kQRows * 128));
              const uint64_t db = make_kmajor_sw128_desc(va + kb * (kHeadDim * 128));
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                umma<true>(d_pv, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), p.idesc_pv, first ? 0u : 1u);
                first = 0;
              }
            }
          }
        }
        umma_commit(&pv_full[t & 1]);
        umma_commit(&v_empty[s]);
        return true;
      };
      if (ok && n_proc > 0) ok = issue_qk(0);
      if (ok && n_proc > 1) ok = issue_qk(1);
      for (int t = 0; t < n_proc && ok; ++t) {
        ok = issue_pv(t);
        if (ok && t + 2 < n_proc) ok = issue_qk(t + 2);
      }
    }
  } else {
    // ---- softmax: two threads per query row, each owning half of the tile's keys and half of the
    //      output columns; the row max and the row sum are combined through shared memory -----------
    const int wg = (warp - 2) >> 2;                 // 0 / 1: which half
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may read
    const int r_in_tile = quarter * 32 + lane;
    const int row = q0 + r_in_tile;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    constexpr int HK = BKV / 2;                     // keys per thread per tile
    constexpr int HD = kHeadDim / 2;                // output columns per thread
    float o[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) o[d] = 0.f;
    float m = -CUDART_INF_F, l = 0.f;
    float alpha_prev = 1.f;
    float scale = p.scale;
    const bool per_elem_scale = p.scale_buf != nullptr && !(p.scale_uniform && *p.scale_uniform);
    if (p.scale_buf && !per_elem_scale) scale = p.scale_buf[0];
    const size_t score_row = ((size_t)(b * p.H + h) * p.Sq + (row < p.Sq ? row : 0)) * (size_t)p.Sk;
    const size_t mask_row = (size_t)b * p.mask_sb + (size_t)h * p.mask_sh + (size_t)(row < p.Sq ? row : 0) * p.Sk;
    bool ok = true;
    int t = 0;
    auto fold_pv = [&](int tt, float alpha) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_full[tt & 1], (uint32_t)(tt >> 1) & 1u, abort_flag))) return false;
      tc_fence_after();
      uint32_t r[32];
      tmem_ld32(tmem_pv + (uint32_t)((tt & 1) * kHeadDim + wg * HD) + lane_sel, r);
#pragma unroll
      for (int i = 0; i < HD; ++i) o[i] = fmaf(o[i], alpha, __uint_as_float(r[i]));
      return true;
    };
    for (int j = 0; j < n_kv; ++j) {
      const int tclass = cls ? cls[j] : (p.mask ? 3 : 1);
      if (tclass == 0) continue;
      const int buf = t & 1;
      // a thread whose wait ran out keeps walking the tiles (its values no longer matter) so that the named
      // barrier below still sees all 256 softmax threads once per tile
      if (ok) ok = mbar_wait(&s_full[buf], (uint32_t)(t >> 1) & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);      // tensor-memory loads are warp-wide: keep the warp together
      tc_fence_after();
      const int k0 = j * BKV + wg * HK;             // first key of this thread's half
      float sv[HK];
      {
        const uint32_t src = tmem_s + (uint32_t)(buf * C::SCols + wg * HK) + lane_sel;
        uint32_t r[32];
        tmem_ld32(src, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[i] = __uint_as_float(r[i]);
      }
      // Probabilities: p = 2^((x - m) * log2(e)) with x = scale * s (+ mask).  The common case -- whole
      // tile in range, no mask to apply, one positive scale -- folds scale and log2(e) into a single FMA
      // per score ahead of the hardware exp2; anything else takes the element-wise path.
      constexpr float kLog2e = 1.4426950408889634f;
      // (autocast graphs round S to the 16-bit dtype between the two products; the fused kernel keeps
      //  the scores in fp32, which stays inside the 2e-2 autocast tolerance)
      const bool simple_scale = !per_elem_scale && scale > 0.f;
        // a binary mask is applied from its bit words only on the folded-scale path; otherwise element by element
        const bool need_mask = p.mask && (tclass == 3 || (tclass == 2 && !simple_scale));
      const bool fast = !need_mask && simple_scale && (tclass == 2 || j * BKV + BKV <= p.Sk);
      float mt = -CUDART_INF_F;
      if (fast && tclass == 2) {
        // binary mask: one word of "masked" bits covers 32 keys of this row
        const uint32_t* wrow = p.mask_bits + (size_t)(row < p.Sq ? row : 0) * p.mask_words + (k0 >> 5);
#pragma unroll
        for (int w = 0; w < (HK + 31) / 32; ++w) {
          uint32_t word = wrow[w] >> (k0 & 31);
#pragma unroll
          for (int i = 0; i < (HK < 32 ? HK : 32); ++i)
            if ((word >> i) & 1u) sv[w * 32 + i] = -CUDART_INF_F;
        }
      }
      if (fast) {
        // four independent chains: a single running max would serialise HK dependent instructions
        float mx[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
        for (int i = 4; i < HK; i += 2) mx[(i >> 1) & 3] = fmax3(mx[(i >> 1) & 3], sv[i], sv[i + 1]);
        mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale;
      } else {
#pragma unroll
        for (int i = 0; i < HK; ++i) {
          const int key = k0 + i;
          const bool in_range = key < p.Sk;
          float x = __fmul_rn(sv[i], per_elem_scale ? (in_range ? p.scale_buf[score_row + key] : 0.f) : scale);
          if (need_mask && in_range) {
            if (p.mask_is_bool) { if (reinterpret_cast<const unsigned char*>(p.mask)[mask_row + key]) x = -CUDART_INF_F; }
            else x = __fadd_rn(x, reinterpret_cast<const float*>(p.mask)[mask_row + key]);
          }
          if (!in_range) x = -CUDART_INF_F;
          sv[i] = x;
          mt = fmaxf(mt, x);
        }
      }
      // the two halves of a row agree on the tile max
      pmax[(buf * 2 + wg) * kQRows + r_in_tile] = mt;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mt = fmaxf(mt, pmax[(buf * 2 + (wg ^ 1)) * kQRows + r_in_tile]);
      const float m_new = fmaxf(m, mt);
      const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
      float psum = 0.f;
      if (fast) {
        const float c = scale * kLog2e, ml = m_use * kLog2e;
        float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < HK; ++i) {
          sv[i] = ex2_approx(fmaf(sv[i], c, -ml));
          ps[i & 3] += sv[i];
        }
        psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
      } else {
#pragma unroll
        for (int i = 0; i < HK; ++i) {
          sv[i] = ex2_approx((sv[i] - m_use) * kLog2e);
          psum += sv[i];
        }
      }
      const float alpha = ex2_approx((m - m_use) * kLog2e);    // m = -inf gives 0: nothing accumulated yet
      l = fmaf(l, alpha, psum);
      m = m_new;
      // publish P in the K-major 128-byte-swizzled operand layout: row r_in_tile, 16-byte chunk c of
      // a 128-byte row lands at chunk (c ^ (row & 7))
      // with a single P buffer the previous tile's P.V must have consumed it first; its result is folded here
      if (ok && C::NP == 1 && t > 0) ok = __all_sync(0xffffffffu, fold_pv(t - 1, alpha_prev));
      const int pbuf = t % C::NP;
      unsigned char* pb = sP + pbuf * C::PBytes;
      const int sw = r_in_tile & 7;
      {
        // this thread's 32 keys are k-block `wg`: one 128-byte row in the hi plane and one in the lo plane
        unsigned char* hi_row = pb + wg * (kQRows * 128) + r_in_tile * 128;
        unsigned char* lo_row = pb + (2 + wg) * (kQRows * 128) + r_in_tile * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t hbits;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hbits) : "f"(sv[c * 4 + e]));
            hi[e] = __uint_as_float(hbits);
            lo[e] = sv[c * 4 + e] - hi[e];
          }
          const int chunk = c ^ sw;
          *reinterpret_cast<float4*>(hi_row + (chunk << 4)) = make_float4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<float4*>(lo_row + (chunk << 4)) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        }
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&p_full[pbuf]);
      // fold the previous tile's P.V while the tensor core works on this one
      if (ok && C::NP == 2 && t > 0) ok = __all_sync(0xffffffffu, fold_pv(t - 1, alpha_prev));
      alpha_prev = alpha;
      ++t;
    }
    if (ok && t > 0) ok = fold_pv(t - 1, alpha_prev);
    // combine the two halves' row sums (pmax is idle now; every softmax thread reaches this barrier)
    pmax[wg * kQRows + r_in_tile] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += pmax[(wg ^ 1) * kQRows + r_in_tile];
    if (ok && row < p.Sq) {
      const float inv = 1.0f / l;   // l = 0 for a fully masked row: 0 * inf = NaN, as the reference's softmax gives
      const size_t base = (size_t)((long long)b * p.out_sb + (long long)h * p.out_sh + (long long)row * p.out_ss) + wg * HD;
      if (p.out_dtype == BG_F32) {
        float* out = reinterpret_cast<float*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 4)
          *reinterpret_cast<float4*>(out + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
      } else if (p.out_dtype == BG_F64) {
        double* out = reinterpret_cast<double*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<double2*>(out + d) = make_double2((double)(o[d] * inv), (double)(o[d + 1] * inv));
      } else if (p.out_dtype == BG_F16) {
        __half* out = reinterpret_cast<__half*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<__half2*>(out + d) = __floats2half2_rn(o[d] * inv, o[d + 1] * inv);
      } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<__nv_bfloat162*>(out + d) = __floats2bfloat162_rn(o[d] * inv, o[d + 1] * inv);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, BG_ERR_DEVICE_TIMEOUT);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TmemCols) : "memory");
  }
}


// ---- 16-bit operands: 128-key tiles, output accumulated in tensor memory ------------------------------
// Differences from the kernel above, which the 3xTF32 encoding keeps:
//   * a tile is 128 keys, so the per-tile handshakes and address arithmetic are paid once per 64 keys per thread;
//   * P.V accumulates in tensor memory across tiles (the MMA's accumulate flag) instead of being folded into
//     registers after every tile.  The exponentials are taken relative to a reference maximum that is only
//     raised when the running maximum exceeds it by more than 2^8 ("lazy rescaling"): then, and only then, a
//     thread multiplies its half row of O in tensor memory (tcgen05.ld / tcgen05.st) and its row sum by
//     2^(old - new).  Until then probabilities may reach 2^8, which bf16 / fp16 and the fp32 sums hold easily;
//     the final O / l is the same quotient.
//   * S has one buffer (128 columns) and P one; with O that is 192 tensor-memory columns, and with Q, two K
//     tiles, one V^T tile and P 96 KB of shared memory: two CTAs per SM, each reading S twice (row maximum,
//     then exponentials) so that no thread holds more than 32 scores.
struct Attn16 {
  static constexpr int BKV = 128;
  static constexpr int NK = 2;
  static constexpr int QBytes = kQRows * 128;
  static constexpr int KBytes = BKV * 128;
  static constexpr int VBytes = 2 * kHeadDim * 128;     // V^T: two k-blocks of 64 keys
  static constexpr int PBytes = 2 * kQRows * 128;       // two k-blocks of 64 keys
  static constexpr int SmemBytes = QBytes + NK * KBytes + VBytes + PBytes;
  static constexpr int TmemCols = 256;                  // S: columns [0, 128), O: [128, 192)
};
constexpr float kLazyRescaleLog2 = 8.0f;

template <bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn16_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ AttnParams p) {
  using C = Attn16;
  constexpr int BKV = C::BKV;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;
  unsigned char* sK = sQ + C::QBytes;
  unsigned char* sV = sK + C::NK * C::KBytes;
  unsigned char* sP = sV + C::VBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::PBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;          // [2]
  uint64_t* k_empty = k_full + C::NK;     // [2]
  uint64_t* v_full = k_empty + C::NK;
  uint64_t* v_empty = v_full + 1;
  uint64_t* s_full = v_empty + 1;         // Q.K^T of a tile has completed
  uint64_t* s_empty = s_full + 1;         // the softmax warps have read S for the last time (8 arrivals)
  uint64_t* p_full = s_empty + 1;         // P is in shared memory (8 arrivals)
  uint64_t* pv_full = p_full + 1;         // P.V of a tile has completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* pmax = reinterpret_cast<float*>(tmem_holder + 4);   // [2 buffers][2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_tile * kQRows;
  const int n_kv = (p.Sk + BKV - 1) / BKV;
  const unsigned char* cls = p.tile_class ? p.tile_class + (size_t)q_tile * n_kv : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    mbar_init(v_full, 1); mbar_init(v_empty, 1);
    mbar_init(s_full, 1); mbar_init(s_empty, 8);
    mbar_init(p_full, 8); mbar_init(pv_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(C::TmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + BKV;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, C::QBytes);
      tma_load_4d(&tmQ, sQ, q_full, 0, q0, h, b);
      auto next_tile = [&](int j) { while (j < n_kv && cls && cls[j] == 0) ++j; return j; };
      int jk = next_tile(0), jv = jk, tk = 0, tv = 0;
      bool okp = true;
      while (jv < n_kv && okp) {
        while (okp && jk < n_kv && tk <= tv + 1) {
          const int s = tk % C::NK;
          if (!mbar_wait(&k_empty[s], ((uint32_t)(tk / C::NK) & 1u) ^ 1u, abort_flag)) { okp = false; break; }
          mbar_expect_tx(&k_full[s], C::KBytes);
          tma_load_4d(&tmK, sK + s * C::KBytes, &k_full[s], 0, jk * BKV, h, b);
          ++tk;
          jk = next_tile(jk + 1);
        }
        if (!okp) break;
        if (!mbar_wait(v_empty, ((uint32_t)tv & 1u) ^ 1u, abort_flag)) break;
        mbar_expect_tx(v_full, C::VBytes);
        tma_load_4d(&tmV, sV, v_full, jv * BKV, 0, h, b);
        tma_load_4d(&tmV, sV + kHeadDim * 128, v_full, jv * BKV + 64, 0, h, b);
        ++tv;
        jv = next_tile(jv + 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int n_proc = 0;
      for (int j = 0; j < n_kv; ++j) n_proc += !(cls && cls[j] == 0);
      bool ok = n_proc == 0 || mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_qk = [&](int t) -> bool {
        const int s = t % C::NK;
        // the single S buffer is free once the softmax warps have taken tile t-1 out of it
        if (t > 0 && !mbar_wait(s_empty, (uint32_t)(t - 1) & 1u, abort_flag)) return false;
        if (!mbar_wait(&k_full[s], (uint32_t)(t / C::NK) & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint64_t da = make_kmajor_sw128_desc(q_addr), db = make_kmajor_sw128_desc(smem_u32(sK + s * C::KBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma<false>(tmem_s, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), p.idesc_qk, k ? 1u : 0u);
        umma_commit(s_full);
        umma_commit(&k_empty[s]);
        return true;
      };
      auto issue_pv = [&](int t) -> bool {
        if (!mbar_wait(p_full, (uint32_t)t & 1u, abort_flag)) return false;
        if (!mbar_wait(v_full, (uint32_t)t & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP), v_addr = smem_u32(sV);
        for (int kb = 0; kb < 2; ++kb) {
          const uint64_t da = make_kmajor_sw128_desc(p_addr + kb * (kQRows * 128));
          const uint64_t db = make_kmajor_sw128_desc(v_addr + kb * (kHeadDim * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma<false>(tmem_o, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), p.idesc_pv, (t > 0 || kb || k) ? 1u : 0u);
        }
        umma_commit(pv_full);
        umma_commit(v_empty);
        return true;
      };
      if (ok && n_proc > 0) ok = issue_qk(0);
      for (int t = 0; t < n_proc && ok; ++t) {
        if (t + 1 < n_proc) ok = issue_qk(t + 1);     // S(t) has been read by the time P(t) is published
        if (ok) ok = issue_pv(t);
      }
    }
  } else {
    const int wg = (warp - 2) >> 2;                 // which 64 keys of a tile / which 32 output columns
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const int row = q0 + r_in_tile;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    constexpr int HD = kHeadDim / 2;
    constexpr float kLog2e = 1.4426950408889634f;
    float m_ref = -CUDART_INF_F, l = 0.f;
    float scale = p.scale;
    const bool per_elem_scale = p.scale_buf != nullptr && !(p.scale_uniform && *p.scale_uniform);
    if (p.scale_buf && !per_elem_scale) scale = p.scale_buf[0];
    const size_t score_row = ((size_t)(b * p.H + h) * p.Sq + (row < p.Sq ? row : 0)) * (size_t)p.Sk;
    const size_t mask_row = (size_t)b * p.mask_sb + (size_t)h * p.mask_sh + (size_t)(row < p.Sq ? row : 0) * p.Sk;
    const int sw = r_in_tile & 7;
    bool ok = true;
    int t = 0;
    for (int j = 0; j < n_kv; ++j) {
      const int tclass = cls ? cls[j] : (p.mask ? 3 : 1);
      if (tclass == 0) continue;
      // a thread whose wait ran out keeps walking the tiles (doing nothing) so that the named barrier below still
      // sees all 256 softmax threads once per tile
      if (ok) ok = mbar_wait(s_full, (uint32_t)t & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);      // tensor-memory loads below are warp-wide: keep the warp together
      tc_fence_after();
      const int k0 = j * BKV + wg * 64;             // first key of this thread's half
      const bool simple_scale = !per_elem_scale && scale > 0.f;
        // a binary mask is applied from its bit words only on the folded-scale path; otherwise element by element
        const bool need_mask = p.mask && (tclass == 3 || (tclass == 2 && !simple_scale));
      const bool fast = !need_mask && simple_scale && (tclass == 2 || j * BKV + BKV <= p.Sk);
      const uint32_t* wrow = (fast && tclass == 2) ? p.mask_bits + (size_t)(row < p.Sq ? row : 0) * p.mask_words + (k0 >> 5) : nullptr;
      // 32 scores (chunk c of this thread's 64), ready for the exponential: raw S with masked keys at -inf on the
      // fast path (scale folded into the exponent later), else scale * S (+ mask) element by element
      auto load_scores = [&](int c, float (&x)[32]) {
        uint32_t r[32];
        tmem_ld32(tmem_s + (uint32_t)(wg * 64 + c * 32) + lane_sel, r);
        if (fast && !wrow) {
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(r[i]);
        } else if (fast) {
          const uint32_t word = wrow[c];
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = ((word >> i) & 1u) ? -CUDART_INF_F : __uint_as_float(r[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = k0 + c * 32 + i;
            const bool in_range = key < p.Sk;
            float v = __fmul_rn(__uint_as_float(r[i]), per_elem_scale ? (in_range ? p.scale_buf[score_row + key] : 0.f) : scale);
            if (need_mask && in_range) {
              if (p.mask_is_bool) { if (reinterpret_cast<const unsigned char*>(p.mask)[mask_row + key]) v = -CUDART_INF_F; }
              else v = __fadd_rn(v, reinterpret_cast<const float*>(p.mask)[mask_row + key]);
            }
            x[i] = in_range ? v : -CUDART_INF_F;
          }
        }
      };
      // pass 1: the tile maximum of this row, in natural units
      float mt = -CUDART_INF_F;
      if (ok) {
        float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          float x[32];
          load_scores(c, x);
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx[(i >> 1) & 3] = fmax3(mx[(i >> 1) & 3], x[i], x[i + 1]);
        }
        mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        if (fast) mt *= scale;
      }
      const int pbuf = t & 1;
      pmax[(pbuf * 2 + wg) * kQRows + r_in_tile] = mt;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mt = fmaxf(mt, pmax[(pbuf * 2 + (wg ^ 1)) * kQRows + r_in_tile]);
      // P of the previous tile has been consumed (and O is quiescent) once its P.V has completed
      if (ok && t > 0) ok = mbar_wait(pv_full, (uint32_t)(t - 1) & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { ++t; continue; }
      // Lazy rescaling.  tcgen05.ld / tcgen05.st are warp-wide instructions: when any row of this warp has to
      // rescale, all 32 lanes run the load / multiply / store, the others with a factor of one.
      const bool raise = m_ref != -CUDART_INF_F && (mt - m_ref) * kLog2e > kLazyRescaleLog2;
      if (__any_sync(0xffffffffu, raise)) {
        const float alpha = raise ? ex2_approx((m_ref - mt) * kLog2e) : 1.0f;
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32(tmem_o + (uint32_t)(wg * HD) + lane_sel, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st32(tmem_o + (uint32_t)(wg * HD) + lane_sel, r);
        if (raise) { l *= alpha; m_ref = mt; }
      }
      if (m_ref == -CUDART_INF_F) m_ref = mt;        // nothing (or only zeros) accumulated so far
      const float m_use = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      const float cc = fast ? scale * kLog2e : kLog2e, ml = m_use * kLog2e;
      // pass 2: exponentials, row sum, P in the operand layout (k-block wg: this thread's 64 keys are one 128-byte row)
      unsigned char* prow = sP + wg * (kQRows * 128) + r_in_tile * 128;
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        float x[32];
        load_scores(c, x);
        if (c == 1) {
          // last read of S: the MMA warp may start the next tile's Q.K^T
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          x[i] = ex2_approx(fmaf(x[i], cc, -ml));
          ps[i & 3] += x[i];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a0 = x[q * 8 + 2 * e], a1 = x[q * 8 + 2 * e + 1];
            if (BF16) { __nv_bfloat162 v2 = __floats2bfloat162_rn(a0, a1); w[e] = *reinterpret_cast<uint32_t*>(&v2); }
            else { __half2 v2 = __floats2half2_rn(a0, a1); w[e] = *reinterpret_cast<uint32_t*>(&v2); }
          }
          *reinterpret_cast<uint4*>(prow + (((c * 4 + q) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      ++t;
    }
    if (ok && t > 0) ok = mbar_wait(pv_full, (uint32_t)(t - 1) & 1u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    // combine the two halves' row sums
    pmax[wg * kQRows + r_in_tile] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += pmax[(wg ^ 1) * kQRows + r_in_tile];
    // the accumulator is read by whole warps (tcgen05.ld is warp-wide); only the stores are per row
    float o[HD];
    {
      tc_fence_after();
      uint32_t r[32];
      tmem_ld32(tmem_o + (uint32_t)(wg * HD) + lane_sel, r);
#pragma unroll
      for (int i = 0; i < HD; ++i) o[i] = t > 0 ? __uint_as_float(r[i]) : 0.f;
    }
    if (ok && row < p.Sq) {
      const float inv = 1.0f / l;   // l = 0 for a fully masked row: 0 * inf = NaN, as the reference's softmax gives
      const size_t base = (size_t)((long long)b * p.out_sb + (long long)h * p.out_sh + (long long)row * p.out_ss) + wg * HD;
      if (p.out_dtype == BG_F32) {
        float* out = reinterpret_cast<float*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 4)
          *reinterpret_cast<float4*>(out + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
      } else if (p.out_dtype == BG_F64) {
        double* out = reinterpret_cast<double*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<double2*>(out + d) = make_double2((double)(o[d] * inv), (double)(o[d + 1] * inv));
      } else if (p.out_dtype == BG_F16) {
        __half* out = reinterpret_cast<__half*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<__half2*>(out + d) = __floats2half2_rn(o[d] * inv, o[d + 1] * inv);
      } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + base;
#pragma unroll
        for (int d = 0; d < HD; d += 2) *reinterpret_cast<__nv_bfloat162*>(out + d) = __floats2bfloat162_rn(o[d] * inv, o[d + 1] * inv);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, BG_ERR_DEVICE_TIMEOUT);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TmemCols) : "memory");
  }
}


// ---- pre-passes ---------------------------------------------------------------------------------
struct PrepView {
  const void* ptr;
  int dtype;
  long long stride[4];   // element strides of the [B,H,S,D] view
};

// Encodings the forward kernel consumes: 16-bit values, or the hi = tf32(x) / lo = x - hi pair.
enum PrepKind : int { PREP_F16 = 0, PREP_BF16 = 1, PREP_TF32 = 2 };

__device__ __forceinline__ double prep_load(const void* p, int dtype, long long off) {
  switch (dtype) {
    case BG_F64: return reinterpret_cast<const double*>(p)[off];
    case BG_F32: return reinterpret_cast<const float*>(p)[off];
    case BG_F16: return __half2float(reinterpret_cast<const __half*>(p)[off]);
    default: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[off]);
  }
}

// Rounds like the graph's CAST node would (float32 -> 16 bit, round to nearest even); 16-bit sources of
// the same type pass through unchanged.
__device__ __forceinline__ void prep_store(void* dst_a, void* dst_b, long long i, double xd, int kind) {
  if (kind == PREP_TF32) {
    const float x = (float)xd;
    uint32_t hb;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x));
    const float fh = __uint_as_float(hb);
    reinterpret_cast<float*>(dst_a)[i] = fh;
    reinterpret_cast<float*>(dst_b)[i] = (float)(xd - (double)fh);   // for fp64 sources lo also carries the bits fp32 dropped
  } else if (kind == PREP_F16) {
    reinterpret_cast<__half*>(dst_a)[i] = __float2half_rn((float)xd);
  } else {
    reinterpret_cast<__nv_bfloat16*>(dst_a)[i] = __float2bfloat16_rn((float)xd);
  }
}

// dst (dense [B,H,S,D], or [B,H,D,S] when `transpose`) = encode(src view): any strides, one element per thread step.
__global__ void attn_prep_kernel(PrepView src, void* dst_a, void* dst_b, int B, int H, int S, int D, int transpose, int kind) {
  const long long n = (long long)B * H * S * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    // i enumerates the destination densely
    long long rem = i;
    int d, s;
    if (transpose) { s = (int)(rem % S); rem /= S; d = (int)(rem % D); rem /= D; }
    else { d = (int)(rem % D); rem /= D; s = (int)(rem % S); rem /= S; }
    const int h = (int)(rem % H);
    const int b = (int)(rem / H);
    const long long off = b * src.stride[0] + h * src.stride[1] + s * src.stride[2] + d * src.stride[3];
    prep_store(dst_a, dst_b, i, prep_load(src.ptr, src.dtype, off), kind);
  }
}

// Same encoding for an fp32 or fp64 source whose rows of D = 64 values are contiguous (strides over b, h, s are
// free multiples of four), four elements per thread step: Q and K of fp32 / fp64 graphs and of autocast graphs
// whose casts were folded into this pass.
template <typename T>
__global__ void attn_prep_rows_kernel(const T* __restrict__ src, long long sb, long long sh, long long ss, void* dst_a,
                                      void* dst_b, int H, int S, long long n4, int kind) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i >> 4;              // 16 groups of four per row of 64
    const int c4 = (int)(i & 15);
    const int sidx = (int)(row % S);
    const long long bh = row / S;
    const int h = (int)(bh % H);
    const long long b = bh / H;
    const T* p = src + b * sb + h * sh + sidx * ss + c4 * 4;
    double xd[4];
    if (sizeof(T) == 8) {
      const double2 v0 = __ldcs(reinterpret_cast<const double2*>(p)), v1 = __ldcs(reinterpret_cast<const double2*>(p) + 1);
      xd[0] = v0.x; xd[1] = v0.y; xd[2] = v1.x; xd[3] = v1.y;
    } else {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(p));
      xd[0] = v.x; xd[1] = v.y; xd[2] = v.z; xd[3] = v.w;
    }
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = (float)xd[e];
    if (kind == PREP_TF32) {
      float hi[4], lo[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t hb;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x[e]));
        hi[e] = __uint_as_float(hb);
        // for fp64 sources lo also carries the bits fp32 dropped
        lo[e] = sizeof(T) == 8 ? (float)(xd[e] - (double)hi[e]) : __fadd_rn(x[e], -hi[e]);
      }
      reinterpret_cast<float4*>(dst_a)[i] = make_float4(hi[0], hi[1], hi[2], hi[3]);
      reinterpret_cast<float4*>(dst_b)[i] = make_float4(lo[0], lo[1], lo[2], lo[3]);
    } else if (kind == PREP_F16) {
      __half2 a = __floats2half2_rn(x[0], x[1]), b2 = __floats2half2_rn(x[2], x[3]);
      reinterpret_cast<uint2*>(dst_a)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b2));
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b2 = __floats2bfloat162_rn(x[2], x[3]);
      reinterpret_cast<uint2*>(dst_a)[i] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b2));
    }
  }
}

// V [B, H, S, 64] (rows of 64 contiguous; fp32, fp64 or the 16-bit operand type) -> V^T [B*H, 64, S] in the kernel's
// encoding.  One CTA transposes 64 keys x 64 columns through shared memory: source rows are read whole, V^T rows
// are written 64 keys at a time.
__global__ void __launch_bounds__(256) attn_prep_vt_kernel(const void* __restrict__ src, int src_dtype, long long sb, long long sh,
                                                           long long ss, void* dst_a, void* dst_b, int H, int S, int kind) {
  __shared__ double tile[64][65];
  const long long bh = blockIdx.y;
  const long long base = (bh / H) * sb + (bh % H) * sh;
  const int s0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;   // 64 x 4
#pragma unroll 4
  for (int r = ty; r < 64; r += 4) {
    const int sidx = s0 + r;
    tile[r][tx] = sidx < S ? prep_load(src, src_dtype, base + sidx * ss + tx) : 0.0;
  }
  __syncthreads();
#pragma unroll 4
  for (int d = ty; d < 64; d += 4) {
    const int sidx = s0 + tx;
    if (sidx < S) prep_store(dst_a, dst_b, (bh * 64 + d) * (long long)S + sidx, tile[tx][d], kind);
  }
}

// Pre-pass over a mask shared by all batches and heads.  Per (128-query, BKV-key) tile it writes a class:
//   0 = every score masked out (skip the tile), 1 = the mask has no effect, 2 = binary (0 / -inf, or
//   boolean) and mixed, 3 = carries finite biases that must be added;
// and per (row, 32 keys) one word of "masked" bits (keys beyond Sk count as masked), so that binary
// tiles are applied from one 32/64-bit load per thread instead of one global load per score.
__global__ void attn_mask_class_kernel(const void* mask, int is_bool, int Sq, int Sk, int bkv, unsigned char* cls, int n_kv,
                                       uint32_t* bits, int words_per_row) {
  const int qt = blockIdx.y, kt = blockIdx.x;
  __shared__ int any_open, any_closed, any_general;
  if (threadIdx.x == 0) { any_open = 0; any_closed = 0; any_general = 0; }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int words = bkv / 32;
  int open = 0, closed = 0, general = 0;
  for (int item = warp; item < kQRows * words; item += n_warps) {
    const int r = qt * kQRows + item / words, w = kt * words + item % words;
    const int key = w * 32 + lane;
    bool is_closed = true, is_general = false;
    if (r < Sq && key < Sk) {
      const size_t off = (size_t)r * Sk + key;
      if (is_bool) is_closed = reinterpret_cast<const unsigned char*>(mask)[off] != 0;
      else {
        const float v = reinterpret_cast<const float*>(mask)[off];
        is_closed = v == -CUDART_INF_F;
        is_general = !is_closed && v != 0.f;
      }
      if (is_closed) closed = 1; else open = 1;
      if (is_general) general = 1;
    }
    const uint32_t word = __ballot_sync(0xffffffffu, is_closed);
    if (lane == 0 && r < Sq && w < words_per_row) bits[(size_t)r * words_per_row + w] = word;
  }
  if (open) atomicOr(&any_open, 1);
  if (closed) atomicOr(&any_closed, 1);
  if (general) atomicOr(&any_general, 1);
  __syncthreads();
  if (threadIdx.x == 0) cls[(size_t)qt * n_kv + kt] = any_general ? 3 : (any_closed ? (any_open ? 2 : 0) : 1);
}

__global__ void attn_uniform_kernel(const float* buf, long long n, int* flag) {
  const float first = buf[0];
  int bad = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    bad |= buf[i] != first;
  if (bad) *flag = 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn attn_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// dense [B, H, rows, cols] tensor, box = 128 bytes of cols x box_rows
bool make_map4(CUtensorMap* map, const void* ptr, int dtype, int B, int H, long long rows, long long cols, int box_rows) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return false;
  const int es = dtype_size(dtype);
  CUtensorMapDataType dt = dtype == BG_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : dtype == BG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)cols * es, (cuuint64_t)cols * rows * es, (cuuint64_t)cols * rows * H * es};
  cuuint32_t box[4] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [B, H, rows, cols] tensor with element strides sb / sh / ss over batch, head and row (rows of `cols` contiguous
// values), box = box_cols x box_rows, 128-byte swizzle.
bool make_map4_strided(CUtensorMap* map, const void* ptr, int dtype, int B, int H, long long rows, long long cols, long long sb,
                       long long sh, long long ss, int box_cols, int box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return false;
  const int es = dtype_size(dtype);
  CUtensorMapDataType dt = dtype == BG_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : dtype == BG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
  // a broadcast batch or head axis (stride 0) is described with extent 1: the kernel then always asks for index 0
  cuuint64_t strides[3] = {(cuuint64_t)ss * es, (cuuint64_t)(sh ? sh : rows * ss) * es, (cuuint64_t)(sb ? sb : rows * ss * H) * es};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

unsigned prep_grid(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return (unsigned)(g < 1 ? 1 : g);
}

}  // namespace

bool attn_tc_supported(const AttnProblem& a) {
  if (!g_tc_assume_available && !attn_encode_fn()) return false;
  if (a.D != kHeadDim || a.B <= 0 || a.H <= 0 || a.Sq <= 0 || a.Sk <= 0) return false;
  if (a.H > 65535 || a.B > 65535) return false;
  if (a.mode == 0 && (a.Sk % 8) != 0) return false;     // V^T rows of Sk 16-bit values must be 16-byte multiples
  if (a.mode == 1 && (a.Sk % 4) != 0) return false;
  return true;
}

void attn_scratch_sizes(const AttnProblem& a, int64_t bytes[8]) {
  const int64_t nq = (int64_t)a.B * a.H * a.Sq * a.D, nk = (int64_t)a.B * a.H * a.Sk * a.D;
  const int es = a.mode == 1 ? 4 : 2;
  const int bkv = a.mode == 1 ? 64 : Attn16::BKV;
  bytes[0] = nq * es;                       // Q (hi)
  bytes[1] = a.mode == 1 ? nq * es : 0;     // Q lo
  bytes[2] = nk * es;                       // K (hi)
  bytes[3] = a.mode == 1 ? nk * es : 0;     // K lo
  bytes[4] = nk * es;                       // V^T (hi)
  bytes[5] = a.mode == 1 ? nk * es : 0;     // V^T lo
  // tile classes (rounded up to 256 bytes) followed by the per-row mask bit words
  const int64_t n_cls = (int64_t)((a.Sq + kQRows - 1) / kQRows) * ((a.Sk + bkv - 1) / bkv);
  const int64_t words = (int64_t)((a.Sk + bkv - 1) / bkv) * (bkv / 32);
  bytes[6] = a.mask ? ((n_cls + 255) & ~(int64_t)255) + (int64_t)a.Sq * words * 4 : 0;
  bytes[7] = a.scale_buf ? 4 : 0;           // uniform-scale flag
}

// 16-bit kernel choice: bit 0 the two-tile (pair) kernel, bit 1 V as an MN-major operand (no transposing pass),
// bit 2 P in tensor memory.  0 selects the single-tile kernel.
int g_attn16_variant = kAttn16DefaultVariant;
// 3xTF32 kernel choice: 0 two threads per row with P in shared memory, 1 one thread per row with P and O in tensor
// memory, 3 the same with fp32 Q and K rows split into planes inside the kernel.
int g_attn32_variant = kAttn32DefaultVariant;

cudaError_t launch_attention_tc(const AttnProblem& a, void* const scratch[8], bool check_uniform, bool classify_mask, int* status,
                                cudaStream_t s) {
  const bool tf32 = a.mode == 1;
  const int bkv = tf32 ? 64 : Attn16::BKV;
  const int sdt = tf32 ? BG_F32 : a.ab_dtype;
  const bool pair = !tf32 && (g_attn16_variant & 1) && attn16_pair_usable(a.Sk, a.out_dtype, a.out, a.out_sb, a.out_sh, a.out_ss);
  const bool v_mn = pair && (g_attn16_variant & 2);
  const bool p_tmem = pair && (g_attn16_variant & 4);
  // fp32 K and V converted inside the kernel: rows of 64 contiguous values, every stride a positive multiple of 16 bytes
  auto fp32_rows = [&](const AttnOperand& o) {
    return o.dtype == BG_F32 && o.stride[3] == 1 && (reinterpret_cast<uintptr_t>(o.ptr) & 15) == 0 && o.stride[0] > 0 && o.stride[1] > 0 &&
           o.stride[2] >= a.D && o.stride[0] % 4 == 0 && o.stride[1] % 4 == 0 && o.stride[2] % 4 == 0;
  };
  const bool kv32 = v_mn && p_tmem && (g_attn16_variant & 8) && fp32_rows(a.k) && fp32_rows(a.v);
  // 3xTF32, one thread per row: fp32 Q, K and V rows are split into hi / lo planes inside the kernel
  const bool row32 = tf32 && (g_attn32_variant & 1);
  const bool raw_rows = row32 && (g_attn32_variant & 2) && fp32_rows(a.q) && fp32_rows(a.k) && fp32_rows(a.v) &&
                      attn_tf32_row_usable(a.Sk, a.out_dtype, a.out, a.out_sb, a.out_sh, a.out_ss, true);
  // operand staging: dense Q, K, V^T (or V) in the kernel's encoding
  const int kind = tf32 ? PREP_TF32 : (a.ab_dtype == BG_F16 ? PREP_F16 : PREP_BF16);
  const AttnOperand* ops[3] = {&a.q, &a.k, &a.v};
  const int seq[3] = {a.Sq, a.Sk, a.Sk};
  const void* staged[3] = {scratch[0], scratch[2], scratch[4]};
  bool q_in_kernel = false;
  for (int i = 0; i < 3; ++i) {
    const long long n = (long long)a.B * a.H * seq[i] * a.D;
    const bool dense = ops[i]->stride[3] == 1 && ops[i]->stride[2] == a.D && ops[i]->stride[1] == (long long)seq[i] * a.D &&
                       ops[i]->stride[0] == (long long)a.H * seq[i] * a.D;
    const bool aligned = (reinterpret_cast<uintptr_t>(ops[i]->ptr) & 15) == 0;
    const bool as_rows = i < 2 || v_mn;        // consumed as [S, 64] rows (not transposed)
    // the pair kernel reads query rows itself: fp32 or operand-type rows of 64 contiguous values, 16-byte aligned
    if (pair && i == 0 && ops[i]->stride[3] == 1 && aligned && (ops[i]->dtype == BG_F32 || ops[i]->dtype == a.ab_dtype)) {
      const long long per16 = ops[i]->dtype == BG_F32 ? 4 : 8;
      if (ops[i]->stride[0] % per16 == 0 && ops[i]->stride[1] % per16 == 0 && ops[i]->stride[2] % per16 == 0) {
        q_in_kernel = true;
        continue;
      }
    }
    if (kv32 && i > 0) continue;
    if (raw_rows) continue;
    // 16-bit operands that are already dense [B,H,S,D] feed the TMA maps directly
    if (!tf32 && as_rows && dense && ops[i]->dtype == a.ab_dtype && aligned) {
      staged[i] = ops[i]->ptr;
      continue;
    }
    const bool rows_contig = ops[i]->stride[3] == 1 && a.D == 64;
    // an fp64 source only ever feeds the 3xTF32 encoding here (16-bit operands never derive from fp64 values)
    const bool rows_vec = rows_contig && (ops[i]->dtype == BG_F32 || (ops[i]->dtype == BG_F64 && tf32)) &&
                          (reinterpret_cast<uintptr_t>(ops[i]->ptr) & 31) == 0 && (ops[i]->stride[0] & 3) == 0 &&
                          (ops[i]->stride[1] & 3) == 0 && (ops[i]->stride[2] & 3) == 0;
    if (!as_rows && rows_contig) {
      attn_prep_vt_kernel<<<dim3((unsigned)((seq[i] + 63) / 64), (unsigned)(a.B * a.H)), 256, 0, s>>>(
          ops[i]->ptr, ops[i]->dtype, ops[i]->stride[0], ops[i]->stride[1], ops[i]->stride[2], scratch[4], scratch[5], a.H, seq[i], kind);
    } else if (as_rows && rows_vec && ops[i]->dtype == BG_F32) {
      attn_prep_rows_kernel<float><<<prep_grid(n / 4), 256, 0, s>>>(reinterpret_cast<const float*>(ops[i]->ptr), ops[i]->stride[0],
                                                                   ops[i]->stride[1], ops[i]->stride[2], scratch[2 * i],
                                                                   scratch[2 * i + 1], a.H, seq[i], n / 4, kind);
    } else if (as_rows && rows_vec) {
      attn_prep_rows_kernel<double><<<prep_grid(n / 4), 256, 0, s>>>(reinterpret_cast<const double*>(ops[i]->ptr), ops[i]->stride[0],
                                                                    ops[i]->stride[1], ops[i]->stride[2], scratch[2 * i],
                                                                    scratch[2 * i + 1], a.H, seq[i], n / 4, kind);
    } else {
      PrepView v{ops[i]->ptr, ops[i]->dtype, {ops[i]->stride[0], ops[i]->stride[1], ops[i]->stride[2], ops[i]->stride[3]}};
      attn_prep_kernel<<<prep_grid(n), 256, 0, s>>>(v, scratch[2 * i], scratch[2 * i + 1], a.B, a.H, seq[i], a.D, !as_rows, kind);
    }
  }
  unsigned char* cls = nullptr;
  uint32_t* bits = nullptr;
  const int n_kv_tiles = (a.Sk + bkv - 1) / bkv;
  const int words_per_row = n_kv_tiles * (bkv / 32);
  if (a.mask && a.mask_sb == 0 && a.mask_sh == 0) {
    cls = reinterpret_cast<unsigned char*>(scratch[6]);
    const int n_q = (a.Sq + kQRows - 1) / kQRows;
    bits = reinterpret_cast<uint32_t*>(cls + (((size_t)n_q * n_kv_tiles + 255) & ~(size_t)255));
    if (classify_mask)
      attn_mask_class_kernel<<<dim3(n_kv_tiles, n_q), 256, 0, s>>>(a.mask, a.mask_is_bool, a.Sq, a.Sk, bkv, cls, n_kv_tiles, bits, words_per_row);
  }
  int* uniform = nullptr;
  if (a.scale_buf) {
    uniform = reinterpret_cast<int*>(scratch[7]);
    if (check_uniform) {
      cudaError_t e = cudaMemsetAsync(uniform, 1, 1, s);   // low byte 1 -> flag != 0 (the other bytes are cleared next)
      if (e != cudaSuccess) return e;
      e = cudaMemsetAsync(reinterpret_cast<char*>(uniform) + 1, 0, 3, s);
      if (e != cudaSuccess) return e;
      const long long n = (long long)a.B * a.H * a.Sq * a.Sk;
      attn_uniform_kernel<<<prep_grid(n), 256, 0, s>>>(a.scale_buf, n, uniform);
    }
  }
  CUtensorMap q0, q1, k0, k1, v0, v1;
  if (raw_rows) {
    if (!make_map4_strided(&q0, a.q.ptr, BG_F32, a.B, a.H, a.Sq, a.D, a.q.stride[0], a.q.stride[1], a.q.stride[2], 32, kQRows) ||
        !make_map4_strided(&k0, a.k.ptr, BG_F32, a.B, a.H, a.Sk, a.D, a.k.stride[0], a.k.stride[1], a.k.stride[2], 32, bkv) ||
        // rows of V feed the tensor core as an MN-major operand of 32-bit values: that takes the swizzle of 32-byte pieces
        !make_map4_strided(&v0, a.v.ptr, BG_F32, a.B, a.H, a.Sk, a.D, a.v.stride[0], a.v.stride[1], a.v.stride[2], 32, bkv,
                           CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
      return cudaErrorInvalidValue;
  } else if (!pair && !make_map4(&q0, staged[0], sdt, a.B, a.H, a.Sq, a.D, kQRows)) return cudaErrorInvalidValue;
  if (raw_rows) {
  } else if (kv32) {
    if (!make_map4_strided(&k0, a.k.ptr, BG_F32, a.B, a.H, a.Sk, a.D, a.k.stride[0], a.k.stride[1], a.k.stride[2], 32, bkv) ||
        !make_map4_strided(&v0, a.v.ptr, BG_F32, a.B, a.H, a.Sk, a.D, a.v.stride[0], a.v.stride[1], a.v.stride[2], 32, bkv))
      return cudaErrorInvalidValue;
  } else if (!make_map4(&k0, staged[1], sdt, a.B, a.H, a.Sk, a.D, bkv)) return cudaErrorInvalidValue;
  if (kv32 || raw_rows) {
  } else if (v_mn) {
    if (!make_map4(&v0, staged[2], sdt, a.B, a.H, a.Sk, a.D, bkv)) return cudaErrorInvalidValue;
  } else if (!make_map4(&v0, staged[2], sdt, a.B, a.H, a.D, a.Sk, kHeadDim)) return cudaErrorInvalidValue;
  q1 = q0; k1 = k0; v1 = v0;
  if (tf32) {
    if (!raw_rows && !make_map4(&q1, scratch[1], sdt, a.B, a.H, a.Sq, a.D, kQRows)) return cudaErrorInvalidValue;
    if (!raw_rows && !make_map4(&k1, scratch[3], sdt, a.B, a.H, a.Sk, a.D, bkv)) return cudaErrorInvalidValue;
    if (!raw_rows && !make_map4(&v1, scratch[5], sdt, a.B, a.H, a.D, a.Sk, kHeadDim)) return cudaErrorInvalidValue;
  }
  AttnParams p{};
  p.B = a.B; p.H = a.H; p.Sq = a.Sq; p.Sk = a.Sk;
  p.scale = a.scale;
  p.scale_buf = a.scale_buf;
  p.scale_uniform = uniform;
  p.mask = a.mask;
  p.mask_is_bool = a.mask_is_bool;
  p.mask_sb = a.mask_sb;
  p.mask_sh = a.mask_sh;
  p.tile_class = cls;
  p.mask_bits = bits;
  p.mask_words = words_per_row;
  p.out = a.out;
  p.out_sb = a.out_sb; p.out_sh = a.out_sh; p.out_ss = a.out_ss;
  p.out_dtype = a.out_dtype;
  p.round_scores = tf32 ? 0 : a.ab_dtype + 1;
  p.status = status;
  const uint32_t fmt = tf32 ? 2u : (a.ab_dtype == BG_BF16 ? 1u : 0u);
  p.idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bkv >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);
  p.idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kHeadDim >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);
  if (pair) {
    if (v_mn) p.idesc_pv |= 1u << 16;      // B operand (V) is MN-major
    if (q_in_kernel) {
      p.q_ptr = a.q.ptr; p.q_sb = a.q.stride[0]; p.q_sh = a.q.stride[1]; p.q_ss = a.q.stride[2];
      p.q_f32 = a.q.dtype == BG_F32;
    } else {
      p.q_ptr = staged[0]; p.q_sb = (long long)a.H * a.Sq * a.D; p.q_sh = (long long)a.Sq * a.D; p.q_ss = a.D;
      p.q_f32 = 0;
    }
    return launch_attn16_pair(p, a.ab_dtype == BG_BF16, v_mn, p_tmem, kv32, k0, v0, s);
  }
  dim3 grid((a.Sq + kQRows - 1) / kQRows, a.H, a.B);
  cudaError_t e;
  const long long n_out = (long long)a.B * a.H * a.Sq * a.D;
  if (row32 && (raw_rows || attn_tf32_row_usable(a.Sk, a.out_dtype, a.out, a.out_sb, a.out_sh, a.out_ss, false))) {
    // (row offsets that keep `out` 16-byte aligned keep the planes' fp32 rows 16- and bf16 rows 8-byte aligned)
    if (a.planes_hi) {
      p.planes_hi = reinterpret_cast<float*>(a.planes_hi);
      p.planes_16 = reinterpret_cast<__nv_bfloat16*>(a.planes_lo);
      p.planes_n = n_out;
    }
    const CUtensorMap maps[6] = {q0, q1, k0, k1, v0, v1};
    return launch_attn_tf32_row(p, maps, raw_rows, s);
  }
  if (tf32) {
    const size_t smem = AttnCfg::SmemBytes + 256 + 2048 + 1024;
    e = cudaFuncSetAttribute(attn_tf32_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attn_tf32_fwd_kernel<<<grid, kAttnThreads, smem, s>>>(q0, q1, k0, k1, v0, v1, p);
    // this kernel stores `out` only: the planes a consumer was promised are made from it
    {
      const cudaError_t le = cudaGetLastError();
      if (le != cudaSuccess || !a.planes_hi) return le;
      return launch_tf32_split(a.out, a.out_dtype, reinterpret_cast<float*>(a.planes_hi), reinterpret_cast<float*>(a.planes_lo), n_out, 8, s);
    }
  } else {
    const size_t smem = Attn16::SmemBytes + 256 + 2048 + 1024;
    auto kern = a.ab_dtype == BG_BF16 ? attn16_fwd_kernel<true> : attn16_fwd_kernel<false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kern<<<grid, kAttnThreads, smem, s>>>(q0, k0, v0, p);
  }
  return cudaGetLastError();
}

}  // namespace bg
