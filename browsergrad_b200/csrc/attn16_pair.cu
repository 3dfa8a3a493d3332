// Fused softmax attention forward for f16 / bf16 operands, head dimension 64, two query tiles per CTA (sm_100a).
//
// One CTA owns 256 query rows of one (batch, head) as two tiles of 128 ("A" and "B") that share every K and V tile
// brought into shared memory and take turns on the tensor core: while the softmax threads of one tile work on their
// scores, the products of the other tile run.
//   warp 0      producer: lane 0 fetches K tiles, lane 1 V tiles (TMA, rings of their own)
//   warps 1, 2  MMA issuers (warp 1 for tile A, warp 2 for tile B; all lanes run the loop, an elected lane issues):
//               S = Q K^T into tensor memory, O += P V
//   warps 4-7   softmax of tile A: one thread per query row, the row's 128 scores in registers
//   warps 8-11  softmax of tile B
// (warp 3 only fills the first warpgroup, which hands most of its registers to the softmax warpgroups with
// setmaxnreg: a softmax thread holds a whole row of scores.)
// A softmax thread reads its row of S once (tcgen05.ld), frees S for the next Q K^T at once, takes the row maximum,
// the exponentials against a lazily raised reference maximum (O in tensor memory is rescaled only when the running
// maximum exceeds the reference by more than 2^8) and the row sum without any exchange with other threads, and
// publishes P either in shared memory (operand layout, 128-byte swizzle) or in tensor memory (the A operand of the
// P V product is then read from there).  Query rows are read by the softmax threads themselves from the tensor the
// graph names (fp32 rows are rounded to the operand type as the graph's CAST would), so Q needs no staging pass.
// V is consumed either as V^T tiles (K-major) or directly as rows of V (MN-major operand), chosen at launch.
// CTAs are numbered heaviest first (late query tiles see the most keys under a causal mask).
// No cluster multicast; every wait is clock-bounded; tensor-memory loads and stores are issued by whole warps.
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

struct PairCfg {
  static constexpr int BKV = 128;
  static constexpr int NK = 2, NV = 2;
  static constexpr int QBytes = kQRows * 128;          // one query tile: 128 rows of 64 16-bit values
  static constexpr int KBytes = BKV * 128;
  static constexpr int VBytes = BKV * 128;
  static constexpr int PBytes = 2 * kQRows * 128;      // two k-blocks of 64 keys
  static constexpr int TmemCols = 512;
  static constexpr int ColS = 0;                       // S of tile A, S of tile B: 2 x 128 columns
  static constexpr int ColO = 256;                     // O of tile A, of tile B: 2 x 64
  static constexpr int ColP = 384;                     // P of tile A, of tile B (16-bit pairs): 2 x 64
  static constexpr int StageBytes = BKV * 256;         // one fp32 tile of 128 rows x 64 values, as two 128-byte-wide boxes
  static constexpr int smem_bytes(bool p_in_tmem, bool kv32) {
    return 2 * QBytes + NK * KBytes + NV * VBytes + (kv32 ? 2 * StageBytes : 0) + (p_in_tmem ? 0 : 2 * PBytes);
  }
};
constexpr float kLazyRescaleLog2 = 8.0f;
// Threads and registers.  Without in-kernel conversion: three warpgroups (producer + MMA issuers, softmax A, softmax
// B); with it a fourth one converts fp32 K / V tiles to the operand type.
// The register pool of a CTA is what it was launched with (Launch registers per thread); the light warpgroups
// shrink to Light so that the softmax warpgroups can grow to Softmax.  A request beyond the pool would wait for ever,
// hence the assertions (and the check of the compiled register count at launch).
template <bool KV32>
struct PairRegs {
  static constexpr int Threads = KV32 ? 512 : 384;
  static constexpr int Launch = KV32 ? 128 : 168;
  static constexpr int Light = 72;
  static constexpr int Softmax = KV32 ? 184 : 216;
  static_assert((Threads - 256) * Light + 256 * Softmax <= Launch * Threads, "setmaxnreg requests exceed the CTA's register pool");
  static_assert(Light % 8 == 0 && Softmax % 8 == 0, "setmaxnreg takes multiples of 8");
};

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float a0, float a1) {
  if (BF16) { __nv_bfloat162 v = __floats2bfloat162_rn(a0, a1); return *reinterpret_cast<uint32_t*>(&v); }
  __half2 v = __floats2half2_rn(a0, a1);
  return *reinterpret_cast<uint32_t*>(&v);
}

// The rare per-tile work of a softmax thread lives in functions of their own, away from the straight-line code of
// the common case: a taken branch over a long cold block costs an instruction fetch the loop cannot afford.

// Puts a score tile into the form the main path expects (see the kernel): masked and out-of-range scores become
// -inf; with `by_element` the scores become scale * s (+ mask), element by element.  32 scores per step.  Returns a
// bit per 32-key piece of the row that is masked out entirely (bit-word masks only).
__device__ __noinline__ uint32_t fixup_scores(const AttnParams& p, uint32_t t_s, int k0, bool by_element, int tclass, uint4 w4, float scale,
                                          bool per_elem_scale, size_t score_row, size_t mask_row) {
  if (!by_element) {
    // bit words: the whole row at once (the caller holds no scores yet, so the registers are free)
    uint32_t r[128];
    tmem_ld32_issue(t_s, r);
    tmem_ld32_issue(t_s + 32, r + 32);
    tmem_ld32_issue(t_s + 64, r + 64);
    tmem_ld32_issue(t_s + 96, r + 96);
    uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int left = p.Sk - (k0 + c * 32);            // keys of this piece that exist
      if (left < 32) w[c] |= left <= 0 ? 0xffffffffu : (0xffffffffu << left);
    }
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 128; ++i)
      if ((w[i >> 5] >> (i & 31)) & 1u) r[i] = __float_as_uint(-CUDART_INF_F);
    tmem_st32_issue(t_s, r);
    tmem_st32_issue(t_s + 32, r + 32);
    tmem_st32_issue(t_s + 64, r + 64);
    tmem_st32_issue(t_s + 96, r + 96);
    tmem_st_wait();
    return (w[0] == 0xffffffffu ? 1u : 0u) | (w[1] == 0xffffffffu ? 2u : 0u) | (w[2] == 0xffffffffu ? 4u : 0u) | (w[3] == 0xffffffffu ? 8u : 0u);
  }
  const bool with_mask = p.mask && tclass >= 2;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t r[32];
    tmem_ld32(t_s + (uint32_t)(c * 32), r);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int key = k0 + c * 32 + i;
      const bool in_range = key < p.Sk;
      float v = __fmul_rn(__uint_as_float(r[i]), per_elem_scale ? (in_range ? p.scale_buf[score_row + key] : 0.f) : scale);
      if (with_mask && in_range) {
        if (p.mask_is_bool) { if (reinterpret_cast<const unsigned char*>(p.mask)[mask_row + key]) v = -CUDART_INF_F; }
        else v = __fadd_rn(v, reinterpret_cast<const float*>(p.mask)[mask_row + key]);
      }
      r[i] = __float_as_uint(in_range ? v : -CUDART_INF_F);
    }
    tmem_st32(t_s + (uint32_t)(c * 32), r);
  }
  return 0u;
}

// O[row, 0..63] *= alpha in tensor memory (tcgen05.ld / st are warp-wide: every lane of the warp calls this).
__device__ __noinline__ void rescale_o(uint32_t t_o, float alpha) {
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    uint32_t r[32];
    tmem_ld32(t_o + (uint32_t)(half * 32), r);
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
    tmem_st32(t_o + (uint32_t)(half * 32), r);
  }
}

// VMN: V tiles are rows of V (MN-major B operand), else V^T tiles (K-major).  PT: P lives in tensor memory.
// KV32: K and V are fp32 in global memory; their tiles land in a staging buffer (TMA) and a converter warpgroup
// rounds them to the operand type into the operand rings, as the graph's CAST nodes would (needs VMN and PT).
template <bool BF16, bool VMN, bool PT, bool KV32>
__global__ void __launch_bounds__(PairRegs<KV32>::Threads, 1)
attn16_pair_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const __grid_constant__ AttnParams p) {
  using C = PairCfg;
  constexpr int BKV = C::BKV;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;                                   // [2][QBytes]
  unsigned char* sK = sQ + 2 * C::QBytes;                     // [NK][KBytes]
  unsigned char* sV = sK + C::NK * C::KBytes;                 // [NV][VBytes]
  unsigned char* sStage = sV + C::NV * C::VBytes;             // [2][StageBytes] fp32 K tile, fp32 V tile (KV32)
  unsigned char* sP = sStage + (KV32 ? 2 * C::StageBytes : 0); // [2][PBytes] unless PT
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + (PT ? 0 : 2 * C::PBytes));
  uint64_t* q_full = bars;                // [2] query rows of a tile are in shared memory (4 arrivals)
  uint64_t* k_full = q_full + 2;          // [NK]
  uint64_t* k_empty = k_full + C::NK;     // [NK]
  uint64_t* v_full = k_empty + C::NK;     // [NV]
  uint64_t* v_empty = v_full + C::NV;     // [NV]
  uint64_t* s_full = v_empty + C::NV;     // [2] Q K^T of the tile's current key tile has completed
  uint64_t* s_empty = s_full + 2;         // [2] its softmax warps hold the scores in registers (4 arrivals)
  uint64_t* p_full = s_empty + 2;         // [2] P is published (4 arrivals)
  uint64_t* pv_full = p_full + 2;         // [2] P V has completed
  uint64_t* stage_full = pv_full + 2;     // [2] an fp32 K (0) / V (1) tile has landed in its staging buffer
  uint64_t* stage_empty = stage_full + 2; // [2] the converter warps have read it (4 arrivals)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(stage_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  unsigned char* s_cls = reinterpret_cast<unsigned char*>(tmem_holder + 4);   // [2][n_kv] tile classes of the two query tiles

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // the same in every lane, and known to be
  const int lane = threadIdx.x & 31;
  const int n_bh = p.B * p.H;
  const int n_qt = (p.Sq + kQRows - 1) / kQRows;
  const int n_pairs = (n_qt + 1) / 2;
  const int pair = n_pairs - 1 - (int)(blockIdx.x / (unsigned)n_bh);
  const int bh = (int)(blockIdx.x % (unsigned)n_bh);
  const int b = bh / p.H, h = bh % p.H;
  const int n_kv = (p.Sk + BKV - 1) / BKV;
  // Tile classes of the two query tiles, copied to shared memory once: every role consults them once or more per
  // key tile, and a global load in the MMA thread's loop delays every product behind it.  Without a class table
  // every key tile is processed (class 3 with a mask, else 1); a tile B that does not exist has class 0 throughout.
  const bool has_b = 2 * pair + 1 < n_qt;
  grid_dependency_wait();       // the tile classes below may come from a kernel of the same plan
  grid_launch_dependents();
  {
    const unsigned char* cls_a = p.tile_class ? p.tile_class + (size_t)(2 * pair) * n_kv : nullptr;
    const unsigned char* cls_b = p.tile_class && has_b ? p.tile_class + (size_t)(2 * pair + 1) * n_kv : nullptr;
    const unsigned char dflt = p.mask ? 3 : 1;
    for (int j = threadIdx.x; j < n_kv; j += PairRegs<KV32>::Threads) {
      s_cls[j] = cls_a ? cls_a[j] : dflt;
      s_cls[n_kv + j] = has_b ? (cls_b ? cls_b[j] : dflt) : (unsigned char)0;
    }
  }
  auto need_a = [&](int j) { return s_cls[j] != 0; };
  auto need_b = [&](int j) { return s_cls[n_kv + j] != 0; };
  auto next_union = [&](int j) { while (j < n_kv && !need_a(j) && !need_b(j)) ++j; return j; };

  // The softmax threads fetch their query rows now: the loads are in flight while the barriers are set up and tensor
  // memory is allocated (64 fp32 values, or 64 16-bit values, per thread).
  uint4 qraw[16];
  bool q_row_ok = false;
  if (warp >= 4 && warp < 12) {
    const int g = (warp - 4) >> 2;
    const int row = (2 * pair + g) * kQRows + (warp & 3) * 32 + lane;
    q_row_ok = (g == 0 || has_b) && row < p.Sq;
    const long long qoff = (long long)b * p.q_sb + (long long)h * p.q_sh + (long long)(q_row_ok ? row : 0) * p.q_ss;
    if (p.q_f32) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p.q_ptr) + qoff);
#pragma unroll
      for (int c = 0; c < 16; ++c) qraw[c] = q_row_ok ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q_ptr) + qoff);
#pragma unroll
      for (int c = 0; c < 8; ++c) qraw[c] = q_row_ok ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
    }
  }

  if (threadIdx.x == 0) {
    for (int g = 0; g < 2; ++g) {
      mbar_init(&q_full[g], 4);
      mbar_init(&s_full[g], 1); mbar_init(&s_empty[g], 4);
      mbar_init(&p_full[g], 4); mbar_init(&pv_full[g], 1);
    }
    // a K or V slot is free once both issuers are done with it
    // an operand tile is complete when its TMA bytes have landed, or (KV32) when the four converter warps have written it
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], KV32 ? 4 : 1); mbar_init(&k_empty[s], 2); }
    for (int s = 0; s < C::NV; ++s) { mbar_init(&v_full[s], KV32 ? 4 : 1); mbar_init(&v_empty[s], 2); }
    for (int i = 0; i < 2; ++i) { mbar_init(&stage_full[i], 1); mbar_init(&stage_empty[i], 4); }
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

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PairRegs<KV32>::Light));
    if (warp == 0) {
      if (KV32) {
        // fp32 tiles into the staging buffers: lane 0 K, lane 1 V; two boxes of 32 values (128 bytes) per row
        if (lane < 2) {
          const CUtensorMap* tm = lane == 0 ? &tmK : &tmV;
          unsigned char* st = sStage + lane * C::StageBytes;
          int u = 0;
          for (int j = next_union(0); j < n_kv; j = next_union(j + 1), ++u) {
            if (!mbar_wait(&stage_empty[lane], ((uint32_t)u & 1u) ^ 1u, abort_flag)) break;
            mbar_expect_tx(&stage_full[lane], C::StageBytes);
            tma_load_4d(tm, st, &stage_full[lane], 0, j * BKV, h, b);
            tma_load_4d(tm, st + C::StageBytes / 2, &stage_full[lane], 32, j * BKV, h, b);
          }
        }
      } else if (lane == 0) {
        int u = 0;
        for (int j = next_union(0); j < n_kv; j = next_union(j + 1), ++u) {
          const int s = u % C::NK;
          if (!mbar_wait(&k_empty[s], ((uint32_t)(u / C::NK) & 1u) ^ 1u, abort_flag)) break;
          mbar_expect_tx(&k_full[s], C::KBytes);
          tma_load_4d(&tmK, sK + s * C::KBytes, &k_full[s], 0, j * BKV, h, b);
        }
      } else if (lane == 1) {
        int u = 0;
        for (int j = next_union(0); j < n_kv; j = next_union(j + 1), ++u) {
          const int s = u % C::NV;
          if (!mbar_wait(&v_empty[s], ((uint32_t)(u / C::NV) & 1u) ^ 1u, abort_flag)) break;
          mbar_expect_tx(&v_full[s], C::VBytes);
          unsigned char* st = sV + s * C::VBytes;
          if (VMN) {
            tma_load_4d(&tmV, st, &v_full[s], 0, j * BKV, h, b);
          } else {
            tma_load_4d(&tmV, st, &v_full[s], j * BKV, 0, h, b);
            tma_load_4d(&tmV, st + kHeadDim * 128, &v_full[s], j * BKV + 64, 0, h, b);
          }
        }
      }
    } else if (warp <= 2) {
      // One issuer warp per query tile (warp 1: tile A, warp 2: tile B): neither tile's products wait behind a
      // barrier of the other.  All 32 lanes run the loop (see elect_one); the elected lane issues.  Key tiles are
      // walked in the producers' order; a tile this query tile skips is released with a plain arrival once it has
      // landed (so that the arrival counts for that tile and no earlier one).
      const int g = warp - 1;
      auto need = [&](int j) { return s_cls[g * n_kv + j] != 0; };
      const uint64_t desc_q = make_kmajor_sw128_desc(smem_u32(sQ + g * C::QBytes));
      const uint32_t d_s = tmem_base + (uint32_t)(C::ColS + g * BKV);
      const uint32_t d_o = tmem_base + (uint32_t)(C::ColO + g * kHeadDim);
      const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
      bool ok = true;
      int n_qk = 0, n_pv = 0;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0; };
      auto issue_qk = [&](int slot) -> bool {
        const int n = n_qk++;
        if (n == 0 && !wait_all(&q_full[g], 0)) return false;
        if (n > 0 && !wait_all(&s_empty[g], (uint32_t)(n - 1) & 1u)) return false;
        tc_fence_after();
        const uint64_t db = make_kmajor_sw128_desc(smem_u32(sK + slot * C::KBytes));
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 4; ++k) umma<false>(d_s, desc_q + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_qk, k ? 1u : 0u);
          umma_commit(&s_full[g]);
        }
        __syncwarp();
        return true;
      };
      auto issue_pv = [&](int slot) -> bool {
        const int n = n_pv++;
        if (!wait_all(&p_full[g], (uint32_t)n & 1u)) return false;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + slot * C::VBytes);
        const uint32_t p_addr = smem_u32(sP + g * C::PBytes);
        const uint32_t first = n > 0 ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t db = VMN ? make_mnmajor_sw128_desc(v_addr + (uint32_t)(k * 2048))
                                    : make_kmajor_sw128_desc(v_addr + (uint32_t)((k >> 2) * (kHeadDim * 128))) + (uint64_t)((k & 3) * 2);
            const uint32_t acc = k > 0 ? 1u : first;
            if (PT) {
              umma_ts_f16(d_o, tmem_base + (uint32_t)(C::ColP + g * 64 + k * 8), db, idesc_pv, acc);
            } else {
              const uint64_t da = make_kmajor_sw128_desc(p_addr + (uint32_t)((k >> 2) * (kQRows * 128))) + (uint64_t)((k & 3) * 2);
              umma<false>(d_o, da, db, idesc_pv, acc);
            }
          }
          umma_commit(&pv_full[g]);
        }
        __syncwarp();
        return true;
      };
      auto release = [&](uint64_t* bar, bool used) {
        if (elect_one()) { if (used) umma_commit(bar); else mbar_arrive(bar); }
        __syncwarp();
      };
      // tile u+1's Q K^T is issued ahead of tile u's P V: S(u+1) is ready when the softmax warps finish tile u
      int jc = next_union(0), u = 0;
      if (jc < n_kv) {
        ok = wait_all(&k_full[0], 0);
        const bool used = need(jc);
        if (ok && used) ok = issue_qk(0);
        if (ok) release(&k_empty[0], used);
      }
      while (jc < n_kv && ok) {
        const int jn = next_union(jc + 1), un = u + 1;
        const int ks = un % C::NK, vs = u % C::NV;
        if (jn < n_kv) {
          ok = wait_all(&k_full[ks], (uint32_t)(un / C::NK) & 1u);
          const bool used = need(jn);
          if (ok && used) ok = issue_qk(ks);
          if (ok) release(&k_empty[ks], used);
        }
        if (ok) ok = wait_all(&v_full[vs], (uint32_t)(u / C::NV) & 1u);
        const bool used = need(jc);
        if (ok && used) ok = issue_pv(vs);
        if (ok) release(&v_empty[vs], used);
        jc = jn;
        u = un;
      }
    }
  } else if (KV32 && warp >= 12) {
    // ---- converter warpgroup: staging buffer (fp32, two 128-byte-swizzled boxes per tile) -> operand ring (16 bit,
    //      128-byte swizzle); thread r owns row r of the tile.  K tiles and V tiles alternate.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PairRegs<KV32>::Light));
    const int r = threadIdx.x & 127, sw = r & 7;
    bool ok = true;
    int u = 0;
    for (int j = next_union(0); j < n_kv && ok; j = next_union(j + 1), ++u) {
#pragma unroll 1
      for (int which = 0; which < 2 && ok; ++which) {       // 0: K, 1: V
        const int slot = u % (which == 0 ? C::NK : C::NV);
        uint64_t* full = which == 0 ? &k_full[slot] : &v_full[slot];
        uint64_t* empty = which == 0 ? &k_empty[slot] : &v_empty[slot];
        unsigned char* dst = (which == 0 ? sK + slot * C::KBytes : sV + slot * C::VBytes) + r * 128;
        const unsigned char* src = sStage + which * C::StageBytes + r * 128;
        ok = __all_sync(0xffffffffu, mbar_wait(&stage_full[which], (uint32_t)u & 1u, abort_flag) &&
                                         mbar_wait(empty, ((uint32_t)(u / (which == 0 ? C::NK : C::NV)) & 1u) ^ 1u, abort_flag));
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < 8; ++c) {                         // eight output chunks of eight values
          const unsigned char* box = src + (c >> 2) * (C::StageBytes / 2);
          const float4 lo = *reinterpret_cast<const float4*>(box + ((((2 * c) & 7) ^ sw) << 4));
          const float4 hi = *reinterpret_cast<const float4*>(box + ((((2 * c + 1) & 7) ^ sw) << 4));
          *reinterpret_cast<uint4*>(dst + ((c ^ sw) << 4)) =
              make_uint4(pack16<BF16>(lo.x, lo.y), pack16<BF16>(lo.z, lo.w), pack16<BF16>(hi.x, hi.y), pack16<BF16>(hi.z, hi.w));
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) { mbar_arrive(full); mbar_arrive(&stage_empty[which]); }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PairRegs<KV32>::Softmax));
    const int g = (warp - 4) >> 2;                  // query tile of this warp
    const int quarter = warp & 3;                   // tensor-memory lane quarter this warp may access
    const int r_in_tile = quarter * 32 + lane;
    const int q_tile = 2 * pair + g;
    const bool active = g == 0 || has_b;
    const int row = q_tile * kQRows + r_in_tile;
    const bool row_ok = active && row < p.Sq;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const int sw = r_in_tile & 7;
    constexpr float kLog2e = 1.4426950408889634f;
    const unsigned char* cls = s_cls + g * n_kv;

    if (active) {
      // ---- this thread's query row (fetched at the top of the kernel) -> shared memory in the operand layout ----
      unsigned char* qrow = sQ + g * C::QBytes + r_in_tile * 128;
      if (p.q_f32) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 lo = qraw[2 * c], hi = qraw[2 * c + 1];
          *reinterpret_cast<uint4*>(qrow + ((c ^ sw) << 4)) =
              make_uint4(pack16<BF16>(__uint_as_float(lo.x), __uint_as_float(lo.y)), pack16<BF16>(__uint_as_float(lo.z), __uint_as_float(lo.w)),
                         pack16<BF16>(__uint_as_float(hi.x), __uint_as_float(hi.y)), pack16<BF16>(__uint_as_float(hi.z), __uint_as_float(hi.w)));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(qrow + ((c ^ sw) << 4)) = qraw[c];
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[g]);

      float m_ref = -CUDART_INF_F, l = 0.f;
      float scale = p.scale;
      const bool per_elem_scale = p.scale_buf != nullptr && !(p.scale_uniform && *p.scale_uniform);
      if (p.scale_buf && !per_elem_scale) scale = p.scale_buf[0];
      const size_t score_row = ((size_t)(b * p.H + h) * p.Sq + (row_ok ? row : 0)) * (size_t)p.Sk;
      const size_t mask_row = (size_t)b * p.mask_sb + (size_t)h * p.mask_sh + (size_t)(row_ok ? row : 0) * p.Sk;
      const uint32_t t_s = tmem_base + (uint32_t)(C::ColS + g * BKV) + lane_sel;
      const uint32_t t_o = tmem_base + (uint32_t)(C::ColO + g * kHeadDim) + lane_sel;
      const uint32_t t_p = tmem_base + (uint32_t)(C::ColP + g * 64) + lane_sel;
      bool ok = true;
      int t = 0;
      const bool simple_scale = !per_elem_scale && scale > 0.f;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int tclass = cls[j];
        if (tclass == 0) continue;
        const int k0 = j * BKV;
        // The main path below is straight-line code over the row's 128 scores and assumes a plain tile: every key
        // in range, nothing masked, one positive scale (folded into the exponent).  Any other tile is first put
        // into that form in tensor memory by a short loop over 32-score pieces (`fixup`): masked or out-of-range
        // scores become -inf; with a per-element scale or an additive mask the scores are replaced by
        // scale * s (+ mask) and the exponent scale becomes one.  Keeping the rare cases out of the unrolled path
        // keeps it small enough for the instruction cache.
        const bool ragged = k0 + BKV > p.Sk;
        const bool by_element = !simple_scale || (p.mask && tclass == 3);
        const bool fixup = by_element || tclass == 2 || ragged;
        // binary mask: four words of "masked" bits cover this row's 128 keys (fetched ahead of the wait for S)
        uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
        if (!by_element && tclass == 2)
          w4 = __ldg(reinterpret_cast<const uint4*>(p.mask_bits + (size_t)(row_ok ? row : 0) * p.mask_words + (k0 >> 5)));
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[g], (uint32_t)t & 1u, abort_flag));
        if (!ok) break;
        tc_fence_after();
        // 32-key pieces that are masked for every row of this warp (the far side of a causal diagonal) need no
        // exponentials: their probabilities are zero
        uint32_t dead = 0u;
        if (fixup) dead = __reduce_and_sync(0xffffffffu, fixup_scores(p, t_s, k0, by_element, tclass, w4, scale, per_elem_scale, score_row, mask_row));
        const bool fast = !by_element;      // scale still to be applied (folded into the exponent)
        float x[BKV];
        {
          uint32_t* xu = reinterpret_cast<uint32_t*>(x);
          tmem_ld32_issue(t_s, xu);
          tmem_ld32_issue(t_s + 32, xu + 32);
          tmem_ld32_issue(t_s + 64, xu + 64);
          tmem_ld32_issue(t_s + 96, xu + 96);
          tmem_ld_wait();
        }
        // the scores are in registers: the next Q K^T of this query tile may overwrite S
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[g]);
        // row maximum of the tile, in natural units
        float mt;
        {
          float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
          for (int i = 4; i < BKV; i += 2) mx[(i >> 1) & 3] = fmax3(mx[(i >> 1) & 3], x[i], x[i + 1]);
          mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
          if (fast) mt *= scale;
        }
        // Lazy rescaling.  O must be quiescent (the previous P V complete) before it is touched; tcgen05.ld / st are
        // warp-wide, so when any row of this warp has to rescale all 32 lanes do, the others by a factor of one.
        bool pv_done = t == 0;
        const bool raise = m_ref != -CUDART_INF_F && (mt - m_ref) * kLog2e > kLazyRescaleLog2;
        if (__any_sync(0xffffffffu, raise)) {
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_full[g], (uint32_t)(t - 1) & 1u, abort_flag));
          if (!ok) break;
          pv_done = true;
          tc_fence_after();
          const float alpha = raise ? ex2_approx((m_ref - mt) * kLog2e) : 1.0f;
          rescale_o(t_o, alpha);
          tc_fence_before();
          if (raise) { l *= alpha; m_ref = mt; }
        }
        if (m_ref == -CUDART_INF_F) m_ref = mt;        // nothing (or only zeros) accumulated so far
        const float m_use = m_ref == -CUDART_INF_F ? 0.f : m_ref;
        const float cc = fast ? scale * kLog2e : kLog2e, ml = m_use * kLog2e;
        {
          float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int c = 0; c < BKV / 32; ++c) {
            if ((dead >> c) & 1u) {
#pragma unroll
              for (int i = c * 32; i < c * 32 + 32; ++i) x[i] = 0.f;
            } else {
#pragma unroll
              for (int i = c * 32; i < c * 32 + 32; ++i) {
                x[i] = ex2_approx(fmaf(x[i], cc, -ml));
                ps[i & 3] += x[i];
              }
            }
          }
          l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
        }
        // P of the previous key tile has been consumed once its P V has completed
        if (!pv_done) {
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_full[g], (uint32_t)(t - 1) & 1u, abort_flag));
          if (!ok) break;
          tc_fence_after();
        }
        if (PT) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t w[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) w[i] = pack16<BF16>(x[half * 64 + 2 * i], x[half * 64 + 2 * i + 1]);
            tmem_st32_issue(t_p + (uint32_t)(half * 32), w);
          }
          tmem_st_wait();
        } else {
          unsigned char* prow = sP + g * C::PBytes + r_in_tile * 128;
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) w[e] = pack16<BF16>(x[q * 8 + 2 * e], x[q * 8 + 2 * e + 1]);
            *reinterpret_cast<uint4*>(prow + (q >> 3) * (kQRows * 128) + (((q & 7) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          fence_async_smem();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[g]);
        ++t;
      }
      if (ok && t > 0) ok = __all_sync(0xffffffffu, mbar_wait(&pv_full[g], (uint32_t)(t - 1) & 1u, abort_flag));
      if (ok) {
        tc_fence_after();
        const float inv = 1.0f / l;   // l = 0 for a fully masked row: 0 * inf = NaN, as the reference's softmax gives
        const size_t base = (size_t)((long long)b * p.out_sb + (long long)h * p.out_sh + (long long)(row_ok ? row : 0) * p.out_ss);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32(t_o + (uint32_t)(half * 32), r);     // warp-wide; only the stores are per row
          float o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = (t > 0 ? __uint_as_float(r[i]) : 0.f) * inv;
          if (!row_ok) continue;
          if (p.out_dtype == BG_F32) {
            float* out = reinterpret_cast<float*>(p.out) + base + half * 32;
#pragma unroll
            for (int d = 0; d < 32; d += 4) *reinterpret_cast<float4*>(out + d) = make_float4(o[d], o[d + 1], o[d + 2], o[d + 3]);
          } else if (p.out_dtype == BG_F64) {
            double* out = reinterpret_cast<double*>(p.out) + base + half * 32;
#pragma unroll
            for (int d = 0; d < 32; d += 2) *reinterpret_cast<double2*>(out + d) = make_double2((double)o[d], (double)o[d + 1]);
          } else {
            uint32_t* out = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(p.out) + base + half * 32);
#pragma unroll
            for (int d = 0; d < 32; d += 8) {
              uint4 v;
              if (p.out_dtype == BG_BF16) v = make_uint4(pack16<true>(o[d], o[d + 1]), pack16<true>(o[d + 2], o[d + 3]), pack16<true>(o[d + 4], o[d + 5]), pack16<true>(o[d + 6], o[d + 7]));
              else v = make_uint4(pack16<false>(o[d], o[d + 1]), pack16<false>(o[d + 2], o[d + 3]), pack16<false>(o[d + 4], o[d + 5]), pack16<false>(o[d + 6], o[d + 7]));
              *reinterpret_cast<uint4*>(out + d / 2) = v;
            }
          }
        }
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

template <bool BF16>
cudaError_t launch_variant(bool vmn, bool pt, bool kv32, dim3 grid, size_t smem, cudaStream_t s, const CUtensorMap& k, const CUtensorMap& v,
                           const AttnParams& p) {
  void (*kern)(const CUtensorMap, const CUtensorMap, const AttnParams) =
      kv32 ? attn16_pair_kernel<BF16, true, true, true>
           : vmn ? (pt ? attn16_pair_kernel<BF16, true, true, false> : attn16_pair_kernel<BF16, true, false, false>)
                 : (pt ? attn16_pair_kernel<BF16, false, true, false> : attn16_pair_kernel<BF16, false, false, false>);
  // the register hand-over in the kernel assumes the pool of a launch at PairRegs::Launch registers per thread
  cudaFuncAttributes fa;
  cudaError_t e = cudaFuncGetAttributes(&fa, kern);
  if (e != cudaSuccess) return e;
  if (fa.numRegs < (kv32 ? PairRegs<true>::Launch : PairRegs<false>::Launch)) return cudaErrorLaunchOutOfResources;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_dependent(kern, dim3(grid), dim3(kv32 ? PairRegs<true>::Threads : PairRegs<false>::Threads), smem, s, k, v, p);
}

}  // namespace

bool attn16_pair_usable(int Sk, int out_dtype, const void* out, long long out_sb, long long out_sh, long long out_ss) {
  // the tile classes of both query tiles are kept in shared memory beside the operand tiles
  const int n_kv = (Sk + PairCfg::BKV - 1) / PairCfg::BKV;
  if ((size_t)PairCfg::smem_bytes(false, false) + 256 + 1024 + 2 * (size_t)n_kv > 227 * 1024) return false;
  // output rows are written in 16-byte pieces
  const int es = dtype_size(out_dtype);
  const long long per16 = 16 / es;
  return (reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_sb % per16 == 0 && out_sh % per16 == 0 && out_ss % per16 == 0;
}

cudaError_t launch_attn16_pair(const attn::AttnParams& p, bool bf16, bool v_mn, bool p_in_tmem, bool kv_fp32, const CUtensorMap& tm_k,
                               const CUtensorMap& tm_v, cudaStream_t s) {
  if (kv_fp32 && !(v_mn && p_in_tmem)) return cudaErrorInvalidValue;
  const int n_qt = (p.Sq + kQRows - 1) / kQRows;
  const long long n_cta = (long long)((n_qt + 1) / 2) * p.B * p.H;
  if (n_cta <= 0 || n_cta > 0x7fffffffll) return cudaErrorInvalidValue;
  const int n_kv = (p.Sk + PairCfg::BKV - 1) / PairCfg::BKV;
  const size_t smem = (size_t)PairCfg::smem_bytes(p_in_tmem, kv_fp32) + 256 + 1024 + 2 * (size_t)n_kv;
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  dim3 grid((unsigned)n_cta);
  return bf16 ? launch_variant<true>(v_mn, p_in_tmem, kv_fp32, grid, smem, s, tm_k, tm_v, p)
              : launch_variant<false>(v_mn, p_in_tmem, kv_fp32, grid, smem, s, tm_k, tm_v, p);
}

}  // namespace bg
