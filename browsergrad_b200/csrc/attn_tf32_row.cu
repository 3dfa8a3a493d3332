// Fused softmax attention forward with 3xTF32 products (fp32-faithful results), head dimension 64, sm_100a:
// one thread per query row, probabilities and output kept in tensor memory.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key tiles (64 keys) that its mask classes keep:
//   warp 0      producer: lane 0 Q once and the K tiles, lane 1 the V tiles (TMA, rings of their own); an operand
//               arrives pre-split into hi = tf32(x) and lo = x - hi planes (V transposed: a K-major operand), or (RAW)
//               Q, K and V arrive as the caller's fp32 rows in the hi planes' places and converter warps round them in
//               place and write the lo planes (V then stays as rows: an MN-major operand)
//   warp 1      MMA issuer (all lanes run the loop, an elected lane issues): S = Q K^T as the three products
//               lo.hi, hi.lo, hi.hi into a double-buffered S; O += P V likewise, with P read from tensor memory
//   4 warps     softmax (warps 2-5; 4-7 under RAW, where warps 2, 3 convert V and 8-11 convert Q and K, so that whole
//               warpgroups trade registers with setmaxnreg): one thread per query row.  A thread reads its 64 scores of a tile once (tcgen05.ld), frees
//               S at once, takes the row maximum, the exponentials against a lazily raised reference maximum and the
//               row sum with no exchange between threads, splits the probabilities into hi / lo and stores both
//               planes to tensor memory (double-buffered: tile t+1's probabilities are written while P.V of tile t
//               runs).
// The tensor core adds into its accumulator with truncation, so O is accumulated in tensor memory for at most
// kChunkTiles key tiles (512 keys x 3 products); at a chunk boundary the softmax threads add it into registers with
// round-to-nearest adds and the next P.V starts a fresh accumulator.  The reference maximum is raised only when the
// running maximum exceeds it by more than 2^8; then the thread rescales its row of O in tensor memory, its register
// part and its row sum.
// An MMA instruction occupies the tensor pipe for some 50 cycles however small it is and a burst of them starts after
// some 270: the loop keeps the pipe fed (Q K^T of tile t+2 is issued ahead of P V of tile t) and nothing in the
// softmax waits for a product to finish except at chunk boundaries and rescales.
// No cluster multicast; every wait is clock-bounded; tensor-memory loads and stores are issued by whole warps.
#include "common.h"

#include <math_constants.h>

#include "attn_common.cuh"
#include "tc_common.cuh"

namespace bg {
namespace {

using namespace tc;
using namespace attn;

template <bool RAW>
struct RowCfg {
  static constexpr int BKV = 64;
  // RAW halves what a K tile asks of the TMA unit but puts the converters between the load and the product: a
  // third K stage covers that hop
  static constexpr int NK = RAW ? 3 : 2, NV = 2;
  // planes of a tile: hi k-block 0, hi k-block 1, lo k-block 0, lo k-block 1 (a k-block is 32 floats = 128 bytes)
  static constexpr int QBytes = 4 * kQRows * 128;
  static constexpr int KBytes = 4 * BKV * 128;
  static constexpr int VBytes = 4 * kHeadDim * 128;            // V^T: 64 rows x (2 x 32) keys, hi and lo
  static constexpr int SmemBytes = QBytes + NK * KBytes + NV * VBytes;   // 192 KB (224 KB under RAW)
  static constexpr int Threads = RAW ? 384 : 192;
  static constexpr int SoftmaxWarp0 = RAW ? 4 : 2;
  // setmaxnreg (RAW): the CTA's register pool is Launch per thread; two warpgroups shrink to Light, the softmax
  // warpgroup grows to Softmax.  A request beyond the pool would wait for ever, hence the assertion and the check of
  // the compiled register count at launch.
  static constexpr int Launch = 168, Light = 72, Softmax = 248;
  static_assert(256 * Light + 128 * Softmax <= Launch * 384, "setmaxnreg requests exceed the CTA's register pool");
  static constexpr int TmemCols = 512;
  static constexpr int ColS = 0;                               // 2 x 64
  static constexpr int ColP = 128;                             // 2 x (hi 64 | lo 64)
  static constexpr int ColO = 384;                             // 64
};
constexpr int kChunkTiles = 8;            // key tiles accumulated in tensor memory before O is folded into registers
constexpr float kLazyRescaleLog2 = 8.0f;

// O[row, 0..63] *= alpha in tensor memory (every lane of the warp calls this).
__device__ __noinline__ void rescale_o_row(uint32_t t_o, float alpha) {
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    uint32_t r[32];
    tmem_ld32(t_o + (uint32_t)(half * 32), r);
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
    tmem_st32(t_o + (uint32_t)(half * 32), r);
  }
}

__device__ __forceinline__ void umma_ts_tf32(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

// RAW: split the fp32 values that the TMA unit left in a tile's hi planes (`bytes` of them) into hi = tf32(x), in
// place, and lo = x - hi in the lo planes that follow.  Same offsets in both, so the swizzle does not matter.
template <int THREADS>
__device__ __forceinline__ void split_planes(unsigned char* hi_planes, int bytes, int tid) {
  float4* h = reinterpret_cast<float4*>(hi_planes);
  float4* l = reinterpret_cast<float4*>(hi_planes + bytes);
#pragma unroll 4
  for (int c = tid; c < bytes / 16; c += THREADS) {
    const float4 x = h[c];
    uint32_t a, b, cc, d;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(a) : "f"(x.x));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(b) : "f"(x.y));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(cc) : "f"(x.z));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(d) : "f"(x.w));
    const float4 hi = make_float4(__uint_as_float(a), __uint_as_float(b), __uint_as_float(cc), __uint_as_float(d));
    h[c] = hi;
    l[c] = make_float4(x.x - hi.x, x.y - hi.y, x.z - hi.z, x.w - hi.w);
  }
}

// RAW: rows of V as an MN-major operand of 32-bit values: a key (K index) is a 128-byte row of 32 head-dimension
// values, stored with the 128-byte swizzle of 32-byte pieces (the TMA map's SWIZZLE_128B_ATOM_32B, the descriptor's
// layout type 1), whose pattern repeats every 4 keys = 512 bytes (the stride byte offset); the second half of the head
// dimension is a tile of its own `kRawVHalf` bytes on (the leading byte offset).  One tf32 instruction (K = 8) reads
// 8 keys = 1024 bytes from its start address.
constexpr uint32_t kRawVHalf = 64 * 128;
__device__ __forceinline__ uint64_t make_v_rows_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(kRawVHalf >> 4) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;
  return d;
}

template <bool RAW>
__global__ void __launch_bounds__(RowCfg<RAW>::Threads, 1)
attn_tf32_row_kernel(const __grid_constant__ CUtensorMap tmQ0, const __grid_constant__ CUtensorMap tmQ1,
                     const __grid_constant__ CUtensorMap tmK0, const __grid_constant__ CUtensorMap tmK1,
                     const __grid_constant__ CUtensorMap tmV0, const __grid_constant__ CUtensorMap tmV1,
                     const __grid_constant__ AttnParams p) {
  using C = RowCfg<RAW>;
  constexpr int BKV = C::BKV;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;
  unsigned char* sK = sQ + C::QBytes;
  unsigned char* sV = sK + C::NK * C::KBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + C::NV * C::VBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;          // [NK]
  uint64_t* k_empty = k_full + C::NK;     // [NK]
  uint64_t* v_full = k_empty + C::NK;     // [NV]
  uint64_t* v_empty = v_full + C::NV;     // [NV]
  uint64_t* s_full = v_empty + C::NV;     // [2] Q K^T of a tile has completed
  uint64_t* s_empty = s_full + 2;         // [2] the softmax warps hold its scores in registers (4 arrivals)
  uint64_t* p_full = s_empty + 2;         // [2] its probabilities are in tensor memory (4 arrivals)
  uint64_t* pv_full = p_full + 2;         // [2] its P V has completed
  uint64_t* q_raw = pv_full + 2;          // RAW: the fp32 rows of Q have landed
  uint64_t* k_raw = q_raw + 1;            // [NK] RAW: the fp32 rows of a K tile have landed
  uint64_t* v_raw = k_raw + C::NK;        // [NV] RAW: likewise of a V tile
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(v_raw + C::NV);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  unsigned char* s_cls = reinterpret_cast<unsigned char*>(tmem_holder + 4);   // [n_kv] tile classes of this query tile

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  // CTAs are numbered heaviest first: late query tiles see the most keys under a causal mask
  const int n_bh = p.B * p.H;
  const int n_qt = (p.Sq + kQRows - 1) / kQRows;
  const int q_tile = n_qt - 1 - (int)(blockIdx.x / (unsigned)n_bh);
  const int bh = (int)(blockIdx.x % (unsigned)n_bh);
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = q_tile * kQRows;
  const int n_kv = (p.Sk + BKV - 1) / BKV;
  grid_dependency_wait();       // the tile classes below may come from a kernel of the same plan
  grid_launch_dependents();
  {
    const unsigned char* cls = p.tile_class ? p.tile_class + (size_t)q_tile * n_kv : nullptr;
    const unsigned char dflt = p.mask ? 3 : 1;
    for (int j = threadIdx.x; j < n_kv; j += C::Threads) s_cls[j] = cls ? cls[j] : dflt;
  }
  auto next_tile = [&](int j) { while (j < n_kv && s_cls[j] == 0) ++j; return j; };

  if (threadIdx.x == 0) {
    mbar_init(q_full, RAW ? 4 : 1);       // RAW: the four converter warps publish an operand
    mbar_init(q_raw, 1);
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], RAW ? 4 : 1); mbar_init(&k_empty[s], 1); mbar_init(&k_raw[s], 1); }
    for (int s = 0; s < C::NV; ++s) { mbar_init(&v_full[s], RAW ? 2 : 1); mbar_init(&v_empty[s], 1); mbar_init(&v_raw[s], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4); mbar_init(&pv_full[i], 1);
    }
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

  const bool softmax_warp = warp >= C::SoftmaxWarp0 && warp < C::SoftmaxWarp0 + 4;
  if (!softmax_warp) {
  if constexpr (RAW) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::Light));
  if (warp == 0) {
    if (lane == 0) {
      if constexpr (RAW) {
        mbar_expect_tx(q_raw, C::QBytes / 2);
        for (int kb = 0; kb < 2; ++kb) tma_load_4d(&tmQ0, sQ + kb * (kQRows * 128), q_raw, kb * 32, q0, h, b);
      } else {
        mbar_expect_tx(q_full, C::QBytes);
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(&tmQ0, sQ + kb * (kQRows * 128), q_full, kb * 32, q0, h, b);
          tma_load_4d(&tmQ1, sQ + (2 + kb) * (kQRows * 128), q_full, kb * 32, q0, h, b);
        }
      }
      int t = 0;
      for (int j = next_tile(0); j < n_kv; j = next_tile(j + 1), ++t) {
        const int s = t % C::NK;
        if (!mbar_wait(&k_empty[s], ((uint32_t)(t / C::NK) & 1u) ^ 1u, abort_flag)) break;
        unsigned char* st = sK + s * C::KBytes;
        if constexpr (RAW) {
          mbar_expect_tx(&k_raw[s], C::KBytes / 2);
          for (int kb = 0; kb < 2; ++kb) tma_load_4d(&tmK0, st + kb * (BKV * 128), &k_raw[s], kb * 32, j * BKV, h, b);
        } else {
          mbar_expect_tx(&k_full[s], C::KBytes);
          for (int kb = 0; kb < 2; ++kb) {
            tma_load_4d(&tmK0, st + kb * (BKV * 128), &k_full[s], kb * 32, j * BKV, h, b);
            tma_load_4d(&tmK1, st + (2 + kb) * (BKV * 128), &k_full[s], kb * 32, j * BKV, h, b);
          }
        }
      }
    } else if (lane == 1) {
      int t = 0;
      for (int j = next_tile(0); j < n_kv; j = next_tile(j + 1), ++t) {
        const int s = t % C::NV;
        if (!mbar_wait(&v_empty[s], ((uint32_t)(t / C::NV) & 1u) ^ 1u, abort_flag)) break;
        unsigned char* st = sV + s * C::VBytes;
        if constexpr (RAW) {
          // rows of V: the two halves of the head dimension as tiles of [64 keys, 32 values]
          mbar_expect_tx(&v_raw[s], C::VBytes / 2);
          for (int half = 0; half < 2; ++half) tma_load_4d(&tmV0, st + half * kRawVHalf, &v_raw[s], half * 32, j * BKV, h, b);
        } else {
          mbar_expect_tx(&v_full[s], C::VBytes);
          for (int kb = 0; kb < 2; ++kb) {
            tma_load_4d(&tmV0, st + kb * (kHeadDim * 128), &v_full[s], j * BKV + kb * 32, 0, h, b);
            tma_load_4d(&tmV1, st + (2 + kb) * (kHeadDim * 128), &v_full[s], j * BKV + kb * 32, 0, h, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    int n_proc = 0;
    for (int j = 0; j < n_kv; ++j) n_proc += s_cls[j] != 0;
    auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0; };
    const uint32_t q_addr = smem_u32(sQ);
    const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
    auto issue_qk = [&](int t) -> bool {
      const int s = t % C::NK, buf = t & 1;
      // S buffer `buf` was last used by tile t - 2
      if (t >= 2 && !wait_all(&s_empty[buf], (uint32_t)((t >> 1) - 1) & 1u)) return false;
      if (!wait_all(&k_full[s], (uint32_t)(t / C::NK) & 1u)) return false;
      tc_fence_after();
      const uint32_t k_addr = smem_u32(sK + s * C::KBytes);
      const uint32_t d_s = tmem_base + (uint32_t)(C::ColS + buf * BKV);
      if (elect_one()) {
        // passes lo.hi, hi.lo, hi.hi; each: 2 k-blocks x 4 k-steps of 8 floats
#pragma unroll
        for (int pass = 0; pass < 3; ++pass) {
          const uint32_t qa = q_addr + (pass == 0 ? 2 * (kQRows * 128) : 0);
          const uint32_t ka = k_addr + (pass == 1 ? 2 * (BKV * 128) : 0);
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            const uint64_t da = make_kmajor_sw128_desc(qa + kb * (kQRows * 128));
            const uint64_t db = make_kmajor_sw128_desc(ka + kb * (BKV * 128));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma<true>(d_s, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_qk, (pass | kb | k) ? 1u : 0u);
          }
        }
        umma_commit(&s_full[buf]);
        umma_commit(&k_empty[s]);
      }
      __syncwarp();
      return true;
    };
    auto issue_pv = [&](int t) -> bool {
      const int s = t % C::NV, pbuf = t & 1;
      if (!wait_all(&p_full[pbuf], (uint32_t)(t >> 1) & 1u)) return false;
      if (!wait_all(&v_full[s], (uint32_t)(t / C::NV) & 1u)) return false;
      tc_fence_after();
      const uint32_t v_addr = smem_u32(sV + s * C::VBytes);
      const uint32_t t_p = tmem_base + (uint32_t)(C::ColP + pbuf * 2 * BKV);
      const uint32_t d_o = tmem_base + (uint32_t)C::ColO;
      const uint32_t fresh = (t % kChunkTiles) == 0 ? 0u : 1u;       // a chunk's first product starts a new accumulator
      if (elect_one()) {
        // passes P_lo.V_hi, P_hi.V_lo, P_hi.V_hi over the tile's two k-blocks of 32 keys
#pragma unroll
        for (int pass = 0; pass < 3; ++pass) {
          const uint32_t pa = t_p + (pass == 0 ? (uint32_t)BKV : 0u);
          const uint32_t va = v_addr + (pass == 1 ? 2 * (kHeadDim * 128) : 0);
          if constexpr (RAW) {
#pragma unroll
            for (int g = 0; g < 8; ++g)      // groups of 8 keys
              umma_ts_tf32(d_o, pa + (uint32_t)(g * 8), make_v_rows_desc(va + (uint32_t)(g * 1024)), idesc_pv, (pass | g) ? 1u : fresh);
          } else {
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
              const uint64_t db = make_kmajor_sw128_desc(va + kb * (kHeadDim * 128));
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ts_tf32(d_o, pa + (uint32_t)(kb * 32 + k * 8), db + (uint64_t)(k * 2), idesc_pv, (pass | kb | k) ? 1u : fresh);
            }
          }
        }
        umma_commit(&pv_full[pbuf]);
        umma_commit(&v_empty[s]);
      }
      __syncwarp();
      return true;
    };
    bool ok = n_proc == 0 || wait_all(q_full, 0);
    if (ok && n_proc > 0) ok = issue_qk(0);
    if (ok && n_proc > 1) ok = issue_qk(1);
    for (int t = 0; t < n_proc && ok; ++t) {
      // S(t) was taken into registers early in tile t's softmax, P(t) comes at its end: Q K^T of tile t + 2 first
      if (t + 2 < n_proc) ok = issue_qk(t + 2);
      if (ok) ok = issue_pv(t);
    }
  } else if (RAW && warp >= 8) {
    // converters: Q once, then every K tile in the producer's order
    const int ctid = (int)threadIdx.x - 256;
    auto publish = [&](uint64_t* bar) {
      fence_async_smem();                           // the planes are read by the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    bool ok = __all_sync(0xffffffffu, mbar_wait(q_raw, 0, abort_flag)) != 0;
    if (ok) {
      split_planes<128>(sQ, C::QBytes / 2, ctid);
      publish(q_full);
    }
    int t = 0;
    for (int j = next_tile(0); j < n_kv && ok; j = next_tile(j + 1), ++t) {
      const int s = t % C::NK;
      ok = __all_sync(0xffffffffu, mbar_wait(&k_raw[s], (uint32_t)(t / C::NK) & 1u, abort_flag)) != 0;
      if (!ok) break;
      split_planes<128>(sK + s * C::KBytes, C::KBytes / 2, ctid);
      publish(&k_full[s]);
    }
  } else if (RAW && warp >= 2 && warp < 4) {
    // converters of the V tiles
    const int ctid = (int)threadIdx.x - 64;
    bool ok = true;
    int t = 0;
    for (int j = next_tile(0); j < n_kv && ok; j = next_tile(j + 1), ++t) {
      const int s = t % C::NV;
      ok = __all_sync(0xffffffffu, mbar_wait(&v_raw[s], (uint32_t)(t / C::NV) & 1u, abort_flag)) != 0;
      if (!ok) break;
      split_planes<64>(sV + s * C::VBytes, C::VBytes / 2, ctid);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&v_full[s]);
    }
  }
  } else {
    if constexpr (RAW) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::Softmax));
    const int quarter = warp & 3;                   // tensor-memory lane quarter this warp may access
    const int r_in_tile = quarter * 32 + lane;
    const int row = q0 + r_in_tile;
    const bool row_ok = row < p.Sq;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    constexpr float kLog2e = 1.4426950408889634f;
    float o[kHeadDim];                              // the chunks folded so far, relative to m_ref
#pragma unroll
    for (int d = 0; d < kHeadDim; ++d) o[d] = 0.f;
    float m_ref = -CUDART_INF_F, l = 0.f;
    float scale = p.scale;
    const bool per_elem_scale = p.scale_buf != nullptr && !(p.scale_uniform && *p.scale_uniform);
    if (p.scale_buf && !per_elem_scale) scale = p.scale_buf[0];
    const bool simple_scale = !per_elem_scale && scale > 0.f;
    const size_t score_row = ((size_t)(b * p.H + h) * p.Sq + (row_ok ? row : 0)) * (size_t)p.Sk;
    const size_t mask_row = (size_t)b * p.mask_sb + (size_t)h * p.mask_sh + (size_t)(row_ok ? row : 0) * p.Sk;
    const uint32_t t_o = tmem_base + (uint32_t)C::ColO + lane_sel;
    bool ok = true;
    int t = 0;
    auto wait_warp = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0; };
    // o += O (tensor memory): both are relative to m_ref
    auto fold_chunk = [&]() {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld32(t_o + (uint32_t)(half * 32), r);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[half * 32 + i] = __fadd_rn(o[half * 32 + i], __uint_as_float(r[i]));
      }
    };
    for (int j = 0; j < n_kv && ok; ++j) {
      const int tclass = s_cls[j];
      if (tclass == 0) continue;
      const int buf = t & 1;
      const int k0 = j * BKV;
      const bool ragged = k0 + BKV > p.Sk;
      const bool by_element = !simple_scale || (p.mask && tclass == 3);
      uint2 w2 = make_uint2(0u, 0u);
      if (!by_element && tclass == 2)
        w2 = __ldg(reinterpret_cast<const uint2*>(p.mask_bits + (size_t)(row_ok ? row : 0) * p.mask_words + (k0 >> 5)));
      ok = wait_warp(&s_full[buf], (uint32_t)(t >> 1) & 1u);
      if (!ok) break;
      tc_fence_after();
      float x[BKV];
      {
        uint32_t* xu = reinterpret_cast<uint32_t*>(x);
        const uint32_t t_s = tmem_base + (uint32_t)(C::ColS + buf * BKV) + lane_sel;
        tmem_ld32_issue(t_s, xu);
        tmem_ld32_issue(t_s + 32, xu + 32);
        tmem_ld_wait();
      }
      // the scores are in registers: Q K^T of tile t + 2 may overwrite this S buffer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);

      if (by_element) {
        const bool with_mask = p.mask && tclass >= 2;
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int key = k0 + i;
          const bool in_range = key < p.Sk;
          float v = __fmul_rn(x[i], per_elem_scale ? (in_range ? p.scale_buf[score_row + key] : 0.f) : scale);
          if (with_mask && in_range) {
            if (p.mask_is_bool) { if (reinterpret_cast<const unsigned char*>(p.mask)[mask_row + key]) v = -CUDART_INF_F; }
            else v = __fadd_rn(v, reinterpret_cast<const float*>(p.mask)[mask_row + key]);
          }
          x[i] = in_range ? v : -CUDART_INF_F;
        }
      } else if (tclass == 2 || ragged) {
        uint32_t w[2] = {w2.x, w2.y};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int left = p.Sk - (k0 + c * 32);
          if (left < 32) w[c] |= left <= 0 ? 0xffffffffu : (0xffffffffu << left);
        }
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if ((w[i >> 5] >> (i & 31)) & 1u) x[i] = -CUDART_INF_F;
      }
      const bool fast = !by_element;                // scale still to be applied (folded into the exponent)
      float mt;
      {
        float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
        for (int i = 4; i < BKV; i += 2) mx[(i >> 1) & 3] = fmax3(mx[(i >> 1) & 3], x[i], x[i + 1]);
        mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        if (fast) mt *= scale;
      }
      // Chunk boundary: the products of the previous chunk are complete and O is folded into registers before this
      // tile's probabilities are published (its P V then starts a fresh accumulator).
      bool o_quiet = t == 0;
      if (t > 0 && (t % kChunkTiles) == 0) {
        ok = wait_warp(&pv_full[(t - 1) & 1], (uint32_t)((t - 1) >> 1) & 1u);
        if (!ok) break;
        tc_fence_after();
        fold_chunk();
        o_quiet = true;
      }
      // Lazy rescaling of everything accumulated so far (tensor memory, registers, row sum).
      const bool raise = m_ref != -CUDART_INF_F && (mt - m_ref) * kLog2e > kLazyRescaleLog2;
      if (__any_sync(0xffffffffu, raise)) {
        const float alpha = raise ? ex2_approx((m_ref - mt) * kLog2e) : 1.0f;
        if ((t % kChunkTiles) != 0) {               // the current chunk holds products: they must be complete
          if (!o_quiet) {
            ok = wait_warp(&pv_full[(t - 1) & 1], (uint32_t)((t - 1) >> 1) & 1u);
            if (!ok) break;
            tc_fence_after();
          }
          rescale_o_row(t_o, alpha);
          tc_fence_before();
        }
#pragma unroll
        for (int d = 0; d < kHeadDim; ++d) o[d] *= alpha;
        if (raise) { l *= alpha; m_ref = mt; }
      }
      if (m_ref == -CUDART_INF_F) m_ref = mt;       // nothing (or only zeros) accumulated so far
      const float m_use = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      const float cc = fast ? scale * kLog2e : kLog2e, ml = m_use * kLog2e;
      {
        float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          x[i] = ex2_approx(fmaf(x[i], cc, -ml));
          ps[i & 3] += x[i];
        }
        l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
      }
      // this P buffer was read by the P V of tile t - 2
      if (t >= 2) {
        ok = wait_warp(&pv_full[buf], (uint32_t)((t - 2) >> 1) & 1u);
        if (!ok) break;
      }
      {
        const uint32_t t_p = tmem_base + (uint32_t)(C::ColP + buf * 2 * BKV) + lane_sel;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = x[half * 32 + i];
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi[i]) : "f"(v));
            lo[i] = __float_as_uint(v - __uint_as_float(hi[i]));
          }
          tmem_st32_issue(t_p + (uint32_t)(half * 32), hi);
          tmem_st32_issue(t_p + (uint32_t)(BKV + half * 32), lo);
        }
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[buf]);
      ++t;
    }
    if (ok && t > 0) ok = wait_warp(&pv_full[(t - 1) & 1], (uint32_t)((t - 1) >> 1) & 1u);
    if (ok) {
      tc_fence_after();
      if (t > 0) fold_chunk();                      // the last chunk (warp-wide loads; only the stores are per row)
      if (row_ok) {
        const float inv = 1.0f / l;   // l = 0 for a fully masked row: 0 * inf = NaN, as the reference's softmax gives
        const size_t base = (size_t)((long long)b * p.out_sb + (long long)h * p.out_sh + (long long)row * p.out_ss);
        if (p.planes_hi) {
          float* hi = p.planes_hi + base;
          __nv_bfloat16* x16 = p.planes_16 + base;
          __nv_bfloat16* lo16 = x16 + p.planes_n;
#pragma unroll
          for (int d = 0; d < kHeadDim; d += 4) {
            uint32_t hw[4];
            float y[4], lw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              y[e] = o[d + e] * inv;
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hw[e]) : "f"(y[e]));
              lw[e] = __fadd_rn(y[e], -__uint_as_float(hw[e]));
            }
            *reinterpret_cast<uint4*>(hi + d) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            __nv_bfloat162 a0 = __floats2bfloat162_rn(y[0], y[1]), a1 = __floats2bfloat162_rn(y[2], y[3]);
            __nv_bfloat162 l0 = __floats2bfloat162_rn(lw[0], lw[1]), l1 = __floats2bfloat162_rn(lw[2], lw[3]);
            *reinterpret_cast<uint2*>(x16 + d) = make_uint2(*reinterpret_cast<uint32_t*>(&a0), *reinterpret_cast<uint32_t*>(&a1));
            *reinterpret_cast<uint2*>(lo16 + d) = make_uint2(*reinterpret_cast<uint32_t*>(&l0), *reinterpret_cast<uint32_t*>(&l1));
          }
        } else if (p.out_dtype == BG_F32) {
          float* out = reinterpret_cast<float*>(p.out) + base;
#pragma unroll
          for (int d = 0; d < kHeadDim; d += 4)
            *reinterpret_cast<float4*>(out + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
        } else {
          double* out = reinterpret_cast<double*>(p.out) + base;
#pragma unroll
          for (int d = 0; d < kHeadDim; d += 2) *reinterpret_cast<double2*>(out + d) = make_double2((double)(o[d] * inv), (double)(o[d + 1] * inv));
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

}  // namespace

bool attn_tf32_row_usable(int Sk, int out_dtype, const void* out, long long out_sb, long long out_sh, long long out_ss, bool raw) {
  if (out_dtype != BG_F32 && out_dtype != BG_F64) return false;
  const int n_kv = (Sk + 63) / 64;
  if ((size_t)(raw ? RowCfg<true>::SmemBytes : RowCfg<false>::SmemBytes) + 256 + 1024 + (size_t)n_kv > 227 * 1024) return false;
  const long long per16 = 16 / dtype_size(out_dtype);
  return (reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_sb % per16 == 0 && out_sh % per16 == 0 && out_ss % per16 == 0;
}

template <bool RAW>
static cudaError_t launch_row(const attn::AttnParams& p, const CUtensorMap maps[6], unsigned n_cta, size_t n_kv, cudaStream_t s) {
  using C = RowCfg<RAW>;
  const size_t smem = (size_t)C::SmemBytes + 256 + 1024 + n_kv;
  auto kern = attn_tf32_row_kernel<RAW>;
  attn::AttnParams pr = p;
  if (RAW) pr.idesc_pv |= 1u << 16;         // V rows: the B operand of P V is MN-major
  if (RAW) {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return e;
    if (fa.numRegs < C::Launch) return cudaErrorLaunchOutOfResources;   // the pool that setmaxnreg draws on
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_dependent(kern, dim3(n_cta), dim3(C::Threads), smem, s, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], pr);
}

cudaError_t launch_attn_tf32_row(const attn::AttnParams& p, const CUtensorMap maps[6], bool raw, cudaStream_t s) {
  const int n_qt = (p.Sq + kQRows - 1) / kQRows;
  const long long n_cta = (long long)n_qt * p.B * p.H;
  if (n_cta <= 0 || n_cta > 0x7fffffffll) return cudaErrorInvalidValue;
  const size_t n_kv = (size_t)((p.Sk + 63) / 64);
  return raw ? launch_row<true>(p, maps, (unsigned)n_cta, n_kv, s) : launch_row<false>(p, maps, (unsigned)n_cta, n_kv, s);
}

}  // namespace bg
