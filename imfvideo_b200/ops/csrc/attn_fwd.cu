// Dense flash attention forward on tcgen05 / TMEM, with an optional fused
// forward-mode tangent (JVP):
//
//   S = Q K^T * scale,  P = softmax(S),  O = P V
//   dS = (dQ K^T + Q dK^T) * scale,  T = P .* dS,
//   dO = (T V + P dV) / l - (rowsum(T) / l) O          (l = rowsum exp)
//
// i.e. the primal, its tangent and the log-sum-exp in ONE pass over K/V, with
// O(L) memory.  Replaces the reference's CuTeDSL mma.sync kernel and Triton
// flash-JVP kernel (reference models/flash_jvp_kernel.py:51-570,
// models/triton_block_jvp.py:228-346) and the FA/SDPA primal forward.
//
// Work item = NT 128-row query tiles that share every K/V tile, of one (batch,
// head): NT = 3 tiles against 64-row K/V tiles in the primal kernel (2 tiles
// against 128-row K/V tiles when three would leave SMs without an item), 2
// tiles in the tangent kernel.  Warps 4t .. 4t+3: softmax + O-correction + epilogue
// of tile t (one query row per thread, rows live in TMEM lanes); then one warp
// with the single-thread tcgen05.mma issuer, one TMA producer warp and two
// warps that only donate registers (setmaxnreg).  The tiles take turns: while
// one tile's softmax runs on the CUDA cores the tensor core works on another.
// The softmax warps are bound by instruction issue and dependency latency
// (two of them per scheduler reach 0.43 instructions per cycle), which is why
// the primal kernel keeps three tiles in flight.  P (and T) are written back
// to TMEM as bf16 over the S (dS) columns and are the A operand of the second
// GEMM.  In the primal kernel V carries 16 extra columns of ones, so the row
// sum l comes out of the tensor core as column 64 of O.  O is rescaled lazily
// (only when the running max grows by > 2^8).
//
// Scheduling: the grid is persistent (one CTA per SM).  The flattened
// (item, K/V tile) iteration space is cut into equal contiguous shares, so an
// item may be split between two neighbouring CTAs; such partial results
// (un-normalised accumulators + running max) go to a scratch buffer and a
// small second kernel merges them.  This removes the wave quantisation that
// equal items on 148 SMs would cost (304 items = 2.05 waves at 29,140 rows).
//
// Tensors are (B, L, H, 64) bf16 with arbitrary 16-byte-aligned strides;
// ragged L is handled by TMA zero fill + masking of the last K/V tile.
#include "attn_fwd128.h"
#include "common.cuh"
#include "host_util.h"

namespace imf {

constexpr int ATT_HD = 64;
constexpr int ATT_TILE_M = 128;

// Work item = NT query tiles of 128 rows that share every K/V tile.
//   tangent kernel : NT 2, K/V tiles of 64 rows, TMEM per tile S|dS|O|dO
//   primal kernel  : NT 2, K/V tiles of 128 rows, row sum on the tensor core (ones column)
//                    NT 3, K/V tiles of 64 rows, ones column
//                    NT 4, K/V tiles of 64 rows, row sum in registers
// More tiles in flight put more softmax warps on each scheduler (the softmax
// warps are bound by instruction issue and dependency latency, not by a pipe).
template <bool TANGENT, int NTP>
struct AttCfg {
  static constexpr int NT = TANGENT ? 2 : NTP;
  static constexpr int ITEM_M = NT * ATT_TILE_M;
  static constexpr int BN = (TANGENT || NT > 2) ? 64 : 128;
  static constexpr int NQ = TANGENT ? 2 : 1;       // q + dq
  static constexpr int NKV = TANGENT ? 4 : 2;      // k, v (+ dk, dv)
  static constexpr int STAGES = (!TANGENT && NT > 2) ? 4 : 3;
  static constexpr bool ONES = !TANGENT && NT < 4; // row sum on the tensor core
  static constexpr int N_PV = ONES ? ATT_HD + 16 : ATT_HD;
  static constexpr int SOFT_WARPS = 4 * NT;
  static constexpr int WARP_MMA = SOFT_WARPS, WARP_TMA = SOFT_WARPS + 1;
  // softmax warps + one warpgroup holding the MMA warp, the TMA warp and two warps that
  // only donate registers (setmaxnreg is a warpgroup-wide instruction)
  static constexpr int THREADS = (SOFT_WARPS + 4) * 32;
  static constexpr int REG_SOFT = NT == 2 ? 216 : (NT == 3 ? 136 : 104);
  static constexpr int REG_OTHER = NT == 2 ? 72 : (NT == 3 ? 104 : 64);
  // setmaxnreg.inc draws from what the CTA was launched with (threads x registers per
  // thread as compiled: 168 / 128 / 96 for 384 / 512 / 640 threads); a request beyond
  // that pool blocks for ever
  static constexpr int REG_LAUNCH = NT == 2 ? 168 : (NT == 3 ? 128 : 96);
  static_assert(SOFT_WARPS * 32 * REG_SOFT + (THREADS - SOFT_WARPS * 32) * REG_OTHER <=
                    THREADS * REG_LAUNCH, "register pool exceeded");
  // TMEM columns per query tile
  static constexpr int COL_S = 0;
  static constexpr int COL_DS = BN;
  static constexpr int COL_O = TANGENT ? 2 * BN : BN;
  static constexpr int COL_DO = COL_O + ATT_HD;    // tangent only
  static constexpr int TILE_COLS = NT == 2 ? 256 : (NT == 3 ? 160 : 128);
  static constexpr int TMEM_COLS = 512;
  static_assert(COL_O + (TANGENT ? 2 * ATT_HD : N_PV) <= TILE_COLS && NT * TILE_COLS <= 512, "");
  static constexpr int ACC = TANGENT ? 2 * ATT_HD : ATT_HD;   // fp32 accumulators per row
};

// scratch record of one half of a split item: [ITEM_M][ACC] accumulators,
// then m, l, mu per row
template <bool TANGENT, int NTP>
constexpr size_t att_part_floats() {
  return (size_t)AttCfg<TANGENT, NTP>::ITEM_M * (AttCfg<TANGENT, NTP>::ACC + 3);
}

template <bool TANGENT, int NTP>
struct AttSmem {
  using C = AttCfg<TANGENT, NTP>;
  alignas(1024) uint8_t q[C::NQ][C::NT][ATT_TILE_M * 128];           // [q|dq][tile]
  alignas(1024) uint8_t kv[C::STAGES][C::NKV][C::BN * 128];          // k, v, dk, dv
  alignas(1024) uint8_t ones[C::ONES ? C::BN * 128 : 1024];          // bf16 1.0 panel
  uint64_t q_full, q_empty;
  uint64_t kv_full[C::STAGES];
  uint64_t kv_empty[C::STAGES];
  uint64_t s_full[C::NT];
  uint64_t p_full[C::NT];
  uint64_t o_done[C::NT];
  uint64_t o_free[C::NT];
  uint32_t tmem_base;
  int abort_flag;
};

struct AttParams {
  __nv_bfloat16* o;
  __nv_bfloat16* dout;     // tangent output (TANGENT only)
  float* lse;              // (B, H, L) natural-log LSE of scaled scores
  float* scratch;          // split-item partials: [grid][2][part floats]
  int B, H, L;
  int n_qblk, n_items, n_kv;
  long total_iters;        // n_items * n_kv
  int64_t o_sb, o_sl, o_sh;   // output strides in elements
  float scale;
  int* status;
};

struct Segment {
  int item, j0, j1;        // K/V tile range [j0, j1)
  int slot, part;          // scratch slot / half when partial (slot < 0: complete item)
};

// Segment `s` of CTA `c` (its share is iterations [c*T/G, (c+1)*T/G)).
__device__ __forceinline__ bool get_segment(const AttParams& p, int c, int G, int s, Segment& sg) {
  const long it0 = (long)c * p.total_iters / G, it1 = (long)(c + 1) * p.total_iters / G;
  const int first_item = (int)(it0 / p.n_kv);
  const int item = first_item + s;
  const long base = (long)item * p.n_kv;
  if (base >= it1 || item >= p.n_items) return false;
  sg.item = item;
  sg.j0 = (int)(it0 > base ? it0 - base : 0);
  sg.j1 = (int)(it1 < base + p.n_kv ? it1 - base : p.n_kv);
  if (sg.j0 >= sg.j1) return false;
  if (sg.j0 == 0 && sg.j1 == p.n_kv) {
    sg.slot = -1;
    sg.part = 0;
  } else if (sg.j0 == 0) {   // head half: the item continues in CTA c + 1
    sg.slot = c;
    sg.part = 0;
  } else {                   // tail half: the item started in CTA c - 1
    sg.slot = c - 1;
    sg.part = 1;
  }
  return true;
}

template <bool TANGENT, int NTP>
__global__ void __launch_bounds__(AttCfg<TANGENT, NTP>::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_dq,
                const __grid_constant__ CUtensorMap tm_dk,
                const __grid_constant__ CUtensorMap tm_dv, const AttParams p) {
  using C = AttCfg<TANGENT, NTP>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<AttSmem<TANGENT, NTP>*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    mbar_init(&s.q_empty, 1);
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[i], 1);
    }
    for (int t = 0; t < C::NT; ++t) {
      mbar_init(&s.s_full[t], 1);
      mbar_init(&s.p_full[t], ATT_TILE_M);
      mbar_init(&s.o_done[t], 1);
      mbar_init(&s.o_free[t], ATT_TILE_M);
    }
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (C::ONES) {
    uint32_t* o32 = reinterpret_cast<uint32_t*>(s.ones);
    for (int i = threadIdx.x; i < BN * 128 / 4; i += C::THREADS) o32[i] = 0x3f803f80u;  // bf16 1.0 x2
    fence_proxy_async_smem();
  }
  if (warp == C::WARP_MMA) {
    tmem_alloc(&s.tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;

  if (warp >= C::SOFT_WARPS) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::REG_OTHER));
    if (warp == C::WARP_TMA) {
      // ---------------------------------------------------- TMA producer --
      if (elect_one()) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
        long kv_it = 0;
        Segment sg;
        bool ok = true;
        for (int si = 0; ok && get_segment(p, cta, G, si, sg); ++si) {
          const int qb = sg.item % p.n_qblk, h = (sg.item / p.n_qblk) % p.H,
                    b = sg.item / (p.n_qblk * p.H);
          const int q0 = qb * C::ITEM_M;
          if (si > 0) ok = mbar_wait(&s.q_empty, (si - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY);
          if (!ok) break;
          mbar_arrive_expect_tx(&s.q_full, C::NQ * C::NT * ATT_TILE_M * 128);
          for (int t = 0; t < C::NT; ++t) {
            tma_load_4d(s.q[0][t], &tm_q, &s.q_full, 0, h, q0 + t * ATT_TILE_M, b);
            if (TANGENT)
              tma_load_4d(s.q[C::NQ - 1][t], &tm_dq, &s.q_full, 0, h, q0 + t * ATT_TILE_M, b);
          }
          for (int j = sg.j0; j < sg.j1; ++j, ++kv_it) {
            const int st = (int)(kv_it % C::STAGES);
            if (kv_it >= C::STAGES) {
              ok = mbar_wait(&s.kv_empty[st], (uint32_t)((kv_it / C::STAGES) & 1) ^ 1, abort_flag,
                             p.status, STATUS_TIMEOUT_EMPTY);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(&s.kv_full[st], C::NKV * BN * 128);
            tma_load_4d(s.kv[st][0], &tm_k, &s.kv_full[st], 0, h, j * BN, b);
            tma_load_4d(s.kv[st][1], &tm_v, &s.kv_full[st], 0, h, j * BN, b);
            if (TANGENT) {
              tma_load_4d(s.kv[st][C::NKV - 2], &tm_dk, &s.kv_full[st], 0, h, j * BN, b);
              tma_load_4d(s.kv[st][C::NKV - 1], &tm_dv, &s.kv_full[st], 0, h, j * BN, b);
            }
          }
        }
      }
    } else if (warp == C::WARP_MMA) {
      // ------------------------------------------------------ MMA issuer --
      if (elect_one()) {
        constexpr uint32_t idesc_qk = idesc_bf16(ATT_TILE_M, BN, 0, 0);
        constexpr uint32_t idesc_pv = idesc_bf16(ATT_TILE_M, C::N_PV, 0, 1);
        constexpr uint32_t idesc_pv64 = idesc_bf16(ATT_TILE_M, ATT_HD, 0, 1);
        const uint32_t ones_a = smem_u32(s.ones);
        auto issue_qk = [&](int t, int st, uint64_t* done) {
          const uint32_t tb = tmem + t * C::TILE_COLS;
          const uint32_t qa = smem_u32(s.q[0][t]), ka = smem_u32(s.kv[st][0]);
#pragma unroll
          for (int ks = 0; ks < ATT_HD / 16; ++ks)
            mma_ss(tb + C::COL_S, sdesc_kmajor(qa + ks * 32), sdesc_kmajor(ka + ks * 32), idesc_qk,
                   ks != 0);
          if (TANGENT) {
            const uint32_t dqa = smem_u32(s.q[C::NQ - 1][t]);
            const uint32_t dka = smem_u32(s.kv[st][C::NKV - 2]);
#pragma unroll
            for (int ks = 0; ks < ATT_HD / 16; ++ks)
              mma_ss(tb + C::COL_DS, sdesc_kmajor(dqa + ks * 32), sdesc_kmajor(ka + ks * 32),
                     idesc_qk, ks != 0);
#pragma unroll
            for (int ks = 0; ks < ATT_HD / 16; ++ks)
              mma_ss(tb + C::COL_DS, sdesc_kmajor(qa + ks * 32), sdesc_kmajor(dka + ks * 32),
                     idesc_qk, 1);
          }
          tc_commit(done);
        };
        auto issue_pv = [&](int t, int st, bool first) {
          const uint32_t tb = tmem + t * C::TILE_COLS;
          const uint32_t va = smem_u32(s.kv[st][1]);
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            // B = [V | ones]: panel 0 is the V tile, panel 1 (LBO away) the ones panel
            const uint32_t vk = va + ks * 2048;
            const uint64_t db = C::ONES ? sdesc_mnmajor(vk, (ones_a + ks * 2048) - vk)
                                        : sdesc_mnmajor(vk, BN * 128);
            mma_ts(tb + C::COL_O, tb + C::COL_S + ks * 8, db, idesc_pv, !(first && ks == 0));
          }
          if (TANGENT) {
            const uint32_t dva = smem_u32(s.kv[st][C::NKV - 1]);
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              mma_ts(tb + C::COL_DO, tb + C::COL_DS + ks * 8,
                     sdesc_mnmajor(va + ks * 2048, BN * 128), idesc_pv64, !(first && ks == 0));
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              mma_ts(tb + C::COL_DO, tb + C::COL_S + ks * 8,
                     sdesc_mnmajor(dva + ks * 2048, BN * 128), idesc_pv64, 1);
          }
          tc_commit(&s.o_done[t]);
        };
        long kv_it = 0, it = 0;
        Segment sg;
        bool ok = true;
        for (int si = 0; ok && get_segment(p, cta, G, si, sg); ++si) {
          const int n_j = sg.j1 - sg.j0;
          ok = mbar_wait(&s.q_full, si & 1, abort_flag, p.status, STATUS_TIMEOUT_TMA) &&
               mbar_wait(&s.kv_full[kv_it % C::STAGES], (uint32_t)((kv_it / C::STAGES) & 1),
                         abort_flag, p.status, STATUS_TIMEOUT_TMA);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < C::NT; ++t) issue_qk(t, (int)(kv_it % C::STAGES), &s.s_full[t]);
          if (n_j == 1) tc_commit(&s.q_empty);
          for (int jj = 0; jj < n_j && ok; ++jj, ++kv_it, ++it) {
            const int st = (int)(kv_it % C::STAGES);
#pragma unroll
            for (int t = 0; t < C::NT; ++t) {
              if (!ok) break;
              ok = mbar_wait(&s.p_full[t], (uint32_t)(it & 1), abort_flag, p.status,
                             STATUS_TIMEOUT_SOFTMAX);
              if (ok && jj == 0 && si > 0)   // epilogue of the previous segment has drained O
                ok = mbar_wait(&s.o_free[t], (uint32_t)((si - 1) & 1), abort_flag, p.status,
                               STATUS_TIMEOUT_SOFTMAX);
              if (!ok) break;
              tc_fence_after();
              issue_pv(t, st, jj == 0);
              if (t == C::NT - 1) tc_commit(&s.kv_empty[st]);
              if (jj + 1 < n_j) {
                const long nk = kv_it + 1;
                const int st1 = (int)(nk % C::STAGES);
                if (t == 0) {
                  ok = mbar_wait(&s.kv_full[st1], (uint32_t)((nk / C::STAGES) & 1), abort_flag,
                                 p.status, STATUS_TIMEOUT_TMA);
                  if (!ok) break;
                  tc_fence_after();
                }
                issue_qk(t, st1, &s.s_full[t]);
                if (t == C::NT - 1 && jj + 2 == n_j) tc_commit(&s.q_empty);   // last Q read of the item
              }
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------- softmax / correction / epilogue --
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::REG_SOFT));
    const int t = warp >> 2;
    const int wl = warp & 3;
    const int row_in_item = t * ATT_TILE_M + wl * 32 + lane;
    const uint32_t tb = tmem_addr(tmem, wl * 32, t * C::TILE_COLS);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    long it = 0;
    Segment sg;
    bool ok = true;
    for (int si = 0; ok && get_segment(p, cta, G, si, sg); ++si) {
      const int qb = sg.item % p.n_qblk, h = (sg.item / p.n_qblk) % p.H,
                b = sg.item / (p.n_qblk * p.H);
      const int q_row = qb * C::ITEM_M + row_in_item;
      float m_used = -INFINITY, l_sum = 0.f, l_sum2 = 0.f, mu_sum = 0.f, mu_sum2 = 0.f;
      for (int j = sg.j0; j < sg.j1 && ok; ++j, ++it) {
        ok = __all_sync(0xffffffffu, mbar_wait(&s.s_full[t], (uint32_t)(it & 1), abort_flag,
                                               p.status, STATUS_TIMEOUT_MMA));
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[BN];
#pragma unroll
        for (int c = 0; c < BN; c += 32) tmem_ld32(tb + C::COL_S + c, sv + c);
        uint32_t dsv[TANGENT ? BN : 1];
        if (TANGENT) {
#pragma unroll
          for (int c = 0; c < BN; c += 32) tmem_ld32(tb + C::COL_DS + c, dsv + c);
        }
        tc_wait_ld();
        const int kv_rem = p.L - j * BN;
        if (kv_rem < BN) {
#pragma unroll
          for (int i = 0; i < BN; ++i)
            if (i >= kv_rem) sv[i] = 0xff800000u;  // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < BN; i += 4) {
          asm("max.f32 %0, %0, %1, %2;" : "+f"(mx0) : "f"(__uint_as_float(sv[i])), "f"(__uint_as_float(sv[i + 1])));
          asm("max.f32 %0, %0, %1, %2;" : "+f"(mx1) : "f"(__uint_as_float(sv[i + 2])), "f"(__uint_as_float(sv[i + 3])));
        }
        const float mx = fmaxf(mx0, mx1);
        if (j == sg.j0) {
          m_used = mx;
        } else {
          const bool need = (mx - m_used) * scale_log2 > 8.0f;
          if (__any_sync(0xffffffffu, need)) {
            float alpha = 1.f;
            if (need) {
              alpha = ex2((m_used - mx) * scale_log2);
              m_used = mx;
            }
            l_sum *= alpha;
            l_sum2 *= alpha;
            mu_sum *= alpha;
            mu_sum2 *= alpha;
            ok = __all_sync(0xffffffffu, mbar_wait(&s.o_done[t], (uint32_t)((it - 1) & 1),
                                                   abort_flag, p.status, STATUS_TIMEOUT_MMA));
            if (!ok) break;
            tc_fence_after();
            constexpr int NRES = TANGENT ? 2 * ATT_HD : C::N_PV;   // 128 or 80 columns
#pragma unroll
            for (int c = 0; c + 32 <= NRES; c += 32) {
              uint32_t ov[32];
              tmem_ld32(tb + C::COL_O + c, ov);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              tmem_st32(tb + C::COL_O + c, ov);
            }
            if (NRES % 32) {
              uint32_t ov[16];
              tmem_ld16(tb + C::COL_O + (NRES / 32) * 32, ov);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              tmem_st16(tb + C::COL_O + (NRES / 32) * 32, ov);
            }
            tc_wait_st();
          }
        }
        const float neg_m = -m_used * scale_log2;
#pragma unroll
        for (int c = 0; c < BN; c += 64) {
          uint32_t pk[32];
          uint32_t tk[TANGENT ? 32 : 1];
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(sv[c + i]), scale_log2, neg_m));
            const float p1 = ex2(fmaf(__uint_as_float(sv[c + i + 1]), scale_log2, neg_m));
            pk[i / 2] = pack_bf16(p0, p1);
            if (!C::ONES) {
              l_sum += p0;
              l_sum2 += p1;
            }
            if (TANGENT) {
              const float t0 = p0 * __uint_as_float(dsv[c + i]) * p.scale;
              const float t1 = p1 * __uint_as_float(dsv[c + i + 1]) * p.scale;
              mu_sum += t0;
              mu_sum2 += t1;
              tk[i / 2] = pack_bf16(t0, t1);
            }
          }
          tmem_st32(tb + C::COL_S + c / 2, pk);
          if (TANGENT) tmem_st32(tb + C::COL_DS + c / 2, tk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&s.p_full[t]);
      }
      // ---- epilogue of this segment ----
      if (ok)
        ok = mbar_wait(&s.o_done[t], (uint32_t)((it - 1) & 1), abort_flag, p.status,
                       STATUS_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float l_tot = l_sum + l_sum2;
      const float mu_tot = mu_sum + mu_sum2;
      if (C::ONES) {
        uint32_t lv[8];
        tmem_ld8(tb + C::COL_O + ATT_HD, lv);
        tc_wait_ld();
        l_tot = __uint_as_float(lv[0]);
      }
      const bool live = q_row < p.L;
      if (sg.slot < 0) {
        const float inv_l = 1.f / l_tot;
        const int64_t off = (int64_t)b * p.o_sb + (int64_t)q_row * p.o_sl + (int64_t)h * p.o_sh;
#pragma unroll
        for (int c = 0; c < ATT_HD; c += 32) {
          uint32_t ov[32];
          tmem_ld32(tb + C::COL_O + c, ov);
          tc_wait_ld();
          uint32_t ob[16];
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * inv_l);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            ob[i] = pack_bf16(__uint_as_float(ov[2 * i]), __uint_as_float(ov[2 * i + 1]));
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(p.o + off + c);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_uint4(ob[4 * i], ob[4 * i + 1], ob[4 * i + 2], ob[4 * i + 3]);
          }
          if (TANGENT) {
            uint32_t dv_[32];
            tmem_ld32(tb + C::COL_DO + c, dv_);
            tc_wait_ld();
            const float mul = mu_tot * inv_l;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float d0 = __uint_as_float(dv_[2 * i]) * inv_l - mul * __uint_as_float(ov[2 * i]);
              const float d1 =
                  __uint_as_float(dv_[2 * i + 1]) * inv_l - mul * __uint_as_float(ov[2 * i + 1]);
              ob[i] = pack_bf16(d0, d1);
            }
            if (live) {
              uint4* dst = reinterpret_cast<uint4*>(p.dout + off + c);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                dst[i] = make_uint4(ob[4 * i], ob[4 * i + 1], ob[4 * i + 2], ob[4 * i + 3]);
            }
          }
        }
        if (live && p.lse)
          p.lse[((int64_t)b * p.H + h) * p.L + q_row] = m_used * p.scale + __logf(l_tot);
      } else {
        // partial result of a split item: raw accumulators + (m, l, mu)
        float* part = p.scratch + ((size_t)sg.slot * 2 + sg.part) * att_part_floats<TANGENT, NTP>();
        float* acc = part + (size_t)row_in_item * C::ACC;
#pragma unroll
        for (int c = 0; c < C::ACC; c += 32) {
          uint32_t ov[32];
          tmem_ld32(tb + C::COL_O + c, ov);
          tc_wait_ld();
          float4* dst = reinterpret_cast<float4*>(acc + c);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(ov[4 * i]), __uint_as_float(ov[4 * i + 1]),
                                 __uint_as_float(ov[4 * i + 2]), __uint_as_float(ov[4 * i + 3]));
        }
        float* stats = part + (size_t)C::ITEM_M * C::ACC;
        stats[row_in_item] = m_used;
        stats[C::ITEM_M + row_in_item] = l_tot;
        stats[2 * C::ITEM_M + row_in_item] = mu_tot;
      }
      tc_fence_before();
      mbar_arrive(&s.o_free[t]);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == C::WARP_MMA) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// Merge the two halves of every split item (one CTA per share boundary).
constexpr int ATT_COMBINE_THREADS = 1024;
template <bool TANGENT, int NTP>
__global__ void __launch_bounds__(ATT_COMBINE_THREADS)
attn_fwd_combine_kernel(const AttParams p, int G) {
  using C = AttCfg<TANGENT, NTP>;
  const int c = blockIdx.x;              // boundary between CTA c and c + 1
  const long bound = (long)(c + 1) * p.total_iters / G;
  if (bound % p.n_kv == 0) return;       // boundary falls on an item start: nothing was split
  const int item = (int)(bound / p.n_kv);
  if (item >= p.n_items) return;
  const int qb = item % p.n_qblk, h = (item / p.n_qblk) % p.H, b = item / (p.n_qblk * p.H);
  const float* pa = p.scratch + ((size_t)c * 2 + 0) * att_part_floats<TANGENT, NTP>();
  const float* pb = p.scratch + ((size_t)c * 2 + 1) * att_part_floats<TANGENT, NTP>();
  const float* sa = pa + (size_t)C::ITEM_M * C::ACC;
  const float* sb = pb + (size_t)C::ITEM_M * C::ACC;
  const float scale_log2 = p.scale * 1.4426950408889634f;
  // one warp per row, a lane per pair of columns: 256-byte reads of the two partial rows and
  // a 128-byte write of the merged row (a thread per row would touch a cache line per value).
  // The CTA is alone on its SM with one item to merge, so it is as wide as a CTA gets (32
  // warps) and the row loop is unrolled: the time goes into load latency, not into bytes.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll 4
  for (int r = warp; r < C::ITEM_M; r += nwarps) {
    const int q_row = qb * C::ITEM_M + r;
    if (q_row >= p.L) continue;
    const float ma = sa[r], mb = sb[r];
    const float m = fmaxf(ma, mb);
    const float wa = ex2((ma - m) * scale_log2), wb = ex2((mb - m) * scale_log2);
    const float l = sa[C::ITEM_M + r] * wa + sb[C::ITEM_M + r] * wb;
    const float mu = sa[2 * C::ITEM_M + r] * wa + sb[2 * C::ITEM_M + r] * wb;
    const float inv_l = 1.f / l;
    const float* aa = pa + (size_t)r * C::ACC;
    const float* ab = pb + (size_t)r * C::ACC;
    const int64_t off = (int64_t)b * p.o_sb + (int64_t)q_row * p.o_sl + (int64_t)h * p.o_sh;
    const int col = 2 * lane;
    const float2 xa = *reinterpret_cast<const float2*>(aa + col);
    const float2 xb = *reinterpret_cast<const float2*>(ab + col);
    const float o0 = (xa.x * wa + xb.x * wb) * inv_l;
    const float o1 = (xa.y * wa + xb.y * wb) * inv_l;
    *reinterpret_cast<uint32_t*>(p.o + off + col) = pack_bf16(o0, o1);
    if (TANGENT) {
      const float2 ya = *reinterpret_cast<const float2*>(aa + ATT_HD + col);
      const float2 yb = *reinterpret_cast<const float2*>(ab + ATT_HD + col);
      const float d0 = (ya.x * wa + yb.x * wb) * inv_l - mu * inv_l * o0;
      const float d1 = (ya.y * wa + yb.y * wb) * inv_l - mu * inv_l * o1;
      *reinterpret_cast<uint32_t*>(p.dout + off + col) = pack_bf16(d0, d1);
    }
    if (p.lse && lane == 0) p.lse[((int64_t)b * p.H + h) * p.L + q_row] = m * p.scale + __logf(l);
  }
}

static int make_qkv_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int64_t sb,
                        int64_t sl, int64_t sh, int rows) {
  uint64_t dims[4] = {(uint64_t)ATT_HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)sh * 2, (uint64_t)sl * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {(uint32_t)ATT_HD, 1, (uint32_t)rows, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, str, box);
}

// SM count of the CURRENT device (cached per device index: a host may hold GPUs of
// different sizes, and a persistent grid larger than the device would not be co-resident).
static int att_grid(int n_items) {
  constexpr int MAX_DEVICES = 64;
  static int sms_of_device[MAX_DEVICES] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = (dev >= 0 && dev < MAX_DEVICES) ? sms_of_device[dev] : 0;
  if (!sms) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    if (dev >= 0 && dev < MAX_DEVICES) sms_of_device[dev] = sms;   // same value from every thread
  }
  return n_items < sms ? n_items : sms;
}

// Query tiles per work item of the primal kernel: three, unless that leaves SMs without an
// item while two tiles per item would not (problems of about one wave).
static int primal_nt(int B, int L, int H) {
  const int items3 = ((L + 383) / 384) * H * B, items2 = ((L + 255) / 256) * H * B;
  const int sms = att_grid(1 << 30);
  return (items3 < sms && items2 > items3) ? 2 : 3;
}

template <bool TANGENT, int NTP>
static int launch_attn_fwd(const void* q, const void* k, const void* v, const void* dq,
                           const void* dk, const void* dv, const int64_t* strides, AttParams prm,
                           size_t scratch_bytes, cudaStream_t stream) {
  using C = AttCfg<TANGENT, NTP>;
  CUtensorMap mq, mk, mv, mdq, mdk, mdv;
  int rc;
  const int B = prm.B, L = prm.L, H = prm.H;
  prm.n_qblk = (L + C::ITEM_M - 1) / C::ITEM_M;
  prm.n_items = prm.n_qblk * H * B;
  prm.n_kv = (L + C::BN - 1) / C::BN;
  prm.total_iters = (long)prm.n_items * prm.n_kv;
  const int G = att_grid(prm.n_items);
  if (G > 1 && prm.n_items > G) {
    if (prm.scratch == nullptr ||
        scratch_bytes < (size_t)G * 2 * att_part_floats<TANGENT, NTP>() * sizeof(float))
      return IMF_ERR_ARG;
  }
  // strides: [q_sb,q_sl,q_sh, k_sb,k_sl,k_sh, v_sb,v_sl,v_sh, dq.., dk.., dv..]
  if ((rc = make_qkv_map(&mq, q, B, L, H, strides[0], strides[1], strides[2], ATT_TILE_M))) return rc;
  if ((rc = make_qkv_map(&mk, k, B, L, H, strides[3], strides[4], strides[5], C::BN))) return rc;
  if ((rc = make_qkv_map(&mv, v, B, L, H, strides[6], strides[7], strides[8], C::BN))) return rc;
  if (TANGENT) {
    if ((rc = make_qkv_map(&mdq, dq, B, L, H, strides[9], strides[10], strides[11], ATT_TILE_M)))
      return rc;
    if ((rc = make_qkv_map(&mdk, dk, B, L, H, strides[12], strides[13], strides[14], C::BN)))
      return rc;
    if ((rc = make_qkv_map(&mdv, dv, B, L, H, strides[15], strides[16], strides[17], C::BN)))
      return rc;
  } else {
    mdq = mq;
    mdk = mk;
    mdv = mv;
  }
  auto kern = attn_fwd_kernel<TANGENT, NTP>;
  const size_t smem = sizeof(AttSmem<TANGENT, NTP>) + 1024;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return IMF_ERR_LAUNCH;
  kern<<<G, C::THREADS, smem, stream>>>(mq, mk, mv, mdq, mdk, mdv, prm);
  if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  if (G > 1 && prm.n_items > G) {
    attn_fwd_combine_kernel<TANGENT, NTP><<<G - 1, ATT_COMBINE_THREADS, 0, stream>>>(prm, G);
    if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  }
  return IMF_OK;
}

}  // namespace imf

// Bytes of scratch the forward needs for (B, L, H): 0 when no item is split.
extern "C" long imf_attn_fwd_scratch_bytes(int B, int L, int H, int tangent) {
  using namespace imf;
  const int nt = tangent ? 2 : primal_nt(B, L, H);
  const int item_m = nt * ATT_TILE_M;
  const int n_items = ((L + item_m - 1) / item_m) * H * B;
  const int G = att_grid(n_items);
  if (G <= 1 || n_items <= G) return 0;
  const size_t per = tangent ? att_part_floats<true, 2>()
                             : (nt == 3 ? att_part_floats<false, 3>() : att_part_floats<false, 2>());
  return (long)((size_t)G * 2 * per * sizeof(float));
}

// Same for either head_dim (64 or 128).
extern "C" long imf_attn_fwd_scratch_bytes_hd(int B, int L, int H, int tangent, int head_dim) {
  if (head_dim == 128) return imf::attn_fwd128_scratch_bytes(B, L, H, tangent);
  return imf_attn_fwd_scratch_bytes(B, L, H, tangent);
}

// Dense attention forward (+ optional tangent).  All tensors (B, L, H, head_dim)
// bf16, head_dim 64 or 128; `strides` holds (batch, row, head) element strides for q, k, v and,
// when tangents are given, dq, dk, dv.  o/dout contiguous-in-last-dim with
// strides (o_sb, o_sl, o_sh).  lse: (B, H, L) fp32 or null.  scratch: device
// buffer of at least imf_attn_fwd_scratch_bytes() bytes (may be null if 0).
extern "C" int imf_attn_fwd(const void* q, const void* k, const void* v, const void* dq,
                            const void* dk, const void* dv, void* o, void* dout, float* lse,
                            int B, int L, int H, int head_dim, const int64_t* strides,
                            int64_t o_sb, int64_t o_sl, int64_t o_sh, float scale, void* scratch,
                            long scratch_bytes, int* status, void* stream) {
  using namespace imf;
  if ((head_dim != ATT_HD && head_dim != 128) || B <= 0 || L <= 0 || H <= 0) return IMF_ERR_ARG;
  if ((o_sl & 7) || (o_sh & 7) || (o_sb & 7) || (reinterpret_cast<uintptr_t>(o) & 15))
    return IMF_ERR_ARG;
  if (head_dim == 128) {
    if (dq != nullptr && (dout == nullptr || (reinterpret_cast<uintptr_t>(dout) & 15)))
      return IMF_ERR_ARG;
    Fwd128Args a{q, k, v, dq, dk, dv, o, dout, lse, B, L, H, strides, o_sb, o_sl, o_sh, scale,
                 scratch, scratch_bytes, status, stream};
    return attn_fwd128_launch(a);
  }
  AttParams prm;
  prm.o = static_cast<__nv_bfloat16*>(o);
  prm.dout = static_cast<__nv_bfloat16*>(dout);
  prm.lse = lse;
  prm.scratch = static_cast<float*>(scratch);
  prm.B = B;
  prm.H = H;
  prm.L = L;
  prm.o_sb = o_sb;
  prm.o_sl = o_sl;
  prm.o_sh = o_sh;
  prm.scale = scale;
  prm.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dq != nullptr) {
    if (dout == nullptr || (reinterpret_cast<uintptr_t>(dout) & 15)) return IMF_ERR_ARG;
    return launch_attn_fwd<true, 2>(q, k, v, dq, dk, dv, strides, prm, (size_t)scratch_bytes, st);
  }
  if (primal_nt(B, L, H) == 3)
    return launch_attn_fwd<false, 3>(q, k, v, nullptr, nullptr, nullptr, strides, prm,
                                     (size_t)scratch_bytes, st);
  return launch_attn_fwd<false, 2>(q, k, v, nullptr, nullptr, nullptr, strides, prm,
                                   (size_t)scratch_bytes, st);
}

// ---------------------------------------------------------------------------
// Allocation-free entry point (see attn_noalloc.h for who needs it and why).
// ---------------------------------------------------------------------------
#include "attn_noalloc.h"

namespace imf {
constexpr size_t NOALLOC_FLOATS =
    (size_t)IMF_ATTN_NOALLOC_MAX_CTAS * 2 * ((size_t)AttCfg<false, 3>::ITEM_M * (ATT_HD + 3));
// Split-item partials of the primal forward.  In host code this name is only a
// stand-in for the symbol, not a device address: the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_attn_noalloc_scratch[NOALLOC_FLOATS];
}  // namespace imf

extern "C" int imf_attn_fwd_noalloc(const void* q, const void* k, const void* v, void* o,
                                    float* lse, int B, int L, int H, int head_dim,
                                    const int64_t* strides, int64_t o_sb, int64_t o_sl,
                                    int64_t o_sh, float scale, int* status, void* stream) {
  using namespace imf;
  static_assert(NOALLOC_FLOATS == (size_t)IMF_ATTN_NOALLOC_MAX_CTAS * 2 * att_part_floats<false, 3>(),
                "scratch array and partial record size disagree");
  constexpr int MAX_DEVICES = 64;
  static float* scratch_of_device[MAX_DEVICES] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return IMF_ERR_DRIVER;
  if (scratch_of_device[dev] == nullptr) {
    // once per device, with that device current; do this outside stream capture
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_attn_noalloc_scratch) != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "imf_attn_fwd_noalloc: cudaGetSymbolAddress failed on device %d\n", dev);
      return IMF_ERR_DRIVER;
    }
    scratch_of_device[dev] = static_cast<float*>(ptr);
  }
  if (head_dim != ATT_HD) return IMF_ERR_ARG;     // the built-in scratch is sized for head_dim 64
  const long need = imf_attn_fwd_scratch_bytes(B, L, H, 0);
  if (need > (long)(NOALLOC_FLOATS * sizeof(float))) {
    fprintf(stderr,
            "imf_attn_fwd_noalloc: problem needs %ld bytes of partial-result scratch, the "
            "built-in array holds %zu (at most %d thread blocks)\n",
            need, NOALLOC_FLOATS * sizeof(float), IMF_ATTN_NOALLOC_MAX_CTAS);
    return IMF_ERR_TOO_LARGE;
  }
  return imf_attn_fwd(q, k, v, nullptr, nullptr, nullptr, o, nullptr, lse, B, L, H, head_dim,
                      strides, o_sb, o_sl, o_sh, scale, scratch_of_device[dev],
                      (long)(NOALLOC_FLOATS * sizeof(float)), status, stream);
}
