// Dense flash attention forward for head_dim 128 on tcgen05 / TMEM, primal and
// fused forward-mode tangent (same math as attn_fwd.cu, which serves head_dim 64):
//
//   S = Q K^T * scale,  P = softmax(S),  O = P V
//   dS = (dQ K^T + Q dK^T) * scale,  T = P .* dS,
//   dO = (T V + P dV) / l - (rowsum(T) / l) O
//
// The reference's JVP kernels are pinned to head_dim 64 (reference
// models/triton_mla_block_jvp.py:689); its model is shape-generic only through
// the library SDPA plug-ins (reference models/imf_dit_video.py:81-104).  This
// kernel is what lets the Wan2.1-1.3B-shaped geometry (12 heads of 128) run on
// the fused primal+tangent path.
//
// A head_dim-128 row is two 64-element (128-byte, SWIZZLE_128B) panels in shared
// memory; Q K^T runs 8 K-steps across the two panels, P V has N = 128.
// TMEM budget (512 columns of fp32 per SM) decides the shapes:
//   primal  : two 128-row query tiles per item, per tile S (64) + O (128);
//             four softmax warps per tile, the tiles take turns on the tensor core.
//   tangent : ONE query tile per item, O (128) + dO (128) and TWO S|dS buffers
//             (64 + 64 each), so Q K^T of K/V tile j+1 runs on the tensor core
//             while the CUDA cores do the softmax of tile j.  Eight softmax
//             warps share the tile: two threads per query row, 32 score columns
//             each; they exchange the row maximum through shared memory (bounded
//             mbarrier wait, like every other wait here).
// K (+dK) and V (+dV) travel in separate TMA rings: a K stage is free again as
// soon as its Q K^T has run, long before the matching V stage.
// Scheduling, split items, scratch layout and the merge kernel follow
// attn_fwd.cu: persistent grid, equal shares of the flattened (item, K/V tile)
// space, partial results of an item split between two CTAs merged afterwards.
#include "attn_fwd128.h"
#include "common.cuh"
#include "host_util.h"

namespace imf {
namespace a128 {

constexpr int HD = 128;
constexpr int TM = 128;              // query rows per tile
constexpr int BN = 64;               // K/V rows per tile
constexpr int QPANEL = TM * 128;     // bytes of one 64-column panel of a query tile
constexpr int KPANEL = BN * 128;     // bytes of one 64-column panel of a K/V tile

template <bool TANGENT>
struct Cfg {
  static constexpr int NT = TANGENT ? 1 : 2;
  static constexpr int ITEM_M = NT * TM;
  static constexpr int NQ = TANGENT ? 2 : 1;       // q (+ dq)
  static constexpr int NK = TANGENT ? 2 : 1;       // k (+ dk) per K stage, v (+ dv) per V stage
  static constexpr int STAGES = TANGENT ? 2 : 4;   // per ring
  static constexpr int SBUF = TANGENT ? 2 : 1;     // S (dS) buffers per tile
  static constexpr bool SPLIT = TANGENT;           // two threads per query row
  static constexpr int SOFT_WARPS = 8;
  static constexpr int WARP_MMA = 8, WARP_TMA = 9;
  static constexpr int THREADS = 12 * 32;
  static constexpr int REG_SOFT = 216, REG_OTHER = 72, REG_LAUNCH = 168;
  static_assert(SOFT_WARPS * 32 * REG_SOFT + (THREADS - SOFT_WARPS * 32) * REG_OTHER <=
                    THREADS * REG_LAUNCH, "register pool exceeded");
  static constexpr int TILE_COLS = TANGENT ? 512 : 256;
  static constexpr int COL_O = TANGENT ? 128 : 64;
  static constexpr int COL_DO = 256;               // tangent only
  __host__ __device__ static constexpr int col_s(int buf) { return TANGENT ? (buf ? 384 : 0) : 0; }
  __host__ __device__ static constexpr int col_ds(int buf) { return col_s(buf) + BN; }
  static constexpr int ACC = TANGENT ? 2 * HD : HD;          // fp32 accumulators per row
  static constexpr int NC = SPLIT ? BN / 2 : BN;             // score columns per thread
  static constexpr int ROW_THREADS = SPLIT ? 2 * TM : TM;    // softmax threads of one tile
  static_assert(NT * TILE_COLS <= 512, "TMEM budget");
};

template <bool TANGENT>
constexpr size_t part_floats() {
  return (size_t)Cfg<TANGENT>::ITEM_M * (Cfg<TANGENT>::ACC + 3);
}

template <bool TANGENT>
struct Smem {
  using C = Cfg<TANGENT>;
  alignas(1024) uint8_t q[C::NQ][C::NT][2 * QPANEL];
  alignas(1024) uint8_t k[C::STAGES][C::NK][2 * KPANEL];
  alignas(1024) uint8_t v[C::STAGES][C::NK][2 * KPANEL];
  float xmx[2][2][TM];      // row-maximum exchange [parity][half][row]
  float xlm[2][2][TM];      // (l, mu) exchange [half][which][row]
  uint64_t q_full, q_empty;
  uint64_t k_full[C::STAGES], k_empty[C::STAGES];
  uint64_t v_full[C::STAGES], v_empty[C::STAGES];
  uint64_t s_full[C::NT][C::SBUF];
  uint64_t p_full[C::NT][C::SBUF];
  uint64_t o_done[C::NT];      // every P V (waited on only by a rescale of the next iteration)
  uint64_t o_final[C::NT];     // last P V of a segment (one phase per segment, never skipped)
  uint64_t o_free[C::NT];
  uint64_t xbar;
  uint32_t tmem_base;
  int abort_flag;
};

struct Params {
  __nv_bfloat16* o;
  __nv_bfloat16* dout;
  float* lse;
  float* scratch;
  int B, H, L;
  int n_qblk, n_items, n_kv;
  long total_iters;
  int64_t o_sb, o_sl, o_sh;
  float scale;
  int* status;
};

struct Segment {
  int item, j0, j1;
  int slot, part;
};

__device__ __forceinline__ bool get_segment(const Params& p, int c, int G, int s, Segment& sg) {
  const long it0 = (long)c * p.total_iters / G, it1 = (long)(c + 1) * p.total_iters / G;
  const int item = (int)(it0 / p.n_kv) + s;
  const long base = (long)item * p.n_kv;
  if (base >= it1 || item >= p.n_items) return false;
  sg.item = item;
  sg.j0 = (int)(it0 > base ? it0 - base : 0);
  sg.j1 = (int)(it1 < base + p.n_kv ? it1 - base : p.n_kv);
  if (sg.j0 >= sg.j1) return false;
  if (sg.j0 == 0 && sg.j1 == p.n_kv) {
    sg.slot = -1;
    sg.part = 0;
  } else if (sg.j0 == 0) {
    sg.slot = c;
    sg.part = 0;
  } else {
    sg.slot = c - 1;
    sg.part = 1;
  }
  return true;
}

template <bool TANGENT>
__global__ void __launch_bounds__(Cfg<TANGENT>::THREADS, 1)
attn_fwd128_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_dq,
                   const __grid_constant__ CUtensorMap tm_dk,
                   const __grid_constant__ CUtensorMap tm_dv, const Params p) {
  using C = Cfg<TANGENT>;
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<Smem<TANGENT>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    mbar_init(&s.q_empty, 1);
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
      mbar_init(&s.v_full[i], 1);
      mbar_init(&s.v_empty[i], 1);
    }
    for (int t = 0; t < C::NT; ++t) {
      for (int b = 0; b < C::SBUF; ++b) {
        mbar_init(&s.s_full[t][b], 1);
        mbar_init(&s.p_full[t][b], C::ROW_THREADS);
      }
      mbar_init(&s.o_done[t], 1);
      mbar_init(&s.o_final[t], 1);
      mbar_init(&s.o_free[t], C::ROW_THREADS);
    }
    mbar_init(&s.xbar, C::SOFT_WARPS);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == C::WARP_MMA) {
    tmem_alloc(&s.tmem_base, 512);
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
      // ------------------------------------------------------ TMA producer --
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
          mbar_arrive_expect_tx(&s.q_full, C::NQ * C::NT * 2 * QPANEL);
          for (int t = 0; t < C::NT; ++t)
            for (int pn = 0; pn < 2; ++pn) {
              tma_load_4d(s.q[0][t] + pn * QPANEL, &tm_q, &s.q_full, pn * 64, h, q0 + t * TM, b);
              if (TANGENT)
                tma_load_4d(s.q[C::NQ - 1][t] + pn * QPANEL, &tm_dq, &s.q_full, pn * 64, h,
                            q0 + t * TM, b);
            }
          for (int j = sg.j0; j < sg.j1; ++j, ++kv_it) {
            const int st = (int)(kv_it % C::STAGES);
            const uint32_t par = (uint32_t)((kv_it / C::STAGES) & 1) ^ 1;
            if (kv_it >= C::STAGES) {
              ok = mbar_wait(&s.k_empty[st], par, abort_flag, p.status, STATUS_TIMEOUT_EMPTY);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(&s.k_full[st], C::NK * 2 * KPANEL);
            for (int pn = 0; pn < 2; ++pn) {
              tma_load_4d(s.k[st][0] + pn * KPANEL, &tm_k, &s.k_full[st], pn * 64, h, j * BN, b);
              if (TANGENT)
                tma_load_4d(s.k[st][C::NK - 1] + pn * KPANEL, &tm_dk, &s.k_full[st], pn * 64, h,
                            j * BN, b);
            }
            if (kv_it >= C::STAGES) {
              ok = mbar_wait(&s.v_empty[st], par, abort_flag, p.status, STATUS_TIMEOUT_EMPTY);
              if (!ok) break;
            }
            mbar_arrive_expect_tx(&s.v_full[st], C::NK * 2 * KPANEL);
            for (int pn = 0; pn < 2; ++pn) {
              tma_load_4d(s.v[st][0] + pn * KPANEL, &tm_v, &s.v_full[st], pn * 64, h, j * BN, b);
              if (TANGENT)
                tma_load_4d(s.v[st][C::NK - 1] + pn * KPANEL, &tm_dv, &s.v_full[st], pn * 64, h,
                            j * BN, b);
            }
          }
        }
      }
    } else if (warp == C::WARP_MMA) {
      // -------------------------------------------------------- MMA issuer --
      if (elect_one()) {
        constexpr uint32_t idesc_qk = idesc_bf16(TM, BN, 0, 0);
        constexpr uint32_t idesc_pv = idesc_bf16(TM, HD, 0, 1);
        // S[buf] (and dS[buf]) of tile t from K stage st
        auto issue_qk = [&](int t, int buf, int st) {
          const uint32_t tb = tmem + t * C::TILE_COLS;
          const uint32_t qa = smem_u32(s.q[0][t]), ka = smem_u32(s.k[st][0]);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            mma_ss(tb + C::col_s(buf), sdesc_kmajor(qa + (ks / 4) * QPANEL + (ks % 4) * 32),
                   sdesc_kmajor(ka + (ks / 4) * KPANEL + (ks % 4) * 32), idesc_qk, ks != 0);
          if (TANGENT) {
            const uint32_t dqa = smem_u32(s.q[C::NQ - 1][t]);
            const uint32_t dka = smem_u32(s.k[st][C::NK - 1]);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
              mma_ss(tb + C::col_ds(buf), sdesc_kmajor(dqa + (ks / 4) * QPANEL + (ks % 4) * 32),
                     sdesc_kmajor(ka + (ks / 4) * KPANEL + (ks % 4) * 32), idesc_qk, ks != 0);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
              mma_ss(tb + C::col_ds(buf), sdesc_kmajor(qa + (ks / 4) * QPANEL + (ks % 4) * 32),
                     sdesc_kmajor(dka + (ks / 4) * KPANEL + (ks % 4) * 32), idesc_qk, 1);
          }
          tc_commit(&s.s_full[t][buf]);
          tc_commit(&s.k_empty[st]);      // counted once per stage: see the calls
        };
        // `last`: the segment's final P V.  The epilogue waits on o_final, whose phases are
        // each waited on exactly once.  It cannot use o_done: with Q K^T issued ahead, the
        // softmax warps may get there while o_done is still two phases back, and a parity
        // wait cannot tell a phase from the one two before it.
        auto issue_pv = [&](int t, int buf, int st, bool first, bool last) {
          const uint32_t tb = tmem + t * C::TILE_COLS;
          const uint32_t va = smem_u32(s.v[st][0]);
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)
            mma_ts(tb + C::COL_O, tb + C::col_s(buf) + ks * 8, sdesc_mnmajor(va + ks * 2048, KPANEL),
                   idesc_pv, !(first && ks == 0));
          if (TANGENT) {
            const uint32_t dva = smem_u32(s.v[st][C::NK - 1]);
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              mma_ts(tb + C::COL_DO, tb + C::col_ds(buf) + ks * 8,
                     sdesc_mnmajor(va + ks * 2048, KPANEL), idesc_pv, !(first && ks == 0));
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              mma_ts(tb + C::COL_DO, tb + C::col_s(buf) + ks * 8,
                     sdesc_mnmajor(dva + ks * 2048, KPANEL), idesc_pv, 1);
          }
          tc_commit(&s.o_done[t]);
          if (last) tc_commit(&s.o_final[t]);
        };
        long kv_it = 0, it = 0;
        Segment sg;
        bool ok = true;
        for (int si = 0; ok && get_segment(p, cta, G, si, sg); ++si) {
          const int n_j = sg.j1 - sg.j0;
          ok = mbar_wait(&s.q_full, si & 1, abort_flag, p.status, STATUS_TIMEOUT_TMA) &&
               mbar_wait(&s.k_full[kv_it % C::STAGES], (uint32_t)((kv_it / C::STAGES) & 1),
                         abort_flag, p.status, STATUS_TIMEOUT_TMA);
          if (!ok) break;
          tc_fence_after();
          if constexpr (C::SBUF == 2) {
            // one tile, two S buffers: Q K^T of iteration it + 1 is issued before waiting for
            // the softmax of iteration it
            issue_qk(0, (int)(it & 1), (int)(kv_it % C::STAGES));
            if (n_j == 1) tc_commit(&s.q_empty);
            for (int jj = 0; jj < n_j && ok; ++jj, ++kv_it, ++it) {
              const int st = (int)(kv_it % C::STAGES);
              if (jj + 1 < n_j) {
                const long nk = kv_it + 1;
                const int st1 = (int)(nk % C::STAGES);
                ok = mbar_wait(&s.k_full[st1], (uint32_t)((nk / C::STAGES) & 1), abort_flag,
                               p.status, STATUS_TIMEOUT_TMA);
                if (!ok) break;
                tc_fence_after();
                issue_qk(0, (int)((it + 1) & 1), st1);
                if (jj + 2 == n_j) tc_commit(&s.q_empty);
              }
              ok = mbar_wait(&s.p_full[0][it & 1], (uint32_t)((it >> 1) & 1), abort_flag, p.status,
                             STATUS_TIMEOUT_SOFTMAX) &&
                   mbar_wait(&s.v_full[st], (uint32_t)((kv_it / C::STAGES) & 1), abort_flag,
                             p.status, STATUS_TIMEOUT_TMA);
              if (ok && jj == 0 && si > 0)
                ok = mbar_wait(&s.o_free[0], (uint32_t)((si - 1) & 1), abort_flag, p.status,
                               STATUS_TIMEOUT_SOFTMAX);
              if (!ok) break;
              tc_fence_after();
              issue_pv(0, (int)(it & 1), st, jj == 0, jj + 1 == n_j);
              tc_commit(&s.v_empty[st]);
            }
          } else {
            // two tiles, one S buffer each: the tiles take turns
#pragma unroll
            for (int t = 0; t < C::NT; ++t) {
              const uint32_t tb = tmem + t * C::TILE_COLS;
              const uint32_t qa = smem_u32(s.q[0][t]), ka = smem_u32(s.k[kv_it % C::STAGES][0]);
#pragma unroll
              for (int ks = 0; ks < HD / 16; ++ks)
                mma_ss(tb + C::col_s(0), sdesc_kmajor(qa + (ks / 4) * QPANEL + (ks % 4) * 32),
                       sdesc_kmajor(ka + (ks / 4) * KPANEL + (ks % 4) * 32), idesc_qk, ks != 0);
              tc_commit(&s.s_full[t][0]);
            }
            tc_commit(&s.k_empty[kv_it % C::STAGES]);
            if (n_j == 1) tc_commit(&s.q_empty);
            for (int jj = 0; jj < n_j && ok; ++jj, ++kv_it, ++it) {
              const int st = (int)(kv_it % C::STAGES);
              ok = mbar_wait(&s.v_full[st], (uint32_t)((kv_it / C::STAGES) & 1), abort_flag, p.status,
                             STATUS_TIMEOUT_TMA);
#pragma unroll
              for (int t = 0; t < C::NT; ++t) {
                if (!ok) break;
                ok = mbar_wait(&s.p_full[t][0], (uint32_t)(it & 1), abort_flag, p.status,
                               STATUS_TIMEOUT_SOFTMAX);
                if (ok && jj == 0 && si > 0)
                  ok = mbar_wait(&s.o_free[t], (uint32_t)((si - 1) & 1), abort_flag, p.status,
                                 STATUS_TIMEOUT_SOFTMAX);
                if (!ok) break;
                tc_fence_after();
                issue_pv(t, 0, st, jj == 0, jj + 1 == n_j);
                if (t == C::NT - 1) tc_commit(&s.v_empty[st]);
                if (jj + 1 < n_j) {
                  const long nk = kv_it + 1;
                  const int st1 = (int)(nk % C::STAGES);
                  if (t == 0) {
                    ok = mbar_wait(&s.k_full[st1], (uint32_t)((nk / C::STAGES) & 1), abort_flag,
                                   p.status, STATUS_TIMEOUT_TMA);
                    if (!ok) break;
                    tc_fence_after();
                  }
                  const uint32_t tb = tmem + t * C::TILE_COLS;
                  const uint32_t qa = smem_u32(s.q[0][t]), ka = smem_u32(s.k[st1][0]);
#pragma unroll
                  for (int ks = 0; ks < HD / 16; ++ks)
                    mma_ss(tb + C::col_s(0), sdesc_kmajor(qa + (ks / 4) * QPANEL + (ks % 4) * 32),
                           sdesc_kmajor(ka + (ks / 4) * KPANEL + (ks % 4) * 32), idesc_qk, ks != 0);
                  tc_commit(&s.s_full[t][0]);
                  if (t == C::NT - 1) {
                    tc_commit(&s.k_empty[st1]);
                    if (jj + 2 == n_j) tc_commit(&s.q_empty);
                  }
                }
              }
            }
          }
        }
      }
    }
  } else {
    // --------------------------------------- softmax / correction / epilogue --
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::REG_SOFT));
    constexpr int NC = C::NC;
    const int grp = warp >> 2, wl = warp & 3;
    const int t = C::SPLIT ? 0 : grp;
    const int half = C::SPLIT ? grp : 0;
    const int c0 = half * NC;                       // first score column of this thread
    const int row = wl * 32 + lane;
    const int row_in_item = t * TM + row;
    const uint32_t tb = tmem_addr(tmem, wl * 32, t * C::TILE_COLS);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    long it = 0;
    uint32_t xn = 0;                                // exchanges done so far (phase of xbar)
    Segment sg;
    bool ok = true;
    for (int si = 0; ok && get_segment(p, cta, G, si, sg); ++si) {
      const int qb = sg.item % p.n_qblk, h = (sg.item / p.n_qblk) % p.H,
                b = sg.item / (p.n_qblk * p.H);
      const int q_row = qb * C::ITEM_M + row_in_item;
      float m_used = -INFINITY, l_sum = 0.f, l_sum2 = 0.f, mu_sum = 0.f, mu_sum2 = 0.f;
      for (int j = sg.j0; j < sg.j1 && ok; ++j, ++it) {
        const int buf = C::SBUF == 2 ? (int)(it & 1) : 0;
        const uint32_t sph = C::SBUF == 2 ? (uint32_t)((it >> 1) & 1) : (uint32_t)(it & 1);
        ok = __all_sync(0xffffffffu, mbar_wait(&s.s_full[t][buf], sph, abort_flag, p.status,
                                               STATUS_TIMEOUT_MMA));
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[NC];
        uint32_t dsv[TANGENT ? NC : 1];
#pragma unroll
        for (int c = 0; c < NC; c += 32) tmem_ld32(tb + C::col_s(buf) + c0 + c, sv + c);
        if (TANGENT) {
#pragma unroll
          for (int c = 0; c < NC; c += 32) tmem_ld32(tb + C::col_ds(buf) + c0 + c, dsv + c);
        }
        tc_wait_ld();
        const int kv_rem = p.L - j * BN - c0;
        if (kv_rem < NC) {
#pragma unroll
          for (int i = 0; i < NC; ++i)
            if (i >= kv_rem) sv[i] = 0xff800000u;  // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < NC; i += 4) {
          asm("max.f32 %0, %0, %1, %2;" : "+f"(mx0) : "f"(__uint_as_float(sv[i])), "f"(__uint_as_float(sv[i + 1])));
          asm("max.f32 %0, %0, %1, %2;" : "+f"(mx1) : "f"(__uint_as_float(sv[i + 2])), "f"(__uint_as_float(sv[i + 3])));
        }
        float mx = fmaxf(mx0, mx1);
        if (C::SPLIT) {
          // both column halves of a row must use the same maximum.  The exchange is also the
          // point after which every S / dS column of this buffer has been read, so the bf16
          // P / T written below may overlap the partner's score columns.
          s.xmx[it & 1][half][row] = mx;
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.xbar);
          ok = __all_sync(0xffffffffu, mbar_wait(&s.xbar, xn & 1, abort_flag, p.status,
                                                 STATUS_TIMEOUT_SOFTMAX));
          ++xn;
          if (!ok) break;
          mx = fmaxf(mx, s.xmx[it & 1][half ^ 1][row]);
        }
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
            // split rows: half 0 rescales O, half 1 rescales dO
            const uint32_t rb = tb + (C::SPLIT && half ? C::COL_DO : C::COL_O);
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
              uint32_t ov[32];
              tmem_ld32(rb + c, ov);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              tmem_st32(rb + c, ov);
            }
            tc_wait_st();
          }
        }
        const float neg_m = -m_used * scale_log2;
#pragma unroll
        for (int c = 0; c < NC; c += 32) {
          uint32_t pk[16];
          uint32_t tk[TANGENT ? 16 : 1];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(sv[c + i]), scale_log2, neg_m));
            const float p1 = ex2(fmaf(__uint_as_float(sv[c + i + 1]), scale_log2, neg_m));
            pk[i / 2] = pack_bf16(p0, p1);
            l_sum += p0;
            l_sum2 += p1;
            if (TANGENT) {
              const float t0 = p0 * __uint_as_float(dsv[c + i]) * p.scale;
              const float t1 = p1 * __uint_as_float(dsv[c + i + 1]) * p.scale;
              mu_sum += t0;
              mu_sum2 += t1;
              tk[i / 2] = pack_bf16(t0, t1);
            }
          }
          tmem_st16(tb + C::col_s(buf) + (c0 + c) / 2, pk);
          if (TANGENT) tmem_st16(tb + C::col_ds(buf) + (c0 + c) / 2, tk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&s.p_full[t][buf]);
      }
      // ---- epilogue of this segment ----
      if (ok)
        ok = mbar_wait(&s.o_final[t], (uint32_t)(si & 1), abort_flag, p.status,
                       STATUS_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float l_tot = l_sum + l_sum2;
      float mu_tot = mu_sum + mu_sum2;
      if (C::SPLIT) {
        s.xlm[half][0][row] = l_tot;
        s.xlm[half][1][row] = mu_tot;
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.xbar);
        ok = __all_sync(0xffffffffu, mbar_wait(&s.xbar, xn & 1, abort_flag, p.status,
                                               STATUS_TIMEOUT_SOFTMAX));
        ++xn;
        if (!ok) break;
        l_tot += s.xlm[half ^ 1][0][row];
        mu_tot += s.xlm[half ^ 1][1][row];
      }
      const bool live = q_row < p.L;
      if (sg.slot < 0) {
        const float inv_l = 1.f / l_tot;
        const int64_t off = (int64_t)b * p.o_sb + (int64_t)q_row * p.o_sl + (int64_t)h * p.o_sh;
        // split rows: each half writes 64 of the 128 output columns (of o and of dout)
        const int cb = C::SPLIT ? half * (HD / 2) : 0, ce = C::SPLIT ? cb + HD / 2 : HD;
        for (int c = cb; c < ce; c += 32) {
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
        if (live && p.lse && half == 0)
          p.lse[((int64_t)b * p.H + h) * p.L + q_row] = m_used * p.scale + __logf(l_tot);
      } else {
        // partial result of a split item: raw accumulators + (m, l, mu); with split rows half 0
        // stores the O accumulators (columns 0-127), half 1 the dO accumulators (128-255)
        float* part = p.scratch + ((size_t)sg.slot * 2 + sg.part) * part_floats<TANGENT>();
        float* acc = part + (size_t)row_in_item * C::ACC + (C::SPLIT ? half * HD : 0);
        const uint32_t rb = tb + (C::SPLIT && half ? C::COL_DO : C::COL_O);
        for (int c = 0; c < HD; c += 32) {
          uint32_t ov[32];
          tmem_ld32(rb + c, ov);
          tc_wait_ld();
          float4* dst = reinterpret_cast<float4*>(acc + c);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(ov[4 * i]), __uint_as_float(ov[4 * i + 1]),
                                 __uint_as_float(ov[4 * i + 2]), __uint_as_float(ov[4 * i + 3]));
        }
        if (half == 0) {
          float* stats = part + (size_t)C::ITEM_M * C::ACC;
          stats[row_in_item] = m_used;
          stats[C::ITEM_M + row_in_item] = l_tot;
          stats[2 * C::ITEM_M + row_in_item] = mu_tot;
        }
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
    tmem_dealloc(tmem, 512);
  }
}

// Merge the two halves of every split item (one CTA per share boundary).
template <bool TANGENT>
__global__ void __launch_bounds__(Cfg<TANGENT>::ITEM_M)
attn_fwd128_combine_kernel(const Params p, int G) {
  using C = Cfg<TANGENT>;
  const int c = blockIdx.x;
  const long bound = (long)(c + 1) * p.total_iters / G;
  if (bound % p.n_kv == 0) return;
  const int item = (int)(bound / p.n_kv);
  if (item >= p.n_items) return;
  const int qb = item % p.n_qblk, h = (item / p.n_qblk) % p.H, b = item / (p.n_qblk * p.H);
  const int r = threadIdx.x;
  const int q_row = qb * C::ITEM_M + r;
  if (q_row >= p.L) return;
  const float* pa = p.scratch + ((size_t)c * 2 + 0) * part_floats<TANGENT>();
  const float* pb = p.scratch + ((size_t)c * 2 + 1) * part_floats<TANGENT>();
  const float* sa = pa + (size_t)C::ITEM_M * C::ACC;
  const float* sb = pb + (size_t)C::ITEM_M * C::ACC;
  const float ma = sa[r], mb = sb[r];
  const float m = fmaxf(ma, mb);
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const float wa = ex2((ma - m) * scale_log2), wb = ex2((mb - m) * scale_log2);
  const float l = sa[C::ITEM_M + r] * wa + sb[C::ITEM_M + r] * wb;
  const float mu = sa[2 * C::ITEM_M + r] * wa + sb[2 * C::ITEM_M + r] * wb;
  const float inv_l = 1.f / l;
  const float* aa = pa + (size_t)r * C::ACC;
  const float* ab = pb + (size_t)r * C::ACC;
  const int64_t off = (int64_t)b * p.o_sb + (int64_t)q_row * p.o_sl + (int64_t)h * p.o_sh;
  for (int col = 0; col < HD; col += 2) {
    const float o0 = (aa[col] * wa + ab[col] * wb) * inv_l;
    const float o1 = (aa[col + 1] * wa + ab[col + 1] * wb) * inv_l;
    *reinterpret_cast<uint32_t*>(p.o + off + col) = pack_bf16(o0, o1);
    if (TANGENT) {
      const float d0 = (aa[HD + col] * wa + ab[HD + col] * wb) * inv_l - mu * inv_l * o0;
      const float d1 = (aa[HD + col + 1] * wa + ab[HD + col + 1] * wb) * inv_l - mu * inv_l * o1;
      *reinterpret_cast<uint32_t*>(p.dout + off + col) = pack_bf16(d0, d1);
    }
  }
  if (p.lse) p.lse[((int64_t)b * p.H + h) * p.L + q_row] = m * p.scale + __logf(l);
}

// 4-D map over a (B, L, H, 128) bf16 tensor whose box is one 64-column panel of `rows` rows
static int make_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int64_t sb, int64_t sl,
                    int64_t sh, int rows) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)sh * 2, (uint64_t)sl * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)rows, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, str, box);
}

static int grid_for(int n_items) {
  constexpr int MAX_DEVICES = 64;
  static int sms_of_device[MAX_DEVICES] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = (dev >= 0 && dev < MAX_DEVICES) ? sms_of_device[dev] : 0;
  if (!sms) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    if (dev >= 0 && dev < MAX_DEVICES) sms_of_device[dev] = sms;
  }
  return n_items < sms ? n_items : sms;
}

template <bool TANGENT>
static int launch(const Fwd128Args& a) {
  using C = Cfg<TANGENT>;
  Params prm;
  prm.o = static_cast<__nv_bfloat16*>(a.o);
  prm.dout = static_cast<__nv_bfloat16*>(a.dout);
  prm.lse = a.lse;
  prm.scratch = static_cast<float*>(a.scratch);
  prm.B = a.B; prm.H = a.H; prm.L = a.L;
  prm.o_sb = a.o_sb; prm.o_sl = a.o_sl; prm.o_sh = a.o_sh;
  prm.scale = a.scale;
  prm.status = a.status;
  prm.n_qblk = (a.L + C::ITEM_M - 1) / C::ITEM_M;
  prm.n_items = prm.n_qblk * a.H * a.B;
  prm.n_kv = (a.L + BN - 1) / BN;
  prm.total_iters = (long)prm.n_items * prm.n_kv;
  const int G = grid_for(prm.n_items);
  if (G > 1 && prm.n_items > G) {
    if (prm.scratch == nullptr ||
        (size_t)a.scratch_bytes < (size_t)G * 2 * part_floats<TANGENT>() * sizeof(float))
      return IMF_ERR_ARG;
  }
  CUtensorMap mq, mk, mv, mdq, mdk, mdv;
  int rc;
  const int64_t* st = a.strides;
  if ((rc = make_map(&mq, a.q, a.B, a.L, a.H, st[0], st[1], st[2], TM))) return rc;
  if ((rc = make_map(&mk, a.k, a.B, a.L, a.H, st[3], st[4], st[5], BN))) return rc;
  if ((rc = make_map(&mv, a.v, a.B, a.L, a.H, st[6], st[7], st[8], BN))) return rc;
  if (TANGENT) {
    if ((rc = make_map(&mdq, a.dq, a.B, a.L, a.H, st[9], st[10], st[11], TM))) return rc;
    if ((rc = make_map(&mdk, a.dk, a.B, a.L, a.H, st[12], st[13], st[14], BN))) return rc;
    if ((rc = make_map(&mdv, a.dv, a.B, a.L, a.H, st[15], st[16], st[17], BN))) return rc;
  } else {
    mdq = mq;
    mdk = mk;
    mdv = mv;
  }
  auto kern = attn_fwd128_kernel<TANGENT>;
  const size_t smem = sizeof(Smem<TANGENT>) + 1024;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return IMF_ERR_LAUNCH;
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  kern<<<G, C::THREADS, smem, stream>>>(mq, mk, mv, mdq, mdk, mdv, prm);
  if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  if (G > 1 && prm.n_items > G) {
    attn_fwd128_combine_kernel<TANGENT><<<G - 1, C::ITEM_M, 0, stream>>>(prm, G);
    if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  }
  return IMF_OK;
}

}  // namespace a128

long attn_fwd128_scratch_bytes(int B, int L, int H, int tangent) {
  const int item_m = tangent ? a128::Cfg<true>::ITEM_M : a128::Cfg<false>::ITEM_M;
  const int n_items = ((L + item_m - 1) / item_m) * H * B;
  const int G = a128::grid_for(n_items);
  if (G <= 1 || n_items <= G) return 0;
  const size_t per = tangent ? a128::part_floats<true>() : a128::part_floats<false>();
  return (long)((size_t)G * 2 * per * sizeof(float));
}

int attn_fwd128_launch(const Fwd128Args& a) {
  return a.dq != nullptr ? a128::launch<true>(a) : a128::launch<false>(a);
}

}  // namespace imf
