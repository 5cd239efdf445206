// Block-sparse softmax attention forward for SLA2 (1-D blocks and 3-D cube
// tiles) with INT8 scores on the tensor core and an optional fused tangent.
//
//   S   = (Q8 K8^T) * sq[q block] * sk[k block] * scale     tcgen05 kind::i8, s32 in TMEM
//   P   = round(127 * exp2(S - m)) / 127                    (QAT grid of the probabilities)
//   O  += P V~                                              V~ = fake-quantised V (bf16)
//   dS  = (dQ K^T + Q dK^T) * scale,  T = P .* dS           bf16 MMAs (straight-through)
//   dO  = (T V~ + P dV) / l - (rowsum T / l) O
//
// over the key blocks listed for each 128-row query tile.  A query tile may
// hold two routing blocks of 64 rows; the list is then the union of their
// routed blocks and a 2-bit flag per entry says which half attends it.
// Replaces the reference's `_attn_fwd_qat`, `_attn_fwd`, `_sla2_sparse_jvp_kernel`,
// `_mla_video_sparse_jvp_kernel` and `_sla2_cube_jvp_qat_kernel` (reference
// models/sla2_vendor/kernel_sparse_qat.py:28-117, models/sla2_cube_qat.py:59-169,
// models/sla2_mla_jvp.py:108-197); `imf_quantize_blocks` replaces `_quant_blocks`.
//
// A CTA runs NT independent query tiles side by side (4 in the primal kernel,
// 1 with the tangent, where two CTAs share an SM): warps 4t .. 4t+3 are the
// softmax / correction / epilogue warps of tile slot t (one row per thread),
// one thread of the MMA warp issues every slot's tcgen05.mma stream and one
// thread of the TMA warp loads every slot's K/V blocks, both by probing the
// slots' barriers without blocking, so the slots never wait for one another.
// Slots walk over the query tiles with a fixed stride (persistent grid).  The
// softmax warps are bound by instruction issue and latency, so what matters is
// how many of them each scheduler can pick from (four per scheduler) and how
// few instructions an element costs: the de-quantisation scale and the softmax
// scale are one FMA, the x127 of the QAT grid is folded into the exponent, the
// rounding is a magic-number add, P is stored as the integer grid value (the
// 1/127 cancels in O / l), and a 64-row half that does not attend a block
// writes zeros without touching the scores.
#include <type_traits>

#include "common.cuh"
#include "host_util.h"

namespace imf {

constexpr int SP_HD = 64;
constexpr int SP_M = 128;
constexpr int SP_BK = 64;          // key block

template <bool TANGENT, bool INT8>
struct SpCfg {
  static constexpr int NT = TANGENT ? 1 : 4;
  static constexpr int STAGES = (!TANGENT && INT8) ? 3 : 2;   // K/V ring per slot (shared memory bound)
  static constexpr bool NEED_QK = TANGENT || !INT8;     // bf16 q / k tiles are needed
  static constexpr int SOFT_WARPS = 4 * NT;
  static constexpr int WARP_MMA = SOFT_WARPS, WARP_TMA = SOFT_WARPS + 1;
  // NT 4: one more warpgroup (MMA, TMA, two register donors); NT 1: MMA and TMA warps only
  static constexpr int THREADS = NT == 1 ? 192 : (SOFT_WARPS + 4) * 32;
  static constexpr int CTAS_PER_SM = NT == 1 ? 2 : 1;
  static constexpr bool SETMAXNREG = NT > 1;
  // 640 threads are launched with 96 registers each; setmaxnreg.inc draws from that pool only
  static constexpr int REG_SOFT = 104, REG_OTHER = 64;
  static_assert(!SETMAXNREG || SOFT_WARPS * 32 * REG_SOFT + 128 * REG_OTHER <= THREADS * 96, "");
  // TMEM columns of one slot: S (P in place) | dS (T in place) | O | dO
  static constexpr int SC_S = 0;
  static constexpr int SC_DS = 64;
  static constexpr int SC_O = TANGENT ? 128 : 64;
  static constexpr int SC_DO = 192;
  static constexpr int TILE_COLS = TANGENT ? 256 : 128;
  static constexpr int TMEM_COLS = NT * TILE_COLS < 256 ? 256 : NT * TILE_COLS;
  static constexpr int NQ = NEED_QK ? (TANGENT ? 2 : 1) : 0;          // q, dq (bf16)
  static constexpr int NKV = 1 + (NEED_QK ? 1 : 0) + (TANGENT ? 2 : 0);   // v, k, dk, dv
};

template <bool TANGENT, bool INT8>
struct SpSlot {
  using C = SpCfg<TANGENT, INT8>;
  alignas(1024) uint8_t q8[INT8 ? SP_M * 64 : 1024];           // int8, 64-byte rows, SWIZZLE_64B
  alignas(1024) uint8_t q[C::NQ ? C::NQ : 1][C::NQ ? SP_M * 128 : 1024];
  alignas(1024) uint8_t k8[C::STAGES][INT8 ? SP_BK * 64 : 1024];
  alignas(1024) uint8_t kv[C::STAGES][C::NKV][SP_BK * 128];    // v, k, dk, dv (bf16)
  uint64_t q_full, q_empty;
  uint64_t kv_full[C::STAGES], kv_empty[C::STAGES];
  uint64_t s_full, p_full, o_done, o_free;
  uint32_t tmem_base;        // used in slot 0 only (kept here: the slot's padding has room)
  int abort_flag;
};

template <bool TANGENT, bool INT8>
struct SpSmem {
  SpSlot<TANGENT, INT8> slot[SpCfg<TANGENT, INT8>::NT];
};
// 228 KB of shared memory per SM, 1 KB of it reserved per resident CTA, 227 KB per CTA at most
static_assert(sizeof(SpSmem<false, true>) <= 232448 && sizeof(SpSmem<false, false>) <= 232448 &&
                  2 * (sizeof(SpSmem<true, true>) + 1024) <= 233472 &&
                  2 * (sizeof(SpSmem<true, false>) + 1024) <= 233472,
              "shared memory per CTA / per SM exceeded");

struct SpParams {
  const int* lut;            // (B, H, n_mt, tmax) key-block ids, -1 = end of list
  const uint8_t* flags;      // (B, H, n_mt, tmax) bit0: rows 0-63 attend, bit1: rows 64-127
  const int* cnt;            // (B, H, n_mt) entries per list
  const float* q_scale;      // (B, H, n_qblk)  per `qblk` rows
  const float* k_scale;      // (B, H, n_kblk)
  __nv_bfloat16* o;
  __nv_bfloat16* dout;
  float* lse;                // (B, H, L) natural log
  int B, H, L, n_mt, tmax, n_qblk, n_kblk, qblk;   // qblk: rows per query scale block (64 or 128)
  int n_tiles;
  int64_t o_sb, o_sl, o_sh;
  float scale;
  int quant_p;               // quantise P to the 127-level grid
  int* status;
};

// descriptor for 64-byte-swizzled K-major int8 operands ([rows][64 B])
IMF_DEVICE uint64_t sdesc_kmajor_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;   // 8 rows x 64 B
  d |= 1ull << 46;
  d |= 4ull << 61;                               // SWIZZLE_64B
  return d;
}

struct SpTile {
  int mt, h, b, n_j;
  const int* lut;
  const uint8_t* flg;
};
IMF_DEVICE SpTile sp_tile(const SpParams& p, int ti) {
  SpTile t;
  t.mt = ti % p.n_mt;
  t.h = (ti / p.n_mt) % p.H;
  t.b = ti / (p.n_mt * p.H);
  const size_t lrow = (size_t)ti * p.tmax;       // (b, h, mt) is the tile order
  t.lut = p.lut + lrow;
  t.flg = p.flags + lrow;
  t.n_j = p.cnt[ti];
  return t;
}

template <bool TANGENT, bool INT8>
__global__ void __launch_bounds__(SpCfg<TANGENT, INT8>::THREADS, SpCfg<TANGENT, INT8>::CTAS_PER_SM)
attn_sparse_fwd_kernel(const __grid_constant__ CUtensorMap tm_q8,
                       const __grid_constant__ CUtensorMap tm_k8,
                       const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v,
                       const __grid_constant__ CUtensorMap tm_dq,
                       const __grid_constant__ CUtensorMap tm_dk,
                       const __grid_constant__ CUtensorMap tm_dv, const SpParams p) {
  using C = SpCfg<TANGENT, INT8>;
  constexpr int NT = C::NT;
  constexpr bool NEED_QK = C::NEED_QK;
  constexpr int VI = 0, KI = 1, DKI = 2, DVI = 3;          // kv[stage][...]
  // no slack for a manual round-up (the tangent kernel needs every byte for two CTAs per
  // SM): the swizzled TMA tiles need the base on a 1024-byte boundary, checked here
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, STATUS_BAD_ARG);
    return;
  }
  auto& s = *reinterpret_cast<SpSmem<TANGENT, INT8>*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_stride = gridDim.x * NT;

  if (threadIdx.x == 0) {
    for (int t = 0; t < NT; ++t) {
      auto& sl = s.slot[t];
      mbar_init(&sl.q_full, 1);
      mbar_init(&sl.q_empty, 1);
      for (int i = 0; i < C::STAGES; ++i) {
        mbar_init(&sl.kv_full[i], 1);
        mbar_init(&sl.kv_empty[i], 1);
      }
      mbar_init(&sl.s_full, 1);
      mbar_init(&sl.p_full, 4);        // one arrival per softmax warp
      mbar_init(&sl.o_done, 1);
      mbar_init(&sl.o_free, 4);
    }
    s.slot[0].abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == C::WARP_MMA) {
    tmem_alloc(&s.slot[0].tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.slot[0].tmem_base;
  volatile int* abort_flag = &s.slot[0].abort_flag;

  if (warp >= C::SOFT_WARPS) {
    if (C::SETMAXNREG) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::REG_OTHER));
    // The TMA producer and the MMA issuer are one thread each for ALL slots: a loop that
    // probes every slot's barriers without blocking (mbarrier.test_wait) and serves whichever
    // slot is ready, so that no slot's wait holds up another slot's work.
    if (warp == C::WARP_TMA && elect_one()) {
      // ------------------------------------------------------- TMA producer --
      int ti[NT] = {}, n_j[NT] = {}, jj[NT] = {}, kbn[NT] = {}, hq[NT] = {}, bq[NT] = {};
      uint32_t kv_it[NT], qn[NT];
      bool q_sent[NT];
      const int* lutp[NT];
      int n_active = 0;
      auto open_tile = [&](int t) {      // skip tiles with empty lists, read the first entry
        while (ti[t] < p.n_tiles) {
          const SpTile tl = sp_tile(p, ti[t]);
          if (tl.n_j > 0) {
            n_j[t] = tl.n_j; jj[t] = 0; lutp[t] = tl.lut; kbn[t] = tl.lut[0];
            hq[t] = tl.h; bq[t] = tl.b; q_sent[t] = false;
            return;
          }
          ti[t] += tile_stride;
        }
        n_j[t] = 0;
      };
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        // slot t of every CTA takes tile t * grid + cta of each round: a last, partial round
        // then leaves every CTA with fewer busy slots (whose steps run faster) instead of
        // some CTAs with all four busy and the others idle
        ti[t] = t * (int)gridDim.x + blockIdx.x; kv_it[t] = 0; qn[t] = 0;
        open_tile(t);
        n_active += n_j[t] > 0;
      }
      uint32_t spins = 0;
      uint64_t t_start = globaltimer_ns();
      while (n_active > 0) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (n_j[t] == 0) continue;
          auto& sl = s.slot[t];
          if (!q_sent[t]) {
            if (qn[t] > 0 && !mbar_test(&sl.q_empty, (qn[t] - 1) & 1)) continue;
            const int q0 = (ti[t] % p.n_mt) * SP_M;
            mbar_arrive_expect_tx(&sl.q_full, (INT8 ? SP_M * 64 : 0) + C::NQ * SP_M * 128);
            if (INT8) tma_load_4d(sl.q8, &tm_q8, &sl.q_full, 0, hq[t], q0, bq[t]);
            if (NEED_QK) tma_load_4d(sl.q[0], &tm_q, &sl.q_full, 0, hq[t], q0, bq[t]);
            if (TANGENT) tma_load_4d(sl.q[C::NQ - 1], &tm_dq, &sl.q_full, 0, hq[t], q0, bq[t]);
            q_sent[t] = true;
          }
          const int st = kv_it[t] % C::STAGES;
          if (kv_it[t] >= C::STAGES &&
              !mbar_test(&sl.kv_empty[st], ((kv_it[t] / C::STAGES) - 1) & 1))
            continue;
          const int k0 = kbn[t] * SP_BK;
          mbar_arrive_expect_tx(&sl.kv_full[st], (INT8 ? SP_BK * 64 : 0) + C::NKV * SP_BK * 128);
          if (INT8) tma_load_4d(sl.k8[st], &tm_k8, &sl.kv_full[st], 0, hq[t], k0, bq[t]);
          tma_load_4d(sl.kv[st][VI], &tm_v, &sl.kv_full[st], 0, hq[t], k0, bq[t]);
          if (NEED_QK) tma_load_4d(sl.kv[st][KI], &tm_k, &sl.kv_full[st], 0, hq[t], k0, bq[t]);
          if (TANGENT) {
            tma_load_4d(sl.kv[st][DKI], &tm_dk, &sl.kv_full[st], 0, hq[t], k0, bq[t]);
            tma_load_4d(sl.kv[st][DVI], &tm_dv, &sl.kv_full[st], 0, hq[t], k0, bq[t]);
          }
          ++kv_it[t];
          spins = 0;
          if (++jj[t] < n_j[t]) {
            kbn[t] = lutp[t][jj[t]];           // in flight until this slot's next turn
          } else {
            ++qn[t];
            ti[t] += tile_stride;
            open_tile(t);
            n_active -= n_j[t] == 0;
          }
        }
        if ((++spins & 1023u) == 0) {
          if (*abort_flag) break;
          if (spins == 1024u) t_start = globaltimer_ns();
          else if (globaltimer_ns() - t_start > IMF_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_EMPTY);
            break;
          }
        }
      }
    } else if (warp == C::WARP_MMA && elect_one()) {
      // --------------------------------------------------------- MMA issuer --
      // s32 accumulate, signed 8-bit operands, both K-major
      constexpr uint32_t id_i8 = make_idesc(SP_M, SP_BK, FMT_S8, FMT_S8, 2, 0, 0);
      constexpr uint32_t id_qk = idesc_bf16(SP_M, SP_BK, 0, 0);
      constexpr uint32_t id_pv = idesc_bf16(SP_M, SP_HD, 0, 1);
      int ti[NT] = {}, n_j[NT] = {}, jj[NT] = {};
      uint32_t kv_it[NT], step[NT], qn[NT];
      bool want_pv[NT];
      int n_active = 0;
      auto open_tile = [&](int t) {
        while (ti[t] < p.n_tiles) {
          const int n = p.cnt[ti[t]];
          if (n > 0) {
            n_j[t] = n; jj[t] = 0; want_pv[t] = false;
            return;
          }
          ti[t] += tile_stride;
        }
        n_j[t] = 0;
      };
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        ti[t] = t * (int)gridDim.x + blockIdx.x; kv_it[t] = 0; step[t] = 0; qn[t] = 0;
        open_tile(t);
        n_active += n_j[t] > 0;
      }
      uint32_t spins = 0;
      uint64_t t_start = globaltimer_ns();
      // score product of slot t's next step, if its operands have landed.  It is tried in
      // the same visit that issued the previous step's PV product as well (the tensor pipe
      // runs the two in order, so P is read before the new scores land on it): a slot then
      // does not wait a whole round over the other slots between the two.
      auto issue_s = [&](int t) -> bool {
        auto& sl = s.slot[t];
        const uint32_t tb = tmem + t * C::TILE_COLS;
        const int st = kv_it[t] % C::STAGES;
        if (jj[t] == 0 && !mbar_test(&sl.q_full, qn[t] & 1)) return false;
        if (!mbar_test(&sl.kv_full[st], (kv_it[t] / C::STAGES) & 1)) return false;
        tc_fence_after();
        // S (s32) = Q8 K8^T : K = 64 int8 = two k-steps of 32 bytes
        if (INT8) {
          const uint32_t q8a = smem_u32(sl.q8), k8a = smem_u32(sl.k8[st]);
#pragma unroll
          for (int ks = 0; ks < 2; ++ks)
            mma_ss_i8(tb + C::SC_S, sdesc_kmajor_sw64(q8a + ks * 32),
                      sdesc_kmajor_sw64(k8a + ks * 32), id_i8, ks != 0);
        } else {
          const uint32_t qa = smem_u32(sl.q[0]), ka = smem_u32(sl.kv[st][KI]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tb + C::SC_S, sdesc_kmajor(qa + ks * 32), sdesc_kmajor(ka + ks * 32), id_qk,
                   ks != 0);
        }
        if (TANGENT) {
          const uint32_t qa = smem_u32(sl.q[0]), dqa = smem_u32(sl.q[C::NQ - 1]);
          const uint32_t ka = smem_u32(sl.kv[st][KI]), dka = smem_u32(sl.kv[st][DKI]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tb + C::SC_DS, sdesc_kmajor(dqa + ks * 32), sdesc_kmajor(ka + ks * 32),
                   id_qk, ks != 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tb + C::SC_DS, sdesc_kmajor(qa + ks * 32), sdesc_kmajor(dka + ks * 32),
                   id_qk, 1);
        }
        tc_commit(&sl.s_full);
        if (jj[t] == n_j[t] - 1) tc_commit(&sl.q_empty);      // last read of this tile's Q
        want_pv[t] = true;
        spins = 0;
        return true;
      };
      while (n_active > 0) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (n_j[t] == 0) continue;
          auto& sl = s.slot[t];
          const uint32_t tb = tmem + t * C::TILE_COLS;
          if (!want_pv[t]) {
            issue_s(t);
          } else {
            const int st = kv_it[t] % C::STAGES;
            if (!mbar_test(&sl.p_full, step[t] & 1)) continue;
            // first PV of a tile overwrites O: the previous tile's epilogue must have read it
            if (jj[t] == 0 && qn[t] > 0 && !mbar_test(&sl.o_free, (qn[t] - 1) & 1)) continue;
            tc_fence_after();
            const uint32_t va = smem_u32(sl.kv[st][VI]);
            const int j0 = jj[t];
#pragma unroll
            for (int ks = 0; ks < SP_BK / 16; ++ks)
              mma_ts(tb + C::SC_O, tb + C::SC_S + ks * 8,
                     sdesc_mnmajor(va + ks * 2048, SP_BK * 128), id_pv, (j0 | ks) != 0);
            if (TANGENT) {
              const uint32_t dva = smem_u32(sl.kv[st][DVI]);
#pragma unroll
              for (int ks = 0; ks < SP_BK / 16; ++ks)
                mma_ts(tb + C::SC_DO, tb + C::SC_DS + ks * 8,
                       sdesc_mnmajor(va + ks * 2048, SP_BK * 128), id_pv, (j0 | ks) != 0);
#pragma unroll
              for (int ks = 0; ks < SP_BK / 16; ++ks)
                mma_ts(tb + C::SC_DO, tb + C::SC_S + ks * 8,
                       sdesc_mnmajor(dva + ks * 2048, SP_BK * 128), id_pv, 1);
            }
            tc_commit(&sl.o_done);
            tc_commit(&sl.kv_empty[st]);
            want_pv[t] = false;
            spins = 0;
            ++kv_it[t];
            ++step[t];
            if (++jj[t] == n_j[t]) {
              ++qn[t];
              ti[t] += tile_stride;
              open_tile(t);
              n_active -= n_j[t] == 0;
            }
            if (n_j[t] != 0) issue_s(t);
          }
        }
        if ((++spins & 1023u) == 0) {
          if (*abort_flag) break;
          if (spins == 1024u) t_start = globaltimer_ns();
          else if (globaltimer_ns() - t_start > IMF_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_MMA);
            break;
          }
        }
      }
    }
  } else {
    // --------------------------------------- softmax / correction / epilogue --
    if (C::SETMAXNREG) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::REG_SOFT));
    const int t = warp >> 2, wl = warp & 3;
    auto& sl = s.slot[t];
    const int row = wl * 32 + lane;
    const int half = wl >> 1;                      // warp-uniform
    const uint32_t tb = tmem_addr(tmem, wl * 32, t * C::TILE_COLS);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    // with the QAT grid, 127 * 2^x = 2^(x + log2 127) and P is stored as the integer grid value
    const float grid_log2 = p.quant_p ? 6.9886846867721655f : 0.f;
    uint32_t step = 0;
    bool ok = true;
    for (int ti = t * (int)gridDim.x + blockIdx.x; ti < p.n_tiles && ok; ti += tile_stride) {
      const SpTile tl = sp_tile(p, ti);
      const int q_row = tl.mt * SP_M + row;
      const bool live = q_row < p.L;
      const int64_t off = (int64_t)tl.b * p.o_sb + (int64_t)q_row * p.o_sl + (int64_t)tl.h * p.o_sh;
      if (tl.n_j == 0) {                           // no key block at all: zero output
        if (live) {
          for (int c = 0; c < SP_HD; c += 8) {
            *reinterpret_cast<uint4*>(p.o + off + c) = make_uint4(0, 0, 0, 0);
            if (TANGENT) *reinterpret_cast<uint4*>(p.dout + off + c) = make_uint4(0, 0, 0, 0);
          }
          if (p.lse) p.lse[((int64_t)tl.b * p.H + tl.h) * p.L + q_row] = -INFINITY;
        }
        continue;
      }
      const int qb_idx = q_row / p.qblk;
      const float sq = INT8 ? p.q_scale[((size_t)tl.b * p.H + tl.h) * p.n_qblk +
                                        (qb_idx < p.n_qblk ? qb_idx : p.n_qblk - 1)]
                            : 1.f;
      const float* ksc = p.k_scale + ((size_t)tl.b * p.H + tl.h) * p.n_kblk;
      float m2 = -INFINITY, l_sum = 0.f, l_sum2 = 0.f, mu_sum = 0.f, mu_sum2 = 0.f;   // m2: log2 units
      // list entries are read two steps ahead and the key scale one step ahead, so that no
      // step waits for a dependent pair of global loads
      int kb1 = tl.lut[0], kb2 = tl.n_j > 1 ? tl.lut[1] : 0;
      uint32_t fl1 = tl.flg[0];
      float ks1 = INT8 ? ksc[kb1] : 1.f;
      for (int j = 0; j < tl.n_j && ok; ++j, ++step) {
        const int kb = kb1;
        const uint32_t fl = fl1;
        const float ks = ks1;
        kb1 = kb2;
        if (j + 1 < tl.n_j) {
          fl1 = tl.flg[j + 1];
          if (INT8) ks1 = ksc[kb1];
        }
        if (j + 2 < tl.n_j) kb2 = tl.lut[j + 2];
        ok = __all_sync(0xffffffffu, mbar_wait(&sl.s_full, step & 1, abort_flag, p.status,
                                               STATUS_TIMEOUT_MMA));
        if (!ok) break;
        tc_fence_after();
        if (!((fl >> half) & 1)) {
          // this half of the tile does not attend the block: P = T = 0
          uint32_t z[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) z[i] = 0u;
          tmem_st16(tb + C::SC_S, z);
          tmem_st16(tb + C::SC_S + 16, z);
          if (TANGENT) {
            tmem_st16(tb + C::SC_DS, z);
            tmem_st16(tb + C::SC_DS + 16, z);
          }
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sl.p_full);
          continue;
        }
        // raw score -> log2 units: one factor for de-quantisation and softmax scale
        const float cf = INT8 ? sq * ks * scale_log2 : scale_log2;
        const int kv_rem = p.L - kb * SP_BK;
        // pass 1: row maximum of the raw scores (integer compare for INT8 scores).  The
        // scores are read from TMEM again in pass 2, 32 columns at a time, so that a row
        // never needs 64 score registers next to the packed results.
        float mx2;
        {
          uint32_t a[32], c[32];
          tmem_ld32(tb + C::SC_S, a);
          tmem_ld32(tb + C::SC_S + 32, c);
          tc_wait_ld();
          if (kv_rem < SP_BK) {
            const uint32_t lowest = INT8 ? 0x80000000u : 0xff800000u;   // INT_MIN / -inf
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i >= kv_rem) a[i] = lowest;
              if (i + 32 >= kv_rem) c[i] = lowest;
            }
          }
          if (INT8) {
            int m0 = (int)a[0], m1 = (int)c[0];
#pragma unroll
            for (int i = 1; i + 1 < 32; i += 2) {
              m0 = __vimax3_s32(m0, (int)a[i], (int)a[i + 1]);
              m1 = __vimax3_s32(m1, (int)c[i], (int)c[i + 1]);
            }
            mx2 = static_cast<float>(__vimax3_s32(m0, m1, max((int)a[31], (int)c[31]))) * cf;
          } else {
            float m0 = __uint_as_float(a[0]), m1 = __uint_as_float(c[0]);
#pragma unroll
            for (int i = 1; i + 1 < 32; i += 2) {
              asm("max.f32 %0, %0, %1, %2;" : "+f"(m0) : "f"(__uint_as_float(a[i])), "f"(__uint_as_float(a[i + 1])));
              asm("max.f32 %0, %0, %1, %2;" : "+f"(m1) : "f"(__uint_as_float(c[i])), "f"(__uint_as_float(c[i + 1])));
            }
            mx2 = fmaxf(fmaxf(m0, m1), fmaxf(__uint_as_float(a[31]), __uint_as_float(c[31]))) * cf;
          }
        }
        if (m2 == -INFINITY) {
          m2 = mx2;                                // first attended block: O and l are still zero
        } else {
          // with the QAT grid the running max is tracked exactly (P <= 1), otherwise lazily
          const bool need = p.quant_p ? (mx2 > m2) : (mx2 - m2 > 8.0f);
          if (__any_sync(0xffffffffu, need)) {
            float alpha = 1.f;
            if (need) {
              alpha = ex2(m2 - mx2);
              m2 = mx2;
            }
            l_sum *= alpha; l_sum2 *= alpha; mu_sum *= alpha; mu_sum2 *= alpha;
            ok = __all_sync(0xffffffffu, mbar_wait(&sl.o_done, (step - 1) & 1, abort_flag, p.status,
                                                   STATUS_TIMEOUT_MMA));
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < (TANGENT ? 128 : 64); c += 32) {
              uint32_t ov[32];
              tmem_ld32(tb + C::SC_O + c, ov);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              tmem_st32(tb + C::SC_O + c, ov);
            }
            tc_wait_st();
          }
        }
        const float magic = 12582912.f;            // 1.5 * 2^23: (x + magic) - magic rounds to nearest
        // INT8 scores become floats without a conversion instruction (which would share the
        // exponential's pipe): the bit pattern of magic plus the integer IS the float
        // magic + x (|x| <= 64 * 127^2 < 2^22), and the FMA takes magic * cf back out
        const float neg_m = INT8 ? (grid_log2 - m2) - magic * cf : grid_log2 - m2;
        // pass 2: P (and T) for 32 columns at a time; the packed bf16 results go over the
        // first columns of S (dS), which have been read by then.  Only the last key block of
        // the sequence can be ragged: every other block runs the loop without the per-column
        // bound test (two instructions per score).
        auto pass2 = [&](auto ragged_tag) {
          constexpr bool RAGGED = decltype(ragged_tag)::value;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t sv[32];
            uint32_t dsv[TANGENT ? 32 : 1];
            tmem_ld32(tb + C::SC_S + hh * 32, sv);
            if (TANGENT) tmem_ld32(tb + C::SC_DS + hh * 32, dsv);
            tc_wait_ld();
            uint32_t pk[16];
            uint32_t tk[TANGENT ? 16 : 1];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float x0 = __uint_as_float(INT8 ? sv[i] + 0x4B400000u : sv[i]);
              const float x1 = __uint_as_float(INT8 ? sv[i + 1] + 0x4B400000u : sv[i + 1]);
              float p0 = ex2(fmaf(x0, cf, neg_m));
              float p1 = ex2(fmaf(x1, cf, neg_m));
              if (RAGGED) {
                if (hh * 32 + i >= kv_rem) p0 = 0.f;
                if (hh * 32 + i + 1 >= kv_rem) p1 = 0.f;
              }
              if (p.quant_p) {
                p0 = (p0 + magic) - magic;
                p1 = (p1 + magic) - magic;
              }
              l_sum += p0;
              l_sum2 += p1;
              pk[i / 2] = pack_bf16(p0, p1);
              if (TANGENT) {
                const float t0 = p0 * __uint_as_float(dsv[i]) * p.scale;
                const float t1 = p1 * __uint_as_float(dsv[i + 1]) * p.scale;
                mu_sum += t0;
                mu_sum2 += t1;
                tk[i / 2] = pack_bf16(t0, t1);
              }
            }
            tmem_st16(tb + C::SC_S + hh * 16, pk);
            if (TANGENT) tmem_st16(tb + C::SC_DS + hh * 16, tk);
          }
        };
        if (kv_rem >= SP_BK) pass2(std::false_type{});
        else pass2(std::true_type{});
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sl.p_full);
      }
      if (ok)
        ok = mbar_wait(&sl.o_done, (step - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float l_tot = l_sum + l_sum2, mu_tot = mu_sum + mu_sum2;
      const float inv_l = l_tot > 0.f ? 1.f / l_tot : 0.f;
#pragma unroll
      for (int c = 0; c < SP_HD; c += 32) {
        uint32_t ov[32];
        tmem_ld32(tb + C::SC_O + c, ov);
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
          tmem_ld32(tb + C::SC_DO + c, dv_);
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
      if (live && p.lse)        // natural log; the grid factor 127 of l is taken out again
        p.lse[((int64_t)tl.b * p.H + tl.h) * p.L + q_row] =
            m2 * 0.6931471805599453f + __logf(l_tot) - grid_log2 * 0.6931471805599453f;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sl.o_free);
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

// Per-block symmetric INT8 quantiser: one warp per (b, h, block); writes the
// int8 values, the fp32 scale (amax / 127 + 1e-12, round half away from zero)
// and optionally the de-quantised bf16 copy ("fake quant") in one pass.
__global__ void quantize_blocks_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ xq,
                                       float* __restrict__ xs, __nv_bfloat16* __restrict__ xfq,
                                       int B, int L, int H, int block, int n_blk, int64_t sb,
                                       int64_t sl, int64_t sh) {
  const int lane = threadIdx.x & 31;
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long total = (long)B * H * n_blk;
  if (wid >= total) return;
  const int blk = (int)(wid % n_blk), h = (int)((wid / n_blk) % H), b = (int)(wid / ((long)n_blk * H));
  const int r0 = blk * block, r1 = min(L, r0 + block);
  const __nv_bfloat16* base = x + b * sb + h * sh;
  float amax = 0.f;
  for (int r = r0; r < r1; ++r) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(base + (int64_t)r * sl + lane * 2);
    amax = fmaxf(amax, fmaxf(fabsf(__low2float(v)), fabsf(__high2float(v))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = amax / 127.f + 1e-12f;
  if (lane == 0) xs[wid] = sc;
  for (int r = r0; r < r1; ++r) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(base + (int64_t)r * sl + lane * 2);
    float a = __fdiv_rn(__low2float(v), sc), c = __fdiv_rn(__high2float(v), sc);
    a = copysignf(floorf(fabsf(a) + 0.5f), a);
    c = copysignf(floorf(fabsf(c) + 0.5f), c);
    a = fminf(fmaxf(a, -127.f), 127.f);
    c = fminf(fmaxf(c, -127.f), 127.f);
    const size_t o = (((size_t)b * L + r) * H + h) * 64 + lane * 2;
    if (xq) {
      char2 q2;
      q2.x = (signed char)a;
      q2.y = (signed char)c;
      *reinterpret_cast<char2*>(xq + o) = q2;
    }
    if (xfq) *reinterpret_cast<__nv_bfloat162*>(xfq + o) = __floats2bfloat162_rn(a * sc, c * sc);
  }
}

// Same result with the block held in registers: four warps per (b, h, block), a lane owns
// 8 columns (16 bytes) of NR rows, so every row is read once with NR independent loads in
// flight and written with 8-byte (int8) / 16-byte (bf16) stores.  block = 16 * NR rows.
template <int NR>
__device__ __forceinline__ void quantize_block_vec(const __nv_bfloat16* __restrict__ x,
                                                   int8_t* __restrict__ xq, float* __restrict__ xs,
                                                   __nv_bfloat16* __restrict__ xfq, int L, int H,
                                                   int n_blk, int64_t sb, int64_t sl, int64_t sh,
                                                   int b) {
  __shared__ float s_max[4];
  const int blk = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rsub = lane >> 3, c8 = (lane & 7) * 8;
  const int r0 = blk * (16 * NR) + warp * (4 * NR);
  const __nv_bfloat16* base = x + b * sb + h * sh + c8;
  uint4 v[NR];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int row = r0 + i * 4 + rsub;
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row < L) v[i] = *reinterpret_cast<const uint4*>(base + (int64_t)row * sl);
  }
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      amax = fmaxf(amax, fmaxf(fabsf(__low2float(h2[j])), fabsf(__high2float(h2[j]))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) s_max[warp] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3]));
  const float sc = amax / 127.f + 1e-12f;
  if (threadIdx.x == 0) xs[((size_t)b * H + h) * n_blk + blk] = sc;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int row = r0 + i * 4 + rsub;
    if (row >= L) continue;
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a = __fdiv_rn(__low2float(h2[j]), sc), c = __fdiv_rn(__high2float(h2[j]), sc);
      a = copysignf(floorf(fabsf(a) + 0.5f), a);
      c = copysignf(floorf(fabsf(c) + 0.5f), c);
      f[2 * j] = fminf(fmaxf(a, -127.f), 127.f);
      f[2 * j + 1] = fminf(fmaxf(c, -127.f), 127.f);
    }
    const size_t o = (((size_t)b * L + row) * H + h) * 64 + c8;
    if (xq) {
      uint2 q;
      q.x = ((unsigned)(int)f[0] & 0xffu) | (((unsigned)(int)f[1] & 0xffu) << 8) |
            (((unsigned)(int)f[2] & 0xffu) << 16) | (((unsigned)(int)f[3] & 0xffu) << 24);
      q.y = ((unsigned)(int)f[4] & 0xffu) | (((unsigned)(int)f[5] & 0xffu) << 8) |
            (((unsigned)(int)f[6] & 0xffu) << 16) | (((unsigned)(int)f[7] & 0xffu) << 24);
      *reinterpret_cast<uint2*>(xq + o) = q;
    }
    if (xfq) {
      uint4 w;
      __nv_bfloat162* w2 = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) w2[j] = __floats2bfloat162_rn(f[2 * j] * sc, f[2 * j + 1] * sc);
      *reinterpret_cast<uint4*>(xfq + o) = w;
    }
  }
}

template <int NR>
__global__ void __launch_bounds__(128)
quantize_blocks_vec_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ xq,
                           float* __restrict__ xs, __nv_bfloat16* __restrict__ xfq, int L, int H,
                           int n_blk, int64_t sb, int64_t sl, int64_t sh) {
  quantize_block_vec<NR>(x, xq, xs, xfq, L, H, n_blk, sb, sl, sh, blockIdx.z);
}

// Up to three tensors of one shape (q, k, v of an attention call) in one launch:
// blockIdx.z = tensor * B + batch.
struct QuantMany {
  const __nv_bfloat16* x[3];
  int8_t* xq[3];
  float* xs[3];
  __nv_bfloat16* xfq[3];
  int64_t sb[3], sl[3], sh[3];
};
template <int NR>
__global__ void __launch_bounds__(128)
quantize_blocks_many_kernel(const __grid_constant__ QuantMany a, int B, int L, int H, int n_blk) {
  const int t = blockIdx.z / B, b = blockIdx.z % B;
  quantize_block_vec<NR>(a.x[t], a.xq[t], a.xs[t], a.xfq[t], L, H, n_blk, a.sb[t], a.sl[t],
                         a.sh[t], b);
}

static int map_rows(CUtensorMap* m, const void* ptr, int B, int L, int H, int64_t sb, int64_t sl,
                    int64_t sh, int rows, bool int8) {
  uint64_t dims[4] = {64, (uint64_t)H, (uint64_t)L, (uint64_t)B};
  const uint64_t es = int8 ? 1 : 2;
  uint64_t str[4] = {es, (uint64_t)sh * es, (uint64_t)sl * es, (uint64_t)sb * es};
  uint32_t box[4] = {64, 1, (uint32_t)rows, 1};
  return make_tmap(m, int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   const_cast<void*>(ptr), dims, str, box,
                   int8 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace imf

using namespace imf;

// x: (B, L, H, 64) bf16 with strides (sb, sl, sh); outputs contiguous (B, L, H, 64).
extern "C" int imf_quantize_blocks(const void* x, void* xq, float* xs, void* xfq, int B, int L,
                                   int H, int block, int64_t sb, int64_t sl, int64_t sh,
                                   void* stream) {
  if (B <= 0 || L <= 0 || H <= 0 || block <= 0) return IMF_ERR_ARG;
  const int n_blk = (L + block - 1) / block;
  const bool vec = (block == 64 || block == 128) && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                   !((sb | sl | sh) & 7);
  if (vec) {
    const dim3 grid(n_blk, H, B);
    if (block == 64)
      quantize_blocks_vec_kernel<4><<<grid, 128, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)x, (int8_t*)xq, xs, (__nv_bfloat16*)xfq, L, H, n_blk, sb, sl, sh);
    else
      quantize_blocks_vec_kernel<8><<<grid, 128, 0, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)x, (int8_t*)xq, xs, (__nv_bfloat16*)xfq, L, H, n_blk, sb, sl, sh);
    return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
  }
  const long warps = (long)B * H * n_blk;
  const long blocks = (warps * 32 + 255) / 256;
  quantize_blocks_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (int8_t*)xq, xs, (__nv_bfloat16*)xfq, B, L, H, block, n_blk, sb, sl, sh);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}

// The same for n <= 3 tensors of one shape with 64-row blocks in ONE launch.  ptrs: n records of
// (x, xq | null, xs, xfq | null); strides: n records of (sb, sl, sh).  Needs 16-byte aligned
// rows (returns IMF_ERR_ARG otherwise: the caller then quantises the tensors one by one).
extern "C" int imf_quantize_blocks_many(void** ptrs, const int64_t* strides, int n, int B, int L,
                                        int H, void* stream) {
  if (n <= 0 || n > 3 || B <= 0 || L <= 0 || H <= 0) return IMF_ERR_ARG;
  QuantMany a;
  for (int t = 0; t < 3; ++t) {
    const int u = t < n ? t : 0;
    a.x[t] = static_cast<const __nv_bfloat16*>(ptrs[4 * u]);
    a.xq[t] = static_cast<int8_t*>(ptrs[4 * u + 1]);
    a.xs[t] = static_cast<float*>(ptrs[4 * u + 2]);
    a.xfq[t] = static_cast<__nv_bfloat16*>(ptrs[4 * u + 3]);
    a.sb[t] = strides[3 * u]; a.sl[t] = strides[3 * u + 1]; a.sh[t] = strides[3 * u + 2];
    if (!a.x[t] || !a.xs[t] || (reinterpret_cast<uintptr_t>(a.x[t]) & 15) ||
        ((a.sb[t] | a.sl[t] | a.sh[t]) & 7))
      return IMF_ERR_ARG;
  }
  const int n_blk = (L + 63) / 64;
  const dim3 grid(n_blk, H, n * B);
  quantize_blocks_many_kernel<4><<<grid, 128, 0, (cudaStream_t)stream>>>(a, B, L, H, n_blk);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}

// q8/k8: contiguous (B, L, H, 64) int8; q/k/v/dq/dk/dv bf16 with `strides`
// (18 element strides, (batch, row, head) each, in the order q, k, v, dq, dk, dv;
// q, k, dq, dk, dv may be null for the primal-only call).
extern "C" int imf_attn_sparse_fwd(const void* q8, const void* k8, const float* q_scale,
                                   const float* k_scale, const void* q, const void* k,
                                   const void* v, const void* dq, const void* dk, const void* dv,
                                   const int* lut, const uint8_t* flags, const int* cnt, void* o,
                                   void* dout,
                                   float* lse, int B, int L, int H, int tmax, int qblk,
                                   const int64_t* strides, int64_t o_sb, int64_t o_sl, int64_t o_sh,
                                   float scale, int quant_p, int int8_qk, int* status, void* stream) {
  if (B <= 0 || L <= 0 || H <= 0 || tmax <= 0 || (qblk != 64 && qblk != 128) || cnt == nullptr)
    return IMF_ERR_ARG;
  const bool tang = dq != nullptr;
  CUtensorMap mq8, mk8, mq, mk, mv, mdq, mdk, mdv;
  int rc;
  const int64_t c8b = (int64_t)L * H * 64, c8l = (int64_t)H * 64, c8h = 64;
  if ((rc = map_rows(&mv, v, B, L, H, strides[6], strides[7], strides[8], SP_BK, false))) return rc;
  mq8 = mk8 = mq = mk = mdq = mdk = mdv = mv;
  if (int8_qk) {
    if ((rc = map_rows(&mq8, q8, B, L, H, c8b, c8l, c8h, SP_M, true))) return rc;
    if ((rc = map_rows(&mk8, k8, B, L, H, c8b, c8l, c8h, SP_BK, true))) return rc;
  }
  if (tang || !int8_qk) {
    if ((rc = map_rows(&mq, q, B, L, H, strides[0], strides[1], strides[2], SP_M, false))) return rc;
    if ((rc = map_rows(&mk, k, B, L, H, strides[3], strides[4], strides[5], SP_BK, false))) return rc;
  }
  if (tang) {
    if ((rc = map_rows(&mdq, dq, B, L, H, strides[9], strides[10], strides[11], SP_M, false))) return rc;
    if ((rc = map_rows(&mdk, dk, B, L, H, strides[12], strides[13], strides[14], SP_BK, false))) return rc;
    if ((rc = map_rows(&mdv, dv, B, L, H, strides[15], strides[16], strides[17], SP_BK, false))) return rc;
  }
  SpParams p;
  p.lut = lut; p.flags = flags; p.cnt = cnt; p.q_scale = q_scale; p.k_scale = k_scale;
  p.o = (__nv_bfloat16*)o; p.dout = (__nv_bfloat16*)dout; p.lse = lse;
  p.B = B; p.H = H; p.L = L; p.n_mt = (L + SP_M - 1) / SP_M; p.tmax = tmax;
  p.qblk = qblk; p.n_qblk = (L + qblk - 1) / qblk; p.n_kblk = (L + SP_BK - 1) / SP_BK;
  p.o_sb = o_sb; p.o_sl = o_sl; p.o_sh = o_sh; p.scale = scale; p.quant_p = quant_p;
  p.status = status;
  p.n_tiles = p.n_mt * H * B;
  cudaStream_t st = (cudaStream_t)stream;
  // SM count of the CURRENT device, cached per device index (a host may hold GPUs of
  // different sizes; every thread that fills a slot writes the same value)
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
#define IMF_SP_LAUNCH(T_, I_)                                                                   \
  do {                                                                                          \
    using C_ = SpCfg<T_, I_>;                                                                   \
    const size_t smem = sizeof(SpSmem<T_, I_>);                                                 \
    int grid = (p.n_tiles + C_::NT - 1) / C_::NT;                                               \
    if (grid > sms * C_::CTAS_PER_SM) grid = sms * C_::CTAS_PER_SM;                             \
    if (cudaFuncSetAttribute(attn_sparse_fwd_kernel<T_, I_>,                                    \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return IMF_ERR_LAUNCH;                                                                    \
    attn_sparse_fwd_kernel<T_, I_><<<grid, C_::THREADS, smem, st>>>(mq8, mk8, mq, mk, mv, mdq,  \
                                                                    mdk, mdv, p);               \
  } while (0)
  if (tang && int8_qk) IMF_SP_LAUNCH(true, true);
  else if (tang) IMF_SP_LAUNCH(true, false);
  else if (int8_qk) IMF_SP_LAUNCH(false, true);
  else IMF_SP_LAUNCH(false, false);
#undef IMF_SP_LAUNCH
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}
