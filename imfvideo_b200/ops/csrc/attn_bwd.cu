// Dense flash attention backward (reverse mode) on tcgen05 / TMEM.
//
// Given Q, K, V, O, dO and the forward's log-sum-exp, computes dQ, dK, dV with
// O(L) memory by recomputing P tile by tile:
//
//   S^T = K Q^T,  P^T = exp2(S^T * scale*log2e - lse2),  dP^T = V dO^T,
//   dS^T = P^T .* (dP^T - delta),   delta = rowsum(dO .* O)
//   dV += P^T dO,   dK += scale * dS^T Q,   dQ += scale * dS K
//
// Replaces FA4 / SDPA backward in the reference (reference
// models/attention_op.py:38-60) and `_attn_bwd_*` of its SLA2 backend for the
// dense case.
//
// CTA = one 128-row K/V tile of one (batch, head); it walks over all 128-row
// Q tiles.  Everything is computed TRANSPOSED (K/V rows on the TMEM lanes), so
// P^T can stay in TMEM as the A operand of the dV GEMM, and dK/dV accumulate
// in TMEM for the whole walk.  dS^T goes through shared memory once and feeds
// both the dK GEMM (K-major view) and the dQ GEMM (MN-major view).  dQ tiles
// are added to an fp32 accumulator in global memory by TMA (reduce-add),
// converted to bf16 by a small epilogue kernel.  On request the adds to one
// query tile happen in a FIXED order (a turn counter per query tile), so the
// result is bit-identical from run to run: the grid is ordered so that a CTA
// only ever waits for CTAs with a smaller linear block index (dispatched
// before it), consecutive K/V tiles of one head are `chains` blocks apart, and
// every CTA of a chain walks the query tiles in the same direction, so a CTA
// runs about one tile behind its predecessor.  The resident CTAs of a chain
// then move in lockstep at the pace of the slowest of them, which costs 13 %
// of the kernel's time (dense, 29,140 tokens), hence an option.
//
// The per-query constants ride on the tensor core: the query tile carries Q * scale*log2e
// and 16 extra K columns [-lse2_hi, -lse2_lo, 0 ...] (bf16 pair = fp32 to 2^-17), the K tile
// 16 columns of ones, so the S^T accumulator already holds the exponent S*scale*log2e - lse2;
// dO / V likewise carry -delta, so the dP^T accumulator holds dP - delta.  The math warps are
// left with one ex2, one multiply and two packs per pair of elements (they, not the tensor
// pipe, set the pace of this kernel), and read no per-row statistics at all.
//
// Warps 0-3 / 4-7: exp / dS math for columns 0-63 / 64-127 of the S^T tile;
// warps 8-11: dQ tile TMEM -> global reduction; warp 12: tcgen05.mma issuer;
// warp 13: TMA producer.  S^T/dP^T of tile i+1 are issued as soon as tile i
// has been pulled into registers, so the tensor core overlaps the exp math.
#include "attn_bwd128.h"
#include "common.cuh"
#include "host_util.h"

namespace imf {

constexpr int BW_HD = 64;
constexpr int BW_T = 128;            // tile rows (both q and kv)
constexpr int BW_THREADS = 512;
constexpr int BW_QSTAGES = 2;

// TMEM columns
constexpr int BC_S = 0, BC_DP = 128, BC_P = 256, BC_DK = 320, BC_DV = 384, BC_DQ = 448;

struct BwSmem {
  alignas(1024) uint8_t k[BW_T * 128];
  alignas(1024) uint8_t v[BW_T * 128];
  alignas(1024) uint8_t q[BW_QSTAGES][BW_T * 128];
  alignas(1024) uint8_t d_o[BW_QSTAGES][BW_T * 128];
  alignas(1024) uint8_t ds[2][2 * BW_T * 128];       // dS^T: [kv 128][q 128] as two 64-col panels
  alignas(1024) float dq_stage[BW_T * BW_HD];        // dQ tile staged for the TMA reduce-add
  alignas(1024) uint8_t ones[BW_T * 32];             // [128][16] bf16 1.0, 32-byte rows (SWIZZLE_32B)
  alignas(1024) uint8_t augq[BW_QSTAGES][BW_T * 32]; // [q 128][16]: -lse2 as (hi, lo), zeros
  alignas(1024) uint8_t augd[BW_QSTAGES][BW_T * 32]; // [q 128][16]: -delta as (hi, lo), zeros
  uint64_t kv_full;
  uint64_t q_full[BW_QSTAGES], q_empty[BW_QSTAGES];
  uint64_t s_full, s_taken, p_ready, p_free;
  uint64_t ds_free[2];
  uint64_t dq_full, dq_free;
  uint64_t final_bar;
  uint32_t tmem_base;
  int abort_flag;
};

struct BwParams {
  float* dq_acc;          // (B, L, H, 64) fp32, zeroed
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int B, H, L, Lp;
  int64_t dk_sb, dk_sl, dk_sh, dv_sb, dv_sl, dv_sh;
  float scale;
  int* status;
  // block-sparse mode (null = dense): per K/V tile the list of query tiles that attend it
  // (-1 terminated, at most qmax entries) and, per entry, 4 flag bits
  // (kv half * 2 + q half) saying which 64 x 64 quadrants are live
  const int* qlist;
  const uint8_t* qflags;
  int qmax;
  // dense mode: the query tiles of a K/V tile are split over `qsplit` CTAs (blockIdx.z =
  // batch * qsplit + part) to even out the last wave; each writes unscaled fp32 partial
  // dK / dV to part[r] = (B, L, H, 64) and a second kernel adds them up
  int qsplit;
  float* part_dk;
  float* part_dv;
  // fixed-order dQ (null = adds land in arrival order): one counter per (batch, head, query
  // tile), zeroed before the launch.  The CTA whose ordinal equals the counter adds its tile
  // and then raises the counter.  Dense: ordinal = K/V tile index; block-sparse: qrank[entry]
  int* turn;
  const uint16_t* qrank;
};

IMF_DEVICE void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
IMF_DEVICE void red_add_v4(float* gptr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gptr), "f"(a), "f"(b),
               "f"(c), "f"(d)
               : "memory");
}

template <bool SPARSE>      // block-sparse lists given (keeps the dense instance free of their tests)
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_augq,
                const __grid_constant__ CUtensorMap tm_augd, const BwParams p) {
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<BwSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                       ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // block-sparse lists can be very uneven (the always-attended tail tiles are attended by every
  // query tile and sit at the end): walk the K/V tiles from the back so the long ones start first
  // grid = (chains, K/V tiles): blockIdx.x = head + H * (batch * qsplit + part) varies fastest,
  // so the resident CTAs are a few K/V tiles of EVERY chain rather than many of one
  const int kvb = p.qlist ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
  const int h = blockIdx.x % p.H, bz = blockIdx.x / p.H;
  const int b = bz / p.qsplit, qpart = bz % p.qsplit;
  const size_t lrow = (((size_t)b * p.H + h) * gridDim.y + kvb) * (size_t)p.qmax;
  const int* qlist = p.qlist ? p.qlist + lrow : nullptr;
  const uint8_t* qflags = p.qflags ? p.qflags + lrow : nullptr;
  const uint16_t* qrank = (p.qlist && p.qrank) ? p.qrank + lrow : nullptr;
  int n_q = (p.L + BW_T - 1) / BW_T;       // query tiles this CTA walks over
  int* turn = p.turn ? p.turn + ((size_t)b * p.H + h) * n_q : nullptr;
  int q_first = 0;                          // dense: they are q_first .. q_first + n_q - 1
  if (qlist) {
    n_q = 0;
    while (n_q < p.qmax && qlist[n_q] >= 0) ++n_q;
  } else {
    q_first = (int)((long)qpart * n_q / p.qsplit);
    n_q = (int)((long)(qpart + 1) * n_q / p.qsplit) - q_first;
  }

  if (threadIdx.x == 0) {
    mbar_init(&s.kv_full, 1);
    for (int i = 0; i < BW_QSTAGES; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.q_empty[i], 1);
    }
    mbar_init(&s.s_full, 1);
    mbar_init(&s.s_taken, 8);      // one arrival per exp warp
    mbar_init(&s.p_ready, 8);
    mbar_init(&s.p_free, 1);
    mbar_init(&s.ds_free[0], 1);
    mbar_init(&s.ds_free[1], 1);
    mbar_init(&s.dq_full, 1);
    mbar_init(&s.dq_free, 4);
    mbar_init(&s.final_bar, 1);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  {
    uint32_t* o32 = reinterpret_cast<uint32_t*>(s.ones);       // every element 1.0: the swizzle
    for (int i = threadIdx.x; i < BW_T * 32 / 4; i += BW_THREADS) o32[i] = 0x3f803f80u;   // is moot
    fence_proxy_async_smem();
  }
  if (warp == 12) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;

  if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 13) {
      // ---------------------------------------------------- TMA producer --
      if (elect_one()) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
        prefetch_tmap(&tm_do);
        mbar_arrive_expect_tx(&s.kv_full, 2 * BW_T * 128);
        tma_load_4d(s.k, &tm_k, &s.kv_full, 0, h, kvb * BW_T, b);
        tma_load_4d(s.v, &tm_v, &s.kv_full, 0, h, kvb * BW_T, b);
        const int bh = b * p.H + h;
        for (int i = 0; i < n_q; ++i) {
          const int st = i % BW_QSTAGES;
          if (i >= BW_QSTAGES &&
              !mbar_wait(&s.q_empty[st], (uint32_t)(((i / BW_QSTAGES) - 1) & 1), abort_flag,
                         p.status, STATUS_TIMEOUT_EMPTY))
            break;
          const int qt = qlist ? qlist[i] : q_first + i;
          mbar_arrive_expect_tx(&s.q_full[st], 2 * BW_T * 128 + 2 * BW_T * 32);
          tma_load_4d(s.q[st], &tm_q, &s.q_full[st], 0, h, qt * BW_T, b);
          tma_load_4d(s.d_o[st], &tm_do, &s.q_full[st], 0, h, qt * BW_T, b);
          tma_load_3d(s.augq[st], &tm_augq, &s.q_full[st], 0, qt * BW_T, bh);
          tma_load_3d(s.augd[st], &tm_augd, &s.q_full[st], 0, qt * BW_T, bh);
        }
      }
    } else if (warp == 12) {
      // ------------------------------------------------------ MMA issuer --
      if (elect_one()) {
        constexpr uint32_t id_st = idesc_bf16(BW_T, BW_T, 0, 0);     // S^T, dP^T
        constexpr uint32_t id_kn = idesc_bf16(BW_T, BW_HD, 0, 1);    // dV (TS), dK (SS, A K-major)
        constexpr uint32_t id_mn = idesc_bf16(BW_T, BW_HD, 1, 1);    // dQ (A MN-major)
        const uint32_t ka = smem_u32(s.k), va = smem_u32(s.v);
        const uint64_t ones_d = sdesc_kmajor_sw32(smem_u32(s.ones));
        constexpr uint32_t id_st64 = idesc_bf16(BW_T, 64, 0, 0);     // one 64-row query half
        // Block-sparse tiles: `f` has one bit per 64 x 64 quadrant (kv half * 2 + q half).  A
        // query half that attends neither K/V half is left out of the score products (N = 64)
        // and of the K dimension of dV / dK; a K/V half that no query half attends is left out
        // of the K dimension of dQ.  The math warps write zeros for dead quadrants, so the
        // skipped products would only have added zeros.  Dense: f = 15.
        auto issue_s = [&](int st, uint32_t f) {
          const uint32_t qa = smem_u32(s.q[st]), doa = smem_u32(s.d_o[st]);
          const uint32_t qh = ((f & 5u) ? 1u : 0u) | ((f & 10u) ? 2u : 0u);   // live query halves
          if (qh == 3u) {
#pragma unroll
            for (int ks = 0; ks < BW_HD / 16; ++ks)
              mma_ss(tmem + BC_S, sdesc_kmajor(ka + ks * 32), sdesc_kmajor(qa + ks * 32), id_st, ks != 0);
            // + ones[kv] x (-lse2[q])  ->  the accumulator holds the exponent itself
            mma_ss(tmem + BC_S, ones_d, sdesc_kmajor_sw32(smem_u32(s.augq[st])), id_st, 1);
#pragma unroll
            for (int ks = 0; ks < BW_HD / 16; ++ks)
              mma_ss(tmem + BC_DP, sdesc_kmajor(va + ks * 32), sdesc_kmajor(doa + ks * 32), id_st, ks != 0);
            // + ones[kv] x (-delta[q])  ->  dP - delta
            mma_ss(tmem + BC_DP, ones_d, sdesc_kmajor_sw32(smem_u32(s.augd[st])), id_st, 1);
          } else {
            const uint32_t h = qh >> 1;                     // the live half: rows 64 h .. 64 h + 63
            const uint32_t qo = h * (64 * 128), ao = h * (64 * 32), co = h * 64;
#pragma unroll
            for (int ks = 0; ks < BW_HD / 16; ++ks)
              mma_ss(tmem + BC_S + co, sdesc_kmajor(ka + ks * 32), sdesc_kmajor(qa + qo + ks * 32),
                     id_st64, ks != 0);
            mma_ss(tmem + BC_S + co, ones_d, sdesc_kmajor_sw32(smem_u32(s.augq[st]) + ao), id_st64, 1);
#pragma unroll
            for (int ks = 0; ks < BW_HD / 16; ++ks)
              mma_ss(tmem + BC_DP + co, sdesc_kmajor(va + ks * 32), sdesc_kmajor(doa + qo + ks * 32),
                     id_st64, ks != 0);
            mma_ss(tmem + BC_DP + co, ones_d, sdesc_kmajor_sw32(smem_u32(s.augd[st]) + ao), id_st64, 1);
          }
          tc_commit(&s.s_full);
        };
        bool ok = n_q > 0 &&      // a K/V tile that no query tile attends has zero gradients
                  mbar_wait(&s.kv_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA) &&
                  mbar_wait(&s.q_full[0], 0, abort_flag, p.status, STATUS_TIMEOUT_TMA);
        if (ok) {
          tc_fence_after();
          issue_s(0, SPARSE ? qflags[0] : 15u);
        }
        bool kv_started = false;     // dK / dV accumulators hold something
        for (int i = 0; i < n_q && ok; ++i) {
          const int st = i % BW_QSTAGES;
          const uint32_t par = (uint32_t)(i & 1);
          ok = mbar_wait(&s.s_taken, par, abort_flag, p.status, STATUS_TIMEOUT_SOFTMAX);
          if (!ok) break;
          if (i + 1 < n_q) {
            const int st1 = (i + 1) % BW_QSTAGES;
            ok = mbar_wait(&s.q_full[st1], (uint32_t)(((i + 1) / BW_QSTAGES) & 1), abort_flag,
                           p.status, STATUS_TIMEOUT_TMA);
            if (!ok) break;
            tc_fence_after();
            issue_s(st1, SPARSE ? qflags[i + 1] : 15u);
          }
          ok = mbar_wait(&s.p_ready, par, abort_flag, p.status, STATUS_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          const uint32_t qa = smem_u32(s.q[st]), doa = smem_u32(s.d_o[st]);
          const uint32_t dsa = smem_u32(s.ds[i & 1]);
          const uint32_t f = SPARSE ? qflags[i] : 15u;
          // k-steps of 16 query rows that belong to a live query half / of 16 K/V rows that
          // belong to a live K/V half
          const int q0 = (f & 5u) ? 0 : 4, q1 = (f & 10u) ? 8 : 4;
          const int k0 = (f & 3u) ? 0 : 4, k1 = (f & 12u) ? 8 : 4;
          // dV += P^T dO   (A = P^T in TMEM: 128 q as K -> 8 k-steps of 8 columns)
#pragma unroll
          for (int ks = 0; ks < BW_T / 16; ++ks)
            if (ks >= q0 && ks < q1)
              mma_ts(tmem + BC_DV, tmem + BC_P + ks * 8,
                     sdesc_mnmajor(doa + ks * 2048, BW_T * 128), id_kn, kv_started || ks != q0);
          tc_commit(&s.p_free);
          // dK += dS^T Q   (A = dS^T from smem, K-major view: K = q)
#pragma unroll
          for (int ks = 0; ks < BW_T / 16; ++ks)
            if (ks >= q0 && ks < q1)
              mma_ss(tmem + BC_DK, sdesc_kmajor(dsa + (ks / 4) * (BW_T * 128) + (ks % 4) * 32),
                     sdesc_mnmajor(qa + ks * 2048, BW_T * 128), id_kn, kv_started || ks != q0);
          kv_started = true;
          // the query-side stage (Q, dO, bands) has had its last reader: hand it back to the
          // TMA producer now, not after the dQ GEMM -- with two stages, the load of tile i+2
          // starts here and its latency sets the pace of the whole pipeline
          tc_commit(&s.q_empty[st]);
          // dQ_i = dS K    (A = dS^T from smem, MN-major view: M = q, K = kv)
          if (i > 0) {
            ok = mbar_wait(&s.dq_free, (uint32_t)((i - 1) & 1), abort_flag, p.status,
                           STATUS_TIMEOUT_SOFTMAX);
            if (!ok) break;
            tc_fence_after();
          }
#pragma unroll
          for (int ks = 0; ks < BW_T / 16; ++ks)
            if (ks >= k0 && ks < k1)
              mma_ss(tmem + BC_DQ, sdesc_mnmajor(dsa + ks * 2048, BW_T * 128),
                     sdesc_mnmajor(ka + ks * 2048, BW_T * 128), id_mn, ks != k0);
          tc_commit(&s.dq_full);
          tc_commit(&s.ds_free[i & 1]);
        }
        if (ok) tc_commit(&s.final_bar);
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------ dQ tile -> global reduction --
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    const int wl = warp & 3;
    const uint32_t tb = tmem_addr(tmem, wl * 32, BC_DQ);
    bool ok = true;
    bool turn_live = true;          // false once a turn wait gave up (the status word says so)
    int prev_qt = -1, prev_ord = 0;
    for (int i = 0; i < n_q && ok; ++i) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s.dq_full, (uint32_t)(i & 1), abort_flag, p.status,
                                             STATUS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      uint32_t r[64];
      tmem_ld32(tb, r);
      tmem_ld32(tb + 32, r + 32);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.dq_free);
      // stage the tile in shared memory (plain [128][64] fp32) and let TMA add it to
      // the fp32 accumulator in global memory: coalesced, asynchronous, rows >= L clipped
      const int qt = qlist ? qlist[i] : q_first + i;
      if (i > 0) {
        if (threadIdx.x == 8 * 32) {
          if (turn && turn_live) {
            // the previous add has been performed (it had the time of this tile's TMEM read):
            // pass its query tile on.  Measured faster than passing it one tile later.
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            turn_pass(turn + prev_qt, prev_ord + 1);
          } else {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      // two 128-byte-swizzled panels [128 rows][32 floats] (columns 0-31 / 32-63)
      const int srow = wl * 32 + lane;
      uint8_t* stage = reinterpret_cast<uint8_t*>(s.dq_stage);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint8_t* dst = stage + (c / 8) * (BW_T * 128) + srow * 128 + (((c & 7) ^ (srow & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 8 * 32) {
        const int ord = qrank ? (int)qrank[i] : kvb;
        if (turn && turn_live) turn_live = turn_wait(turn + qt, ord, abort_flag, p.status);
        if (!turn || turn_live) {
#pragma unroll
          for (int pnl = 0; pnl < 2; ++pnl)
            asm volatile(
                "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group"
                " [%0, {%2, %3, %4, %5}], [%1];"
                ::"l"(reinterpret_cast<uint64_t>(&tm_dq)),
                "r"(smem_u32(stage + pnl * (BW_T * 128))), "r"(pnl * 32), "r"(h), "r"(qt * BW_T),
                "r"(b)
                : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        prev_qt = qt;
        prev_ord = ord;
      }
    }
    if (threadIdx.x == 8 * 32) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (turn && turn_live && n_q > 0 && prev_qt >= 0) turn_pass(turn + prev_qt, prev_ord + 1);
    }
  } else {
    // ---------------------------------------------------- exp / dS math ----
    asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
    const int wg = warp >> 2;           // column half: q columns [64 wg, 64 wg + 64)
    const int wl = warp & 3;
    const int row = wl * 32 + lane;     // kv row of this thread (TMEM lane)
    const uint32_t tb = tmem_addr(tmem, wl * 32, 0);
    bool ok = true;
    for (int i = 0; i < n_q && ok; ++i) {
      const uint32_t par = (uint32_t)(i & 1);
      ok = __all_sync(0xffffffffu,
                      mbar_wait(&s.s_full, par, abort_flag, p.status, STATUS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[64], dp[64];
      tmem_ld32(tb + BC_S + wg * 64, sv);
      tmem_ld32(tb + BC_S + wg * 64 + 32, sv + 32);
      tmem_ld32(tb + BC_DP + wg * 64, dp);
      tmem_ld32(tb + BC_DP + wg * 64 + 32, dp + 32);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.s_taken);
      // P^T goes to TMEM (A operand of the dV GEMM): dV of tile i-1 must have read it;
      // dS^T goes to smem buffer i&1: the GEMMs of tile i-2 must have read it
      if (i > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&s.p_free, (uint32_t)((i - 1) & 1), abort_flag,
                                               p.status, STATUS_TIMEOUT_MMA));
        if (!ok) break;
      }
      if (i >= 2) {
        ok = __all_sync(0xffffffffu,
                        mbar_wait(&s.ds_free[i & 1], (uint32_t)(((i / 2) - 1) & 1), abort_flag,
                                  p.status, STATUS_TIMEOUT_MMA));
        if (!ok) break;
      }
      uint8_t* dsb = s.ds[i & 1] + wg * (BW_T * 128) + row * 128;
      // block-sparse: this thread's 64 columns are one (kv half, q half) quadrant
      const bool live = !qflags || ((qflags[i] >> ((row >> 6) * 2 + wg)) & 1);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t pk[16], dk_[16];
        if (live) {        // warp-uniform: a warp's 32 rows and 64 columns lie in one quadrant
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const int cg = hh * 32 + c;
            // sv = S scale log2e - lse2 and dp = dP - delta, straight from the tensor core
            const float p0 = ex2(__uint_as_float(sv[cg]));
            const float p1 = ex2(__uint_as_float(sv[cg + 1]));
            pk[c / 2] = pack_bf16(p0, p1);
            dk_[c / 2] = pack_bf16(p0 * __uint_as_float(dp[cg]), p1 * __uint_as_float(dp[cg + 1]));
          }
        } else {           // block-sparse: this quadrant is not attended
#pragma unroll
          for (int c = 0; c < 16; ++c) pk[c] = dk_[c] = 0u;
        }
        tmem_st16(tb + BC_P + wg * 32 + hh * 16, pk);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int chunk = hh * 4 + cc;
          uint4 val = make_uint4(dk_[4 * cc], dk_[4 * cc + 1], dk_[4 * cc + 2], dk_[4 * cc + 3]);
          *reinterpret_cast<uint4*>(dsb + ((chunk ^ (row & 7)) << 4)) = val;
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.p_ready);
    }
    // ---- epilogue: WG0 stores dK (scaled), WG1 stores dV ----
    if (ok && n_q > 0) ok = mbar_wait(&s.final_bar, 0, abort_flag, p.status, STATUS_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int kv_row = kvb * BW_T + row;
      // Q in shared memory is Q * scale * log2(e): dK = scale dS^T Q = ln(2) dS^T Q_scaled
      const float mul = n_q == 0 ? 0.f : (wg == 0 ? 0.6931471805599453f : 1.f);
      __nv_bfloat16* base =
          wg == 0 ? p.dk + (int64_t)b * p.dk_sb + (int64_t)kv_row * p.dk_sl + (int64_t)h * p.dk_sh
                  : p.dv + (int64_t)b * p.dv_sb + (int64_t)kv_row * p.dv_sl + (int64_t)h * p.dv_sh;
      float* pbase = nullptr;
      if (p.qsplit > 1)
        pbase = (wg == 0 ? p.part_dk : p.part_dv) +
                ((((size_t)qpart * p.B + b) * p.L + kv_row) * p.H + h) * BW_HD;
#pragma unroll
      for (int c = 0; c < BW_HD; c += 32) {
        uint32_t r[32];
        tmem_ld32(tb + (wg == 0 ? BC_DK : BC_DV) + c, r);
        tc_wait_ld();
        if (kv_row < p.L) {
          if (pbase) {                       // unscaled fp32 partial of this query range
            float4* dst = reinterpret_cast<float4*>(pbase + c);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              dst[e] = n_q == 0 ? make_float4(0.f, 0.f, 0.f, 0.f)
                                : make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                              __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
          } else {
            uint32_t ob[16];
#pragma unroll
            for (int e = 0; e < 16; ++e)
              ob[e] = n_q == 0 ? 0u
                               : pack_bf16(__uint_as_float(r[2 * e]) * mul,
                                           __uint_as_float(r[2 * e + 1]) * mul);
            uint4* dst = reinterpret_cast<uint4*>(base + c);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              dst[e] = make_uint4(ob[4 * e], ob[4 * e + 1], ob[4 * e + 2], ob[4 * e + 3]);
          }
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 12) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// Per (b, l, h) row, one warp:  delta = rowsum(dO .* O) and lse2 = lse * log2(e) as the bf16
// (hi, lo) pairs the main kernel feeds to the tensor core (16 columns per row, the rest zero;
// rows l >= L of the padded length Lp get lse2 = 30000, i.e. P = 0), and Q * scale*log2e as bf16.
// Wide form of the kernel below: a lane owns 8 consecutive channels (one 16-byte access per
// tensor), a row is 8 lanes, a warp takes 4 rows -- the H index fastest, so that a warp reads
// neighbouring heads of one token.  Needs 16-byte aligned rows in q, o and dO.
__global__ void attn_bwd_prep_wide_kernel(const __nv_bfloat16* __restrict__ q,
                                          const __nv_bfloat16* __restrict__ o,
                                          const __nv_bfloat16* __restrict__ d_o,
                                          const float* __restrict__ lse,
                                          __nv_bfloat16* __restrict__ qs, uint32_t* __restrict__ augq,
                                          uint32_t* __restrict__ augd, int B, int L, int H, int Lp,
                                          int64_t q_sb, int64_t q_sl, int64_t q_sh, int64_t o_sb,
                                          int64_t o_sl, int64_t o_sh, int64_t g_sb, int64_t g_sl,
                                          int64_t g_sh, float scale_log2) {
  const int lane = threadIdx.x & 31, sub = lane >> 3, part = lane & 7, c0 = part * 8;
  const long grp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long total = (long)B * H * Lp;
  const long u = grp * 4 + sub;
  const bool in = u < total;             // no early exit: the shuffles below need every lane
  int h = 0, l = 0, b = 0;
  if (in) {
    h = (int)(u % H);
    l = (int)((u / H) % Lp);
    b = (int)(u / ((long)H * Lp));
  }
  const bool live = in && l < L;
  float v = 0.f;
  if (live) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * o_sb + (int64_t)l * o_sl + h * o_sh + c0);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + b * g_sb + (int64_t)l * g_sl + h * g_sh + c0);
    const uint4 qq = *reinterpret_cast<const uint4*>(q + b * q_sb + (int64_t)l * q_sl + h * q_sh + c0);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
    const uint32_t qw[4] = {qq.x, qq.y, qq.z, qq.w};
    uint32_t ow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v += bf16_lo(aw[i]) * bf16_lo(gw[i]) + bf16_hi(aw[i]) * bf16_hi(gw[i]);
      ow[i] = pack_bf16(bf16_lo(qw[i]) * scale_log2, bf16_hi(qw[i]) * scale_log2);
    }
    *reinterpret_cast<uint4*>(qs + (((int64_t)b * L + l) * H + h) * 64 + c0) =
        make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if (!in) return;
  float x = 30000.f, dl = 0.f;           // padding rows: exp2(S - 30000) = 0
  if (live) {
    dl = v;
    x = lse[((long)b * H + h) * L + l] * 1.4426950408889634f;
    x = fminf(fmaxf(x, -30000.f), 30000.f);
  }
  uint32_t wq = 0u, wd = 0u;             // 16 bf16 = 8 words per row, one per lane of the row
  if (part == 0) {
    const float xh = bf16_lo(pack_bf16(-x, 0.f)), dh = bf16_lo(pack_bf16(-dl, 0.f));
    wq = pack_bf16(xh, -x - xh);
    wd = pack_bf16(dh, -dl - dh);
  }
  const long row = ((long)b * H + h) * Lp + l;
  augq[row * 8 + part] = wq;
  augd[row * 8 + part] = wd;
}

__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ q,
                                     const __nv_bfloat16* __restrict__ o,
                                     const __nv_bfloat16* __restrict__ d_o,
                                     const float* __restrict__ lse, __nv_bfloat16* __restrict__ qs,
                                     uint32_t* __restrict__ augq, uint32_t* __restrict__ augd, int B,
                                     int L, int H, int Lp, int64_t q_sb, int64_t q_sl, int64_t q_sh,
                                     int64_t o_sb, int64_t o_sl, int64_t o_sh, int64_t g_sb,
                                     int64_t g_sl, int64_t g_sh, float scale_log2) {
  const int lane = threadIdx.x & 31;
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long total = (long)B * H * Lp;
  if (wid >= total) return;
  const int l = (int)(wid % Lp), h = (int)((wid / Lp) % H), b = (int)(wid / ((long)Lp * H));
  float x = 30000.f, dl = 0.f;          // padding rows: exp2(S - 30000) = 0
  if (l < L) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(
        o + b * o_sb + (int64_t)l * o_sl + h * o_sh + lane * 2);
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(
        d_o + b * g_sb + (int64_t)l * g_sl + h * g_sh + lane * 2);
    float v = __low2float(a) * __low2float(g) + __high2float(a) * __high2float(g);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    dl = v;
    x = lse[((long)b * H + h) * L + l] * 1.4426950408889634f;
    x = fminf(fmaxf(x, -30000.f), 30000.f);
    const __nv_bfloat162 qq = *reinterpret_cast<const __nv_bfloat162*>(
        q + b * q_sb + (int64_t)l * q_sl + h * q_sh + lane * 2);
    *reinterpret_cast<uint32_t*>(qs + (((int64_t)b * L + l) * H + h) * 64 + lane * 2) =
        pack_bf16(__low2float(qq) * scale_log2, __high2float(qq) * scale_log2);
  }
  if (lane < 8) {                        // 16 bf16 = 8 words per row
    uint32_t wq = 0u, wd = 0u;
    if (lane == 0) {
      const float xh = bf16_lo(pack_bf16(-x, 0.f)), dh = bf16_lo(pack_bf16(-dl, 0.f));
      wq = pack_bf16(xh, -x - xh);
      wd = pack_bf16(dh, -dl - dh);
    }
    augq[wid * 8 + lane] = wq;
    augd[wid * 8 + lane] = wd;
  }
}

// dq = bf16(acc * scale (+ add)); `add`: an fp32 (B, L, H, 64) gradient from another branch
__global__ void attn_bwd_post_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                     long n4, float scale, const float* __restrict__ add) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 v = reinterpret_cast<const float4*>(acc)[i];
  v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
  if (add) {
    const float4 a = reinterpret_cast<const float4*>(add)[i];
    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
  }
  uint2 o;
  o.x = pack_bf16(v.x, v.y);
  o.y = pack_bf16(v.z, v.w);
  reinterpret_cast<uint2*>(dq)[i] = o;
}

// dk = scale * sum_r part_dk[r], dv = sum_r part_dv[r] (fixed order), rows of 64 channels.
__global__ void attn_bwd_combine_kernel(const float* __restrict__ part_dk,
                                        const float* __restrict__ part_dv,
                                        __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                                        int qsplit, int B, int L, int H, int64_t dk_sb, int64_t dk_sl,
                                        int64_t dk_sh, int64_t dv_sb, int64_t dv_sl, int64_t dv_sh,
                                        float scale) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;     // one float4 of one row
  const long rows = (long)B * L * H;
  if (i >= rows * 16) return;
  const long row = i >> 4;
  const int c = (int)(i & 15) * 4;
  const int h = (int)(row % H), l = (int)((row / H) % L), b = (int)(row / ((long)H * L));
  const size_t plane = (size_t)rows * 64;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), v = a;
  for (int r = 0; r < qsplit; ++r) {
    const float4 x = *reinterpret_cast<const float4*>(part_dk + r * plane + row * 64 + c);
    const float4 y = *reinterpret_cast<const float4*>(part_dv + r * plane + row * 64 + c);
    a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    v.x += y.x; v.y += y.y; v.z += y.z; v.w += y.w;
  }
  uint2 o;
  o.x = pack_bf16(a.x * scale, a.y * scale);
  o.y = pack_bf16(a.z * scale, a.w * scale);
  *reinterpret_cast<uint2*>(dk + b * dk_sb + (int64_t)l * dk_sl + h * dk_sh + c) = o;
  o.x = pack_bf16(v.x, v.y);
  o.y = pack_bf16(v.z, v.w);
  *reinterpret_cast<uint2*>(dv + b * dv_sb + (int64_t)l * dv_sl + h * dv_sh + c) = o;
}

// Number of CTAs the query tiles of one K/V tile are split over (dense mode): the smallest
// of 1..3 whose last wave wastes less than 6 % on this GPU.
static int bwd_qsplit(int B, int L, int H) {
  int dev = 0, sms = 0;        // of the current device (a host may hold GPUs of different sizes)
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const long n_t = (L + BW_T - 1) / BW_T;
  const long items = n_t * H * B;
  int best = 1;
  double best_w = 1e9;
  for (int s = 1; s <= 3 && s * 8 <= n_t; ++s) {
    const double waves = (double)items * s / sms;
    const double w = (double)((items * s + sms - 1) / sms) / waves;
    if (w < best_w - 0.02) {
      best_w = w;
      best = s;
    }
    if (w < 1.06) break;
  }
  return best;
}

static int make_map64(CUtensorMap* m, const void* ptr, int B, int L, int H, int64_t sb, int64_t sl,
                      int64_t sh) {
  uint64_t dims[4] = {(uint64_t)BW_HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)sh * 2, (uint64_t)sl * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {(uint32_t)BW_HD, 1, (uint32_t)BW_T, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, str, box);
}

}  // namespace imf

// Scratch (bytes) the backward needs: fp32 dQ accumulator + the two 16-column operand bands
// (-lse2, -delta; padded to Lp rows) + the scaled copy of Q + (dense mode, when the query tiles
// are split) fp32 partial dK / dV.
extern "C" long imf_attn_bwd_scratch_bytes(int B, int L, int H) {
  const long Lp = ((L + 127) / 128) * 128;
  const int qs = imf::bwd_qsplit(B, L, H);
  const long part = qs > 1 ? 2L * qs * B * L * H * 64 * 4 : 0;
  const long turns = (long)B * H * (Lp / 128) * 4 + 256;     // fixed-order dQ: one counter per query tile
  return (long)B * L * H * 64 * 4 + turns + 2 * (long)B * H * Lp * 32 + (long)B * L * H * 64 * 2 +
         1024 + part;
}

// Same for either head_dim (64 or 128).
extern "C" long imf_attn_bwd_scratch_bytes_hd(int B, int L, int H, int head_dim) {
  if (head_dim == 128) return imf::attn_bwd128_scratch_bytes(B, L, H);
  return imf_attn_bwd_scratch_bytes(B, L, H);
}

// All tensors (B, L, H, head_dim) bf16, head_dim 64 or 128 (128: dense only); strides[0..11]: (batch,row,head) for q,k,v,do;
// o contiguous-like with its own strides; dq contiguous (B, L, H, 64); dq_add: optional fp32
// (B, L, H, 64) contiguous, added to dq before the rounding to bf16 (another branch's gradient);
// dk/dv with given strides (dv may point into a wider buffer).
extern "C" int imf_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                            const void* d_o, const float* lse, void* dq, void* dk, void* dv, int B,
                            int L, int H, int head_dim, const int64_t* strides,
                            const int64_t* o_strides, const int64_t* dk_strides,
                            const int64_t* dv_strides, float scale, void* scratch,
                            long scratch_bytes, const int* qlist, const uint8_t* qflags,
                            const uint16_t* qrank, int qmax, int fixed_order, const float* dq_add,
                            int* status, void* stream) {
  using namespace imf;
  if ((head_dim != BW_HD && head_dim != 128) || B <= 0 || L <= 0 || H <= 0) return IMF_ERR_ARG;
  if (head_dim == 128) {
    if (qlist != nullptr || dq_add != nullptr) return IMF_ERR_ARG;   // head_dim 64 only
    if ((reinterpret_cast<uintptr_t>(scratch) & 255) || (reinterpret_cast<uintptr_t>(dq) & 15) ||
        (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15))
      return IMF_ERR_ARG;
    for (int i = 0; i < 3; ++i)
      if ((dk_strides[i] & 7) || (dv_strides[i] & 7) || (o_strides[i] & 3) || (strides[9 + i] & 3))
        return IMF_ERR_ARG;
    Bwd128Args a{q, k, v, o, d_o, lse, dq, dk, dv, B, L, H, strides, o_strides, dk_strides,
                 dv_strides, scale, scratch, scratch_bytes, status, stream,
                 fixed_order && status != nullptr};
    return attn_bwd128_launch(a);
  }
  if (scratch == nullptr || scratch_bytes < imf_attn_bwd_scratch_bytes(B, L, H)) return IMF_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(scratch) & 255) || (reinterpret_cast<uintptr_t>(dq) & 15) ||
      (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15) ||
      (reinterpret_cast<uintptr_t>(dq_add) & 15))
    return IMF_ERR_ARG;
  for (int i = 0; i < 3; ++i)
    if ((dk_strides[i] & 7) || (dv_strides[i] & 7) || (o_strides[i] & 1)) return IMF_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Lp = ((L + 127) / 128) * 128;
  float* dq_acc = static_cast<float*>(scratch);
  const size_t acc_bytes = ((size_t)B * L * H * 64 * 4 + 255) & ~size_t(255);
  // the turn counters follow the accumulator, so one memset clears both.  Fixed order needs a
  // status word (how a CTA that gave up tells the others) and, block-sparse, the rank table
  const bool ordered = fixed_order && status != nullptr && (qlist == nullptr || qrank != nullptr);
  int* turn = reinterpret_cast<int*>(static_cast<uint8_t*>(scratch) + acc_bytes);
  const size_t turn_bytes = ((size_t)B * H * (Lp / 128) * 4 + 255) & ~size_t(255);
  uint8_t* cur = static_cast<uint8_t*>(scratch) + acc_bytes + turn_bytes;
  uint32_t* augq = reinterpret_cast<uint32_t*>(cur);
  cur += (size_t)B * H * Lp * 32;
  uint32_t* augd = reinterpret_cast<uint32_t*>(cur);
  cur += (size_t)B * H * Lp * 32;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(cur);
  cur += ((size_t)B * L * H * 64 * 2 + 255) & ~size_t(255);
  const int qsplit = qlist ? 1 : bwd_qsplit(B, L, H);
  float* part_dk = nullptr;
  float* part_dv = nullptr;
  if (qsplit > 1) {
    part_dk = reinterpret_cast<float*>(cur);
    part_dv = part_dk + (size_t)qsplit * B * L * H * 64;
  }
  if (cudaMemsetAsync(dq_acc, 0, acc_bytes + turn_bytes, st) != cudaSuccess) return IMF_ERR_LAUNCH;
  {
    const long rows = (long)B * H * Lp;
    const int threads = 256;
    auto ok16 = [](const void* p, int64_t s0, int64_t s1, int64_t s2) {
      return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && s0 % 8 == 0 && s1 % 8 == 0 && s2 % 8 == 0;
    };
    const bool wide = ok16(q, strides[0], strides[1], strides[2]) &&
                      ok16(o, o_strides[0], o_strides[1], o_strides[2]) &&
                      ok16(d_o, strides[9], strides[10], strides[11]);
    const long warps = wide ? (rows + 3) / 4 : rows;
    const long blocks = (warps * 32 + threads - 1) / threads;
    (wide ? attn_bwd_prep_wide_kernel : attn_bwd_prep_kernel)<<<(unsigned)blocks, threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(o),
        static_cast<const __nv_bfloat16*>(d_o), lse, qs, augq, augd, B, L, H, Lp, strides[0],
        strides[1], strides[2], o_strides[0], o_strides[1], o_strides[2], strides[9], strides[10],
        strides[11], scale * 1.4426950408889634f);
    if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  }
  CUtensorMap mq, mk, mv, mdo, mdq, maq, mad;
  int rc;
  // the query operand is the scaled copy (contiguous (B, L, H, 64))
  if ((rc = make_map64(&mq, qs, B, L, H, (int64_t)L * H * 64, (int64_t)H * 64, 64))) return rc;
  for (int which = 0; which < 2; ++which) {      // (B*H, Lp, 16) bf16, 32-byte rows
    uint64_t dims[3] = {16, (uint64_t)Lp, (uint64_t)B * H};
    uint64_t str[3] = {2, 32, (uint64_t)Lp * 32};
    uint32_t box[3] = {16, (uint32_t)BW_T, 1};
    if ((rc = make_tmap(which ? &mad : &maq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                        which ? (void*)augd : (void*)augq, dims, str, box,
                        CU_TENSOR_MAP_SWIZZLE_32B)))
      return rc;
  }
  if ((rc = make_map64(&mk, k, B, L, H, strides[3], strides[4], strides[5]))) return rc;
  if ((rc = make_map64(&mv, v, B, L, H, strides[6], strides[7], strides[8]))) return rc;
  if ((rc = make_map64(&mdo, d_o, B, L, H, strides[9], strides[10], strides[11]))) return rc;
  {
    uint64_t dims[4] = {(uint64_t)BW_HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
    uint64_t str[4] = {4, (uint64_t)BW_HD * 4, (uint64_t)H * BW_HD * 4, (uint64_t)L * H * BW_HD * 4};
    uint32_t box[4] = {32, 1, (uint32_t)BW_T, 1};
    if ((rc = make_tmap(&mdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, dims, str, box)))
      return rc;
  }
  BwParams prm;
  prm.dq_acc = dq_acc;
  prm.dk = static_cast<__nv_bfloat16*>(dk);
  prm.dv = static_cast<__nv_bfloat16*>(dv);
  prm.B = B; prm.H = H; prm.L = L; prm.Lp = Lp;
  prm.dk_sb = dk_strides[0]; prm.dk_sl = dk_strides[1]; prm.dk_sh = dk_strides[2];
  prm.dv_sb = dv_strides[0]; prm.dv_sl = dv_strides[1]; prm.dv_sh = dv_strides[2];
  prm.scale = scale;
  prm.status = status;
  prm.qlist = qlist;
  prm.qflags = qflags;
  prm.qmax = qlist ? qmax : 0;
  prm.qsplit = qsplit;
  prm.part_dk = part_dk;
  prm.part_dv = part_dv;
  prm.turn = ordered ? turn : nullptr;
  prm.qrank = ordered ? qrank : nullptr;
  const size_t smem = sizeof(BwSmem) + 1024;
  auto kern = (qlist != nullptr && qflags != nullptr) ? attn_bwd_kernel<true> : attn_bwd_kernel<false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return IMF_ERR_LAUNCH;
  dim3 grid(H * B * qsplit, (L + BW_T - 1) / BW_T, 1);
  kern<<<grid, BW_THREADS, smem, st>>>(mq, mk, mv, mdo, mdq, maq, mad, prm);
  if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  if (qsplit > 1) {
    const long n = (long)B * L * H * 16;
    attn_bwd_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        part_dk, part_dv, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), qsplit,
        B, L, H, dk_strides[0], dk_strides[1], dk_strides[2], dv_strides[0], dv_strides[1],
        dv_strides[2], 0.6931471805599453f);      // partial dK = dS^T (Q scale log2e)
    if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  }
  const long n4 = (long)B * L * H * 64 / 4;
  attn_bwd_post_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(
      dq_acc, static_cast<__nv_bfloat16*>(dq), n4, scale, dq_add);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}
