// Dense flash attention backward for head_dim 128 on tcgen05 / TMEM (attn_bwd.cu
// serves head_dim 64 and the block-sparse mode).  Same math:
//
//   S^T = K Q^T,  P^T = exp2(S^T * scale*log2e - lse2),  dP^T = V dO^T,
//   dS^T = P^T .* (dP^T - delta),   delta = rowsum(dO .* O)
//   dV += P^T dO,   dK += scale * dS^T Q,   dQ += scale * dS K
//
// Replaces the library backward the reference falls back to for head dims its own
// kernels do not cover (reference models/imf_dit_video.py:81-104,
// models/attention_op.py:38-60).
//
// CTA = one 128-row K/V tile of one (batch, head); it walks over the query
// sequence in tiles of 64 rows.  dK and dV (128 x 128 fp32 each) stay in TMEM for
// the whole walk and take half of its 512 columns, which is why the query tile is
// 64 rows here: S^T (64) + dP^T (64) + P^T as bf16 (32) + dQ^T (64) fill the rest.
// dQ is produced TRANSPOSED, dQ^T = K^T dS^T (head_dim on the TMEM lanes, M = 128),
// because a 64-row dQ tile would be an M = 64 instruction; the reduction warps
// write it back un-transposed into a shared-memory stage and a TMA reduce-add
// accumulates it into the fp32 dQ buffer in global memory.
//
// Warps 0-3 / 4-7: exp / dS math for query columns 0-31 / 32-63 of the S^T tile;
// warps 8-11: dQ^T tile TMEM -> shared -> global reduction; warp 12: tcgen05.mma
// issuer; warp 13: TMA producer.  S^T / dP^T of tile i+1 are issued as soon as
// tile i has been pulled into registers.
#include "attn_bwd128.h"
#include "common.cuh"
#include "host_util.h"

namespace imf {
namespace b128 {

constexpr int HD = 128;
constexpr int KT = 128;              // K/V rows per CTA
constexpr int QT = 64;               // query rows per step
constexpr int THREADS = 512;         // 16 warps (setmaxnreg works on whole warpgroups; 14, 15 idle)
constexpr int QSTAGES = 2;
constexpr int KPANEL = KT * 128;     // bytes of one 64-column panel of the K (V) tile
constexpr int QPANEL = QT * 128;     // bytes of one 64-column panel of a Q (dO) tile
constexpr int DQPANEL = QT * 128;    // bytes of one 32-float panel of the dQ stage

// TMEM columns
constexpr int BC_S = 0, BC_DP = 64, BC_P = 128, BC_DQ = 192, BC_DK = 256, BC_DV = 384;
// P^T is double-buffered (columns 128-159 and 160-191): the math warps write tile i+1 while the
// dV MMA of tile i still reads its buffer, so they never wait for the tensor core's last tile

struct Smem {
  alignas(1024) uint8_t k[2 * KPANEL];
  alignas(1024) uint8_t v[2 * KPANEL];
  alignas(1024) uint8_t q[QSTAGES][2 * QPANEL];
  alignas(1024) uint8_t d_o[QSTAGES][2 * QPANEL];
  alignas(1024) uint8_t ds[2][KT * 128];              // dS^T: [kv 128][q 64] bf16, one panel
  alignas(1024) uint8_t dq_stage[4 * DQPANEL];        // dQ tile [q 64][hd 128] fp32, 4 panels
  alignas(16) float lse2[QSTAGES][QT];
  alignas(16) float delta[QSTAGES][QT];
  uint64_t kv_full;
  uint64_t q_full[QSTAGES], q_empty[QSTAGES];
  uint64_t s_full, s_taken, p_ready, p_free[2];
  uint64_t ds_free[2];
  uint64_t dq_full, dq_free;
  uint64_t final_bar;
  uint32_t tmem_base;
  int abort_flag;
};

struct Params {
  const float* lse2;      // (B, H, Lp) log2-domain LSE, +inf on padding rows
  const float* delta;     // (B, H, Lp) rowsum(dO .* O), 0 on padding rows
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int B, H, L, Lp;
  int64_t dk_sb, dk_sl, dk_sh, dv_sb, dv_sl, dv_sh;
  float scale;
  int* status;
  // the query tiles of a K/V tile are split over `qsplit` CTAs (blockIdx.z = batch * qsplit +
  // part); each writes unscaled fp32 partial dK / dV and a second kernel adds them up
  int qsplit;
  float* part_dk;
  float* part_dv;
  // fixed-order dQ (null = arrival order): one counter per (batch, head, 64-row query step),
  // zeroed before the launch; the CTA of K/V tile j adds when the counter shows j
  int* turn;
};

IMF_DEVICE void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd128_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_dq, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                     ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid = (chains, K/V tiles) with blockIdx.x = head + H * (batch * qsplit + part) fastest: a
  // CTA waits (fixed-order dQ) only for the K/V tile before it in its chain, whose block index
  // is smaller, and the resident CTAs are a few tiles of every chain
  const int kvb = (int)blockIdx.y;
  const int h = blockIdx.x % p.H, bz = blockIdx.x / p.H;
  const int b = bz / p.qsplit, qpart = bz % p.qsplit;
  int n_q = (p.L + QT - 1) / QT;
  int* turn = p.turn ? p.turn + ((size_t)b * p.H + h) * n_q : nullptr;
  const int q_first = (int)((long)qpart * n_q / p.qsplit);
  n_q = (int)((long)(qpart + 1) * n_q / p.qsplit) - q_first;

  if (threadIdx.x == 0) {
    mbar_init(&s.kv_full, 1);
    for (int i = 0; i < QSTAGES; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.q_empty[i], 1);
    }
    mbar_init(&s.s_full, 1);
    mbar_init(&s.s_taken, 8);      // one arrival per exp warp
    mbar_init(&s.p_ready, 8);
    mbar_init(&s.p_free[0], 1);
    mbar_init(&s.p_free[1], 1);
    mbar_init(&s.ds_free[0], 1);
    mbar_init(&s.ds_free[1], 1);
    mbar_init(&s.dq_full, 1);
    mbar_init(&s.dq_free, 4);
    mbar_init(&s.final_bar, 1);
    s.abort_flag = 0;
    fence_barrier_init();
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
      // ------------------------------------------------------ TMA producer --
      if (elect_one()) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
        prefetch_tmap(&tm_do);
        mbar_arrive_expect_tx(&s.kv_full, 4 * KPANEL);
        for (int pn = 0; pn < 2; ++pn) {
          tma_load_4d(s.k + pn * KPANEL, &tm_k, &s.kv_full, pn * 64, h, kvb * KT, b);
          tma_load_4d(s.v + pn * KPANEL, &tm_v, &s.kv_full, pn * 64, h, kvb * KT, b);
        }
        const float* lse_row = p.lse2 + ((size_t)b * p.H + h) * p.Lp;
        const float* dl_row = p.delta + ((size_t)b * p.H + h) * p.Lp;
        for (int i = 0; i < n_q; ++i) {
          const int st = i % QSTAGES;
          if (i >= QSTAGES &&
              !mbar_wait(&s.q_empty[st], (uint32_t)(((i / QSTAGES) - 1) & 1), abort_flag,
                         p.status, STATUS_TIMEOUT_EMPTY))
            break;
          const int qt = q_first + i;
          mbar_arrive_expect_tx(&s.q_full[st], 4 * QPANEL + 2 * QT * 4);
          for (int pn = 0; pn < 2; ++pn) {
            tma_load_4d(s.q[st] + pn * QPANEL, &tm_q, &s.q_full[st], pn * 64, h, qt * QT, b);
            tma_load_4d(s.d_o[st] + pn * QPANEL, &tm_do, &s.q_full[st], pn * 64, h, qt * QT, b);
          }
          bulk_load_1d(s.lse2[st], lse_row + (size_t)qt * QT, QT * 4, &s.q_full[st]);
          bulk_load_1d(s.delta[st], dl_row + (size_t)qt * QT, QT * 4, &s.q_full[st]);
        }
      }
    } else if (warp == 12) {
      // -------------------------------------------------------- MMA issuer --
      if (elect_one()) {
        constexpr uint32_t id_st = idesc_bf16(KT, QT, 0, 0);     // S^T, dP^T : [kv 128][q 64]
        constexpr uint32_t id_kn = idesc_bf16(KT, HD, 0, 1);     // dV (TS), dK (SS): [kv 128][hd 128]
        constexpr uint32_t id_dq = idesc_bf16(HD, QT, 1, 1);     // dQ^T: [hd 128][q 64]
        const uint32_t ka = smem_u32(s.k), va = smem_u32(s.v);
        auto issue_s = [&](int st) {
          const uint32_t qa = smem_u32(s.q[st]), doa = smem_u32(s.d_o[st]);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            mma_ss(tmem + BC_S, sdesc_kmajor(ka + (ks / 4) * KPANEL + (ks % 4) * 32),
                   sdesc_kmajor(qa + (ks / 4) * QPANEL + (ks % 4) * 32), id_st, ks != 0);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            mma_ss(tmem + BC_DP, sdesc_kmajor(va + (ks / 4) * KPANEL + (ks % 4) * 32),
                   sdesc_kmajor(doa + (ks / 4) * QPANEL + (ks % 4) * 32), id_st, ks != 0);
          tc_commit(&s.s_full);
        };
        bool ok = n_q > 0 &&
                  mbar_wait(&s.kv_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA) &&
                  mbar_wait(&s.q_full[0], 0, abort_flag, p.status, STATUS_TIMEOUT_TMA);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
        for (int i = 0; i < n_q && ok; ++i) {
          const int st = i % QSTAGES;
          const uint32_t par = (uint32_t)(i & 1);
          ok = mbar_wait(&s.s_taken, par, abort_flag, p.status, STATUS_TIMEOUT_SOFTMAX);
          if (!ok) break;
          if (i + 1 < n_q) {
            const int st1 = (i + 1) % QSTAGES;
            ok = mbar_wait(&s.q_full[st1], (uint32_t)(((i + 1) / QSTAGES) & 1), abort_flag,
                           p.status, STATUS_TIMEOUT_TMA);
            if (!ok) break;
            tc_fence_after();
            issue_s(st1);
          }
          ok = mbar_wait(&s.p_ready, par, abort_flag, p.status, STATUS_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          const uint32_t qa = smem_u32(s.q[st]), doa = smem_u32(s.d_o[st]);
          const uint32_t dsa = smem_u32(s.ds[i & 1]);
          // dV += P^T dO   (A = P^T in TMEM: 64 q as K -> 4 k-steps of 8 columns)
#pragma unroll
          for (int ks = 0; ks < QT / 16; ++ks)
            mma_ts(tmem + BC_DV, tmem + BC_P + (i & 1) * 32 + ks * 8,
                   sdesc_mnmajor(doa + ks * 2048, QPANEL), id_kn, (i | ks) != 0);
          tc_commit(&s.p_free[i & 1]);
          // dK += dS^T Q   (A = dS^T from smem, K-major: K = q)
#pragma unroll
          for (int ks = 0; ks < QT / 16; ++ks)
            mma_ss(tmem + BC_DK, sdesc_kmajor(dsa + ks * 32), sdesc_mnmajor(qa + ks * 2048, QPANEL),
                   id_kn, (i | ks) != 0);
          // Q and dO of this step have had their last reader: the stage goes back to the TMA
          // producer before the dQ GEMM (the load latency of step i + QSTAGES sets the pace)
          tc_commit(&s.q_empty[st]);
          // dQ_i^T = K^T dS^T   (A = K as MN-major: M = hd, K = kv; B = dS^T MN-major: N = q)
          if (i > 0) {
            ok = mbar_wait(&s.dq_free, (uint32_t)((i - 1) & 1), abort_flag, p.status,
                           STATUS_TIMEOUT_SOFTMAX);
            if (!ok) break;
            tc_fence_after();
          }
#pragma unroll
          for (int ks = 0; ks < KT / 16; ++ks)
            mma_ss(tmem + BC_DQ, sdesc_mnmajor(ka + ks * 2048, KPANEL),
                   sdesc_mnmajor(dsa + ks * 2048, KT * 128), id_dq, ks != 0);
          tc_commit(&s.dq_full);
          tc_commit(&s.ds_free[i & 1]);
        }
        if (ok) tc_commit(&s.final_bar);
      }
    }
  } else if (warp >= 8) {
    // ---------------------------------------- dQ^T tile -> global reduction --
    asm volatile("setmaxnreg.dec.sync.aligned.u32 112;");
    const int wl = warp & 3;                 // head-dim channels [32 wl, 32 wl + 32) = panel wl
    const uint32_t tb = tmem_addr(tmem, wl * 32, BC_DQ);
    uint8_t* panel = s.dq_stage + wl * DQPANEL;
    bool ok = true;
    bool turn_live = true;          // false once a turn wait gave up (the status word says so)
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
      // this thread holds channel (32 wl + lane) of 64 query rows: write them un-transposed
      // into panel wl ([64 rows][32 floats], 128-byte swizzle) for the TMA reduce-add
      if (i > 0) {
        if (threadIdx.x == 8 * 32) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
#pragma unroll
      for (int qq = 0; qq < QT; ++qq) {
        uint8_t* dst = panel + qq * 128 + ((((lane >> 2) ^ (qq & 7))) << 4) + ((lane & 3) << 2);
        *reinterpret_cast<uint32_t*>(dst) = r[qq];
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 8 * 32) {
        if (turn && turn_live) turn_live = turn_wait(turn + q_first + i, kvb, abort_flag, p.status);
        if (!turn || turn_live) {
#pragma unroll
          for (int pnl = 0; pnl < 4; ++pnl)
            asm volatile(
                "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group"
                " [%0, {%2, %3, %4, %5}], [%1];"
                ::"l"(reinterpret_cast<uint64_t>(&tm_dq)),
                "r"(smem_u32(s.dq_stage + pnl * DQPANEL)), "r"(pnl * 32), "r"(h),
                "r"((q_first + i) * QT), "r"(b)
                : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        // the add before this one has had a whole step's time to be performed: once it has,
        // pass its query rows on (this add stays in flight)
        if (turn && turn_live && i > 0) {
          asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
          turn_pass(turn + q_first + i - 1, kvb + 1);
        }
      }
    }
    if (threadIdx.x == 8 * 32) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (turn && turn_live && ok && n_q > 0) turn_pass(turn + q_first + n_q - 1, kvb + 1);
    }
  } else {
    // ------------------------------------------------------ exp / dS math ----
    asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
    const int wg = warp >> 2;           // query columns [32 wg, 32 wg + 32)
    const int wl = warp & 3;
    const int row = wl * 32 + lane;     // kv row of this thread (TMEM lane)
    const uint32_t tb = tmem_addr(tmem, wl * 32, 0);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    for (int i = 0; i < n_q && ok; ++i) {
      const int st = i % QSTAGES;
      const uint32_t par = (uint32_t)(i & 1);
      ok = __all_sync(0xffffffffu,
                      mbar_wait(&s.s_full, par, abort_flag, p.status, STATUS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[32], dp[32];
      tmem_ld32(tb + BC_S + wg * 32, sv);
      tmem_ld32(tb + BC_DP + wg * 32, dp);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.s_taken);
      const float4* lse4 = reinterpret_cast<const float4*>(s.lse2[st] + wg * 32);
      const float4* dl4 = reinterpret_cast<const float4*>(s.delta[st] + wg * 32);
      // all of the tile's math first, from registers only: it overlaps the dV / dK / dQ MMAs
      // of the previous tile, which still read P^T (TMEM) and dS^T (shared memory)
      uint32_t pk[16], dk_[16];
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        const float4 l4 = lse4[c / 4], d4 = dl4[c / 4];
        const float p0 = ex2(fmaf(__uint_as_float(sv[c]), scale_log2, -l4.x));
        const float p1 = ex2(fmaf(__uint_as_float(sv[c + 1]), scale_log2, -l4.y));
        const float p2 = ex2(fmaf(__uint_as_float(sv[c + 2]), scale_log2, -l4.z));
        const float p3 = ex2(fmaf(__uint_as_float(sv[c + 3]), scale_log2, -l4.w));
        pk[c / 2] = pack_bf16(p0, p1);
        pk[c / 2 + 1] = pack_bf16(p2, p3);
        dk_[c / 2] = pack_bf16(p0 * (__uint_as_float(dp[c]) - d4.x),
                               p1 * (__uint_as_float(dp[c + 1]) - d4.y));
        dk_[c / 2 + 1] = pack_bf16(p2 * (__uint_as_float(dp[c + 2]) - d4.z),
                                   p3 * (__uint_as_float(dp[c + 3]) - d4.w));
      }
      // P^T goes to TMEM buffer i&1 (A operand of the dV GEMM) and dS^T to smem buffer i&1: the
      // GEMMs of tile i-2 must have read them
      if (i >= 2) {
        ok = __all_sync(0xffffffffu, mbar_wait(&s.p_free[i & 1], (uint32_t)(((i / 2) - 1) & 1),
                                               abort_flag, p.status, STATUS_TIMEOUT_MMA));
        if (!ok) break;
      }
      tmem_st16(tb + BC_P + (i & 1) * 32 + wg * 16, pk);
      if (i >= 2) {
        ok = __all_sync(0xffffffffu,
                        mbar_wait(&s.ds_free[i & 1], (uint32_t)(((i / 2) - 1) & 1), abort_flag,
                                  p.status, STATUS_TIMEOUT_MMA));
        if (!ok) break;
      }
      uint8_t* dsb = s.ds[i & 1] + row * 128;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int chunk = wg * 4 + cc;
        uint4 val = make_uint4(dk_[4 * cc], dk_[4 * cc + 1], dk_[4 * cc + 2], dk_[4 * cc + 3]);
        *reinterpret_cast<uint4*>(dsb + ((chunk ^ (row & 7)) << 4)) = val;
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.p_ready);
    }
    // ---- epilogue: warps 0-3 store dK (scaled), warps 4-7 store dV ----
    if (ok && n_q > 0) ok = mbar_wait(&s.final_bar, 0, abort_flag, p.status, STATUS_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int kv_row = kvb * KT + row;
      const float mul = n_q == 0 ? 0.f : (wg == 0 ? p.scale : 1.f);
      __nv_bfloat16* base =
          wg == 0 ? p.dk + (int64_t)b * p.dk_sb + (int64_t)kv_row * p.dk_sl + (int64_t)h * p.dk_sh
                  : p.dv + (int64_t)b * p.dv_sb + (int64_t)kv_row * p.dv_sl + (int64_t)h * p.dv_sh;
      float* pbase = nullptr;
      if (p.qsplit > 1)
        pbase = (wg == 0 ? p.part_dk : p.part_dv) +
                ((((size_t)qpart * p.B + b) * p.L + kv_row) * p.H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
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

// delta = rowsum(dO .* O), lse2 = lse * log2(e), both padded to Lp rows per (b, h); one warp
// per (b, l, h) row of 128 channels.
__global__ void attn_bwd128_prep_kernel(const __nv_bfloat16* __restrict__ o,
                                        const __nv_bfloat16* __restrict__ d_o,
                                        const float* __restrict__ lse, float* __restrict__ lse2,
                                        float* __restrict__ delta, int B, int L, int H, int Lp,
                                        int64_t o_sb, int64_t o_sl, int64_t o_sh, int64_t g_sb,
                                        int64_t g_sl, int64_t g_sh) {
  const int lane = threadIdx.x & 31;
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long total = (long)B * H * Lp;
  if (wid >= total) return;
  const int l = (int)(wid % Lp), h = (int)((wid / Lp) % H), b = (int)(wid / ((long)Lp * H));
  if (l >= L) {
    if (lane == 0) {
      lse2[wid] = INFINITY;
      delta[wid] = 0.f;
    }
    return;
  }
  const uint2 a = *reinterpret_cast<const uint2*>(o + b * o_sb + (int64_t)l * o_sl + h * o_sh + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(d_o + b * g_sb + (int64_t)l * g_sl + h * g_sh + lane * 4);
  float v = bf16_lo(a.x) * bf16_lo(g.x) + bf16_hi(a.x) * bf16_hi(g.x) +
            bf16_lo(a.y) * bf16_lo(g.y) + bf16_hi(a.y) * bf16_hi(g.y);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if (lane == 0) {
    delta[wid] = v;
    lse2[wid] = lse[((long)b * H + h) * L + l] * 1.4426950408889634f;
  }
}

__global__ void attn_bwd128_post_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq,
                                        long n4, float scale) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v = reinterpret_cast<const float4*>(acc)[i];
  uint2 o;
  o.x = pack_bf16(v.x * scale, v.y * scale);
  o.y = pack_bf16(v.z * scale, v.w * scale);
  reinterpret_cast<uint2*>(dq)[i] = o;
}

// dk = scale * sum_r part_dk[r], dv = sum_r part_dv[r] (fixed order), rows of 128 channels.
__global__ void attn_bwd128_combine_kernel(const float* __restrict__ part_dk,
                                           const float* __restrict__ part_dv,
                                           __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                                           int qsplit, int B, int L, int H, int64_t dk_sb,
                                           int64_t dk_sl, int64_t dk_sh, int64_t dv_sb, int64_t dv_sl,
                                           int64_t dv_sh, float scale) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;     // one float4 of one row
  const long rows = (long)B * L * H;
  if (i >= rows * (HD / 4)) return;
  const long row = i / (HD / 4);
  const int c = (int)(i % (HD / 4)) * 4;
  const int h = (int)(row % H), l = (int)((row / H) % L), b = (int)(row / ((long)H * L));
  const size_t plane = (size_t)rows * HD;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), v = a;
  for (int r = 0; r < qsplit; ++r) {
    const float4 x = *reinterpret_cast<const float4*>(part_dk + r * plane + row * HD + c);
    const float4 y = *reinterpret_cast<const float4*>(part_dv + r * plane + row * HD + c);
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

// Number of CTAs the query tiles of one K/V tile are split over: the smallest of 1..3 whose
// last wave wastes less than 6 % on this GPU.
static int qsplit_for(int B, int L, int H) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const long n_t = (L + KT - 1) / KT;
  const long items = n_t * H * B;
  int best = 1;
  double best_w = 1e9;
  for (int sp = 1; sp <= 3 && sp * 8 <= n_t; ++sp) {
    const double waves = (double)items * sp / sms;
    const double w = (double)((items * sp + sms - 1) / sms) / waves;
    if (w < best_w - 0.02) {
      best_w = w;
      best = sp;
    }
    if (w < 1.06) break;
  }
  return best;
}

static int make_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int64_t sb, int64_t sl,
                    int64_t sh, int rows) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)sh * 2, (uint64_t)sl * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, 1, (uint32_t)rows, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, str, box);
}

}  // namespace b128

long attn_bwd128_scratch_bytes(int B, int L, int H) {
  const long Lp = ((L + 127) / 128) * 128;
  const int qs = b128::qsplit_for(B, L, H);
  const long part = qs > 1 ? 2L * qs * B * L * H * b128::HD * 4 : 0;
  const long turns = (long)B * H * (Lp / b128::QT) * 4 + 256;   // fixed-order dQ counters
  return (long)B * L * H * b128::HD * 4 + turns + 2 * (long)B * H * Lp * 4 + 512 + part;
}

int attn_bwd128_launch(const Bwd128Args& a) {
  using namespace b128;
  const int B = a.B, L = a.L, H = a.H;
  if (a.scratch == nullptr || a.scratch_bytes < attn_bwd128_scratch_bytes(B, L, H)) return IMF_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(a.stream);
  const int Lp = ((L + 127) / 128) * 128;
  float* dq_acc = static_cast<float*>(a.scratch);
  const size_t acc_bytes = ((size_t)B * L * H * HD * 4 + 255) & ~size_t(255);
  // the turn counters follow the accumulator, so one memset clears both
  int* turn = reinterpret_cast<int*>(static_cast<uint8_t*>(a.scratch) + acc_bytes);
  const size_t turn_bytes = ((size_t)B * H * (Lp / QT) * 4 + 255) & ~size_t(255);
  float* lse2 = reinterpret_cast<float*>(static_cast<uint8_t*>(a.scratch) + acc_bytes + turn_bytes);
  float* delta = lse2 + (size_t)B * H * Lp;
  const int qsplit = qsplit_for(B, L, H);
  float* part_dk = nullptr;
  float* part_dv = nullptr;
  if (qsplit > 1) {
    const uintptr_t end = (reinterpret_cast<uintptr_t>(delta + (size_t)B * H * Lp) + 255) & ~uintptr_t(255);
    part_dk = reinterpret_cast<float*>(end);
    part_dv = part_dk + (size_t)qsplit * B * L * H * HD;
  }
  if (cudaMemsetAsync(dq_acc, 0, acc_bytes + turn_bytes, st) != cudaSuccess) return IMF_ERR_LAUNCH;
  {
    const long warps = (long)B * H * Lp;
    const int threads = 256;
    const long blocks = (warps * 32 + threads - 1) / threads;
    attn_bwd128_prep_kernel<<<(unsigned)blocks, threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(a.o), static_cast<const __nv_bfloat16*>(a.d_o), a.lse, lse2,
        delta, B, L, H, Lp, a.o_strides[0], a.o_strides[1], a.o_strides[2], a.strides[9],
        a.strides[10], a.strides[11]);
    if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  }
  CUtensorMap mq, mk, mv, mdo, mdq;
  int rc;
  const int64_t* s_ = a.strides;
  if ((rc = make_map(&mq, a.q, B, L, H, s_[0], s_[1], s_[2], QT))) return rc;
  if ((rc = make_map(&mk, a.k, B, L, H, s_[3], s_[4], s_[5], KT))) return rc;
  if ((rc = make_map(&mv, a.v, B, L, H, s_[6], s_[7], s_[8], KT))) return rc;
  if ((rc = make_map(&mdo, a.d_o, B, L, H, s_[9], s_[10], s_[11], QT))) return rc;
  {
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
    uint64_t str[4] = {4, (uint64_t)HD * 4, (uint64_t)H * HD * 4, (uint64_t)L * H * HD * 4};
    uint32_t box[4] = {32, 1, (uint32_t)QT, 1};
    if ((rc = make_tmap(&mdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, dims, str, box)))
      return rc;
  }
  Params prm;
  prm.lse2 = lse2;
  prm.delta = delta;
  prm.dk = static_cast<__nv_bfloat16*>(a.dk);
  prm.dv = static_cast<__nv_bfloat16*>(a.dv);
  prm.B = B; prm.H = H; prm.L = L; prm.Lp = Lp;
  prm.dk_sb = a.dk_strides[0]; prm.dk_sl = a.dk_strides[1]; prm.dk_sh = a.dk_strides[2];
  prm.dv_sb = a.dv_strides[0]; prm.dv_sl = a.dv_strides[1]; prm.dv_sh = a.dv_strides[2];
  prm.scale = a.scale;
  prm.status = a.status;
  prm.qsplit = qsplit;
  prm.turn = (a.fixed_order && a.status != nullptr) ? turn : nullptr;
  prm.part_dk = part_dk;
  prm.part_dv = part_dv;
  const size_t smem = sizeof(Smem) + 1024;
  if (cudaFuncSetAttribute(attn_bwd128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return IMF_ERR_LAUNCH;
  dim3 grid(H * B * qsplit, (L + KT - 1) / KT, 1);
  attn_bwd128_kernel<<<grid, THREADS, smem, st>>>(mq, mk, mv, mdo, mdq, prm);
  if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  if (qsplit > 1) {
    const long n = (long)B * L * H * (HD / 4);
    attn_bwd128_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        part_dk, part_dv, prm.dk, prm.dv, qsplit, B, L, H, prm.dk_sb, prm.dk_sl, prm.dk_sh,
        prm.dv_sb, prm.dv_sl, prm.dv_sh, a.scale);
    if (cudaGetLastError() != cudaSuccess) return IMF_ERR_LAUNCH;
  }
  const long n4 = (long)B * L * H * HD / 4;
  attn_bwd128_post_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(
      dq_acc, static_cast<__nv_bfloat16*>(a.dq), n4, a.scale);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}

}  // namespace imf
