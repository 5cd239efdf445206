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
// CTA = 256 query rows (two 128-row tiles that share every K/V tile) of one
// (batch, head).  Warps 0-3 / 4-7: softmax + O-correction + epilogue of tile
// 0 / 1 (one query row per thread, rows live in TMEM lanes); warp 8: single-
// thread tcgen05.mma issuer; warp 9: TMA producer.  The two tiles ping-pong:
// while one tile's softmax runs on the CUDA cores the tensor core works on the
// other tile.  P (and T) are written back to TMEM as bf16 over the S (dS)
// columns and consumed as the A operand of the second GEMM.  O is rescaled
// lazily (only when the running max grows by more than 2^8).
//
// Tensors are (B, L, H, 64) bf16 with arbitrary 16-byte-aligned strides;
// ragged L is handled by TMA zero fill + masking of the last K/V tile.
#include "common.cuh"
#include "host_util.h"

namespace imf {

constexpr int ATT_HD = 64;
constexpr int ATT_TILE_M = 128;
constexpr int ATT_THREADS = 320;
constexpr int ATT_STAGES = 3;

template <bool TANGENT>
struct AttCfg {
  static constexpr int BN = TANGENT ? 64 : 128;
  static constexpr int NQ = TANGENT ? 2 : 1;       // q + dq
  static constexpr int NKV = TANGENT ? 4 : 2;      // k, v (+ dk, dv)
  // TMEM columns per query tile
  static constexpr int COL_S = 0;
  static constexpr int COL_DS = BN;
  static constexpr int COL_O = TANGENT ? 2 * BN : BN;   // primal: S 128 | O 64
  static constexpr int COL_DO = COL_O + ATT_HD;
  static constexpr int TILE_COLS = TANGENT ? 256 : 192;
  static constexpr int TMEM_COLS = 512;
};

template <bool TANGENT>
struct AttSmem {
  using C = AttCfg<TANGENT>;
  alignas(1024) uint8_t q[C::NQ][2][ATT_TILE_M * 128];               // [q|dq][tile]
  alignas(1024) uint8_t kv[ATT_STAGES][C::NKV][C::BN * 128];         // k, v, dk, dv
  uint64_t q_full;
  uint64_t kv_full[ATT_STAGES];
  uint64_t kv_empty[ATT_STAGES];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_done[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct AttParams {
  __nv_bfloat16* o;
  __nv_bfloat16* dout;     // tangent output (TANGENT only)
  float* lse;              // (B, H, L) natural-log LSE of scaled scores
  int B, H, L;
  int64_t o_sb, o_sl, o_sh;   // output strides in elements
  float scale;
  int* status;
};

template <bool TANGENT>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_dq,
                const __grid_constant__ CUtensorMap tm_dk,
                const __grid_constant__ CUtensorMap tm_dv, const AttParams p) {
  using C = AttCfg<TANGENT>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<AttSmem<TANGENT>*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * (2 * ATT_TILE_M);
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_kv = (p.L + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    for (int i = 0; i < ATT_STAGES; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s.s_full[t], 1);
      mbar_init(&s.p_full[t], ATT_TILE_M);
      mbar_init(&s.o_done[t], 1);
    }
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(&s.tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;

  if (warp == 9) {
    // ------------------------------------------------------ TMA producer --
    if (elect_one()) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_arrive_expect_tx(&s.q_full, C::NQ * 2 * ATT_TILE_M * 128);
      for (int t = 0; t < 2; ++t) {
        tma_load_4d(s.q[0][t], &tm_q, &s.q_full, 0, h, q0 + t * ATT_TILE_M, b);
        if (TANGENT) tma_load_4d(s.q[C::NQ - 1][t], &tm_dq, &s.q_full, 0, h, q0 + t * ATT_TILE_M, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % ATT_STAGES;
        if (j >= ATT_STAGES &&
            !mbar_wait(&s.kv_empty[st], ((j / ATT_STAGES) & 1) ^ 1, abort_flag, p.status,
                       STATUS_TIMEOUT_EMPTY))
          break;
        mbar_arrive_expect_tx(&s.kv_full[st], C::NKV * BN * 128);
        tma_load_4d(s.kv[st][0], &tm_k, &s.kv_full[st], 0, h, j * BN, b);
        tma_load_4d(s.kv[st][1], &tm_v, &s.kv_full[st], 0, h, j * BN, b);
        if (TANGENT) {
          tma_load_4d(s.kv[st][C::NKV - 2], &tm_dk, &s.kv_full[st], 0, h, j * BN, b);
          tma_load_4d(s.kv[st][C::NKV - 1], &tm_dv, &s.kv_full[st], 0, h, j * BN, b);
        }
      }
    }
  } else if (warp == 8) {
    // -------------------------------------------------------- MMA issuer --
    if (elect_one()) {
      constexpr uint32_t idesc_qk = idesc_bf16(ATT_TILE_M, BN, 0, 0);
      constexpr uint32_t idesc_pv = idesc_bf16(ATT_TILE_M, ATT_HD, 0, 1);
      auto issue_qk = [&](int t, int st) {
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
        tc_commit(&s.s_full[t]);
      };
      auto issue_pv = [&](int t, int st, int j) {
        const uint32_t tb = tmem + t * C::TILE_COLS;
        const uint32_t va = smem_u32(s.kv[st][1]);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)
          mma_ts(tb + C::COL_O, tb + C::COL_S + ks * 8, sdesc_mnmajor(va + ks * 2048, BN * 128),
                 idesc_pv, (j | ks) != 0);
        if (TANGENT) {
          const uint32_t dva = smem_u32(s.kv[st][C::NKV - 1]);
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)
            mma_ts(tb + C::COL_DO, tb + C::COL_DS + ks * 8,
                   sdesc_mnmajor(va + ks * 2048, BN * 128), idesc_pv, (j | ks) != 0);
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks)
            mma_ts(tb + C::COL_DO, tb + C::COL_S + ks * 8,
                   sdesc_mnmajor(dva + ks * 2048, BN * 128), idesc_pv, 1);
        }
        tc_commit(&s.o_done[t]);
      };
      bool ok = mbar_wait(&s.q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA) &&
                mbar_wait(&s.kv_full[0], 0, abort_flag, p.status, STATUS_TIMEOUT_TMA);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        issue_qk(1, 0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % ATT_STAGES;
        for (int t = 0; t < 2 && ok; ++t) {
          ok = mbar_wait(&s.p_full[t], j & 1, abort_flag, p.status, STATUS_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          issue_pv(t, st, j);
          if (t == 1) tc_commit(&s.kv_empty[st]);
          if (j + 1 < n_kv) {
            const int st1 = (j + 1) % ATT_STAGES;
            if (t == 0) {
              ok = mbar_wait(&s.kv_full[st1], ((j + 1) / ATT_STAGES) & 1, abort_flag, p.status,
                             STATUS_TIMEOUT_TMA);
              if (!ok) break;
              tc_fence_after();
            }
            issue_qk(t, st1);
          }
        }
      }
    }
  } else {
    // ------------------------------------- softmax / correction / epilogue --
    const int t = warp >> 2;
    const int wl = warp & 3;
    const uint32_t tb = tmem_addr(tmem, wl * 32, t * C::TILE_COLS);
    const int q_row = q0 + t * ATT_TILE_M + wl * 32 + lane;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    float m_used = -INFINITY, l_sum = 0.f, mu_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      ok = __all_sync(0xffffffffu,
                      mbar_wait(&s.s_full[t], j & 1, abort_flag, p.status, STATUS_TIMEOUT_MMA));
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
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
      if (j == 0) {
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
          mu_sum *= alpha;
          ok = mbar_wait(&s.o_done[t], (j - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < (TANGENT ? 2 : 1) * ATT_HD; c += 32) {
            uint32_t ov[32];
            tmem_ld32(tb + C::COL_O + c, ov);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(tb + C::COL_O + c, ov);
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
          l_sum += p0 + p1;
          pk[i / 2] = pack_bf16(p0, p1);
          if (TANGENT) {
            const float t0 = p0 * __uint_as_float(dsv[c + i]) * p.scale;
            const float t1 = p1 * __uint_as_float(dsv[c + i + 1]) * p.scale;
            mu_sum += t0 + t1;
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
    // epilogue
    if (ok) ok = mbar_wait(&s.o_done[t], (n_kv - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l_sum;
      const bool live = q_row < p.L;
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
          const float mul = mu_sum * inv_l;
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
        p.lse[((int64_t)b * p.H + h) * p.L + q_row] = m_used * p.scale + __logf(l_sum);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

static int make_qkv_map(CUtensorMap* m, const void* ptr, int B, int L, int H, int64_t sb,
                        int64_t sl, int64_t sh, int rows) {
  uint64_t dims[4] = {(uint64_t)ATT_HD, (uint64_t)H, (uint64_t)L, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)sh * 2, (uint64_t)sl * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {(uint32_t)ATT_HD, 1, (uint32_t)rows, 1};
  return make_tmap(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, str, box);
}

template <bool TANGENT>
static int launch_attn_fwd(const void* q, const void* k, const void* v, const void* dq,
                           const void* dk, const void* dv, const int64_t* strides, AttParams prm,
                           cudaStream_t stream) {
  using C = AttCfg<TANGENT>;
  CUtensorMap mq, mk, mv, mdq, mdk, mdv;
  int rc;
  const int B = prm.B, L = prm.L, H = prm.H;
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
  auto kern = attn_fwd_kernel<TANGENT>;
  const size_t smem = sizeof(AttSmem<TANGENT>) + 1024;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return IMF_ERR_LAUNCH;
  dim3 grid((L + 2 * ATT_TILE_M - 1) / (2 * ATT_TILE_M), H, B);
  kern<<<grid, ATT_THREADS, smem, stream>>>(mq, mk, mv, mdq, mdk, mdv, prm);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}

}  // namespace imf

// Dense attention forward (+ optional tangent).  All tensors (B, L, H, 64)
// bf16; `strides` holds (batch, row, head) element strides for q, k, v and,
// when tangents are given, dq, dk, dv.  o/dout contiguous-in-last-dim with
// strides (o_sb, o_sl, o_sh).  lse: (B, H, L) fp32 or null.
extern "C" int imf_attn_fwd(const void* q, const void* k, const void* v, const void* dq,
                            const void* dk, const void* dv, void* o, void* dout, float* lse,
                            int B, int L, int H, int head_dim, const int64_t* strides,
                            int64_t o_sb, int64_t o_sl, int64_t o_sh, float scale, int* status,
                            void* stream) {
  using namespace imf;
  if (head_dim != ATT_HD || B <= 0 || L <= 0 || H <= 0) return IMF_ERR_ARG;
  if ((o_sl & 7) || (o_sh & 7) || (o_sb & 7) || (reinterpret_cast<uintptr_t>(o) & 15))
    return IMF_ERR_ARG;
  AttParams prm;
  prm.o = static_cast<__nv_bfloat16*>(o);
  prm.dout = static_cast<__nv_bfloat16*>(dout);
  prm.lse = lse;
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
    return launch_attn_fwd<true>(q, k, v, dq, dk, dv, strides, prm, st);
  }
  return launch_attn_fwd<false>(q, k, v, nullptr, nullptr, nullptr, strides, prm, st);
}
