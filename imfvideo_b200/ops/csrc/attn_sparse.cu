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
// CTA = one query tile.  Warps 0-3: softmax / correction / epilogue (one row
// per thread), warp 4: tcgen05.mma issuer, warp 5: TMA producer.  TMEM use is
// 256 columns, so two CTAs share an SM and overlap each other's phases.
#include "common.cuh"
#include "host_util.h"

namespace imf {

constexpr int SP_HD = 64;
constexpr int SP_M = 128;
constexpr int SP_BK = 64;          // key block
constexpr int SP_THREADS = 192;
constexpr int SP_STAGES = 2;

// TMEM columns
constexpr int SC_S = 0, SC_DS = 64, SC_O = 128, SC_DO = 192;

struct SpSmem {
  alignas(1024) uint8_t q8[SP_M * 64];                         // int8, 64-byte rows, SWIZZLE_64B
  alignas(1024) uint8_t q[2][SP_M * 128];                      // q, dq (bf16)
  alignas(1024) uint8_t k8[SP_STAGES][SP_BK * 64];
  alignas(1024) uint8_t kv[SP_STAGES][4][SP_BK * 128];         // k, dk, v, dv (bf16)
  uint64_t q_full;
  uint64_t kv_full[SP_STAGES], kv_empty[SP_STAGES];
  uint64_t s_full, p_full, o_done;
  uint32_t tmem_base;
  int abort_flag;
};

struct SpParams {
  const int* lut;            // (B, H, n_mt, tmax) key-block ids, -1 = end of list
  const uint8_t* flags;      // (B, H, n_mt, tmax) bit0: rows 0-63 attend, bit1: rows 64-127
  const float* q_scale;      // (B, H, n_qblk)  per 64-row... per `qblk` rows
  const float* k_scale;      // (B, H, n_kblk)
  __nv_bfloat16* o;
  __nv_bfloat16* dout;
  float* lse;                // (B, H, L) natural log
  int B, H, L, n_mt, tmax, n_qblk, n_kblk, qblk;   // qblk: rows per query scale block (64 or 128)
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

template <bool TANGENT, bool INT8>
__global__ void __launch_bounds__(SP_THREADS, 2)
attn_sparse_fwd_kernel(const __grid_constant__ CUtensorMap tm_q8,
                       const __grid_constant__ CUtensorMap tm_k8,
                       const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v,
                       const __grid_constant__ CUtensorMap tm_dq,
                       const __grid_constant__ CUtensorMap tm_dk,
                       const __grid_constant__ CUtensorMap tm_dv, const SpParams p) {
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<SpSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                       ~uintptr_t(1023));
  constexpr bool NEED_QK = TANGENT || !INT8;     // bf16 q / k tiles are needed
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = mt * SP_M;
  const size_t lrow = (((size_t)b * p.H + h) * p.n_mt + mt) * p.tmax;
  const int* lut = p.lut + lrow;
  const uint8_t* flg = p.flags + lrow;
  int n_j = 0;
  while (n_j < p.tmax && lut[n_j] >= 0) ++n_j;

  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    for (int i = 0; i < SP_STAGES; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[i], 1);
    }
    mbar_init(&s.s_full, 1);
    mbar_init(&s.p_full, SP_M);
    mbar_init(&s.o_done, 1);
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(&s.tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;
  constexpr int VI = 2;                    // kv[stage] = {k, dk, v, dv}

  if (warp == 5) {
    if (elect_one()) {
      mbar_arrive_expect_tx(&s.q_full, (INT8 ? SP_M * 64 : 0) + (NEED_QK ? SP_M * 128 : 0) +
                                           (TANGENT ? SP_M * 128 : 0));
      if (INT8) tma_load_4d(s.q8, &tm_q8, &s.q_full, 0, h, q0, b);
      if (NEED_QK) tma_load_4d(s.q[0], &tm_q, &s.q_full, 0, h, q0, b);
      if (TANGENT) tma_load_4d(s.q[1], &tm_dq, &s.q_full, 0, h, q0, b);
      for (int j = 0; j < n_j; ++j) {
        const int st = j % SP_STAGES;
        if (j >= SP_STAGES &&
            !mbar_wait(&s.kv_empty[st], (uint32_t)(((j / SP_STAGES) - 1) & 1), abort_flag, p.status,
                       STATUS_TIMEOUT_EMPTY))
          break;
        const int k0 = lut[j] * SP_BK;
        mbar_arrive_expect_tx(&s.kv_full[st], (INT8 ? SP_BK * 64 : 0) +
                                                  (1 + (NEED_QK ? 1 : 0) + (TANGENT ? 2 : 0)) * SP_BK * 128);
        if (INT8) tma_load_4d(s.k8[st], &tm_k8, &s.kv_full[st], 0, h, k0, b);
        tma_load_4d(s.kv[st][VI], &tm_v, &s.kv_full[st], 0, h, k0, b);
        if (NEED_QK) tma_load_4d(s.kv[st][0], &tm_k, &s.kv_full[st], 0, h, k0, b);
        if (TANGENT) {
          tma_load_4d(s.kv[st][1], &tm_dk, &s.kv_full[st], 0, h, k0, b);
          tma_load_4d(s.kv[st][3], &tm_dv, &s.kv_full[st], 0, h, k0, b);
        }
      }
    }
  } else if (warp == 4) {
    if (elect_one()) {
      // s32 accumulate, signed 8-bit operands, both K-major
      constexpr uint32_t id_i8 = make_idesc(SP_M, SP_BK, FMT_S8, FMT_S8, 2, 0, 0);
      constexpr uint32_t id_qk = idesc_bf16(SP_M, SP_BK, 0, 0);
      constexpr uint32_t id_pv = idesc_bf16(SP_M, SP_HD, 0, 1);
      bool ok = mbar_wait(&s.q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA);
      for (int j = 0; j < n_j && ok; ++j) {
        const int st = j % SP_STAGES;
        ok = mbar_wait(&s.kv_full[st], (uint32_t)((j / SP_STAGES) & 1), abort_flag, p.status,
                       STATUS_TIMEOUT_TMA);
        if (!ok) break;
        tc_fence_after();
        // S (s32) = Q8 K8^T : K = 64 int8 = two k-steps of 32 bytes
        if (INT8) {
          const uint32_t q8a = smem_u32(s.q8), k8a = smem_u32(s.k8[st]);
#pragma unroll
          for (int ks = 0; ks < 2; ++ks)
            mma_ss_i8(tmem + SC_S, sdesc_kmajor_sw64(q8a + ks * 32),
                      sdesc_kmajor_sw64(k8a + ks * 32), id_i8, ks != 0);
        } else {
          const uint32_t qa = smem_u32(s.q[0]), ka = smem_u32(s.kv[st][0]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tmem + SC_S, sdesc_kmajor(qa + ks * 32), sdesc_kmajor(ka + ks * 32), id_qk,
                   ks != 0);
        }
        if (TANGENT) {
          const uint32_t qa = smem_u32(s.q[0]), dqa = smem_u32(s.q[1]);
          const uint32_t ka = smem_u32(s.kv[st][0]), dka = smem_u32(s.kv[st][1]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tmem + SC_DS, sdesc_kmajor(dqa + ks * 32), sdesc_kmajor(ka + ks * 32), id_qk,
                   ks != 0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tmem + SC_DS, sdesc_kmajor(qa + ks * 32), sdesc_kmajor(dka + ks * 32), id_qk, 1);
        }
        tc_commit(&s.s_full);
        ok = mbar_wait(&s.p_full, (uint32_t)(j & 1), abort_flag, p.status, STATUS_TIMEOUT_SOFTMAX);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(s.kv[st][VI]);
#pragma unroll
        for (int ks = 0; ks < SP_BK / 16; ++ks)
          mma_ts(tmem + SC_O, tmem + SC_S + ks * 8, sdesc_mnmajor(va + ks * 2048, SP_BK * 128),
                 id_pv, (j | ks) != 0);
        if (TANGENT) {
          const uint32_t dva = smem_u32(s.kv[st][3]);
#pragma unroll
          for (int ks = 0; ks < SP_BK / 16; ++ks)
            mma_ts(tmem + SC_DO, tmem + SC_DS + ks * 8, sdesc_mnmajor(va + ks * 2048, SP_BK * 128),
                   id_pv, (j | ks) != 0);
#pragma unroll
          for (int ks = 0; ks < SP_BK / 16; ++ks)
            mma_ts(tmem + SC_DO, tmem + SC_S + ks * 8, sdesc_mnmajor(dva + ks * 2048, SP_BK * 128),
                   id_pv, 1);
        }
        tc_commit(&s.o_done);
        tc_commit(&s.kv_empty[st]);
      }
    }
  } else {
    const int row = warp * 32 + lane;
    const int half = row >> 6;
    const int q_row = q0 + row;
    const uint32_t tb = tmem_addr(tmem, warp * 32, 0);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int qb_idx = q_row / p.qblk;
    const float sq = p.q_scale[((size_t)b * p.H + h) * p.n_qblk + (qb_idx < p.n_qblk ? qb_idx : p.n_qblk - 1)];
    const float* ksc = p.k_scale + ((size_t)b * p.H + h) * p.n_kblk;
    float m_used = -INFINITY, l_sum = 0.f, l_sum2 = 0.f, mu_sum = 0.f, mu_sum2 = 0.f;
    bool ok = true;
    for (int j = 0; j < n_j && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s.s_full, (uint32_t)(j & 1), abort_flag, p.status,
                                             STATUS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[SP_BK];
      tmem_ld32(tb + SC_S, sv);
      tmem_ld32(tb + SC_S + 32, sv + 32);
      uint32_t dsv[TANGENT ? SP_BK : 1];
      if (TANGENT) {
        tmem_ld32(tb + SC_DS, dsv);
        tmem_ld32(tb + SC_DS + 32, dsv + 32);
      }
      tc_wait_ld();
      const int kb = lut[j];
      const bool attend = (flg[j] >> half) & 1;
      const int kv_rem = p.L - kb * SP_BK;
      const float deq = INT8 ? sq * ksc[kb] : 1.f;   // s32 -> real score (before the softmax scale)
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < SP_BK; ++i) {
        float x = INT8 ? static_cast<float>(static_cast<int>(sv[i])) * deq : __uint_as_float(sv[i]);
        if (!attend || i >= kv_rem) x = -INFINITY;
        sv[i] = __float_as_uint(x);
        mx = fmaxf(mx, x);
      }
      if (j == 0) {
        m_used = mx;
      } else {
        // with the QAT grid on P the running max is tracked exactly (P <= 1), otherwise
        // lazily; both tests are false for NaN (-inf - -inf)
        const bool need = p.quant_p ? (mx > m_used) : ((mx - m_used) * scale_log2 > 8.0f);
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.f;
          if (need) {
            alpha = ex2((m_used - mx) * scale_log2);             // 0 when m_used == -inf
            m_used = mx;
          }
          l_sum *= alpha; l_sum2 *= alpha; mu_sum *= alpha; mu_sum2 *= alpha;
          ok = __all_sync(0xffffffffu, mbar_wait(&s.o_done, (uint32_t)((j - 1) & 1), abort_flag,
                                                 p.status, STATUS_TIMEOUT_MMA));
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < (TANGENT ? 128 : 64); c += 32) {
            uint32_t ov[32];
            tmem_ld32(tb + SC_O + c, ov);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(tb + SC_O + c, ov);
          }
          tc_wait_st();
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used * scale_log2;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t pk[16];
        uint32_t tk[TANGENT ? 16 : 1];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int c = hh * 32 + i;
          float p0 = ex2(fmaf(__uint_as_float(sv[c]), scale_log2, neg_m));
          float p1 = ex2(fmaf(__uint_as_float(sv[c + 1]), scale_log2, neg_m));
          if (p.quant_p) {
            p0 = rintf(p0 * 127.f) * (1.f / 127.f);
            p1 = rintf(p1 * 127.f) * (1.f / 127.f);
          }
          l_sum += p0;
          l_sum2 += p1;
          pk[i / 2] = pack_bf16(p0, p1);
          if (TANGENT) {
            const float t0 = p0 * __uint_as_float(dsv[c]) * p.scale;
            const float t1 = p1 * __uint_as_float(dsv[c + 1]) * p.scale;
            mu_sum += t0;
            mu_sum2 += t1;
            tk[i / 2] = pack_bf16(t0, t1);
          }
        }
        tmem_st16(tb + SC_S + hh * 16, pk);
        if (TANGENT) tmem_st16(tb + SC_DS + hh * 16, tk);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&s.p_full);
    }
    if (ok && n_j > 0)
      ok = mbar_wait(&s.o_done, (uint32_t)((n_j - 1) & 1), abort_flag, p.status, STATUS_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_j > 0) {
      tc_fence_after();
      const float l_tot = l_sum + l_sum2, mu_tot = mu_sum + mu_sum2;
      const float inv_l = l_tot > 0.f ? 1.f / l_tot : 0.f;
      const bool live = q_row < p.L;
      const int64_t off = (int64_t)b * p.o_sb + (int64_t)q_row * p.o_sl + (int64_t)h * p.o_sh;
#pragma unroll
      for (int c = 0; c < SP_HD; c += 32) {
        uint32_t ov[32];
        tmem_ld32(tb + SC_O + c, ov);
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
          tmem_ld32(tb + SC_DO + c, dv_);
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
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 256);
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
  const long warps = (long)B * H * n_blk;
  const long blocks = (warps * 32 + 255) / 256;
  quantize_blocks_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (int8_t*)xq, xs, (__nv_bfloat16*)xfq, B, L, H, block, n_blk, sb, sl, sh);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}

// q8/k8: contiguous (B, L, H, 64) int8; q/k/v/dq/dk/dv bf16 with `strides`
// (18 element strides, (batch, row, head) each, in the order q, k, v, dq, dk, dv;
// q, k, dq, dk, dv may be null for the primal-only call).
extern "C" int imf_attn_sparse_fwd(const void* q8, const void* k8, const float* q_scale,
                                   const float* k_scale, const void* q, const void* k,
                                   const void* v, const void* dq, const void* dk, const void* dv,
                                   const int* lut, const uint8_t* flags, void* o, void* dout,
                                   float* lse, int B, int L, int H, int tmax, int qblk,
                                   const int64_t* strides, int64_t o_sb, int64_t o_sl, int64_t o_sh,
                                   float scale, int quant_p, int int8_qk, int* status, void* stream) {
  if (B <= 0 || L <= 0 || H <= 0 || tmax <= 0 || (qblk != 64 && qblk != 128)) return IMF_ERR_ARG;
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
  p.lut = lut; p.flags = flags; p.q_scale = q_scale; p.k_scale = k_scale;
  p.o = (__nv_bfloat16*)o; p.dout = (__nv_bfloat16*)dout; p.lse = lse;
  p.B = B; p.H = H; p.L = L; p.n_mt = (L + SP_M - 1) / SP_M; p.tmax = tmax;
  p.qblk = qblk; p.n_qblk = (L + qblk - 1) / qblk; p.n_kblk = (L + SP_BK - 1) / SP_BK;
  p.o_sb = o_sb; p.o_sl = o_sl; p.o_sh = o_sh; p.scale = scale; p.quant_p = quant_p;
  p.status = status;
  dim3 grid(p.n_mt, H, B);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = sizeof(SpSmem) + 1024;
#define IMF_SP_LAUNCH(T_, I_)                                                                   \
  do {                                                                                          \
    if (cudaFuncSetAttribute(attn_sparse_fwd_kernel<T_, I_>,                                    \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return IMF_ERR_LAUNCH;                                                                    \
    attn_sparse_fwd_kernel<T_, I_><<<grid, SP_THREADS, smem, st>>>(mq8, mk8, mq, mk, mv, mdq, mdk, \
                                                                   mdv, p);                     \
  } while (0)
  if (tang && int8_qk) IMF_SP_LAUNCH(true, true);
  else if (tang) IMF_SP_LAUNCH(true, false);
  else if (int8_qk) IMF_SP_LAUNCH(false, true);
  else IMF_SP_LAUNCH(false, false);
#undef IMF_SP_LAUNCH
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}
