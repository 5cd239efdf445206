// Remaining per-token kernels of the MLA block, each with forward-mode
// tangent and reverse-mode gradient:
//   * strided RMSNorm over a column band of a wider GEMM output (latent norms)
//   * q/k preparation: per-head RMSNorm of the position-free band, rotary
//     embedding of the rope band, shared k_rope broadcast over heads
//   * sigmoid output gate, SituAndMul activation, gated residual add
// They replace the reference's `_rmsnorm_jvp_strided_kernel`, `_q_prep_kernel`,
// `_kv_prep_kernel`, `_out_gate_jvp_kernel`, `_swiglu_row_jvp_kernel` and
// `_gate_add_kernel` (reference models/triton_mla_block_jvp.py:237-521) and
// add the backward halves the reference leaves to autograd.
#include "rowops_common.cuh"

namespace imf {

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------
// Strided RMSNorm, up to 2 column segments per launch (grid.y = segment)
// ---------------------------------------------------------------------------
struct NormSeg {
  const bf16* x;
  const bf16* dx;
  const float* gain;
  bf16* out;
  bf16* dout;
  const bf16* gy;   // bwd: grad of out
  bf16* gx;         // bwd: grad of x (strided like x)
  float* partial;   // bwd: [grid.x, D]
  int D, ld_x, ld_o;
};
struct NormArgs {
  NormSeg seg[2];
  int rows;
  float eps;
  int has_t;
};

__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_seg_fwd_kernel(const NormArgs a) {
  const NormSeg& s = a.seg[blockIdx.y];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_d = 1.f / s.D;
  if (s.D <= 128) {
    // a row is one 8-byte load per lane: four rows per warp pass, all loads issued before the
    // first reduction, or the kernel is a chain of load latencies
    const int c = lane * 4, step = gridDim.x * ROW_WARPS;
    const bool in = c < s.D;
    const float4 g = in ? ld4(s.gain + c) : f4zero();
    for (int row0 = blockIdx.x * ROW_WARPS + warp; row0 < a.rows; row0 += 4 * step) {
      float4 v[4], dv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int row = row0 + k * step;
        const bool ok = in && row < a.rows;
        v[k] = ok ? ld4(s.x + (size_t)row * s.ld_x + c) : f4zero();
        dv[k] = (ok && a.has_t) ? ld4(s.dx + (size_t)row * s.ld_x + c) : f4zero();
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int row = row0 + k * step;
        const float ss = warp_sum(dot4(v[k], v[k]));
        const float r = rsqrtf(ss * inv_d + a.eps);
        float c2 = 0.f;
        if (a.has_t) c2 = warp_sum(dot4(v[k], dv[k])) * inv_d * r * r * r;
        if (in && row < a.rows) {
          st4(s.out + (size_t)row * s.ld_o + c, v[k] * g * r);
          if (a.has_t) st4(s.dout + (size_t)row * s.ld_o + c, fma4(v[k], -c2, dv[k] * r) * g);
        }
      }
    }
    return;
  }
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    const bf16* x = s.x + (size_t)row * s.ld_x;
    const bf16* dx = a.has_t ? s.dx + (size_t)row * s.ld_x : nullptr;
    float ss = 0.f, xd = 0.f;
    for (int c = lane * 4; c < s.D; c += 128) {
      const float4 v = ld4(x + c);
      ss += dot4(v, v);
      if (a.has_t) xd += dot4(v, ld4(dx + c));
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss * inv_d + a.eps);
    float c2 = 0.f;
    if (a.has_t) c2 = warp_sum(xd) * inv_d * r * r * r;
    for (int c = lane * 4; c < s.D; c += 128) {
      const float4 v = ld4(x + c), g = ld4(s.gain + c);
      st4(s.out + (size_t)row * s.ld_o + c, v * g * r);
      if (a.has_t)
        st4(s.dout + (size_t)row * s.ld_o + c, fma4(v, -c2, ld4(dx + c) * r) * g);
    }
  }
}

__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_seg_bwd_kernel(const NormArgs a) {
  extern __shared__ float smem_acc[];  // [ROW_WARPS][D]
  const NormSeg& s = a.seg[blockIdx.y];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_d = 1.f / s.D;
  float* acc = smem_acc + (size_t)warp * s.D;
  for (int c = lane; c < s.D; c += 32) acc[c] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    const bf16* x = s.x + (size_t)row * s.ld_x;
    const bf16* gy = s.gy + (size_t)row * s.ld_o;
    float ss = 0.f, ux = 0.f;
    for (int c = lane * 4; c < s.D; c += 128) {
      const float4 v = ld4(x + c);
      ss += dot4(v, v);
      ux += dot4(ld4(gy + c) * ld4(s.gain + c), v);
    }
    ss = warp_sum(ss);
    ux = warp_sum(ux);
    const float r = rsqrtf(ss * inv_d + a.eps);
    const float c3 = ux * inv_d * r * r * r;
    for (int c = lane * 4; c < s.D; c += 128) {
      const float4 v = ld4(x + c), g = ld4(gy + c);
      st4(s.gx + (size_t)row * s.ld_x + c, fma4(v, -c3, g * ld4(s.gain + c) * r));
      st4(acc + c, ld4(acc + c) + g * v * r);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < s.D; c += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < ROW_WARPS; ++w) t += smem_acc[(size_t)w * s.D + c];
    s.partial[(size_t)blockIdx.x * s.D + c] = t;
  }
}

__device__ __forceinline__ void unpack8(const uint4 v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------
// q / k preparation
// ---------------------------------------------------------------------------
struct PrepArgs {
  const bf16 *qb, *dqb;        // [rows, H*HD]
  const bf16 *kvb, *dkvb;      // [rows, H*(dn+dv)]
  const bf16 *kr, *dkr;        // shared rope key, [rows, dr] with row stride ld_kr
  const float *cos_, *sin_;    // [L, dr/2]
  const float *qg, *kg;        // per-head norm gains [dn]
  bf16 *q, *dq, *k, *dk;       // [rows, H, HD]
  // backward
  const bf16 *gq, *gk;         // [rows, H, HD]
  bf16 *g_qb, *g_kvb, *g_kr;   // same layouts as qb / kvb (nope band only) / kr
  float* partial;              // [grid, 2, dn]
  int rows, L, H, dn, dr, dv, ld_kr, ld_gkr;
  float eps;
  int has_t;
};

// one warp per (row, head, q|k); lane owns EPL = HD/32 consecutive channels
template <int EPL>
__global__ void __launch_bounds__(ROW_THREADS) qkprep_fwd_kernel(const PrepArgs a) {
  const int HD = EPL * 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long total = (long)a.rows * a.H * 2;
  const float inv_dn = 1.f / a.dn;
  for (long wid = (long)blockIdx.x * ROW_WARPS + warp; wid < total;
       wid += (long)gridDim.x * ROW_WARPS) {
    const int which = (int)(wid % 2);
    const int h = (int)((wid / 2) % a.H);
    const int row = (int)(wid / (2 * a.H));
    const int c0 = lane * EPL;
    const bool nope = c0 < a.dn;
    const bf16 *src, *dsrc;
    if (which == 0) {
      src = a.qb + (size_t)row * a.H * HD + h * HD + c0;
      dsrc = a.dqb ? a.dqb + (size_t)row * a.H * HD + h * HD + c0 : nullptr;
    } else if (nope) {
      src = a.kvb + (size_t)row * a.H * (a.dn + a.dv) + h * (a.dn + a.dv) + c0;
      dsrc = a.dkvb ? a.dkvb + (size_t)row * a.H * (a.dn + a.dv) + h * (a.dn + a.dv) + c0 : nullptr;
    } else {
      src = a.kr + (size_t)row * a.ld_kr + (c0 - a.dn);
      dsrc = a.dkr ? a.dkr + (size_t)row * a.ld_kr + (c0 - a.dn) : nullptr;
    }
    float x[EPL], dx[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      x[e] = __bfloat162float(src[e]);
      dx[e] = (a.has_t && dsrc) ? __bfloat162float(dsrc[e]) : 0.f;
    }
    float ss = 0.f, xd = 0.f;
    if (nope) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        ss += x[e] * x[e];
        xd += x[e] * dx[e];
      }
    }
    ss = warp_sum(ss);
    xd = warp_sum(xd);
    float y[EPL], dy[EPL];
    if (nope) {
      const float r = rsqrtf(ss * inv_dn + a.eps);
      const float c2 = xd * inv_dn * r * r * r;
      const float* g = (which == 0 ? a.qg : a.kg) + c0;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        y[e] = x[e] * r * g[e];
        dy[e] = (dx[e] * r - x[e] * c2) * g[e];
      }
    } else {
      const int pos = row % a.L;
      const int pr = (c0 - a.dn) / 2;
#pragma unroll
      for (int e = 0; e < EPL; e += 2) {
        const float cs = a.cos_[(size_t)pos * (a.dr / 2) + pr + e / 2];
        const float sn = a.sin_[(size_t)pos * (a.dr / 2) + pr + e / 2];
        y[e] = x[e] * cs - x[e + 1] * sn;
        y[e + 1] = x[e] * sn + x[e + 1] * cs;
        dy[e] = dx[e] * cs - dx[e + 1] * sn;
        dy[e + 1] = dx[e] * sn + dx[e + 1] * cs;
      }
    }
    bf16* dst = (which == 0 ? a.q : a.k) + ((size_t)row * a.H + h) * HD + c0;
    bf16* ddst = (which == 0 ? a.dq : a.dk);
#pragma unroll
    for (int e = 0; e < EPL; e += 2)
      *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(y[e], y[e + 1]);
    if (a.has_t) {
      ddst += ((size_t)row * a.H + h) * HD + c0;
#pragma unroll
      for (int e = 0; e < EPL; e += 2)
        *reinterpret_cast<__nv_bfloat162*>(ddst + e) = __floats2bfloat162_rn(dy[e], dy[e + 1]);
    }
  }
}

// Wide variant of the forward: a lane owns 8 consecutive channels (one 16-byte access), so a
// head is HD / 8 lanes and a warp handles 32 / (HD / 8) (row, head, q|k) units at once; the
// RMS reduction runs inside the lane group.  Needs dn % 8 == 0 and 16-byte aligned rows.
template <int HD>
__global__ void __launch_bounds__(ROW_THREADS) qkprep_fwd_wide_kernel(const PrepArgs a) {
  constexpr int LPH = HD / 8;            // lanes per head: 8 or 16
  constexpr int UPW = 32 / LPH;          // units per warp: 4 or 2
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPH, c0 = (lane % LPH) * 8;
  const bool nope = c0 < a.dn;
  const int total = a.rows * a.H * 2;
  const int n_groups = (total + UPW - 1) / UPW;
  const float inv_dn = 1.f / a.dn;
  const int kvw = a.H * (a.dn + a.dv);
  for (int grp = blockIdx.x * ROW_WARPS + warp; grp < n_groups; grp += gridDim.x * ROW_WARPS) {
    const int wid = grp * UPW + sub;
    const bool live = wid < total;
    const int which = wid & 1, h = (wid >> 1) % a.H, row = (wid >> 1) / a.H;
    float x[8], dx[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = dx[e] = 0.f;
    if (live) {
      const bf16 *src, *dsrc;
      if (which == 0) {
        src = a.qb + (size_t)row * a.H * HD + h * HD + c0;
        dsrc = a.dqb ? a.dqb + (size_t)row * a.H * HD + h * HD + c0 : nullptr;
      } else if (nope) {
        src = a.kvb + (size_t)row * kvw + h * (a.dn + a.dv) + c0;
        dsrc = a.dkvb ? a.dkvb + (size_t)row * kvw + h * (a.dn + a.dv) + c0 : nullptr;
      } else {
        src = a.kr + (size_t)row * a.ld_kr + (c0 - a.dn);
        dsrc = a.dkr ? a.dkr + (size_t)row * a.ld_kr + (c0 - a.dn) : nullptr;
      }
      unpack8(*reinterpret_cast<const uint4*>(src), x);
      if (a.has_t && dsrc) unpack8(*reinterpret_cast<const uint4*>(dsrc), dx);
    }
    float ss = 0.f, xd = 0.f;
    if (nope) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        ss += x[e] * x[e];
        xd += x[e] * dx[e];
      }
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) {       // reduction inside the head's lane group
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      xd += __shfl_xor_sync(0xffffffffu, xd, o);
    }
    if (!live) continue;
    float y[8], dy[8];
    if (nope) {
      const float r = rsqrtf(ss * inv_dn + a.eps);
      const float c2 = xd * inv_dn * r * r * r;
      const float* g = (which == 0 ? a.qg : a.kg) + c0;
      const float4 g0 = ld4(g), g1 = ld4(g + 4);
      const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        y[e] = x[e] * r * gg[e];
        dy[e] = (dx[e] * r - x[e] * c2) * gg[e];
      }
    } else {
      const int pos = row % a.L;
      const size_t ro = (size_t)pos * (a.dr / 2) + (c0 - a.dn) / 2;
      const float4 cs4 = ld4(a.cos_ + ro), sn4 = ld4(a.sin_ + ro);
      const float cs[4] = {cs4.x, cs4.y, cs4.z, cs4.w}, sn[4] = {sn4.x, sn4.y, sn4.z, sn4.w};
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        y[e] = x[e] * cs[e / 2] - x[e + 1] * sn[e / 2];
        y[e + 1] = x[e] * sn[e / 2] + x[e + 1] * cs[e / 2];
        dy[e] = dx[e] * cs[e / 2] - dx[e + 1] * sn[e / 2];
        dy[e + 1] = dx[e] * sn[e / 2] + dx[e + 1] * cs[e / 2];
      }
    }
    const size_t off = ((size_t)row * a.H + h) * HD + c0;
    *reinterpret_cast<uint4*>((which == 0 ? a.q : a.k) + off) = pack8(y);
    if (a.has_t) *reinterpret_cast<uint4*>((which == 0 ? a.dq : a.dk) + off) = pack8(dy);
  }
}

// backward: warps (row, h, q|k) as forward, plus one extra warp slot per row
// (index 2H) that sums the shared rope-key gradient over heads.
template <int EPL>
__global__ void __launch_bounds__(ROW_THREADS) qkprep_bwd_kernel(const PrepArgs a) {
  const int HD = EPL * 32;
  extern __shared__ float smem_acc[];  // [ROW_WARPS][2][dn]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* acc = smem_acc + (size_t)warp * 2 * a.dn;
  for (int c = lane; c < 2 * a.dn; c += 32) acc[c] = 0.f;
  __syncwarp();
  const int per_row = 2 * a.H + 1;
  const long total = (long)a.rows * per_row;
  const float inv_dn = 1.f / a.dn;
  for (long wid = (long)blockIdx.x * ROW_WARPS + warp; wid < total;
       wid += (long)gridDim.x * ROW_WARPS) {
    const int slot = (int)(wid % per_row);
    const int row = (int)(wid / per_row);
    const int pos = row % a.L;
    if (slot == 2 * a.H) {
      // g_k_rope[c'] = sum_h R^T gk[row, h, dn + c']
      const int npair = a.dr / 2;
      for (int pr = lane; pr < npair; pr += 32) {
        const float cs = a.cos_[(size_t)pos * npair + pr], sn = a.sin_[(size_t)pos * npair + pr];
        float gr = 0.f, gi = 0.f;
        for (int h = 0; h < a.H; ++h) {
          const bf16* g = a.gk + ((size_t)row * a.H + h) * HD + a.dn + 2 * pr;
          const float a0 = __bfloat162float(g[0]), a1 = __bfloat162float(g[1]);
          gr += a0 * cs + a1 * sn;
          gi += -a0 * sn + a1 * cs;
        }
        *reinterpret_cast<__nv_bfloat162*>(a.g_kr + (size_t)row * a.ld_gkr + 2 * pr) =
            __floats2bfloat162_rn(gr, gi);
      }
      continue;
    }
    const int which = slot % 2, h = slot / 2;
    const int c0 = lane * EPL;
    const bool nope = c0 < a.dn;
    // k rope lanes are handled by the extra slot: they only join the reductions
    const bool skip = (which == 1 && !nope);
    const bf16* gsrc = (which == 0 ? a.gq : a.gk) + ((size_t)row * a.H + h) * HD + c0;
    float g[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) g[e] = skip ? 0.f : __bfloat162float(gsrc[e]);
    const bf16* src = which == 0 ? a.qb + (size_t)row * a.H * HD + h * HD + c0
                                 : a.kvb + (size_t)row * a.H * (a.dn + a.dv) + h * (a.dn + a.dv) + c0;
    float x[EPL];
    float ss = 0.f, ux = 0.f;
    const float* gain = (which == 0 ? a.qg : a.kg) + c0;
    if (nope) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        x[e] = __bfloat162float(src[e]);
        ss += x[e] * x[e];
        ux += g[e] * gain[e] * x[e];
      }
    }
    ss = warp_sum(ss);
    ux = warp_sum(ux);
    float gx[EPL];
    if (nope) {
      const float r = rsqrtf(ss * inv_dn + a.eps);
      const float c3 = ux * inv_dn * r * r * r;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        gx[e] = g[e] * gain[e] * r - x[e] * c3;
        acc[which * a.dn + c0 + e] += g[e] * x[e] * r;
      }
    } else if (!skip) {
      const int pr = (c0 - a.dn) / 2;
#pragma unroll
      for (int e = 0; e < EPL; e += 2) {
        const float cs = a.cos_[(size_t)pos * (a.dr / 2) + pr + e / 2];
        const float sn = a.sin_[(size_t)pos * (a.dr / 2) + pr + e / 2];
        gx[e] = g[e] * cs + g[e + 1] * sn;
        gx[e + 1] = -g[e] * sn + g[e + 1] * cs;
      }
    }
    if (!skip) {
      bf16* dst = which == 0
                      ? a.g_qb + (size_t)row * a.H * HD + h * HD + c0
                      : a.g_kvb + (size_t)row * a.H * (a.dn + a.dv) + h * (a.dn + a.dv) + c0;
#pragma unroll
      for (int e = 0; e < EPL; e += 2)
        *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(gx[e], gx[e + 1]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * a.dn; c += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < ROW_WARPS; ++w) t += smem_acc[(size_t)w * 2 * a.dn + c];
    a.partial[(size_t)blockIdx.x * 2 * a.dn + c] = t;
  }
}

// Wide variant of the backward, laid out like the wide forward: a lane owns 8 consecutive
// channels, a head is HD / 8 lanes, a warp handles 32 / (HD / 8) heads at once.  A unit of work
// is a row with all its heads, query and key side (a loop over groups of heads when H is larger
// than a warp holds), so that the shared rope key's gradient -- the sum over heads of the rotated
// key gradient -- is formed in registers, in a fixed order, and written once.  The gains'
// gradients accumulate in registers over a warp's rows and are summed over lane groups,
// warps (shared memory) and CTAs (partial buffer) in fixed orders as well.
template <int HD>
__global__ void __launch_bounds__(ROW_THREADS) qkprep_bwd_wide_kernel(const PrepArgs a) {
  constexpr int LPH = HD / 8;            // lanes per head: 8 or 16
  constexpr int UPW = 32 / LPH;          // heads per warp pass: 4 or 2
  extern __shared__ float smem_acc[];    // [ROW_WARPS][2][dn]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPH, c0 = (lane % LPH) * 8;
  const bool nope = c0 < a.dn;
  const float inv_dn = 1.f / a.dn;
  const int kvw = a.H * (a.dn + a.dv);
  const int half_dr = a.dr / 2;
  float accq[8], acck[8], gain_q[8], gain_k[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) accq[e] = acck[e] = gain_q[e] = gain_k[e] = 0.f;
  if (nope) {
    const float4 q0 = ld4(a.qg + c0), q1 = ld4(a.qg + c0 + 4);
    const float4 k0 = ld4(a.kg + c0), k1 = ld4(a.kg + c0 + 4);
    gain_q[0] = q0.x; gain_q[1] = q0.y; gain_q[2] = q0.z; gain_q[3] = q0.w;
    gain_q[4] = q1.x; gain_q[5] = q1.y; gain_q[6] = q1.z; gain_q[7] = q1.w;
    gain_k[0] = k0.x; gain_k[1] = k0.y; gain_k[2] = k0.z; gain_k[3] = k0.w;
    gain_k[4] = k1.x; gain_k[5] = k1.y; gain_k[6] = k1.z; gain_k[7] = k1.w;
  }
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    float cs[4] = {0.f, 0.f, 0.f, 0.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
    if (!nope) {
      const size_t ro = (size_t)(row % a.L) * half_dr + (c0 - a.dn) / 2;
      const float4 c4 = ld4(a.cos_ + ro), s4 = ld4(a.sin_ + ro);
      cs[0] = c4.x; cs[1] = c4.y; cs[2] = c4.z; cs[3] = c4.w;
      sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
    }
    float kr_sum[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) kr_sum[e] = 0.f;
    for (int hb = 0; hb < a.H; hb += UPW) {
      const int h = hb + sub;
      const bool live = h < a.H;
      // all four loads of the pass (q and k side) are issued before any of them is used
      uint4 raw_g[2], raw_x[2];
      raw_g[0] = raw_g[1] = raw_x[0] = raw_x[1] = make_uint4(0u, 0u, 0u, 0u);
      if (live) {
        const size_t go = ((size_t)row * a.H + h) * HD + c0;
        raw_g[0] = *reinterpret_cast<const uint4*>(a.gq + go);
        raw_g[1] = *reinterpret_cast<const uint4*>(a.gk + go);
        if (nope) {
          raw_x[0] = *reinterpret_cast<const uint4*>(a.qb + (size_t)row * a.H * HD + h * HD + c0);
          raw_x[1] = *reinterpret_cast<const uint4*>(a.kvb + (size_t)row * kvw +
                                                     h * (a.dn + a.dv) + c0);
        }
      }
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        float g[8], x[8];
        unpack8(raw_g[which], g);
        unpack8(raw_x[which], x);
        float ss = 0.f, ux = 0.f;
        if (nope) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            ss += x[e] * x[e];
            ux += g[e] * (which == 0 ? gain_q[e] : gain_k[e]) * x[e];
          }
        }
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) {   // reduction inside the head's lane group
          ss += __shfl_xor_sync(0xffffffffu, ss, o);
          ux += __shfl_xor_sync(0xffffffffu, ux, o);
        }
        float gx[8];
        if (nope) {
          const float r = rsqrtf(ss * inv_dn + a.eps);
          const float c3 = ux * inv_dn * r * r * r;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float gn = which == 0 ? gain_q[e] : gain_k[e];
            gx[e] = g[e] * gn * r - x[e] * c3;
            const float ga = g[e] * x[e] * r;     // zero for a head that is not live
            if (which == 0) accq[e] += ga;
            else acck[e] += ga;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            gx[e] = g[e] * cs[e / 2] + g[e + 1] * sn[e / 2];
            gx[e + 1] = -g[e] * sn[e / 2] + g[e + 1] * cs[e / 2];
          }
          if (which == 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) kr_sum[e] += gx[e];
          }
        }
        if (live && (which == 0 || nope)) {
          bf16* dst = which == 0 ? a.g_qb + (size_t)row * a.H * HD + h * HD + c0
                                 : a.g_kvb + (size_t)row * kvw + h * (a.dn + a.dv) + c0;
          *reinterpret_cast<uint4*>(dst) = pack8(gx);
        }
      }
    }
    // sum of the rotated key gradient over the heads of a warp pass (lane groups)
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int o = LPH; o < 32; o <<= 1) kr_sum[e] += __shfl_xor_sync(0xffffffffu, kr_sum[e], o);
    if (!nope && sub == 0)
      *reinterpret_cast<uint4*>(a.g_kr + (size_t)row * a.ld_gkr + (c0 - a.dn)) = pack8(kr_sum);
  }
  // gains' gradients: lane groups -> warp -> CTA, fixed orders
#pragma unroll
  for (int e = 0; e < 8; ++e)
#pragma unroll
    for (int o = LPH; o < 32; o <<= 1) {
      accq[e] += __shfl_xor_sync(0xffffffffu, accq[e], o);
      acck[e] += __shfl_xor_sync(0xffffffffu, acck[e], o);
    }
  float* acc = smem_acc + (size_t)warp * 2 * a.dn;
  if (nope && sub == 0) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      acc[c0 + e] = accq[e];
      acc[a.dn + c0 + e] = acck[e];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * a.dn; c += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < ROW_WARPS; ++w) t += smem_acc[(size_t)w * 2 * a.dn + c];
    a.partial[(size_t)blockIdx.x * 2 * a.dn + c] = t;
  }
}

// ---------------------------------------------------------------------------
// Elementwise: output gate, SituAndMul, gated residual add
// ---------------------------------------------------------------------------
struct EwArgs {
  const bf16 *a0, *da0;    // o / gate-half / y
  const bf16 *b0, *db0;    // g / up-half
  const float *res, *dres; // scale_add: residual
  const float* gate;       // scale_add: per-column gate
  bf16 *out, *dout;
  float *fout, *dfout;     // scale_add: fp32 output
  const bf16* gout;        // bwd: grad of out (bf16)
  const float* gfout;      // bwd: grad of fp32 out
  bf16 *ga, *gb;           // bwd: grads of a0 / b0
  float* partial;          // bwd (scale_add): [grid, D]
  int rows, D, ld_a, ld_b, ld_o, ld_ga, ld_gb;
  float beta, lbeta;
  int has_lbeta, has_t;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(ROW_THREADS) outgate_fwd_kernel(const EwArgs a) {
  const long n4 = (long)a.rows * (a.D / 4);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long)gridDim.x * blockDim.x) {
    const int row = (int)(i / (a.D / 4)), c = (int)(i % (a.D / 4)) * 4;
    const float4 o = ld4(a.a0 + (size_t)row * a.ld_a + c), z = ld4(a.b0 + (size_t)row * a.ld_b + c);
    const float4 s = make_float4(sigmoidf_(z.x), sigmoidf_(z.y), sigmoidf_(z.z), sigmoidf_(z.w));
    st4(a.out + (size_t)row * a.ld_o + c, o * s);
    if (a.has_t) {
      const float4 d_o = ld4(a.da0 + (size_t)row * a.ld_a + c);
      const float4 dz = ld4(a.db0 + (size_t)row * a.ld_b + c);
      const float4 one = make_float4(1.f - s.x, 1.f - s.y, 1.f - s.z, 1.f - s.w);
      st4(a.dout + (size_t)row * a.ld_o + c, d_o * s + o * s * one * dz);
    }
  }
}

__global__ void __launch_bounds__(ROW_THREADS) outgate_bwd_kernel(const EwArgs a) {
  const long n4 = (long)a.rows * (a.D / 4);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long)gridDim.x * blockDim.x) {
    const int row = (int)(i / (a.D / 4)), c = (int)(i % (a.D / 4)) * 4;
    const float4 o = ld4(a.a0 + (size_t)row * a.ld_a + c), z = ld4(a.b0 + (size_t)row * a.ld_b + c);
    const float4 g = ld4(a.gout + (size_t)row * a.ld_o + c);
    const float4 s = make_float4(sigmoidf_(z.x), sigmoidf_(z.y), sigmoidf_(z.z), sigmoidf_(z.w));
    const float4 one = make_float4(1.f - s.x, 1.f - s.y, 1.f - s.z, 1.f - s.w);
    st4(a.ga + (size_t)row * a.ld_ga + c, g * s);
    st4(a.gb + (size_t)row * a.ld_gb + c, g * o * s * one);
  }
}

// situ(g) = beta tanh(g/beta) sigmoid(g); up' = lbeta tanh(up/lbeta).  The hyperbolic
// tangent is the hardware approximation (one MUFU op, error below bf16 resolution) and the
// sigmoid is written through it, sigmoid(x) = 0.5 tanh(x / 2) + 0.5: three special-function
// ops per element, so the kernels below stay memory-bound.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void situ1(float g, float u, float beta, float inv_beta, float lbeta,
                                      float inv_lbeta, int has_lb, float& a, float& da_dg,
                                      float& up, float& dup_du) {
  const float th = tanh_fast(g * inv_beta), sg = fmaf(0.5f, tanh_fast(0.5f * g), 0.5f);
  a = beta * th * sg;
  da_dg = (1.f - th * th) * sg + beta * th * sg * (1.f - sg);
  if (has_lb) {
    const float tu = tanh_fast(u * inv_lbeta);
    up = lbeta * tu;
    dup_du = 1.f - tu * tu;
  } else {
    up = u;
    dup_du = 1.f;
  }
}

// a0 = [gate | up] rows of width 2*D (up at column offset ld_b), out width D.
// VEC elements per thread and access (8 = 16-byte accesses, 2 = any even layout).
template <int VEC>
__global__ void __launch_bounds__(ROW_THREADS) situ_fwd_kernel(const EwArgs a) {
  const int per_row = a.D / VEC;
  const int n = a.rows * per_row;
  const float inv_beta = 1.f / a.beta, inv_lbeta = a.has_lbeta ? 1.f / a.lbeta : 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int row = i / per_row, c = (i - row * per_row) * VEC;
    const size_t ia = (size_t)row * a.ld_a + c, io = (size_t)row * a.ld_o + c;
    float g[VEC], u[VEC], dg[VEC], du[VEC], y[VEC], dy[VEC];
    if (VEC == 8) {
      unpack8(*reinterpret_cast<const uint4*>(a.a0 + ia), g);
      unpack8(*reinterpret_cast<const uint4*>(a.b0 + ia), u);
      if (a.has_t) {
        unpack8(*reinterpret_cast<const uint4*>(a.da0 + ia), dg);
        unpack8(*reinterpret_cast<const uint4*>(a.db0 + ia), du);
      }
    } else {
      const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(a.a0 + ia);
      const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(a.b0 + ia);
      g[0] = __low2float(g2); g[1] = __high2float(g2);
      u[0] = __low2float(u2); u[1] = __high2float(u2);
      if (a.has_t) {
        const __nv_bfloat162 dg2 = *reinterpret_cast<const __nv_bfloat162*>(a.da0 + ia);
        const __nv_bfloat162 du2 = *reinterpret_cast<const __nv_bfloat162*>(a.db0 + ia);
        dg[0] = __low2float(dg2); dg[1] = __high2float(dg2);
        du[0] = __low2float(du2); du[1] = __high2float(du2);
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float av, dav, up, dup;
      situ1(g[e], u[e], a.beta, inv_beta, a.lbeta, inv_lbeta, a.has_lbeta, av, dav, up, dup);
      y[e] = av * up;
      dy[e] = a.has_t ? dav * dg[e] * up + av * dup * du[e] : 0.f;
    }
    if (VEC == 8) {
      *reinterpret_cast<uint4*>(a.out + io) = pack8(y);
      if (a.has_t) *reinterpret_cast<uint4*>(a.dout + io) = pack8(dy);
    } else {
      *reinterpret_cast<__nv_bfloat162*>(a.out + io) = __floats2bfloat162_rn(y[0], y[1]);
      if (a.has_t)
        *reinterpret_cast<__nv_bfloat162*>(a.dout + io) = __floats2bfloat162_rn(dy[0], dy[1]);
    }
  }
}

template <int VEC>
__global__ void __launch_bounds__(ROW_THREADS) situ_bwd_kernel(const EwArgs a) {
  const int per_row = a.D / VEC;
  const int n = a.rows * per_row;
  const float inv_beta = 1.f / a.beta, inv_lbeta = a.has_lbeta ? 1.f / a.lbeta : 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int row = i / per_row, c = (i - row * per_row) * VEC;
    const size_t ia = (size_t)row * a.ld_a + c, io = (size_t)row * a.ld_o + c;
    const size_t ig = (size_t)row * a.ld_ga + c;
    float g[VEC], u[VEC], go[VEC], gg[VEC], gu[VEC];
    if (VEC == 8) {
      unpack8(*reinterpret_cast<const uint4*>(a.a0 + ia), g);
      unpack8(*reinterpret_cast<const uint4*>(a.b0 + ia), u);
      unpack8(*reinterpret_cast<const uint4*>(a.gout + io), go);
    } else {
      const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(a.a0 + ia);
      const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(a.b0 + ia);
      const __nv_bfloat162 go2 = *reinterpret_cast<const __nv_bfloat162*>(a.gout + io);
      g[0] = __low2float(g2); g[1] = __high2float(g2);
      u[0] = __low2float(u2); u[1] = __high2float(u2);
      go[0] = __low2float(go2); go[1] = __high2float(go2);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float av, dav, up, dup;
      situ1(g[e], u[e], a.beta, inv_beta, a.lbeta, inv_lbeta, a.has_lbeta, av, dav, up, dup);
      gg[e] = go[e] * dav * up;
      gu[e] = go[e] * av * dup;
    }
    if (VEC == 8) {
      *reinterpret_cast<uint4*>(a.ga + ig) = pack8(gg);
      *reinterpret_cast<uint4*>(a.gb + ig) = pack8(gu);
    } else {
      *reinterpret_cast<__nv_bfloat162*>(a.ga + ig) = __floats2bfloat162_rn(gg[0], gg[1]);
      *reinterpret_cast<__nv_bfloat162*>(a.gb + ig) = __floats2bfloat162_rn(gu[0], gu[1]);
    }
  }
}

// fout = res + y * gate   (fp32 residual stream; y bf16)
__global__ void __launch_bounds__(ROW_THREADS) scale_add_fwd_kernel(const EwArgs a) {
  const long n4 = (long)a.rows * (a.D / 4);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (long)gridDim.x * blockDim.x) {
    const int row = (int)(i / (a.D / 4)), c = (int)(i % (a.D / 4)) * 4;
    const size_t o = (size_t)row * a.D + c;
    const float4 g = ld4(a.gate + c);
    float4 v = ld4(a.a0 + o) * g;
    if (a.res) v = v + ld4(a.res + o);
    st4(a.fout + o, v);
    if (a.has_t) {
      float4 dv = ld4(a.da0 + o) * g;
      if (a.dres) dv = dv + ld4(a.dres + o);
      st4(a.dfout + o, dv);
    }
  }
}

// g_y = g * gate (bf16); partial[c] += g * y   (g_res is g itself)
__global__ void __launch_bounds__(ROW_THREADS) scale_add_bwd_kernel(const EwArgs a) {
  extern __shared__ float smem_acc[];  // [ROW_WARPS][D]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* acc = smem_acc + (size_t)warp * a.D;
  for (int c = lane; c < a.D; c += 32) acc[c] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    for (int c = lane * 4; c < a.D; c += 128) {
      const size_t o = (size_t)row * a.D + c;
      const float4 g = ld4(a.gfout + o);
      st4(a.ga + o, g * ld4(a.gate + c));
      st4(acc + c, ld4(acc + c) + g * ld4(a.a0 + o));
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < a.D; c += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < ROW_WARPS; ++w) t += smem_acc[(size_t)w * a.D + c];
    a.partial[(size_t)blockIdx.x * a.D + c] = t;
  }
}

static int ew_grid(long n) {
  long g = (n + ROW_THREADS - 1) / ROW_THREADS;
  return (int)(g < 1 ? 1 : (g > 148 * 8 ? 148 * 8 : g));
}

}  // namespace imf

using namespace imf;

// ptrs (per segment s in 0..nseg-1, 8 pointers each):
//   x, dx, gain, out, dout, gy, gx, partial ; dims[s] = {D, ld_x, ld_o}
extern "C" int imf_rmsnorm_seg(void** ptrs, const int* dims, int nseg, int rows, float eps,
                               int has_t, int bwd, void* stream) {
  if (nseg < 1 || nseg > 2 || rows <= 0) return -1;
  NormArgs a;
  int maxd = 0;
  for (int s = 0; s < nseg; ++s) {
    NormSeg& g = a.seg[s];
    void** p = ptrs + 8 * s;
    g.x = (const bf16*)p[0];
    g.dx = (const bf16*)p[1];
    g.gain = (const float*)p[2];
    g.out = (bf16*)p[3];
    g.dout = (bf16*)p[4];
    g.gy = (const bf16*)p[5];
    g.gx = (bf16*)p[6];
    g.partial = (float*)p[7];
    g.D = dims[3 * s];
    g.ld_x = dims[3 * s + 1];
    g.ld_o = dims[3 * s + 2];
    if (g.D % 4 || g.ld_x % 4 || g.ld_o % 4) return -1;
    maxd = g.D > maxd ? g.D : maxd;
  }
  if (nseg == 1) a.seg[1] = a.seg[0];
  a.rows = rows;
  a.eps = eps;
  a.has_t = has_t;
  dim3 grid(row_grid(rows), nseg);
  cudaStream_t st = (cudaStream_t)stream;
  if (!bwd) {
    rmsnorm_seg_fwd_kernel<<<grid, ROW_THREADS, 0, st>>>(a);
  } else {
    const size_t smem = (size_t)ROW_WARPS * maxd * sizeof(float);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(rmsnorm_seg_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return -3;
    rmsnorm_seg_bwd_kernel<<<grid, ROW_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ptrs: 0 qb, 1 dqb, 2 kvb, 3 dkvb, 4 kr, 5 dkr, 6 cos, 7 sin, 8 qg, 9 kg, 10 q, 11 dq, 12 k,
//       13 dk, 14 gq, 15 gk, 16 g_qb, 17 g_kvb, 18 g_kr, 19 partial
extern "C" int imf_qkprep(void** p, int rows, int L, int H, int dn, int dr, int dv, int ld_kr,
                          int ld_gkr, float eps, int has_t, int bwd, void* stream) {
  const int HD = dn + dr;
  if ((HD != 64 && HD != 128) || rows <= 0) return -1;
  const int epl = HD / 32;
  if (dn % epl || dr % 2 || (dn + dv) % 2 || ld_kr % 2) return -1;
  PrepArgs a;
  a.qb = (const bf16*)p[0]; a.dqb = (const bf16*)p[1];
  a.kvb = (const bf16*)p[2]; a.dkvb = (const bf16*)p[3];
  a.kr = (const bf16*)p[4]; a.dkr = (const bf16*)p[5];
  a.cos_ = (const float*)p[6]; a.sin_ = (const float*)p[7];
  a.qg = (const float*)p[8]; a.kg = (const float*)p[9];
  a.q = (bf16*)p[10]; a.dq = (bf16*)p[11]; a.k = (bf16*)p[12]; a.dk = (bf16*)p[13];
  a.gq = (const bf16*)p[14]; a.gk = (const bf16*)p[15];
  a.g_qb = (bf16*)p[16]; a.g_kvb = (bf16*)p[17]; a.g_kr = (bf16*)p[18];
  a.partial = (float*)p[19];
  a.rows = rows; a.L = L; a.H = H; a.dn = dn; a.dr = dr; a.dv = dv;
  a.ld_kr = ld_kr; a.ld_gkr = ld_gkr; a.eps = eps; a.has_t = has_t;
  cudaStream_t st = (cudaStream_t)stream;
  if (!bwd) {
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool wide = dn % 8 == 0 && dr % 8 == 0 && (dn + dv) % 8 == 0 && ld_kr % 8 == 0 &&
                      al16(a.qb) && al16(a.kvb) && al16(a.kr) && al16(a.q) && al16(a.k) &&
                      al16(a.cos_) && al16(a.sin_) && al16(a.qg) && al16(a.kg) &&
                      (!has_t || (al16(a.dqb) && al16(a.dkvb) && al16(a.dkr) && al16(a.dq) && al16(a.dk)));
    if (wide) {
      const int upw = HD == 64 ? 4 : 2;
      const int grid = row_grid((rows * H * 2 + upw - 1) / upw);
      if (HD == 64) qkprep_fwd_wide_kernel<64><<<grid, ROW_THREADS, 0, st>>>(a);
      else qkprep_fwd_wide_kernel<128><<<grid, ROW_THREADS, 0, st>>>(a);
    } else {
      const int grid = row_grid(rows * H * 2);
      if (epl == 2) qkprep_fwd_kernel<2><<<grid, ROW_THREADS, 0, st>>>(a);
      else qkprep_fwd_kernel<4><<<grid, ROW_THREADS, 0, st>>>(a);
    }
  } else {
    const int grid = row_grid(rows);     // partial buffers are sized by imf_row_grid(rows)
    const size_t smem = (size_t)ROW_WARPS * 2 * dn * sizeof(float);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool wide = dn % 8 == 0 && dr % 8 == 0 && (dn + dv) % 8 == 0 && ld_gkr % 8 == 0 &&
                      al16(a.qb) && al16(a.kvb) && al16(a.gq) && al16(a.gk) && al16(a.g_qb) &&
                      al16(a.g_kvb) && al16(a.g_kr) && al16(a.cos_) && al16(a.sin_) &&
                      al16(a.qg) && al16(a.kg);
    if (wide && HD == 64) qkprep_bwd_wide_kernel<64><<<grid, ROW_THREADS, smem, st>>>(a);
    else if (wide && HD == 128) qkprep_bwd_wide_kernel<128><<<grid, ROW_THREADS, smem, st>>>(a);
    else if (epl == 2) qkprep_bwd_kernel<2><<<grid, ROW_THREADS, smem, st>>>(a);
    else qkprep_bwd_kernel<4><<<grid, ROW_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// op: 0 out-gate, 1 situ, 2 scale-add.
// ptrs: 0 a0, 1 da0, 2 b0, 3 db0, 4 res, 5 dres, 6 gate, 7 out, 8 dout, 9 fout, 10 dfout,
//       11 gout, 12 gfout, 13 ga, 14 gb, 15 partial
// dims: rows, D, ld_a, ld_b, ld_o, ld_ga, ld_gb
extern "C" int imf_elementwise(int op, void** p, const int* dims, float beta, float lbeta,
                               int has_lbeta, int has_t, int bwd, void* stream) {
  EwArgs a;
  a.a0 = (const bf16*)p[0]; a.da0 = (const bf16*)p[1];
  a.b0 = (const bf16*)p[2]; a.db0 = (const bf16*)p[3];
  a.res = (const float*)p[4]; a.dres = (const float*)p[5];
  a.gate = (const float*)p[6];
  a.out = (bf16*)p[7]; a.dout = (bf16*)p[8];
  a.fout = (float*)p[9]; a.dfout = (float*)p[10];
  a.gout = (const bf16*)p[11]; a.gfout = (const float*)p[12];
  a.ga = (bf16*)p[13]; a.gb = (bf16*)p[14];
  a.partial = (float*)p[15];
  a.rows = dims[0]; a.D = dims[1]; a.ld_a = dims[2]; a.ld_b = dims[3]; a.ld_o = dims[4];
  a.ld_ga = dims[5]; a.ld_gb = dims[6];
  a.beta = beta; a.lbeta = lbeta; a.has_lbeta = has_lbeta; a.has_t = has_t;
  if (a.rows <= 0 || a.D <= 0 || a.D % 4) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  if (op == 0) {
    if (a.ld_a % 4 || a.ld_b % 4 || a.ld_o % 4) return -1;
    const int grid = ew_grid((long)a.rows * a.D / 4);
    if (!bwd) outgate_fwd_kernel<<<grid, ROW_THREADS, 0, st>>>(a);
    else {
      if (a.ld_ga % 4 || a.ld_gb % 4) return -1;
      outgate_bwd_kernel<<<grid, ROW_THREADS, 0, st>>>(a);
    }
  } else if (op == 1) {
    if (a.ld_a % 2 || a.ld_o % 2 || (long)a.rows * a.D / 2 > 0x7fffffffL) return -1;
    // 16-byte accesses when every row start and the column split are 16-byte aligned
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    bool v8 = a.D % 8 == 0 && a.ld_a % 8 == 0 && a.ld_o % 8 == 0 && al16(a.a0) && al16(a.b0);
    if (!bwd) v8 = v8 && al16(a.out) && (!a.has_t || (al16(a.da0) && al16(a.db0) && al16(a.dout)));
    else v8 = v8 && a.ld_ga % 8 == 0 && al16(a.gout) && al16(a.ga) && al16(a.gb);
    const int grid = ew_grid((long)a.rows * a.D / (v8 ? 8 : 2));
    if (!bwd) {
      if (v8) situ_fwd_kernel<8><<<grid, ROW_THREADS, 0, st>>>(a);
      else situ_fwd_kernel<2><<<grid, ROW_THREADS, 0, st>>>(a);
    } else {
      if (v8) situ_bwd_kernel<8><<<grid, ROW_THREADS, 0, st>>>(a);
      else situ_bwd_kernel<2><<<grid, ROW_THREADS, 0, st>>>(a);
    }
  } else if (op == 2) {
    if (!bwd) {
      scale_add_fwd_kernel<<<ew_grid((long)a.rows * a.D / 4), ROW_THREADS, 0, st>>>(a);
    } else {
      const size_t smem = (size_t)ROW_WARPS * a.D * sizeof(float);
      if (smem > 48 * 1024 &&
          cudaFuncSetAttribute(scale_add_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem) != cudaSuccess)
        return -3;
      scale_add_bwd_kernel<<<row_grid(a.rows), ROW_THREADS, smem, st>>>(a);
    }
  } else {
    return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------
// Column sums of the per-CTA partial gradients that the row kernels leave behind (gains,
// gates, score weights): up to COLSUM_MAX vectors in ONE launch, each summed over its
// partial rows in a fixed order and written -- or accumulated -- straight into its
// destination (a parameter's gradient buffer).  Replaces one framework reduction plus one
// gradient-accumulation add per vector.
// ---------------------------------------------------------------------------
namespace imf {
constexpr int COLSUM_MAX = 12;
struct ColSumEntry {
  const float* part;     // first element of the column block: part[g * stride + d]
  float* dst;            // [D]
  int g, D, stride, accumulate;
};
struct ColSumArgs {
  ColSumEntry e[COLSUM_MAX];
};
// block = 32 columns x 32 row groups: thread (x, y) adds rows y, y + 32, ... of its column
// (four loads in flight: the partial rows are few and the time is load latency), the group
// sums are added in a fixed order
constexpr int COLSUM_GROUPS = 32;
__global__ void __launch_bounds__(32 * COLSUM_GROUPS)
colsum_kernel(const __grid_constant__ ColSumArgs a) {
  const ColSumEntry e = a.e[blockIdx.y];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + x;
  __shared__ float s_part[COLSUM_GROUPS][32];
  float acc = 0.f;
  if (d < e.D) {
#pragma unroll 4
    for (int i = y; i < e.g; i += COLSUM_GROUPS) acc += e.part[(size_t)i * e.stride + d];
  }
  s_part[y][x] = acc;
  __syncthreads();
  if (y == 0 && d < e.D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < COLSUM_GROUPS; ++k) t += s_part[k][x];
    e.dst[d] = e.accumulate ? e.dst[d] + t : t;
  }
}
}  // namespace imf

// entries: host array of n records {const float* part, float* dst, int g, D, stride, accumulate}
extern "C" int imf_colsum(const void* entries, int n, void* stream) {
  if (n <= 0) return 0;
  if (n > imf::COLSUM_MAX) return -1;
  imf::ColSumArgs a;
  int maxd = 0;
  const imf::ColSumEntry* src = static_cast<const imf::ColSumEntry*>(entries);
  for (int i = 0; i < imf::COLSUM_MAX; ++i) {
    a.e[i] = src[i < n ? i : 0];
    if (i < n && a.e[i].D > maxd) maxd = a.e[i].D;
    if (i < n && (a.e[i].g <= 0 || a.e[i].D <= 0)) return -1;
  }
  imf::colsum_kernel<<<dim3((maxd + 31) / 32, n), 32 * imf::COLSUM_GROUPS, 0,
                       (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

