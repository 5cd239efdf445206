// Fused "residual update -> attention-residual re-mix -> RMSNorm" row kernel
// with forward-mode tangent, and its reverse-mode gradient.
//
//   pfx = res + y * gate                       (fp32 residual stream)
//   v_j = {snap_1 .. snap_{J-1}, pfx};  r_j = rsqrt(mean v_j^2 + eps)
//   s_j = r_j <v_j, w>;  p = softmax_j(s);  h = sum_j p_j v_j     (if w given)
//   n   = h * rsqrt(mean h^2 + eps) * gain                        (bf16 out)
//
// Replaces, in one launch, the reference's gate-add, attention-residual and
// RMSNorm kernels plus the torch.stack of the candidates (reference
// models/triton_attn_res_jvp.py:44-209, models/triton_mla_block_jvp.py:506-557,
// models/triton_block_jvp.py:99-168).  Candidates are read through a pointer
// list, never stacked.
#include "rowops_common.cuh"

namespace imf {

struct ResNormArgs {
  const float* res;
  const float* dres;
  const __nv_bfloat16* y;
  const __nv_bfloat16* dy;
  const float* gate;
  const float* snaps[MAX_CANDS];
  const float* dsnaps[MAX_CANDS];   // forward: tangents; backward: gradients added to g_snaps
  int nsnap;
  const float* w;
  const float* gain;
  float eps;
  float* pfx;
  float* dpfx;
  __nv_bfloat16* n;
  __nv_bfloat16* dn;
  int rows;
  int has_t;
  // backward only
  const __nv_bfloat16* gn;
  const float* g_pfx_ext;
  float* g_res;
  __nv_bfloat16* g_y;
  float* g_snaps[MAX_CANDS];
  float* partial;  // [grid, 3, D]: g_gain, g_w, g_gate
};

template <int NV>
__global__ void __launch_bounds__(ROW_THREADS, NV <= 2 ? 4 : 1) resnorm_fwd_kernel(const ResNormArgs a) {
  constexpr int D = NV * 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_d = 1.f / D;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * D + lane * 4;
    float4 pf[NV], dpf[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const size_t o = base + i * 128;
      pf[i] = a.res ? ld4(a.res + o) : f4zero();
      dpf[i] = (a.has_t && a.dres) ? ld4(a.dres + o) : f4zero();
      if (a.y) {
        const float4 g = ld4(a.gate + lane * 4 + i * 128);
        pf[i] = pf[i] + ld4(a.y + o) * g;
        if (a.has_t) dpf[i] = dpf[i] + ld4(a.dy + o) * g;
        st4(a.pfx + o, pf[i]);
        if (a.has_t) st4(a.dpfx + o, dpf[i]);
      }
    }
    if (a.w) {
      // One pass over the candidates with a running maximum, for the value and its tangent:
      //   s_j = r_j <v_j, w>,  ds_j = r_j <dv_j, w> - r_j^3 <v_j, w> <v_j, dv_j> / D,
      //   e_j = exp(s_j - m):  H = sum e_j v_j,  Hd = sum e_j (ds_j v_j + dv_j),
      //   S = sum e_j,  Sd = sum e_j ds_j;   h = H / S,  dh = Hd / S - (Sd / S) h.
      // The running prefix (already in registers) is the first candidate, so pf / dpf turn
      // into H / Hd and every snapshot and snapshot tangent is read exactly once.
      auto score = [&](const float4(&v)[NV], const float4(&dv)[NV], float& sc, float& dsc) {
        float ss = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const float4 w4 = ld4(a.w + lane * 4 + i * 128);
          ss += dot4(v[i], v[i]);
          s1 += dot4(v[i], w4);
          s2 += dot4(dv[i], w4);
          s3 += dot4(v[i], dv[i]);
        }
        ss = warp_sum(ss);
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        s3 = warp_sum(s3) * inv_d;
        const float r = rsqrtf(ss * inv_d + a.eps);
        sc = r * s1;
        dsc = r * s2 - r * r * r * s1 * s3;
      };
      float m, ds0;
      score(pf, dpf, m, ds0);
      float S = 1.f, Sd = ds0;
#pragma unroll
      for (int i = 0; i < NV; ++i) dpf[i] = fma4(pf[i], ds0, dpf[i]);
#pragma unroll 1
      for (int j = 0; j < a.nsnap; ++j) {
        float4 v[NV], dv[NV];
        const bool has_dv = a.has_t && a.dsnaps[j];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const size_t o = base + i * 128;
          v[i] = ld4(a.snaps[j] + o);
          dv[i] = has_dv ? ld4(a.dsnaps[j] + o) : f4zero();
        }
        float sc, dsc;
        score(v, dv, sc, dsc);
        const float mn = fmaxf(m, sc);
        const float al = __expf(m - mn), e = __expf(sc - mn);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          pf[i] = fma4(v[i], e, pf[i] * al);
          dpf[i] = fma4(fma4(v[i], dsc, dv[i]), e, dpf[i] * al);
        }
        S = S * al + e;
        Sd = Sd * al + e * dsc;
        m = mn;
      }
      const float inv = 1.f / S, sd = Sd * inv;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        pf[i] = pf[i] * inv;
        dpf[i] = fma4(pf[i], -sd, dpf[i] * inv);
      }
    }
    float hh = 0.f, hdh = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      hh += dot4(pf[i], pf[i]);
      if (a.has_t) hdh += dot4(pf[i], dpf[i]);
    }
    hh = warp_sum(hh);
    const float rh = rsqrtf(hh * inv_d + a.eps);
    float c2 = 0.f;
    if (a.has_t) c2 = warp_sum(hdh) * inv_d * rh * rh * rh;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const size_t o = base + i * 128;
      const float4 g = ld4(a.gain + lane * 4 + i * 128);
      st4(a.n + o, pf[i] * g * rh);
      if (a.has_t) st4(a.dn + o, fma4(pf[i], -c2, dpf[i] * rh) * g);
    }
  }
}

// Primal-only forward (guidance passes, v branch): the remix is ONE pass over the candidates
// with a running maximum, flash-softmax style,
//   h <- h exp(m - m') + exp(s_j - m') v_j,   den likewise,   h /= den at the end,
// so every snapshot is read once and no tangent registers are carried: twice the occupancy
// and about half the traffic of the two-pass kernel above.
template <int NV>
__global__ void __launch_bounds__(ROW_THREADS, NV <= 2 ? 4 : (NV <= 4 ? 3 : (NV <= 8 ? 2 : 1))) resnorm_fwd_primal_kernel(const ResNormArgs a) {
  constexpr int D = NV * 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_d = 1.f / D;
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * D + lane * 4;
    float4 pf[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const size_t o = base + i * 128;
      pf[i] = a.res ? ld4(a.res + o) : f4zero();
      if (a.y) {
        pf[i] = pf[i] + ld4(a.y + o) * ld4(a.gate + lane * 4 + i * 128);
        st4(a.pfx + o, pf[i]);
      }
    }
    if (a.w) {
      // candidate J-1 (the prefix itself) first: it is already in registers
      float ss = 0.f, s1 = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        ss += dot4(pf[i], pf[i]);
        s1 += dot4(pf[i], ld4(a.w + lane * 4 + i * 128));
      }
      float m = rsqrtf(warp_sum(ss) * inv_d + a.eps) * warp_sum(s1);
      float den = 1.f;                       // exp(s - m) of the first candidate
#pragma unroll 1
      for (int j = 0; j < a.nsnap; ++j) {
        float4 v[NV];
        ss = 0.f;
        s1 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          v[i] = ld4(a.snaps[j] + base + i * 128);
          ss += dot4(v[i], v[i]);
          s1 += dot4(v[i], ld4(a.w + lane * 4 + i * 128));
        }
        const float sc = rsqrtf(warp_sum(ss) * inv_d + a.eps) * warp_sum(s1);
        const float mn = fmaxf(m, sc);
        const float al = __expf(m - mn), pj = __expf(sc - mn);
        den = den * al + pj;
        m = mn;
#pragma unroll
        for (int i = 0; i < NV; ++i) pf[i] = fma4(v[i], pj, pf[i] * al);
      }
      const float inv = 1.f / den;
#pragma unroll
      for (int i = 0; i < NV; ++i) pf[i] = pf[i] * inv;
    }
    float hh = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) hh += dot4(pf[i], pf[i]);
    const float rh = rsqrtf(warp_sum(hh) * inv_d + a.eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const size_t o = base + i * 128;
      st4(a.n + o, pf[i] * ld4(a.gain + lane * 4 + i * 128) * rh);
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(ROW_THREADS, NV <= 2 ? 4 : 1) resnorm_bwd_kernel(const ResNormArgs a) {
  constexpr int D = NV * 128;
  extern __shared__ float smem_acc[];  // [ROW_WARPS][3][D]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_d = 1.f / D;
  float* acc = smem_acc + (size_t)warp * 3 * D;
  for (int i = lane; i < 3 * D; i += 32) acc[i] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * ROW_WARPS + warp; row < a.rows; row += gridDim.x * ROW_WARPS) {
    const size_t base = (size_t)row * D + lane * 4;
    float4 pf[NV], h[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const size_t o = base + i * 128;
      pf[i] = a.res ? ld4(a.res + o) : f4zero();
      if (a.y) pf[i] = pf[i] + ld4(a.y + o) * ld4(a.gate + lane * 4 + i * 128);
    }
    const int J = a.nsnap + 1;
    float r[MAX_CANDS], vw[MAX_CANDS], p[MAX_CANDS];
    if (a.w) {
#pragma unroll 1
      for (int j = 0; j < J; ++j) {
        float ss = 0.f, s1 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const float4 v = j < a.nsnap ? ld4(a.snaps[j] + base + i * 128) : pf[i];
          ss += dot4(v, v);
          s1 += dot4(v, ld4(a.w + lane * 4 + i * 128));
        }
        r[j] = rsqrtf(warp_sum(ss) * inv_d + a.eps);
        vw[j] = warp_sum(s1);
      }
      float mx = -INFINITY, den = 0.f;
      for (int j = 0; j < J; ++j) {
        p[j] = r[j] * vw[j];
        mx = fmaxf(mx, p[j]);
      }
      for (int j = 0; j < J; ++j) {
        p[j] = __expf(p[j] - mx);
        den += p[j];
      }
      for (int j = 0; j < J; ++j) p[j] /= den;
#pragma unroll
      for (int i = 0; i < NV; ++i) h[i] = pf[i] * p[J - 1];
#pragma unroll 1
      for (int j = 0; j < a.nsnap; ++j)
#pragma unroll
        for (int i = 0; i < NV; ++i) h[i] = fma4(ld4(a.snaps[j] + base + i * 128), p[j], h[i]);
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) h[i] = pf[i];
    }
    // RMSNorm backward: u = gn * gain; gh = rh u - h rh^3 mean(u h)
    float hh = 0.f, uh = 0.f;
    float4 u[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float4 gn = ld4(a.gn + base + i * 128);
      u[i] = gn * ld4(a.gain + lane * 4 + i * 128);
      hh += dot4(h[i], h[i]);
      uh += dot4(u[i], h[i]);
      // g_gain += gn * h * rh  (rh applied after the reduction below)
      h[i] = h[i];
    }
    hh = warp_sum(hh);
    uh = warp_sum(uh);
    const float rh = rsqrtf(hh * inv_d + a.eps);
    const float c = uh * inv_d * rh * rh * rh;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float4 gn = ld4(a.gn + base + i * 128);
      float* ag = acc + 0 * D + lane * 4 + i * 128;
      st4(ag, ld4(ag) + gn * h[i] * rh);
      h[i] = fma4(h[i], -c, u[i] * rh);  // h now holds gh
    }
    float4 gp_last[NV];  // gradient w.r.t. the prefix candidate
    if (a.w) {
      float gp[MAX_CANDS];
#pragma unroll 1
      for (int j = 0; j < J; ++j) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
          s += dot4(h[i], j < a.nsnap ? ld4(a.snaps[j] + base + i * 128) : pf[i]);
        gp[j] = warp_sum(s);
      }
      float pg = 0.f;
      for (int j = 0; j < J; ++j) pg += p[j] * gp[j];
#pragma unroll 1
      for (int j = 0; j < J; ++j) {
        const float gs = p[j] * (gp[j] - pg);
        const float c1 = gs * r[j];
        const float c3 = gs * r[j] * r[j] * r[j] * vw[j] * inv_d;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const size_t o = base + i * 128;
          const float4 v = j < a.nsnap ? ld4(a.snaps[j] + o) : pf[i];
          const float4 w4 = ld4(a.w + lane * 4 + i * 128);
          // g_v_j = p_j gh + gs (r_j w - r_j^3 <v_j,w> v_j / D)
          const float4 gv = fma4(v, -c3, fma4(w4, c1, h[i] * p[j]));
          float* aw = acc + 1 * D + lane * 4 + i * 128;
          st4(aw, fma4(v, c1, ld4(aw)));  // g_w += gs r_j v_j
          if (j < a.nsnap)   // backward: dsnaps[j], when given, is a gradient to add in
            st4(a.g_snaps[j] + o, a.dsnaps[j] ? gv + ld4(a.dsnaps[j] + o) : gv);
          else
            gp_last[i] = gv;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) gp_last[i] = h[i];
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const size_t o = base + i * 128;
      float4 g = gp_last[i];
      if (a.g_pfx_ext) g = g + ld4(a.g_pfx_ext + o);
      if (a.g_res) st4(a.g_res + o, g);
      if (a.y) {
        const float4 gate = ld4(a.gate + lane * 4 + i * 128);
        st4(a.g_y + o, g * gate);
        float* agt = acc + 2 * D + lane * 4 + i * 128;
        st4(agt, ld4(agt) + g * ld4(a.y + o));
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 3 * D; c += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < ROW_WARPS; ++w) t += smem_acc[(size_t)w * 3 * D + c];
    a.partial[(size_t)blockIdx.x * 3 * D + c] = t;
  }
}

template <int NV>
static int launch_resnorm(const ResNormArgs& a, bool bwd, cudaStream_t st) {
  const int grid = row_grid(a.rows);
  if (!bwd) {
    if (a.has_t) resnorm_fwd_kernel<NV><<<grid, ROW_THREADS, 0, st>>>(a);
    else resnorm_fwd_primal_kernel<NV><<<grid, ROW_THREADS, 0, st>>>(a);
  } else {
    const size_t smem = (size_t)ROW_WARPS * 3 * NV * 128 * sizeof(float);
    if (cudaFuncSetAttribute(resnorm_bwd_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return -3;
    resnorm_bwd_kernel<NV><<<grid, ROW_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace imf

// Number of CTAs the row kernels use for `rows` rows (size of the leading
// dimension of every `partial` buffer).
extern "C" int imf_row_grid(int rows) { return imf::row_grid(rows); }

// Forward (bwd = 0) / backward (bwd = 1).  `ptrs` layout (void*[]):
//  0 res, 1 dres, 2 y, 3 dy, 4 gate, 5 w, 6 gain, 7 pfx, 8 dpfx, 9 n, 10 dn,
//  11 gn, 12 g_pfx_ext, 13 g_res, 14 g_y, 15 partial,
//  16.. snaps[nsnap], then dsnaps[nsnap], then g_snaps[nsnap].
extern "C" int imf_resnorm(void** ptrs, int nsnap, int rows, int D, float eps, int has_t,
                           int bwd, void* stream) {
  using namespace imf;
  if (D % 128 != 0 || D > 2048 || nsnap < 0 || nsnap >= MAX_CANDS || rows <= 0) return -1;
  ResNormArgs a;
  a.res = (const float*)ptrs[0];
  a.dres = (const float*)ptrs[1];
  a.y = (const __nv_bfloat16*)ptrs[2];
  a.dy = (const __nv_bfloat16*)ptrs[3];
  a.gate = (const float*)ptrs[4];
  a.w = (const float*)ptrs[5];
  a.gain = (const float*)ptrs[6];
  a.pfx = (float*)ptrs[7];
  a.dpfx = (float*)ptrs[8];
  a.n = (__nv_bfloat16*)ptrs[9];
  a.dn = (__nv_bfloat16*)ptrs[10];
  a.gn = (const __nv_bfloat16*)ptrs[11];
  a.g_pfx_ext = (const float*)ptrs[12];
  a.g_res = (float*)ptrs[13];
  a.g_y = (__nv_bfloat16*)ptrs[14];
  a.partial = (float*)ptrs[15];
  for (int j = 0; j < MAX_CANDS; ++j) {
    a.snaps[j] = j < nsnap ? (const float*)ptrs[16 + j] : nullptr;
    a.dsnaps[j] = j < nsnap ? (const float*)ptrs[16 + nsnap + j] : nullptr;
    a.g_snaps[j] = j < nsnap ? (float*)ptrs[16 + 2 * nsnap + j] : nullptr;
  }
  a.nsnap = nsnap;
  a.eps = eps;
  a.rows = rows;
  a.has_t = has_t;
  if (a.w == nullptr && nsnap != 0) return -1;
  if (a.y != nullptr && (a.gate == nullptr || (!bwd && a.pfx == nullptr))) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D / 128) {
#define IMF_CASE(NV_) \
  case NV_:           \
    return launch_resnorm<NV_>(a, bwd != 0, st);
    IMF_CASE(1)
    IMF_CASE(2)
    IMF_CASE(3)
    IMF_CASE(4)
    IMF_CASE(6)
    IMF_CASE(8)
    IMF_CASE(12)
    IMF_CASE(16)
#undef IMF_CASE
    default:
      return -1;
  }
}
