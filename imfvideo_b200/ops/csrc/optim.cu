// Fused optimizer kernels over flat parameter arenas (fp32 master weights).
//
//   muon_momentum : buf = mu buf + c g ; dir = c g + mu buf (Nesterov) or buf
//   muon_apply    : p = p (1 - lr_i wd) - lr_i s_i Phi ;  ema = lerp(ema, p)
//   adamw         : bias-corrected AdamW with decoupled decay ; ema lerp
//
// clip[0] is the gradient-clip factor and clip[1] a skip flag (non-finite
// gradient norm), both read from device memory, so no host round trip
// separates backward from the update.  One launch covers every parameter
// of a class; per-parameter constants come from a small segment table.
// Replaces the reference's per-parameter Python loops (reference
// moonlight.py:395-469, train.py:290-298, train.py:582).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

struct Seg {          // one parameter inside an arena
  long start;         // element offset
  long numel;
  float a;            // muon_apply: 1 - lr wd        adamw: lr
  float b;            // muon_apply: lr * scale       adamw: 1 - lr wd
};

__global__ void muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf,
                                     float* __restrict__ dir, long n, float mu, int nesterov,
                                     const float* __restrict__ clip) {
  if (clip && clip[1] != 0.f) return;      // non-finite gradient: the whole step is skipped
  const float c = clip ? clip[0] : 1.f;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long)gridDim.x * blockDim.x * 4) {
    float4 gv = *reinterpret_cast<const float4*>(g + i);
    float4 bv = *reinterpret_cast<const float4*>(buf + i);
    gv.x *= c; gv.y *= c; gv.z *= c; gv.w *= c;
    bv.x = mu * bv.x + gv.x; bv.y = mu * bv.y + gv.y;
    bv.z = mu * bv.z + gv.z; bv.w = mu * bv.w + gv.w;
    *reinterpret_cast<float4*>(buf + i) = bv;
    float4 dv = bv;
    if (nesterov) {
      dv.x = gv.x + mu * bv.x; dv.y = gv.y + mu * bv.y;
      dv.z = gv.z + mu * bv.z; dv.w = gv.w + mu * bv.w;
    }
    *reinterpret_cast<float4*>(dir + i) = dv;
  }
}

template <typename UT>
__global__ void muon_apply_kernel(float* __restrict__ p, const UT* __restrict__ upd,
                                  float* __restrict__ ema, const Seg* __restrict__ segs,
                                  long upd_offset, float ema_w, const float* __restrict__ clip) {
  if (clip && clip[1] != 0.f) return;
  const Seg s = segs[blockIdx.y];
  if (((s.start | s.numel | upd_offset) & 3) == 0) {   // four elements per thread and access
    for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < s.numel;
         i += (long)gridDim.x * blockDim.x * 4) {
      const long j = s.start + i;
      float u[4];
      if constexpr (sizeof(UT) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(upd + (j - upd_offset));
        u[0] = __uint_as_float(raw.x << 16); u[1] = __uint_as_float(raw.x & 0xffff0000u);
        u[2] = __uint_as_float(raw.y << 16); u[3] = __uint_as_float(raw.y & 0xffff0000u);
      } else {
        const float4 raw = *reinterpret_cast<const float4*>(upd + (j - upd_offset));
        u[0] = raw.x; u[1] = raw.y; u[2] = raw.z; u[3] = raw.w;
      }
      float4 pv = *reinterpret_cast<float4*>(p + j);
      pv.x = pv.x * s.a - s.b * u[0]; pv.y = pv.y * s.a - s.b * u[1];
      pv.z = pv.z * s.a - s.b * u[2]; pv.w = pv.w * s.a - s.b * u[3];
      *reinterpret_cast<float4*>(p + j) = pv;
      if (ema) {
        float4 ev = *reinterpret_cast<float4*>(ema + j);
        ev.x += ema_w * (pv.x - ev.x); ev.y += ema_w * (pv.y - ev.y);
        ev.z += ema_w * (pv.z - ev.z); ev.w += ema_w * (pv.w - ev.w);
        *reinterpret_cast<float4*>(ema + j) = ev;
      }
    }
    return;
  }
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < s.numel;
       i += (long)gridDim.x * blockDim.x) {
    const long j = s.start + i;
    const float u = static_cast<float>(upd[j - upd_offset]);
    const float v = p[j] * s.a - s.b * u;
    p[j] = v;
    if (ema) ema[j] += ema_w * (v - ema[j]);
  }
}

// `t_dev` (optional): device count of applied steps, this one included; the bias
// corrections are then computed here, so a step skipped by the device-side flag never
// needs the host to roll a counter back.  [lo, hi) (absolute arena offsets, hi > lo)
// restricts the update to one rank's shard of the AdamW slice.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ ema, const Seg* __restrict__ segs, long state_offset,
                             float b1, float b2, float eps, float bias1, float bias2,
                             const float* __restrict__ clip, float ema_w,
                             const float* __restrict__ t_dev, long lo, long hi) {
  if (clip && clip[1] != 0.f) return;
  const Seg s = segs[blockIdx.y];
  const float c = clip ? clip[0] : 1.f;
  if (t_dev) {
    const double t = (double)t_dev[0];
    bias1 = (float)(1.0 - pow((double)b1, t));
    bias2 = (float)(1.0 - pow((double)b2, t));
  }
  const float inv_b1 = 1.f / bias1, inv_b2 = 1.f / bias2;
  long i0 = 0, i1 = s.numel;
  if (hi > lo) {
    i0 = lo > s.start ? lo - s.start : 0;
    i1 = hi - s.start < s.numel ? hi - s.start : s.numel;
  }
  for (long i = i0 + (long)blockIdx.x * blockDim.x + threadIdx.x; i < i1;
       i += (long)gridDim.x * blockDim.x) {
    const long j = s.start + i, k = j - state_offset;
    const float gv = g[j] * c;
    const float mv = b1 * m[k] + (1.f - b1) * gv;
    const float vv = b2 * v[k] + (1.f - b2) * gv * gv;
    m[k] = mv;
    v[k] = vv;
    const float den = sqrtf(vv * inv_b2) + eps;
    const float nv = p[j] * s.b - s.a * (mv * inv_b1) / den;
    p[j] = nv;
    if (ema) ema[j] += ema_w * (nv - ema[j]);
  }
}

}  // namespace imf

using namespace imf;

extern "C" int imf_muon_momentum(const float* g, float* buf, float* dir, long n, float mu,
                                 int nesterov, const float* clip, void* stream) {
  if (n <= 0 || (n & 3)) return -1;
  long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  muon_momentum_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(g, buf, dir, n, mu,
                                                                          nesterov, clip);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// segs: device array of nseg records {long start, long numel, float a, float b}
extern "C" int imf_muon_apply(float* p, const void* upd, int upd_bf16, float* ema,
                              const void* segs, int nseg, long max_numel, long upd_offset,
                              float ema_w, const float* clip, void* stream) {
  if (nseg <= 0) return 0;
  long bx = (max_numel + 1023) / 1024;
  if (bx > 256) bx = 256;
  if (bx < 1) bx = 1;
  dim3 grid((unsigned)bx, nseg);
  if (upd_bf16)
    muon_apply_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        p, (const __nv_bfloat16*)upd, ema, (const Seg*)segs, upd_offset, ema_w, clip);
  else
    muon_apply_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(
        p, (const float*)upd, ema, (const Seg*)segs, upd_offset, ema_w, clip);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_adamw(float* p, const float* g, float* m, float* v, float* ema,
                         const void* segs, int nseg, long max_numel, long state_offset, float b1,
                         float b2, float eps, float bias1, float bias2, const float* clip,
                         float ema_w, const float* t_dev, long lo, long hi, void* stream) {
  if (nseg <= 0) return 0;
  long bx = (max_numel + 1023) / 1024;
  if (bx > 256) bx = 256;
  if (bx < 1) bx = 1;
  dim3 grid((unsigned)bx, nseg);
  adamw_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p, g, m, v, ema, (const Seg*)segs,
                                                      state_offset, b1, b2, eps, bias1, bias2,
                                                      clip, ema_w, t_dev, lo, hi);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------
// QK-Clip (MuonClip): for every attention module and head whose maximum logit
// S (log2 units in `stat`) exceeded tau, the rope rows of that head in the q
// up-projection are scaled by tau / S.  One launch for all modules; the number
// of clipped heads and the largest logit come back in `summary` (no host
// round trip inside).  Replaces the per-module loop of the reference
// (reference train.py:301-350).
// ---------------------------------------------------------------------------
namespace imf {

struct ClipMod {
  float* w;             // (H * hd, cols) row-major weight of q_b_proj
  const float* stat;    // (H,) max logit in log2 units
  int H, hd, dn, cols;
  float* ema;           // the same weight in the EMA model, or null
};

// `clip` (optional) is the optimizer's [factor, skip flag] word: a skipped step leaves
// the weights alone here too.  A non-finite statistic clips nothing.  The optimizer
// kernels have already folded the un-clipped weight into the EMA, so for a clipped row
// the EMA is corrected to what lerp(ema, gamma * w) would have given.
__global__ void qk_clip_kernel(const ClipMod* __restrict__ mods, float tau_nat,
                               float* __restrict__ summary, const float* __restrict__ clip,
                               float ema_w) {
  if (clip && clip[1] != 0.f) return;
  const ClipMod m = mods[blockIdx.y];
  const int h = blockIdx.x;
  if (h >= m.H) return;
  const float s_nat = m.stat[h] * 0.6931471805599453f;
  if (!isfinite(s_nat)) return;
  const float gamma = fminf(1.f, tau_nat / fmaxf(s_nat, 1e-20f));
  if (threadIdx.x == 0) {
    // non-negative floats order like their bit patterns
    atomicMax(reinterpret_cast<int*>(summary + 1), __float_as_int(fmaxf(s_nat, 0.f)));
    if (gamma < 1.f) atomicAdd(summary, 1.f);
  }
  if (gamma >= 1.f) return;
  const int rows = m.hd - m.dn;
  const size_t off = ((size_t)h * m.hd + m.dn) * m.cols;
  float* base = m.w + off;
  float* eb = m.ema ? m.ema + off : nullptr;
  for (int i = threadIdx.x; i < rows * m.cols; i += blockDim.x) {
    const float w = base[i];
    base[i] = w * gamma;
    if (eb) eb[i] += ema_w * (gamma - 1.f) * w;
  }
}

}  // namespace imf

// mods: device array of nmod records {float* w, const float* stat, int H, hd, dn, cols, float* ema};
// summary: device float[2], zeroed by the caller (count of clipped heads, max logit in nats);
// clip: the optimizer's device word [factor, skip flag] or null; ema_w = 1 - ema decay.
extern "C" int imf_qk_clip(const void* mods, int nmod, int max_heads, float tau_nat, float* summary,
                           const float* clip, float ema_w, void* stream) {
  if (nmod <= 0) return 0;
  qk_clip_kernel<<<dim3(max_heads, nmod), 256, 0, (cudaStream_t)stream>>>(
      (const ClipMod*)mods, tau_nat, summary, clip, ema_w);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------
// Newton-Schulz input preparation: X[z] = bf16(G[z] / (||G[z]||_F + eps)) for a batch of
// fp32 matrices (n x m, contiguous) into bf16 matrices with row pitch mp >= m (the pad
// columns are zeroed), in two launches with fixed-order sums.  Replaces the norm / divide /
// cast / pad sequence of the reference (reference moonlight.py:228-236).
// ---------------------------------------------------------------------------
namespace imf {

constexpr int NS_CHUNKS = 32;

__global__ void __launch_bounds__(256)
ns_sumsq_kernel(const float* __restrict__ g, long numel, double* __restrict__ part) {
  const float* src = g + (long)blockIdx.y * numel;
  const long per = (numel + NS_CHUNKS - 1) / NS_CHUNKS;
  const long lo = blockIdx.x * per, hi = lo + per < numel ? lo + per : numel;
  double ss = 0.0;
  for (long i = lo + threadIdx.x; i < hi; i += 256) {
    const float v = src[i];
    ss += (double)v * v;
  }
  __shared__ double s_part[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    double b = 0.0;
    for (int w = 0; w < 8; ++w) b += s_part[w];
    part[blockIdx.y * NS_CHUNKS + blockIdx.x] = b;
  }
}

__global__ void __launch_bounds__(256)
ns_scale_kernel(const float* __restrict__ g, __nv_bfloat16* __restrict__ x, int n, int m, int mp,
                const double* __restrict__ part, float eps) {
  const int z = blockIdx.y;
  double tot = 0.0;
  for (int c = 0; c < NS_CHUNKS; ++c) tot += part[z * NS_CHUNKS + c];    // same order everywhere
  const float inv = 1.f / ((float)sqrt(tot) + eps);
  const float* src = g + (long)z * n * m;
  __nv_bfloat16* dst = x + (long)z * n * mp;
  const long total = (long)n * mp;
  for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long)gridDim.x * 256) {
    const int r = (int)(i / mp), c = (int)(i % mp);
    dst[i] = __float2bfloat16_rn(c < m ? src[(long)r * m + c] * inv : 0.f);
  }
}

}  // namespace imf

// g: (k, n, m) fp32 contiguous; x: (k, n, mp) bf16; part: fp64 scratch of k * 32 entries.
extern "C" int imf_ns_prepare(const float* g, void* x, int k, int n, int m, int mp, double* part,
                              float eps, void* stream) {
  if (k <= 0 || n <= 0 || m <= 0 || mp < m) return -1;
  const long numel = (long)n * m;
  ns_sumsq_kernel<<<dim3(NS_CHUNKS, k), 256, 0, (cudaStream_t)stream>>>(g, numel, part);
  long bx = ((long)n * mp + 255) / 256;
  if (bx > 128) bx = 128;
  ns_scale_kernel<<<dim3((unsigned)bx, k), 256, 0, (cudaStream_t)stream>>>(
      g, static_cast<__nv_bfloat16*>(x), n, m, mp, part, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

