// Layout kernels around the transformer: patch rows of a latent video and back,
// row permutation of a token sequence (tile-major order and its inverse), and
// the sinusoidal scalar embedding with its derivative.
//
//   patch_gather   : x (B, C, T, H, W) -> rows (B, N, F), N = gt*gh*gw patches in
//                    (t, h, w) order, F = C*pt*ph*pw features ordered (c, pt, ph, pw)
//                    (the flattened Conv3d weight) or (pt, ph, pw, c) (the output
//                    head's order);
//   patch_scatter  : the inverse (and adjoint) map, rows -> video, fp32 output;
//   permute_rows   : dst[b, j, :] = src[b, idx[j], :], 16 bytes per thread;
//   sinusoid       : emb = [cos(t f_i) | sin(t f_i)], demb = d emb / dt.
//
// Each is a pure index map (one element or one 16-byte vector per thread), so
// results are bit-identical to the reshape / permute / index formulas.  Replaces
// the reference's Conv3d patch embedding input shuffle, `unpatchify` einsum,
// `tile_permutation` gathers and `timestep_embedding` (reference
// models/imf_dit_video.py, models/sla2_cube.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

struct PatchGeom {
  int B, C, T, H, W, pt, ph, pw, gt, gh, gw, F, N;
  int c_last;              // feature order: 0 = (c, pt, ph, pw), 1 = (pt, ph, pw, c)
};

// flat video index of (patch n, feature f)
__device__ __forceinline__ int64_t video_index(const PatchGeom& g, int b, int n, int f) {
  const int iw_g = n % g.gw, ih_g = (n / g.gw) % g.gh, it_g = n / (g.gw * g.gh);
  int c, it, ih, iw;
  if (g.c_last) {
    c = f % g.C;
    const int r = f / g.C;
    iw = r % g.pw;
    ih = (r / g.pw) % g.ph;
    it = r / (g.pw * g.ph);
  } else {
    iw = f % g.pw;
    ih = (f / g.pw) % g.ph;
    it = (f / (g.pw * g.ph)) % g.pt;
    c = f / (g.pw * g.ph * g.pt);
  }
  const int t = it_g * g.pt + it, h = ih_g * g.ph + ih, w = iw_g * g.pw + iw;
  return ((((int64_t)b * g.C + c) * g.T + t) * g.H + h) * g.W + w;
}

template <typename TIn, typename TOut>
__global__ void patch_gather_kernel(const TIn* __restrict__ x, TOut* __restrict__ rows,
                                    const PatchGeom g) {
  const int64_t total = (int64_t)g.B * g.N * g.F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int f = (int)(i % g.F);
    const int n = (int)((i / g.F) % g.N);
    const int b = (int)(i / ((int64_t)g.F * g.N));
    rows[i] = (TOut)(float)x[video_index(g, b, n, f)];
  }
}

template <typename TIn>
__global__ void patch_scatter_kernel(const TIn* __restrict__ rows, float* __restrict__ x,
                                     const PatchGeom g) {
  const int64_t total = (int64_t)g.B * g.N * g.F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int f = (int)(i % g.F);
    const int n = (int)((i / g.F) % g.N);
    const int b = (int)(i / ((int64_t)g.F * g.N));
    x[video_index(g, b, n, f)] = (float)rows[i];
  }
}

// rows of `vecs` 16-byte vectors
__global__ void permute_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                    const int64_t* __restrict__ idx, int B, int L_src, int L_dst,
                                    int vecs) {
  const int64_t total = (int64_t)B * L_dst * vecs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vecs);
    const int j = (int)((i / vecs) % L_dst);
    const int b = (int)(i / ((int64_t)vecs * L_dst));
    const int64_t s = idx[j];
    if (s < 0 || s >= L_src) continue;           // an index outside the source writes nothing
    dst[i] = src[((int64_t)b * L_src + s) * vecs + v];
  }
}

__global__ void sinusoid_kernel(const float* __restrict__ t, float* __restrict__ emb,
                                float* __restrict__ demb, int B, int dim, float log_max_period) {
  const int half = dim / 2;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * dim) return;
  const int b = i / dim, j = i - b * dim;
  float e = 0.f, de = 0.f;
  if (j < 2 * half) {
    const int k = j < half ? j : j - half;
    const float freq = expf(-log_max_period * (float)k / (float)half);
    const float arg = t[b] * freq;
    const float c = cosf(arg), s = sinf(arg);
    e = j < half ? c : s;
    de = j < half ? -s * freq : c * freq;
  }
  emb[i] = e;
  demb[i] = de;
}

static int grid_for(int64_t total, int threads) {
  const int64_t blocks = (total + threads - 1) / threads;
  return (int)(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16);
}

static bool geom(PatchGeom* g, int B, int C, int T, int H, int W, int pt, int ph, int pw,
                 int c_last) {
  if (B <= 0 || C <= 0 || pt <= 0 || ph <= 0 || pw <= 0 || T % pt || H % ph || W % pw) return false;
  g->B = B; g->C = C; g->T = T; g->H = H; g->W = W; g->pt = pt; g->ph = ph; g->pw = pw;
  g->gt = T / pt; g->gh = H / ph; g->gw = W / pw;
  g->F = C * pt * ph * pw;
  g->N = g->gt * g->gh * g->gw;
  g->c_last = c_last;
  return true;
}

}  // namespace imf

using namespace imf;

// in_bf16 / out_bf16: element types of the video and of the rows (0 = fp32).
extern "C" int imf_patch_gather(const void* x, void* rows, int B, int C, int T, int H, int W,
                                int pt, int ph, int pw, int c_last, int in_bf16, int out_bf16,
                                void* stream) {
  PatchGeom g;
  if (!geom(&g, B, C, T, H, W, pt, ph, pw, c_last)) return -1;
  const int64_t total = (int64_t)B * g.N * g.F;
  const int grid = grid_for(total, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (!in_bf16 && !out_bf16)
    patch_gather_kernel<float, float><<<grid, 256, 0, st>>>((const float*)x, (float*)rows, g);
  else if (!in_bf16 && out_bf16)
    patch_gather_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>((const float*)x,
                                                                   (__nv_bfloat16*)rows, g);
  else if (in_bf16 && out_bf16)
    patch_gather_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)rows, g);
  else
    patch_gather_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x,
                                                                   (float*)rows, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_patch_scatter(const void* rows, float* x, int B, int C, int T, int H, int W,
                                 int pt, int ph, int pw, int c_last, int in_bf16, void* stream) {
  PatchGeom g;
  if (!geom(&g, B, C, T, H, W, pt, ph, pw, c_last)) return -1;
  const int64_t total = (int64_t)B * g.N * g.F;
  const int grid = grid_for(total, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (in_bf16)
    patch_scatter_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)rows, x, g);
  else
    patch_scatter_kernel<float><<<grid, 256, 0, st>>>((const float*)rows, x, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// src (B, L_src, row_bytes), dst (B, L_dst, row_bytes), idx (L_dst) int64; row_bytes % 16 == 0.
extern "C" int imf_permute_rows(const void* src, void* dst, const int64_t* idx, int B, int L_src,
                                int L_dst, int row_bytes, void* stream) {
  if (B <= 0 || L_src <= 0 || L_dst <= 0 || row_bytes <= 0) return -1;
  if ((row_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(dst) & 15))
    return -2;
  const int vecs = row_bytes / 16;
  const int64_t total = (int64_t)B * L_dst * vecs;
  permute_rows_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, (uint4*)dst, idx, B, L_src, L_dst, vecs);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_sinusoid(const float* t, float* emb, float* demb, int B, int dim,
                            float max_period, void* stream) {
  if (B <= 0 || dim < 2 || max_period <= 0.f) return -1;
  const int total = B * dim;
  sinusoid_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(t, emb, demb, B, dim,
                                                                        logf(max_period));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
