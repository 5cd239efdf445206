// Helpers for the per-token ("row") kernels: one warp owns one token row,
// a lane owns NV float4 chunks (columns lane*4 + i*128 ... +3).  All row
// kernels are memory-bound; they fuse the residual update, attention-residual
// re-mix, RMSNorm, activation and their forward-mode tangents / reverse-mode
// gradients so each activation tensor is read and written once.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

constexpr int ROW_THREADS = 256;
constexpr int ROW_WARPS = ROW_THREADS / 32;
constexpr int MAX_CANDS = 16;     // candidates of the attention-residual re-mix (snapshots + prefix)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  float4 v;
  v.x = __uint_as_float(u.x << 16);
  v.y = __uint_as_float(u.x & 0xffff0000u);
  v.z = __uint_as_float(u.y << 16);
  v.w = __uint_as_float(u.y & 0xffff0000u);
  return v;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
  __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ float4 f4zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float dot4(float4 a, float4 b) {
  return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
}
__device__ __forceinline__ float4 operator+(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ float4 operator*(float4 a, float4 b) {
  return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
}
__device__ __forceinline__ float4 operator*(float4 a, float s) {
  return make_float4(a.x * s, a.y * s, a.z * s, a.w * s);
}
__device__ __forceinline__ float4 fma4(float4 a, float s, float4 c) {
  return make_float4(fmaf(a.x, s, c.x), fmaf(a.y, s, c.y), fmaf(a.z, s, c.z), fmaf(a.w, s, c.w));
}

// Column sums over rows: each lane keeps NV float4 partials over the rows its
// warp visits; the CTA reduces them through shared memory and writes one
// [D] slice of `partial` (shape [gridDim.x, D]); the host sums the slices, so
// the result is deterministic.
template <int NV>
struct ColAcc {
  float4 v[NV];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = f4zero();
  }
};

template <int NV>
__device__ __forceinline__ void col_flush(const ColAcc<NV>& acc,
                                          float* smem_col /*[ROW_WARPS][NV*128]*/,
                                          float* partial, int lane, int warp) {
  constexpr int D = NV * 128;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; ++i) st4(smem_col + warp * D + i * 128 + lane * 4, acc.v[i]);
  __syncthreads();
  if (partial)
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < ROW_WARPS; ++w) t += smem_col[w * D + c];   // fixed order
      partial[(size_t)blockIdx.x * D + c] = t;
    }
}

inline int row_grid(int rows) {
  int g = (rows + ROW_WARPS - 1) / ROW_WARPS;
  const int cap = 148 * 4;
  return g < cap ? (g < 1 ? 1 : g) : cap;
}

}  // namespace imf
