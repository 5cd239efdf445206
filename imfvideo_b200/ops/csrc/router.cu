// Router of the block-sparse attention kernels on the device, without a host
// round trip: pooled block means (pool_blocks), projected block scores with a
// radix-select top-k (route_topk), and the routing tables built from the
// selection:
//
//   tile lists   : per 128-row query tile the ascending list of 64-row key
//                  blocks selected by its routing block(s), with 2 flag bits
//                  per entry (which 64-row half attends it) and the entry count;
//   inverted     : per 128-row K/V tile the ascending list of query tiles that
//                  attend it, with 4 flag bits (kv half * 2 + q half), for the
//                  backward kernel.
//
// A query tile's selection is scattered into bitmaps in shared memory (one per
// half); lists come out of the bitmaps in ascending order by a prefix sum over
// the words, so the result does not depend on the order of the selection.
// Replaces the reference's `_invert_lut`, the LUT post-processing of
// `route_*` and the sort / unique passes around them, and `_colmean`,
// `_pool_sub`, `_route_pool_kernel` + `torch.topk` (reference
// models/sla2_vendor/kernel.py, models/sla2_cube.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

constexpr int RT_THREADS = 128;
constexpr int RT_MAX_WORDS = 128;         // up to 4096 key blocks

// exclusive prefix sum of one value per thread over RT_THREADS threads
__device__ __forceinline__ int block_excl_scan(int v, int* total) {
  __shared__ int s_warp[RT_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) s_warp[warp] = x;
  __syncthreads();
  int base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < RT_THREADS / 32; ++w) {
    if (w < warp) base += s_warp[w];
    tot += s_warp[w];
  }
  __syncthreads();
  *total = tot;
  return base + x - v;
}

// sel: (B, H, Mb, T) int32 key-block ids (-1 = none).  rpt = routing blocks per query tile
// (1 or 2).  Outputs: lut / flags (B, H, n_mt, tmax), cnt (B, H, n_mt), fm (B, H, n_kvt, n_mt)
// nibble matrix (may be null) and rk (same shape, may be null): for a live (K/V tile, query
// tile) pair, how many HIGHER K/V tiles also attend the query tile -- the backward's place in
// the fixed order of additions to that query tile (it walks the K/V tiles from the back).
__global__ void __launch_bounds__(RT_THREADS)
tile_lut_kernel(const int* __restrict__ sel, int* __restrict__ lut, uint8_t* __restrict__ flags,
                int* __restrict__ cnt, uint8_t* __restrict__ fm, uint16_t* __restrict__ rk, int H,
                int Mb, int T, int rpt, int n_mt, int tmax, int n_kblk, int n_kvt) {
  __shared__ unsigned int bm[2][RT_MAX_WORDS];
  const int mt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int words = (n_kblk + 31) >> 5;
  for (int w = tid; w < RT_MAX_WORDS; w += RT_THREADS) bm[0][w] = bm[1][w] = 0u;
  __syncthreads();
  for (int half = 0; half < rpt; ++half) {
    const int rb = mt * rpt + half;
    if (rb >= Mb) break;
    const int* row = sel + (((size_t)b * H + h) * Mb + rb) * T;
    for (int t = tid; t < T; t += RT_THREADS) {
      const int id = row[t];
      if (id >= 0 && id < n_kblk) {
        if (rpt == 1) {                        // one routing block covers both halves
          atomicOr(&bm[0][id >> 5], 1u << (id & 31));
          atomicOr(&bm[1][id >> 5], 1u << (id & 31));
        } else {
          atomicOr(&bm[half][id >> 5], 1u << (id & 31));
        }
      }
    }
  }
  __syncthreads();
  const unsigned int b0 = tid < words ? bm[0][tid] : 0u, b1 = tid < words ? bm[1][tid] : 0u;
  unsigned int any = b0 | b1;
  int total;
  int pos = block_excl_scan(__popc(any), &total);
  const size_t base = (((size_t)b * H + h) * n_mt + mt) * tmax;
  while (any) {
    const int bit = __ffs(any) - 1;
    any &= any - 1;
    if (pos < tmax) {
      lut[base + pos] = tid * 32 + bit;
      flags[base + pos] = (uint8_t)(((b0 >> bit) & 1u) | (((b1 >> bit) & 1u) << 1));
    }
    ++pos;
  }
  for (int i = total + tid; i < tmax; i += RT_THREADS) {
    lut[base + i] = -1;
    flags[base + i] = 0;
  }
  if (tid == 0) cnt[((size_t)b * H + h) * n_mt + mt] = total < tmax ? total : tmax;
  if (fm && tid < words) {
#pragma unroll
    for (int pp = 0; pp < 16; ++pp) {
      const int kvt = tid * 16 + pp;
      if (kvt < n_kvt) {
        const unsigned int nib = ((b0 >> (2 * pp)) & 1u) | (((b1 >> (2 * pp)) & 1u) << 1) |
                                 (((b0 >> (2 * pp + 1)) & 1u) << 2) |
                                 (((b1 >> (2 * pp + 1)) & 1u) << 3);
        fm[(((size_t)b * H + h) * n_kvt + kvt) * n_mt + mt] = (uint8_t)nib;
      }
    }
  }
  if (rk) {                      // block-uniform
    const unsigned int both = b0 | b1;
    const unsigned int pairs = (both | (both >> 1)) & 0x55555555u;   // bit 2 pp: K/V tile live
    int live_total;
    int below = block_excl_scan(__popc(pairs), &live_total);          // live K/V tiles before mine
    if (tid < words) {
#pragma unroll
      for (int pp = 0; pp < 16; ++pp) {
        const int kvt = tid * 16 + pp;
        if (kvt < n_kvt && ((pairs >> (2 * pp)) & 1u)) {
          rk[(((size_t)b * H + h) * n_kvt + kvt) * n_mt + mt] = (uint16_t)(live_total - 1 - below);
          ++below;
        }
      }
    }
  }
}

// fm: (B, H, n_kvt, n_mt) nibbles -> qlist / qflags (B, H, n_kvt, qmax), -1 terminated.
__global__ void __launch_bounds__(RT_THREADS)
kv_lists_kernel(const uint8_t* __restrict__ fm, const uint16_t* __restrict__ rk,
                int* __restrict__ qlist, uint8_t* __restrict__ qflags,
                uint16_t* __restrict__ qrank, int n_mt, int qmax) {
  const size_t rowi = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  const uint8_t* row = fm + rowi * n_mt;
  const int tid = threadIdx.x;
  const int per = (n_mt + RT_THREADS - 1) / RT_THREADS;
  const int lo = tid * per, hi = min(n_mt, lo + per);
  int n = 0;
  for (int i = lo; i < hi; ++i) n += row[i] != 0;
  int total;
  int pos = block_excl_scan(n, &total);
  for (int i = lo; i < hi; ++i) {
    const uint8_t f = row[i];
    if (f) {
      if (pos < qmax) {
        qlist[rowi * qmax + pos] = i;
        qflags[rowi * qmax + pos] = f;
        if (qrank) qrank[rowi * qmax + pos] = rk[rowi * n_mt + i];
      }
      ++pos;
    }
  }
  for (int i = total + tid; i < qmax; i += RT_THREADS) {
    qlist[rowi * qmax + i] = -1;
    qflags[rowi * qmax + i] = 0;
  }
}

// --------------------------------------------------------------------------
// Block means: x (B, L, H, 64) bf16 with element strides (sb, sl, sh) ->
// out (B, H, nb, 64) fp32, mean over the valid rows of each block.  Fixed
// summation order (rows of a warp in sequence, then the warps in sequence).
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(RT_THREADS)
pool_blocks_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int64_t sb,
                   int64_t sl, int64_t sh, int L, int block, int nb) {
  __shared__ float2 part[RT_THREADS / 32][32];
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = n * block, r1 = min(L, r0 + block);
  const __nv_bfloat16* base = x + b * sb + h * sh + 2 * lane;
  float2 acc = make_float2(0.f, 0.f);
  for (int r = r0 + warp; r < r1; r += RT_THREADS / 32) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + r * sl));
    acc.x += v.x;
    acc.y += v.y;
  }
  part[warp][lane] = acc;
  __syncthreads();
  if (warp == 0) {
    float2 s = part[0][lane];
#pragma unroll
    for (int w = 1; w < RT_THREADS / 32; ++w) {
      s.x += part[w][lane].x;
      s.y += part[w][lane].y;
    }
    const float inv = 1.f / (float)max(1, r1 - r0);
    float* o = out + ((((size_t)b * gridDim.y + h) * nb + n) << 6) + 2 * lane;
    *reinterpret_cast<float2*>(o) = make_float2(s.x * inv, s.y * inv);
  }
}

// order-preserving map of a float to an unsigned key (larger float <=> larger key)
__device__ __forceinline__ unsigned int float_key(float f) {
  const unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// --------------------------------------------------------------------------
// Scores of one pooled query block against the first Nk pooled key blocks and
// the T best of them:
//     score[n] = (Pq qb) . (Pk kb[n]) = (Pk^T Pq qb) . kb[n]
// (a key-side centring would add the same constant to every score of the row
// and cannot change the selection, so it is not applied).  The T-th largest
// score is found by a 4-pass radix select on order-preserving keys; the
// selection is written in ascending block order (scores above the threshold
// first, then as many equal to it as are still needed, lowest index first),
// followed by n_tail always-attended blocks tail0, tail0 + 1, ...
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(RT_THREADS)
route_topk_kernel(const float* __restrict__ qb, const float* __restrict__ kb,
                  const float* __restrict__ Pq, const float* __restrict__ Pk,
                  int* __restrict__ sel, float* __restrict__ scores_out, int Mb, int Nkb, int Nk,
                  int T, int n_tail, int tail0, float scale) {
  extern __shared__ float sc[];                    // Nk scores
  __shared__ __align__(16) float qv[64], uv[64], wv[64];
  __shared__ int hist[256];
  __shared__ unsigned int s_prefix, s_mask;
  __shared__ int s_remaining;
  const int m = blockIdx.x, h = blockIdx.y, b = blockIdx.z, H = gridDim.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t bh = (size_t)b * H + h;
  if (tid < 64) qv[tid] = qb[((bh * Mb + m) << 6) + tid];
  __syncthreads();
  // every global access below is a whole 256-byte row per (half) warp: a divergent
  // row-per-thread access costs one L1 tag look-up per lane
  if (Pq) {                                        // u = Pq q: one row per warp, four in flight
    const float2 q2 = make_float2(qv[2 * lane], qv[2 * lane + 1]);
    for (int i0 = warp * 16; i0 < warp * 16 + 16; i0 += 4) {
      float part[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float2 p2 = __ldg(reinterpret_cast<const float2*>(Pq + (i0 + r) * 64) + lane);
        part[r] = fmaf(p2.x, q2.x, p2.y * q2.y);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < 4; ++r) part[r] += __shfl_xor_sync(0xffffffffu, part[r], o);
      if (lane < 4) uv[i0 + lane] = part[lane == 0 ? 0 : lane == 1 ? 1 : lane == 2 ? 2 : 3];
    }
  } else if (tid < 64) {
    uv[tid] = qv[tid];
  }
  __syncthreads();
  if (Pk) {                                        // w = Pk^T u: column per thread, rows split in two
    const int j = tid & 63, half = tid >> 6;
    float acc = 0.f;
#pragma unroll 8
    for (int i = half * 32; i < half * 32 + 32; ++i) acc = fmaf(__ldg(Pk + i * 64 + j), uv[i], acc);
    if (half) qv[j] = acc;                         // qv is free after the first product
    __syncthreads();
    if (!half) wv[j] = acc + qv[j];
  } else if (tid < 64) {
    wv[tid] = uv[tid];
  }
  __syncthreads();
  {                                                // scores: half a warp per key, eight keys in flight
    const int hl = lane & 15, sub = lane >> 4;
    const float4 w4 = *reinterpret_cast<const float4*>(wv + 4 * hl);
    const float4* kbase = reinterpret_cast<const float4*>(kb + ((bh * Nkb) << 6)) + hl;
    for (int n0 = warp * 8; n0 < Nk; n0 += (RT_THREADS / 32) * 8) {
      float part[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int n = n0 + 2 * r + sub;
        float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < Nk) kv = __ldg(kbase + ((size_t)n << 4));
        part[r] = fmaf(w4.x, kv.x, fmaf(w4.y, kv.y, fmaf(w4.z, kv.z, w4.w * kv.w)));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int r = 0; r < 4; ++r) part[r] += __shfl_xor_sync(0xffffffffu, part[r], o);
      if (hl == 0) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int n = n0 + 2 * r + sub;
          if (n < Nk) sc[n] = part[r] * scale;
        }
      }
    }
  }
  if (tid == 0) {
    s_prefix = 0u;
    s_mask = 0u;
    s_remaining = T;
  }
  __syncthreads();
  if (scores_out)
    for (int n = tid; n < Nk; n += RT_THREADS) scores_out[(bh * Mb + m) * Nk + n] = sc[n];
  // radix select: after the 4 passes s_prefix is the key of the T-th largest score and
  // s_remaining the number of scores equal to it that belong to the selection
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += RT_THREADS) hist[i] = 0;
    __syncthreads();
    const unsigned int prefix = s_prefix, mask = s_mask;
    for (int n = tid; n < Nk; n += RT_THREADS) {
      const unsigned int key = float_key(sc[n]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins 255 - 8l ... 248 - 8l (descending)
      int own = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) own += hist[255 - 8 * lane - i];
      int incl = own;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      const int remaining = s_remaining;
      const int before = incl - own;
      if (before < remaining && remaining <= incl) {
        int cum = before;
        for (int i = 0; i < 8; ++i) {
          const int bin = 255 - 8 * lane - i;
          const int c = hist[bin];
          if (cum + c >= remaining) {
            s_prefix = prefix | ((unsigned int)bin << shift);
            s_mask = mask | (255u << shift);
            s_remaining = remaining - cum;
            break;
          }
          cum += c;
        }
      }
    }
    __syncthreads();
  }
  const unsigned int thr = s_prefix;
  const int n_eq_take = s_remaining;
  const int per = (Nk + RT_THREADS - 1) / RT_THREADS;
  const int lo = tid * per, hi = min(Nk, lo + per);
  int cg = 0, ce = 0;
  for (int n = lo; n < hi; ++n) {
    const unsigned int key = float_key(sc[n]);
    cg += key > thr;
    ce += key == thr;
  }
  int total;
  const int packed = block_excl_scan(cg | (ce << 16), &total);
  int pg = packed & 0xffff, pe = packed >> 16;
  const int n_gt = total & 0xffff;
  int* row = sel + (bh * Mb + m) * (size_t)(T + n_tail);
  for (int n = lo; n < hi; ++n) {
    const unsigned int key = float_key(sc[n]);
    if (key > thr) {
      row[pg++] = n;
    } else if (key == thr) {
      if (pe < n_eq_take) row[n_gt + pe] = n;
      ++pe;
    }
  }
  for (int j = tid; j < n_tail; j += RT_THREADS) row[T + j] = tail0 + j;
}

}  // namespace imf

using namespace imf;

extern "C" int imf_pool_blocks(const void* x, float* out, int B, int L, int H, int block, int nb,
                               int64_t sb, int64_t sl, int64_t sh, void* stream) {
  if (B <= 0 || H <= 0 || L <= 0 || block <= 0 || nb <= 0 || (int64_t)(nb - 1) * block >= L)
    return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 3) || ((sb | sl | sh) & 1)) return -2;
  pool_blocks_kernel<<<dim3(nb, H, B), RT_THREADS, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(x), out, sb, sl, sh, L, block, nb);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// qb (B, H, Mb, 64), kb (B, H, Nkb, 64) fp32 pooled blocks; the first Nk key blocks are
// candidates.  sel (B, H, Mb, T + n_tail) int32.  Pq / Pk: 64 x 64 fp32 row-major projections
// (nn.Linear weights) or null.  scores_out (B, H, Mb, Nk) fp32 or null.
extern "C" int imf_route_topk(const float* qb, const float* kb, const float* Pq, const float* Pk,
                              int* sel, float* scores_out, int B, int H, int Mb, int Nkb, int Nk,
                              int T, int n_tail, int tail0, float scale, void* stream) {
  if (B <= 0 || H <= 0 || Mb <= 0 || Nk <= 0 || Nk > Nkb || T < 1 || T > Nk || n_tail < 0)
    return -1;
  if (Nk > RT_MAX_WORDS * 32) return -4;           // also keeps the packed 16-bit counts exact
  route_topk_kernel<<<dim3(Mb, H, B), RT_THREADS, (size_t)Nk * sizeof(float),
                      (cudaStream_t)stream>>>(qb, kb, Pq, Pk, sel, scores_out, Mb, Nkb, Nk, T,
                                              n_tail, tail0, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_build_tile_lut(const int* sel, int* lut, uint8_t* flags, int* cnt, uint8_t* fm,
                                  uint16_t* rk, int B, int H, int Mb, int T, int qblk, int L,
                                  int tmax, void* stream) {
  if (B <= 0 || H <= 0 || Mb <= 0 || T <= 0 || (qblk != 64 && qblk != 128)) return -1;
  const int rpt = 128 / qblk;
  const int n_mt = (L + 127) / 128, n_kblk = (L + 63) / 64, n_kvt = (L + 127) / 128;
  if (n_kblk > RT_MAX_WORDS * 32 || tmax < 1) return -4;
  tile_lut_kernel<<<dim3(n_mt, H, B), RT_THREADS, 0, (cudaStream_t)stream>>>(
      sel, lut, flags, cnt, fm, rk, H, Mb, T, rpt, n_mt, tmax, n_kblk, n_kvt);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_build_kv_lists(const uint8_t* fm, const uint16_t* rk, int* qlist,
                                  uint8_t* qflags, uint16_t* qrank, int B, int H, int n_kvt,
                                  int n_mt, int qmax, void* stream) {
  if (B <= 0 || H <= 0 || n_kvt <= 0 || n_mt <= 0 || qmax <= 0) return -1;
  if ((rk == nullptr) != (qrank == nullptr)) return -1;
  kv_lists_kernel<<<dim3(n_kvt, H, B), RT_THREADS, 0, (cudaStream_t)stream>>>(
      fm, rk, qlist, qflags, qrank, n_mt, qmax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
