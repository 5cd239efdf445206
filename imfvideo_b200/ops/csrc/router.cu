// Routing tables of the block-sparse attention kernels, built on the device
// in two launches and without a host round trip:
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
// `route_*` and the sort / unique passes around them (reference
// models/sla2_vendor/kernel.py, models/sla2_cube.py).
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
// nibble matrix (may be null).
__global__ void __launch_bounds__(RT_THREADS)
tile_lut_kernel(const int* __restrict__ sel, int* __restrict__ lut, uint8_t* __restrict__ flags,
                int* __restrict__ cnt, uint8_t* __restrict__ fm, int H, int Mb, int T, int rpt,
                int n_mt, int tmax, int n_kblk, int n_kvt) {
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
}

// fm: (B, H, n_kvt, n_mt) nibbles -> qlist / qflags (B, H, n_kvt, qmax), -1 terminated.
__global__ void __launch_bounds__(RT_THREADS)
kv_lists_kernel(const uint8_t* __restrict__ fm, int* __restrict__ qlist,
                uint8_t* __restrict__ qflags, int n_mt, int qmax) {
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
      }
      ++pos;
    }
  }
  for (int i = total + tid; i < qmax; i += RT_THREADS) {
    qlist[rowi * qmax + i] = -1;
    qflags[rowi * qmax + i] = 0;
  }
}

}  // namespace imf

using namespace imf;

extern "C" int imf_build_tile_lut(const int* sel, int* lut, uint8_t* flags, int* cnt, uint8_t* fm,
                                  int B, int H, int Mb, int T, int qblk, int L, int tmax,
                                  void* stream) {
  if (B <= 0 || H <= 0 || Mb <= 0 || T <= 0 || (qblk != 64 && qblk != 128)) return -1;
  const int rpt = 128 / qblk;
  const int n_mt = (L + 127) / 128, n_kblk = (L + 63) / 64, n_kvt = (L + 127) / 128;
  if (n_kblk > RT_MAX_WORDS * 32 || tmax < 1) return -4;
  tile_lut_kernel<<<dim3(n_mt, H, B), RT_THREADS, 0, (cudaStream_t)stream>>>(
      sel, lut, flags, cnt, fm, H, Mb, T, rpt, n_mt, tmax, n_kblk, n_kvt);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_build_kv_lists(const uint8_t* fm, int* qlist, uint8_t* qflags, int B, int H,
                                  int n_kvt, int n_mt, int qmax, void* stream) {
  if (B <= 0 || H <= 0 || n_kvt <= 0 || n_mt <= 0 || qmax <= 0) return -1;
  kv_lists_kernel<<<dim3(n_kvt, H, B), RT_THREADS, 0, (cudaStream_t)stream>>>(fm, qlist, qflags,
                                                                             n_mt, qmax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
