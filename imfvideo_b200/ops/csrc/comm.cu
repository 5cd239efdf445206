// NVLink-side collectives over peer memory for the flat gradient / update
// arenas (one process per GPU; every rank runs the same launch sequence).
//
//   reduce_grads   : cross-rank arrival barrier, then
//                      Muon segment `rank`  <- mean over ranks (fixed order)
//                      AdamW shard  `rank`  <- mean over ranks
//                    read with plain peer loads (or one multimem.ld_reduce per
//                    16 bytes when an NVLS multicast mapping is given), scaled
//                    by 1/W and written to this rank's arena in the same pass.
//                    The same pass accumulates the squared norm of what it wrote
//                    (fp64, fixed order) and publishes it to every rank, so the
//                    global gradient norm needs no second pass and no collective.
//   gather         : barrier, then pull the other ranks' reduced AdamW shards /
//                    orthogonalised update segments into the local arena.
//   muon_apply     : barrier, then p <- p (1 - lr wd) - lr s Phi (+ EMA) for EVERY Muon
//                    parameter with Phi read straight from its owner's memory: the
//                    update all-gather is fused into its consumer.
//
// Barriers are epoch flags in symmetric memory: rank r writes flag[r] = epoch
// into every peer's flag array (st.release.sys) and every CTA polls its LOCAL
// copy (ld.acquire.sys) with a wall-clock bound (2 s unless imf_comm_set_wait_ns
// changed it); on expiry the kernel records STATUS_TIMEOUT_PEER and returns
// without touching data, and the host raises when it next reads the status word
// (the trainer does so once per step).  The signal is sent by whichever CTA of
// the grid gets there first (a ticket in the local flag array), so it does not
// depend on the order in which the hardware schedules the CTAs.  No TMA multicast, no
// library kernel touches peer memory.  Replaces the reference's flat NCCL
// all-reduce (reference train.py:353-371).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

constexpr int MAX_RANKS = 16;
constexpr int TICKET_SLOT = 2 * MAX_RANKS;     // local "someone has signalled epoch e" word
static unsigned long long g_peer_wait_ns = 2000000000ull;

struct CommPeers {
  float* arena[MAX_RANKS];      // peer base pointers of the fp32 arena
  int* flags[MAX_RANKS];        // peer base pointers of the flag arrays [4 * MAX_RANKS]
  unsigned long long wait_ns;   // bound of every wait on a peer
};

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Signal (first block to arrive) and wait (every block).  Returns false on timeout.
__device__ __forceinline__ bool peer_barrier(const CommPeers& peers, int rank, int world, int epoch,
                                             int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    if (atomicMax(peers.flags[rank] + TICKET_SLOT, epoch) < epoch) {
      __threadfence_system();
      for (int q = 0; q < world; ++q) st_release_sys(peers.flags[q] + rank, epoch);
    }
    int ok = 1;
    const unsigned long long t0 = gtime();
    for (int q = 0; q < world && ok; ++q) {
      while (ld_acquire_sys(peers.flags[rank] + q) < epoch) {
        if (gtime() - t0 > peers.wait_ns) {
          ok = 0;
          if (status) atomicCAS(status, 0, 6);
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

struct NormOut {
  double* part;                 // [gridDim.x] per-block partial sums (local scratch)
  unsigned int* done;           // block counter (local, returns to zero)
  double* slots[MAX_RANKS];     // peer base pointers of the per-rank norm arrays [MAX_RANKS]
};

// ranges: [lo0, hi0) = this rank's Muon segment, [lo1, hi1) = its AdamW shard
__global__ void __launch_bounds__(512)
comm_reduce_kernel(const CommPeers peers, const float* mc_arena, int rank, int world, long lo0,
                   long hi0, long lo1, long hi1, int epoch, int* status, const NormOut nrm) {
  if (!peer_barrier(peers, rank, world, epoch, status)) return;
  const float inv = 1.f / world;
  float* mine = peers.arena[rank];
  const long n0 = (hi0 - lo0) / 4, n1 = (hi1 - lo1) / 4;
  double ss = 0.0;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n0 + n1;
       i += (long)gridDim.x * blockDim.x) {
    const long off = i < n0 ? lo0 + i * 4 : lo1 + (i - n0) * 4;
    float4 acc;
    if (mc_arena) {
      acc = multimem_ld_reduce_f32x4(mc_arena + off);
    } else {
      acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = 0; q < world; ++q) {      // fixed order: same bits whoever owns the segment
        const float4 v = *reinterpret_cast<const float4*>(peers.arena[q] + off);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    *reinterpret_cast<float4*>(mine + off) = acc;
    ss += (double)acc.x * acc.x + (double)acc.y * acc.y + (double)acc.z * acc.z +
          (double)acc.w * acc.w;
  }
  if (nrm.part == nullptr) return;
  // squared norm of this rank's reduced slices: warp -> block -> grid, every level in a fixed order
  __shared__ double s_part[16];
  __shared__ bool s_last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    double b = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) b += s_part[w];
    nrm.part[blockIdx.x] = b;
    __threadfence();
    s_last = atomicAdd(nrm.done, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence();
    double tot = 0.0;
    for (unsigned int i = 0; i < gridDim.x; ++i) tot += reinterpret_cast<volatile double*>(nrm.part)[i];
    for (int q = 0; q < world; ++q) nrm.slots[q][rank] = tot;   // visible after the next barrier
    __threadfence_system();
    *nrm.done = 0u;
  }
}

// Pull [base + q*len, base + (q+1)*len) from rank q for every q != rank.
template <typename T>
__global__ void __launch_bounds__(512)
comm_gather_kernel(const CommPeers peers, int rank, int world, long base, long len, int epoch,
                   int* status) {
  if (!peer_barrier(peers, rank, world, epoch, status)) return;
  constexpr int V = 16 / sizeof(T);
  T* mine = reinterpret_cast<T*>(peers.arena[rank]);
  const long nv = len / V;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv * (world - 1);
       i += (long)gridDim.x * blockDim.x) {
    int q = (int)(i / nv);
    if (q >= rank) ++q;
    const long off = base + (long)q * len + (i % nv) * V;
    const T* src = reinterpret_cast<const T*>(peers.arena[q]);
    *reinterpret_cast<uint4*>(mine + off) = *reinterpret_cast<const uint4*>(src + off);
  }
}

__global__ void comm_barrier_kernel(const CommPeers peers, int rank, int world, int epoch,
                                    int* status) {
  peer_barrier(peers, rank, world, epoch, status);
}

struct Seg {          // one parameter inside the arena (same record as the optimizer kernels)
  long start;
  long numel;
  float a;            // 1 - lr wd
  float b;            // lr * scale
};

// p <- a p - b Phi (+ EMA) for every Muon parameter; Phi of a parameter is read from the
// update arena of its owner (start / seg_pad), i.e. over NVLink for the other ranks' segments.
template <typename UT>
__global__ void __launch_bounds__(256)
comm_muon_apply_kernel(const CommPeers peers, int rank, int world, long seg_pad, float* __restrict__ p,
                       float* __restrict__ ema, const Seg* __restrict__ segs, float ema_w,
                       const float* __restrict__ clip, int epoch, int* status) {
  if (!peer_barrier(peers, rank, world, epoch, status)) return;
  if (clip && clip[1] != 0.f) return;       // skipped step (same decision on every rank)
  const Seg sg = segs[blockIdx.y];
  const int owner = (int)(sg.start / seg_pad);
  const UT* upd = reinterpret_cast<const UT*>(peers.arena[owner]);
  if (((sg.start | sg.numel) & 3) == 0) {          // four elements per thread and access
    for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < sg.numel;
         i += (long)gridDim.x * blockDim.x * 4) {
      const long j = sg.start + i;
      float u[4];
      if constexpr (sizeof(UT) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(upd + j);
        u[0] = __uint_as_float(raw.x << 16); u[1] = __uint_as_float(raw.x & 0xffff0000u);
        u[2] = __uint_as_float(raw.y << 16); u[3] = __uint_as_float(raw.y & 0xffff0000u);
      } else {
        const float4 raw = *reinterpret_cast<const float4*>(upd + j);
        u[0] = raw.x; u[1] = raw.y; u[2] = raw.z; u[3] = raw.w;
      }
      float4 pv = *reinterpret_cast<float4*>(p + j);
      pv.x = pv.x * sg.a - sg.b * u[0]; pv.y = pv.y * sg.a - sg.b * u[1];
      pv.z = pv.z * sg.a - sg.b * u[2]; pv.w = pv.w * sg.a - sg.b * u[3];
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
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < sg.numel;
       i += (long)gridDim.x * blockDim.x) {
    const long j = sg.start + i;
    const float u = static_cast<float>(upd[j]);
    const float v = p[j] * sg.a - sg.b * u;
    p[j] = v;
    if (ema) ema[j] += ema_w * (v - ema[j]);
  }
}

static int fill(CommPeers& p, void* const* arena_ptrs, void* const* flag_ptrs, int world) {
  if (world < 1 || world > MAX_RANKS) return -1;
  for (int q = 0; q < MAX_RANKS; ++q) {
    p.arena[q] = q < world ? static_cast<float*>(arena_ptrs[q]) : nullptr;
    p.flags[q] = q < world ? static_cast<int*>(flag_ptrs[q]) : nullptr;
  }
  p.wait_ns = g_peer_wait_ns;
  return 0;
}

}  // namespace imf

using namespace imf;

// Bound (nanoseconds) of every later wait on a peer's flag; returns the previous value.
// A launcher-side setting: kernels already in flight keep the bound they were launched with.
extern "C" unsigned long long imf_comm_set_wait_ns(unsigned long long ns) {
  const unsigned long long old = g_peer_wait_ns;
  if (ns > 0) g_peer_wait_ns = ns;
  return old;
}

// Mean-reduce this rank's Muon segment and AdamW shard of the fp32 arena.
// arena_ptrs / flag_ptrs: host arrays of `world` device pointers (peer mapped).
// mc_arena: NVLS multicast address of the arena or null.
// norm_ptrs: `world` peer pointers of fp64[MAX_RANKS] arrays (slot r receives rank r's squared
// norm of its reduced slices), norm_part: local fp64 scratch of >= 296 entries, norm_done: local
// zeroed counter; all three null to skip the norm.
extern "C" int imf_comm_reduce(void* const* arena_ptrs, void* const* flag_ptrs, const void* mc_arena,
                               int rank, int world, long seg_pad, long muon_total, long adam_numel,
                               int epoch, int* status, void* const* norm_ptrs, double* norm_part,
                               unsigned int* norm_done, void* stream) {
  CommPeers p;
  if (fill(p, arena_ptrs, flag_ptrs, world)) return -1;
  NormOut nrm;
  nrm.part = norm_ptrs ? norm_part : nullptr;
  nrm.done = norm_done;
  for (int q = 0; q < MAX_RANKS; ++q)
    nrm.slots[q] = (norm_ptrs && q < world) ? static_cast<double*>(norm_ptrs[q]) : nullptr;
  if ((seg_pad & 3) || (adam_numel % (4L * world))) return -1;
  const long shard = adam_numel / world;
  const long lo0 = rank * seg_pad, hi0 = lo0 + seg_pad;
  const long lo1 = muon_total + rank * shard, hi1 = lo1 + shard;
  long blocks = ((seg_pad + shard) / 4 + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  comm_reduce_kernel<<<(unsigned)blocks, 512, 0, (cudaStream_t)stream>>>(
      p, static_cast<const float*>(mc_arena), rank, world, lo0, hi0, lo1, hi1, epoch, status, nrm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// All-gather equal slices [base + q*len, ...) of a symmetric buffer; elem_size 4 or 2.
extern "C" int imf_comm_gather(void* const* arena_ptrs, void* const* flag_ptrs, int rank, int world,
                               long base, long len, int elem_size, int epoch, int* status,
                               void* stream) {
  CommPeers p;
  if (fill(p, arena_ptrs, flag_ptrs, world)) return -1;
  if ((len * elem_size) % 16 || (base * elem_size) % 16) return -1;
  long blocks = (len * elem_size / 16 * (world - 1) + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  if (elem_size == 4)
    comm_gather_kernel<float><<<(unsigned)blocks, 512, 0, (cudaStream_t)stream>>>(
        p, rank, world, base, len, epoch, status);
  else if (elem_size == 2)
    comm_gather_kernel<__nv_bfloat16><<<(unsigned)blocks, 512, 0, (cudaStream_t)stream>>>(
        p, rank, world, base, len, epoch, status);
  else
    return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int imf_comm_barrier(void* const* arena_ptrs, void* const* flag_ptrs, int rank, int world,
                                int epoch, int* status, void* stream) {
  CommPeers p;
  if (fill(p, arena_ptrs, flag_ptrs, world)) return -1;
  comm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p, rank, world, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Muon weight update with the update all-gather fused in: u_ptrs are the peer pointers of the
// update arena (bf16 or fp32, owner-major segments of seg_pad elements), segs the device table
// of nseg parameters {start, numel, 1 - lr wd, lr * scale}.
extern "C" int imf_comm_muon_apply(void* const* u_ptrs, void* const* flag_ptrs, int rank, int world,
                                   long seg_pad, float* p, float* ema, const void* segs, int nseg,
                                   long max_numel, float ema_w, const float* clip, int upd_bf16,
                                   int epoch, int* status, void* stream) {
  if (nseg <= 0) return 0;
  CommPeers peers;
  if (fill(peers, u_ptrs, flag_ptrs, world)) return -1;
  long bx = (max_numel + 1023) / 1024;
  if (bx > 256) bx = 256;
  if (bx < 1) bx = 1;
  dim3 grid((unsigned)bx, nseg);
  if (upd_bf16)
    comm_muon_apply_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        peers, rank, world, seg_pad, p, ema, (const Seg*)segs, ema_w, clip, epoch, status);
  else
    comm_muon_apply_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(
        peers, rank, world, seg_pad, p, ema, (const Seg*)segs, ema_w, clip, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------
// Bucketed gradient reduce-scatter with a bf16 wire format, launched bucket by
// bucket on a side stream while the backward pass is still producing the later
// buckets (a bucket = the parameters of one transformer block).  Two launches per
// bucket, neither of which makes one rank's kernel wait for a kernel that another
// rank has not launched yet for longer than the ranks' skew:
//   pack   : this rank's fp32 gradients of the bucket that OTHER ranks own are
//            written as bf16 into its wire arena; the last CTA to finish publishes
//            "bucket b of step e is packed" to every peer (no waiting at all);
//   reduce : waits (bounded) until every peer has published the bucket, then, for
//            the ranges this rank owns: own fp32 gradient + the peers' bf16 copies,
//            summed in rank order in fp32, times 1/W, written back in place, and
//            the squared norm of the result as per-CTA fp64 partials.
// finish_norm adds up all partials in a fixed order, publishes the rank's share of
// the squared gradient norm to every rank and ends with a barrier, so the clip
// factor is known everywhere without a collective.  AdamW then runs on this rank's
// shard only and param_gather pulls the updated parameters (not gradients) from
// their owners, updating the local EMA copy on the way.
// Replaces the reference's blocking flat all-reduce after backward (reference
// train.py:353-371) and its replicated AdamW (reference moonlight.py:439-469).
// ---------------------------------------------------------------------------
namespace imf {

constexpr int BUCKET_FLAG_BASE = 4 * MAX_RANKS;     // flags[BASE + bucket * MAX_RANKS + rank]
constexpr int MAX_BUCKETS = 64;
constexpr int BUCKET_BX = 8;                        // CTAs per range

struct Range {       // one contiguous piece of the arena with a single owner
  long start;
  long numel;
  int owner;
  int pad;
};

__device__ __forceinline__ uint2 pack4_bf16(float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  return u;
}

__global__ void __launch_bounds__(256)
comm_bucket_pack_kernel(const CommPeers peers, const float* __restrict__ g,
                        __nv_bfloat16* __restrict__ wire, const Range* __restrict__ ranges,
                        int rank, int world, int bucket, int epoch, unsigned int* done) {
  const Range r = ranges[blockIdx.y];
  if (r.owner != rank) {
    if (((r.start | r.numel) & 3) == 0) {
      for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < r.numel;
           i += (long)gridDim.x * blockDim.x * 4)
        *reinterpret_cast<uint2*>(wire + r.start + i) =
            pack4_bf16(*reinterpret_cast<const float4*>(g + r.start + i));
    } else {
      for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < r.numel;
           i += (long)gridDim.x * blockDim.x)
        wire[r.start + i] = __float2bfloat16_rn(g[r.start + i]);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    if (atomicAdd(done, 1u) == total - 1) {          // every CTA's stores are fenced
      *done = 0u;
      __threadfence_system();
      for (int q = 0; q < world; ++q)
        if (q != rank)
          st_release_sys(peers.flags[q] + BUCKET_FLAG_BASE + bucket * MAX_RANKS + rank, epoch);
    }
  }
}

struct WirePeers {
  const __nv_bfloat16* wire[MAX_RANKS];
};

__global__ void __launch_bounds__(256)
comm_bucket_reduce_kernel(const CommPeers peers, const WirePeers wp, float* __restrict__ g,
                          const Range* __restrict__ ranges, int rank, int world, int bucket,
                          int epoch, int* status, double* __restrict__ part) {
  const Range r = ranges[blockIdx.y];
  double ss = 0.0;
  __shared__ int s_ok;
  if (r.owner == rank) {
    if (threadIdx.x == 0) {
      int ok = 1;
      const unsigned long long t0 = gtime();
      const int* mine = peers.flags[rank] + BUCKET_FLAG_BASE + bucket * MAX_RANKS;
      for (int q = 0; q < world && ok; ++q) {
        if (q == rank) continue;
        while (ld_acquire_sys(mine + q) < epoch) {
          if (gtime() - t0 > peers.wait_ns) {
            ok = 0;
            if (status) atomicCAS(status, 0, 6);
            break;
          }
        }
      }
      s_ok = ok;
    }
    __syncthreads();
    if (s_ok) {
      const float inv = 1.f / world;
      if (((r.start | r.numel) & 3) == 0) {
        for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < r.numel;
             i += (long)gridDim.x * blockDim.x * 4) {
          const long j = r.start + i;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int q = 0; q < world; ++q) {            // rank order: same bits on every run
            float4 v;
            if (q == rank) {
              v = *reinterpret_cast<const float4*>(g + j);
            } else {
              const uint2 u = *reinterpret_cast<const uint2*>(wp.wire[q] + j);
              v.x = __uint_as_float(u.x << 16); v.y = __uint_as_float(u.x & 0xffff0000u);
              v.z = __uint_as_float(u.y << 16); v.w = __uint_as_float(u.y & 0xffff0000u);
            }
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
          *reinterpret_cast<float4*>(g + j) = acc;
          ss += (double)acc.x * acc.x + (double)acc.y * acc.y + (double)acc.z * acc.z +
                (double)acc.w * acc.w;
        }
      } else {
        for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < r.numel;
             i += (long)gridDim.x * blockDim.x) {
          const long j = r.start + i;
          float acc = 0.f;
          for (int q = 0; q < world; ++q)
            acc += q == rank ? g[j] : __bfloat162float(wp.wire[q][j]);
          acc *= inv;
          g[j] = acc;
          ss += (double)acc * acc;
        }
      }
    }
  }
  // per-CTA partial of the squared norm (zero for ranges of other owners), fixed order
  __shared__ double s_part[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    double b = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) b += s_part[w];
    part[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = b;
  }
}

// One CTA: total = sum of `n` partials in a fixed order; publish to slot `rank` of every rank's
// norm array; barrier, after which every rank's slot array is complete.
__global__ void __launch_bounds__(256)
comm_norm_finish_kernel(const CommPeers peers, const NormOut nrm, const double* __restrict__ part,
                        int n, int rank, int world, int epoch, int* status) {
  __shared__ double s_sum[256];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n; i += 256) acc += part[i];
  s_sum[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) s_sum[threadIdx.x] += s_sum[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    for (int q = 0; q < world; ++q) nrm.slots[q][rank] = s_sum[0];
    __threadfence_system();
  }
  __syncthreads();
  peer_barrier(peers, rank, world, epoch, status);
}

struct ParamPeers {
  const float* p[MAX_RANKS];
};

// Pull the AdamW shard of every other rank from that rank's parameter arena (it holds the
// updated values), and fold them into the local EMA copy.
__global__ void __launch_bounds__(512)
comm_param_gather_kernel(const CommPeers peers, const ParamPeers pp, float* __restrict__ p,
                         float* __restrict__ ema, int rank, int world, long base, long shard,
                         float ema_w, const float* __restrict__ clip, int epoch, int* status) {
  if (!peer_barrier(peers, rank, world, epoch, status)) return;
  if (clip && clip[1] != 0.f) return;       // skipped step: nothing changed anywhere
  const long nv = shard / 4;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv * (world - 1);
       i += (long)gridDim.x * blockDim.x) {
    int q = (int)(i / nv);
    if (q >= rank) ++q;
    const long off = base + (long)q * shard + (i % nv) * 4;
    const float4 v = *reinterpret_cast<const float4*>(pp.p[q] + off);
    *reinterpret_cast<float4*>(p + off) = v;
    if (ema) {
      float4 e = *reinterpret_cast<float4*>(ema + off);
      e.x += ema_w * (v.x - e.x); e.y += ema_w * (v.y - e.y);
      e.z += ema_w * (v.z - e.z); e.w += ema_w * (v.w - e.w);
      *reinterpret_cast<float4*>(ema + off) = e;
    }
  }
}

}  // namespace imf

// Pack bucket `bucket` (device table `ranges`, `nranges` entries) of this rank's gradients `g`
// into its bf16 wire arena and publish it.  `done`: local zeroed counter.  No waits.
extern "C" int imf_comm_bucket_pack(void* const* flag_ptrs, const float* g, void* wire,
                                    const void* ranges, int nranges, int rank, int world,
                                    int bucket, int epoch, unsigned int* done, void* stream) {
  if (nranges <= 0) return 0;
  if (bucket < 0 || bucket >= MAX_BUCKETS || world < 1 || world > MAX_RANKS) return -1;
  CommPeers p;
  for (int q = 0; q < MAX_RANKS; ++q) {
    p.arena[q] = nullptr;
    p.flags[q] = q < world ? static_cast<int*>(flag_ptrs[q]) : nullptr;
  }
  p.wait_ns = g_peer_wait_ns;
  comm_bucket_pack_kernel<<<dim3(BUCKET_BX, nranges), 256, 0, (cudaStream_t)stream>>>(
      p, g, static_cast<__nv_bfloat16*>(wire), static_cast<const Range*>(ranges), rank, world,
      bucket, epoch, done);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Reduce the ranges of bucket `bucket` that this rank owns: g (fp32, in place) = mean over ranks
// of own fp32 + peers' bf16 wire copies.  part: fp64[nranges * 8] partial squared norms.
extern "C" int imf_comm_bucket_reduce(void* const* flag_ptrs, void* const* wire_ptrs, float* g,
                                      const void* ranges, int nranges, int rank, int world,
                                      int bucket, int epoch, int* status, double* part,
                                      void* stream) {
  if (nranges <= 0) return 0;
  if (bucket < 0 || bucket >= MAX_BUCKETS || world < 1 || world > MAX_RANKS) return -1;
  CommPeers p;
  WirePeers wp;
  for (int q = 0; q < MAX_RANKS; ++q) {
    p.arena[q] = nullptr;
    p.flags[q] = q < world ? static_cast<int*>(flag_ptrs[q]) : nullptr;
    wp.wire[q] = q < world ? static_cast<const __nv_bfloat16*>(wire_ptrs[q]) : nullptr;
  }
  p.wait_ns = g_peer_wait_ns;
  comm_bucket_reduce_kernel<<<dim3(BUCKET_BX, nranges), 256, 0, (cudaStream_t)stream>>>(
      p, wp, g, static_cast<const Range*>(ranges), rank, world, bucket, epoch, status, part);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Sum `n` fp64 partials, publish to slot `rank` of every rank's norm array, barrier.
extern "C" int imf_comm_norm_finish(void* const* flag_ptrs, void* const* norm_ptrs,
                                    const double* part, int n, int rank, int world, int epoch,
                                    int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS || n < 0) return -1;
  CommPeers p;
  NormOut nrm;
  nrm.part = nullptr;
  nrm.done = nullptr;
  for (int q = 0; q < MAX_RANKS; ++q) {
    p.arena[q] = nullptr;
    p.flags[q] = q < world ? static_cast<int*>(flag_ptrs[q]) : nullptr;
    nrm.slots[q] = q < world ? static_cast<double*>(norm_ptrs[q]) : nullptr;
  }
  p.wait_ns = g_peer_wait_ns;
  comm_norm_finish_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p, nrm, part, n, rank, world,
                                                              epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// All-gather of updated parameters: shard q ([base + q * shard, + shard), shard % 4 == 0) is read
// from rank q's parameter arena into the local one; ema (optional) follows with weight ema_w.
extern "C" int imf_comm_param_gather(void* const* flag_ptrs, void* const* param_ptrs, float* p,
                                     float* ema, int rank, int world, long base, long shard,
                                     float ema_w, const float* clip, int epoch, int* status,
                                     void* stream) {
  if (world < 1 || world > MAX_RANKS || (shard & 3) || (base & 3)) return -1;
  CommPeers peers;
  ParamPeers pp;
  for (int q = 0; q < MAX_RANKS; ++q) {
    peers.arena[q] = nullptr;
    peers.flags[q] = q < world ? static_cast<int*>(flag_ptrs[q]) : nullptr;
    pp.p[q] = q < world ? static_cast<const float*>(param_ptrs[q]) : nullptr;
  }
  peers.wait_ns = g_peer_wait_ns;
  long blocks = (shard / 4 * (world - 1) + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  comm_param_gather_kernel<<<(unsigned)blocks, 512, 0, (cudaStream_t)stream>>>(
      peers, pp, p, ema, rank, world, base, shard, ema_w, clip, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------
// Element-wise MAX over ranks of a small fp32 vector (the per-head logit maxima of
// every attention module, for QK-clip): every rank reads every rank's copy over
// peer memory after a barrier and writes the maximum to a LOCAL output, so no rank
// overwrites what another is still reading.  One launch, no host read.  Replaces
// the per-module all_reduce(MAX) of the reference (reference train.py:336).
// ---------------------------------------------------------------------------
namespace imf {
__global__ void __launch_bounds__(256)
comm_max_kernel(const CommPeers peers, float* __restrict__ out, int n, int rank, int world,
                int epoch, int* status) {
  if (!peer_barrier(peers, rank, world, epoch, status)) return;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    float m = peers.arena[0][i];
    for (int q = 1; q < world; ++q) m = fmaxf(m, peers.arena[q][i]);   // NaN-ignoring, like MAX
    out[i] = m;
  }
}
}  // namespace imf

// in_ptrs: `world` peer pointers of fp32[n] buffers; out: local fp32[n].
extern "C" int imf_comm_max(void* const* in_ptrs, void* const* flag_ptrs, float* out, int n,
                            int rank, int world, int epoch, int* status, void* stream) {
  if (n <= 0) return 0;
  CommPeers p;
  if (fill(p, in_ptrs, flag_ptrs, world)) return -1;
  int blocks = (n + 255) / 256;
  if (blocks > 64) blocks = 64;
  comm_max_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, out, n, rank, world, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

