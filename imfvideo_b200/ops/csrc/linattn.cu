// Linear-attention complement branch of SLA2 / cube attention (forward,
// forward-mode tangent and reverse mode) on per-block states.
//
//   phi = softmax over the head dimension (64)
//   key block n   : S_n = [ phi(K_n)^T V_n | sum_rows phi(K_n) ]      (64 x 65)
//   query block m : C_m = sum_{n not selected by m} S_n = [ H | z ]
//   row r of m    : o_l = phi(q_r) H / (phi(q_r) . z + eps)
//   output        : o = a o_s + (1 - a) o_l    (o_s: block-sparse softmax branch)
//
// The sum over non-selected blocks is one GEMM with a 0/1 complement mask on
// the tcgen05 GEMM of this library: states are written as bf16 (hi, lo) pairs
// so that the bf16 GEMM reproduces them to 2^-17.  Reverse mode has the same
// two shapes of work: "rows x state" products (lin_apply / lin_bwd_rows /
// lin_bwd_kv) and "rows^T rows" state builds (lin_states, reused with
// (phi(q), dL/dnum | dL/dden) to get dL/dC); both run on the tensor cores
// (mma.sync, TF32 inputs, fp32 accumulation).  Every reduction has a fixed
// order (no atomics).  Replaces the reference's `_hblocks`,
// `_phi_states_kernel`, `_lin_fwd*`, `_linear_jvp`, `_lin_bwd_dq`,
// `_lin_bwd_dkdv` (reference models/sla2_vendor/kernel.py,
// models/triton_sla2_jvp.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace imf {

constexpr int LD = 64;             // head dim
constexpr int LW = 68;             // state row: 64 H columns, z, 3 x pad
constexpr int LSTATE = LD * LW;    // 4352 elements per state
constexpr float LIN_EPS = 1e-5f;

struct RowPtr {
  const void* p;
  int64_t sb, sl, sh;              // element strides of (batch, row, head); last dim contiguous
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float2 ld_bf16x2(const RowPtr& t, int b, int row, int h, int col) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(
      static_cast<const __nv_bfloat16*>(t.p) + b * t.sb + (int64_t)row * t.sl + h * t.sh + col);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float2 ld_f32x2(const RowPtr& t, int b, int row, int h, int col) {
  return *reinterpret_cast<const float2*>(static_cast<const float*>(t.p) + b * t.sb +
                                          (int64_t)row * t.sl + h * t.sh + col);
}

// One warp, one row: lane holds columns 2*lane, 2*lane+1.  phi = softmax(x);
// with a tangent dx: dphi = phi .* (dx - phi . dx).
__device__ __forceinline__ void softmax_row(float2 x, float2& phi) {
  const float m = warp_max(fmaxf(x.x, x.y));
  const float e0 = __expf(x.x - m), e1 = __expf(x.y - m);
  const float inv = 1.f / warp_sum(e0 + e1);
  phi = make_float2(e0 * inv, e1 * inv);
}
__device__ __forceinline__ void softmax_row_jvp(float2 phi, float2 dx, float2& dphi) {
  const float dot = warp_sum(phi.x * dx.x + phi.y * dx.y);
  dphi = make_float2(phi.x * (dx.x - dot), phi.y * (dx.y - dot));
}

// --------------------------------------------------------------------------
// 64 x 64 x 64 products in shared memory, on the tensor cores.  All matrices have pitch
// LP = 68 floats.  `mma.sync.m16n8k8` with TF32 inputs (fp32 values rounded to nearest, 10
// mantissa bits) and fp32 accumulation: the eight warps form a 4 x 2 grid, each with a
// 16 x 32 piece of the result (four 16 x 8 accumulator fragments).  The results go through a
// shared-memory tile S so that every thread ends up with the 4 x 4 block
//     acc[i][j] += sum_k A[r0 + i][k] * Bm[k][c0 + j]        (A_T: A[k][r0 + i])
// of the 16 x 16 thread grid that the row-wise epilogues of the callers are written for.
// Fragment layout (g = lane / 4, t = lane % 4): A (row g | g + 8, col t | t + 4),
// B (k t | t + 4, n g), C (row g | g + 8, col 2 t | 2 t + 1).  Must be called by all 256
// threads.  The result tile S may be one of the operands' tiles: `frags_to_blocks` starts with
// a block-wide barrier, after which no thread reads an operand any more.
// --------------------------------------------------------------------------
constexpr int LP = LW;

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4],
                                         const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// d[n][.] += (A or A^T)[rows mr .. mr + 15][:] * Bm[:][cols nc + 8 n .. + 7], n = 0 .. 3
template <bool A_T>
__device__ __forceinline__ void warp_mm_tf32(const float* __restrict__ A,
                                             const float* __restrict__ Bm, int mr, int nc,
                                             int g, int t, float (&d)[4][4]) {
#pragma unroll 2
  for (int k = 0; k < 64; k += 8) {
    uint32_t a[4];
    if (A_T) {
      a[0] = to_tf32(A[(k + t) * LP + mr + g]);
      a[1] = to_tf32(A[(k + t) * LP + mr + g + 8]);
      a[2] = to_tf32(A[(k + t + 4) * LP + mr + g]);
      a[3] = to_tf32(A[(k + t + 4) * LP + mr + g + 8]);
    } else {
      a[0] = to_tf32(A[(mr + g) * LP + k + t]);
      a[1] = to_tf32(A[(mr + g + 8) * LP + k + t]);
      a[2] = to_tf32(A[(mr + g) * LP + k + t + 4]);
      a[3] = to_tf32(A[(mr + g + 8) * LP + k + t + 4]);
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      uint32_t b[2];
      b[0] = to_tf32(Bm[(k + t) * LP + nc + n * 8 + g]);
      b[1] = to_tf32(Bm[(k + t + 4) * LP + nc + n * 8 + g]);
      mma_tf32(d[n], a, b);
    }
  }
}

// fragments -> S -> 4 x 4 blocks (added to acc)
__device__ __forceinline__ void frags_to_blocks(const float (&d)[4][4], float* __restrict__ S,
                                                int mr, int nc, int g, int t, int r0, int c0,
                                                float (&acc)[4][4]) {
  __syncthreads();                  // earlier readers of S are done
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    *reinterpret_cast<float2*>(S + (mr + g) * LP + nc + n * 8 + 2 * t) = make_float2(d[n][0], d[n][1]);
    *reinterpret_cast<float2*>(S + (mr + g + 8) * LP + nc + n * 8 + 2 * t) = make_float2(d[n][2], d[n][3]);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = *reinterpret_cast<const float4*>(S + (r0 + i) * LP + c0);
    acc[i][0] += v.x; acc[i][1] += v.y; acc[i][2] += v.z; acc[i][3] += v.w;
  }
}

// position of a thread in the warp grid / fragment layout of the products above
struct MmaPos {
  int mr, nc, g, t;
  __device__ __forceinline__ explicit MmaPos(int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    mr = (warp & 3) * 16;
    nc = (warp >> 2) * 32;
    g = lane >> 2;
    t = lane & 3;
  }
};

// --------------------------------------------------------------------------
// State build: per block of `bs` rows, S = [ phi(X)^T Y | phi(X)^T w ] and the
// tangent [ dphi^T Y + phi^T dY | dphi^T w ], written as bf16 hi / lo pairs.
// --------------------------------------------------------------------------
struct StatesArgs {
  RowPtr x, dx, y, dy;
  const float* w;          // (B, H, L) weights of the extra column or null (= 1)
  __nv_bfloat16* out;      // [(b, h)][2 * nblk_pad][LSTATE]: hi rows then lo rows
  __nv_bfloat16* dout;
  int L, H, bs, nblk_pad, lim, y_fp32, tangent;
};

template <bool TANGENT>
__global__ void __launch_bounds__(256) lin_states_kernel(const StatesArgs a) {
  extern __shared__ __align__(16) float sm[];
  float* X = sm;                     // [64][LP]  phi rows
  float* Y = X + 64 * LP;            // [64][LP]  y rows | w
  float* S = X;                      // result tile of the products: X is dead by then
  float* dX = Y + 64 * LP;           // tangent only
  float* dY = dX + 64 * LP;
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int d0 = (tid >> 4) * 4, e0 = (tid & 15) * 4;
  const int g = lane >> 2, t = lane & 3, mr = (warp & 3) * 16, nc = (warp >> 2) * 32;
  float acc[4][4] = {}, dacc[4][4] = {};
  float fr[4][4] = {}, dfr[4][4] = {};       // accumulator fragments of X^T Y and its tangent
  float zacc = 0.f, dzacc = 0.f;
  for (int c0 = 0; c0 < a.bs; c0 += 64) {
    // Every warp has eight rows.  All their loads are issued before the first softmax (a
    // row at a time would put eight global-memory latencies end to end), and the unrolled
    // softmaxes give the scheduler eight independent shuffle chains.
    float2 xr[8], yr[8], dxr[8], dyr[8];
    float wr[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = n * a.bs + c0 + warp + 8 * i;
      xr[i] = yr[i] = dxr[i] = dyr[i] = make_float2(0.f, 0.f);
      wr[i] = 0.f;
      if (row < a.lim) {
        xr[i] = ld_bf16x2(a.x, b, row, h, 2 * lane);
        yr[i] = a.y_fp32 ? ld_f32x2(a.y, b, row, h, 2 * lane) : ld_bf16x2(a.y, b, row, h, 2 * lane);
        wr[i] = a.w ? a.w[((int64_t)b * a.H + h) * a.L + row] : 1.f;
        if (TANGENT) {
          dxr[i] = ld_bf16x2(a.dx, b, row, h, 2 * lane);
          dyr[i] = ld_bf16x2(a.dy, b, row, h, 2 * lane);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = warp + 8 * i;
      const bool valid = n * a.bs + c0 + rr < a.lim;
      float2 phi = make_float2(0.f, 0.f), dphi = phi;
      if (valid) {
        softmax_row(xr[i], phi);
        if (TANGENT) softmax_row_jvp(phi, dxr[i], dphi);
      }
      *reinterpret_cast<float2*>(X + rr * LP + 2 * lane) = phi;
      *reinterpret_cast<float2*>(Y + rr * LP + 2 * lane) = yr[i];
      if (lane == 0) Y[rr * LP + 64] = wr[i];
      if (TANGENT) {
        *reinterpret_cast<float2*>(dX + rr * LP + 2 * lane) = dphi;
        *reinterpret_cast<float2*>(dY + rr * LP + 2 * lane) = dyr[i];
      }
    }
    __syncthreads();
    // [d][e] += sum over the 64 rows of phi[row][d] * y[row][e]: X^T Y on the tensor cores
    warp_mm_tf32<true>(X, Y, mr, nc, g, t, fr);
    if (TANGENT) {
      warp_mm_tf32<true>(dX, Y, mr, nc, g, t, dfr);
      warp_mm_tf32<true>(X, dY, mr, nc, g, t, dfr);
    }
    if (tid < 64) {                  // the extra column: sum of phi weighted by w
#pragma unroll 8
      for (int rr = 0; rr < 64; ++rr) {
        const float wv = Y[rr * LP + 64];
        zacc = fmaf(X[rr * LP + tid], wv, zacc);
        if (TANGENT) dzacc = fmaf(dX[rr * LP + tid], wv, dzacc);
      }
    }
    __syncthreads();
  }
  frags_to_blocks(fr, S, mr, nc, g, t, d0, e0, acc);
  if (TANGENT) frags_to_blocks(dfr, S, mr, nc, g, t, d0, e0, dacc);
  const int64_t base = ((int64_t)b * a.H + h) * 2 * a.nblk_pad * LSTATE + (int64_t)n * LSTATE;
  const int64_t lo_off = (int64_t)a.nblk_pad * LSTATE;
  auto put = [&](__nv_bfloat16* dst, int d, int e, float v) {
    const __nv_bfloat16 hi = __float2bfloat16(v);
    dst[base + d * LW + e] = hi;
    dst[base + lo_off + d * LW + e] = __float2bfloat16(v - __bfloat162float(hi));
  };
  // four columns at a time: one 8-byte store of the hi parts and one of the lo parts
  auto put4 = [&](__nv_bfloat16* dst, int d, int e, const float (&v)[4]) {
    __align__(8) __nv_bfloat16 hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hi[j] = __float2bfloat16(v[j]);
      lo[j] = __float2bfloat16(v[j] - __bfloat162float(hi[j]));
    }
    *reinterpret_cast<uint2*>(dst + base + d * LW + e) = *reinterpret_cast<const uint2*>(hi);
    *reinterpret_cast<uint2*>(dst + base + lo_off + d * LW + e) = *reinterpret_cast<const uint2*>(lo);
  };
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    put4(a.out, d0 + i, e0, acc[i]);
    if (TANGENT) put4(a.dout, d0 + i, e0, dacc[i]);
  }
  if (tid < 64) {
    put(a.out, tid, 64, zacc);
    if (TANGENT) put(a.dout, tid, 64, dzacc);
#pragma unroll
    for (int e = 65; e < LW; ++e) {
      put(a.out, tid, e, 0.f);
      if (TANGENT) put(a.dout, tid, e, 0.f);
    }
  }
}

// sum over the 16 lanes that share a row group (lanes 0-15 / 16-31 of a warp)
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void load_state(float* dst, const float* src, int tid) {
  for (int i = tid * 4; i < LSTATE; i += 256 * 4)
    *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
}

// dst[e][d] = src[d][e] for d, e < 64 (both pitch LP, both in shared memory)
__device__ __forceinline__ void transpose_state(float* dst, const float* src, int tid) {
  const int d = tid & 63;
  for (int e = tid >> 6; e < 64; e += 4) dst[e * LP + d] = src[d * LP + e];
}

__device__ __forceinline__ __nv_bfloat16* row_at(const RowPtr& t, int b, int row, int h) {
  return static_cast<__nv_bfloat16*>(const_cast<void*>(t.p)) + b * t.sb + (int64_t)row * t.sl +
         h * t.sh;
}
__device__ __forceinline__ void ld_bf16x4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void st_bf16x4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned int*>(&lo);
  u.y = *reinterpret_cast<const unsigned int*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}

// --------------------------------------------------------------------------
// Apply (forward): o_l = phi(q) H / (phi(q) z + eps) per query block and the
// mix with the sparse branch; optional tangent.
// --------------------------------------------------------------------------
struct ApplyArgs {
  RowPtr q, dq, os, dos;
  const float* C;          // [(b, h)][Mb][LSTATE] complement states
  const float* dC;
  const float* a_rows;     // (H, L) mixing ratio per row
  RowPtr o, dout;          // bf16 outputs
  int L, H, Mb, qblk;
};

template <bool TANGENT>
__global__ void __launch_bounds__(256) lin_apply_kernel(const ApplyArgs a) {
  extern __shared__ __align__(16) float sm[];
  float* C = sm;                      // [64][LP]: H | z
  float* P = C + LSTATE;              // phi rows [64][LP]
  float* dC = P + 64 * LP;            // tangent only
  float* dP = dC + LSTATE;
  float* S = P;                       // result tile of the products (P is dead by then)
  __shared__ float Den[64], dDen[64];
  const int m = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t sidx = (((int64_t)b * a.H + h) * a.Mb + m) * LSTATE;
  load_state(C, a.C + sidx, tid);
  if (TANGENT) load_state(dC, a.dC + sidx, tid);
  __syncthreads();
  const float z0 = C[(2 * lane) * LP + 64], z1 = C[(2 * lane + 1) * LP + 64];
  const float dz0 = TANGENT ? dC[(2 * lane) * LP + 64] : 0.f;
  const float dz1 = TANGENT ? dC[(2 * lane + 1) * LP + 64] : 0.f;
  const int r0 = (tid >> 4) * 4, c0 = (tid & 15) * 4;
  for (int ch = 0; ch < a.qblk; ch += 64) {
    if (ch) __syncthreads();
    float2 qr[8], dqr[8];           // this warp's eight rows: loads first, then the softmaxes
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = m * a.qblk + ch + warp + 8 * i;
      qr[i] = dqr[i] = make_float2(0.f, 0.f);
      if (row < a.L) {
        qr[i] = ld_bf16x2(a.q, b, row, h, 2 * lane);
        if (TANGENT) dqr[i] = ld_bf16x2(a.dq, b, row, h, 2 * lane);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = warp + 8 * i;
      const int row = m * a.qblk + ch + rr;
      float2 phi = make_float2(0.f, 0.f), dphi = phi;
      if (row < a.L) {
        softmax_row(qr[i], phi);
        if (TANGENT) softmax_row_jvp(phi, dqr[i], dphi);
      }
      *reinterpret_cast<float2*>(P + rr * LP + 2 * lane) = phi;
      const float den = warp_sum(fmaf(phi.x, z0, phi.y * z1));
      if (TANGENT) {
        *reinterpret_cast<float2*>(dP + rr * LP + 2 * lane) = dphi;
        const float dd = warp_sum(fmaf(dphi.x, z0, dphi.y * z1) + fmaf(phi.x, dz0, phi.y * dz1));
        if (lane == 0) dDen[rr] = dd;
      }
      if (lane == 0) Den[rr] = den + LIN_EPS;
    }
    __syncthreads();
    float num[4][4] = {}, dnum[4][4] = {};
    {
      const MmaPos mp(tid);
      float fr[4][4] = {}, dfr[4][4] = {};
      warp_mm_tf32<false>(P, C, mp.mr, mp.nc, mp.g, mp.t, fr);
      if (TANGENT) {
        warp_mm_tf32<false>(dP, C, mp.mr, mp.nc, mp.g, mp.t, dfr);
        warp_mm_tf32<false>(P, dC, mp.mr, mp.nc, mp.g, mp.t, dfr);
      }
      frags_to_blocks(fr, S, mp.mr, mp.nc, mp.g, mp.t, r0, c0, num);
      if (TANGENT) frags_to_blocks(dfr, S, mp.mr, mp.nc, mp.g, mp.t, r0, c0, dnum);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = m * a.qblk + ch + r0 + i;
      if (row >= a.L) continue;
      const float inv = 1.f / Den[r0 + i];
      const float al = a.a_rows[(int64_t)h * a.L + row], bl = 1.f - al;
      float s[4], l[4];
      ld_bf16x4(row_at(a.os, b, row, h) + c0, s);
#pragma unroll
      for (int j = 0; j < 4; ++j) l[j] = num[i][j] * inv;
      st_bf16x4(row_at(a.o, b, row, h) + c0, al * s[0] + bl * l[0], al * s[1] + bl * l[1],
                al * s[2] + bl * l[2], al * s[3] + bl * l[3]);
      if (TANGENT) {
        const float dden = dDen[r0 + i];
        float t[4], g[4];
        ld_bf16x4(row_at(a.dos, b, row, h) + c0, t);
#pragma unroll
        for (int j = 0; j < 4; ++j) g[j] = (dnum[i][j] - l[j] * dden) * inv;
        st_bf16x4(row_at(a.dout, b, row, h) + c0, al * t[0] + bl * g[0], al * t[1] + bl * g[1],
                  al * t[2] + bl * g[2], al * t[3] + bl * g[3]);
      }
    }
  }
}

// --------------------------------------------------------------------------
// Reverse mode, row side.  Per query row with upstream gradient go of the mixed
// output:  u = (1 - a) go,  g_num = u / den,  g_den = -(u . o_l) / den,
//   g_phi = H g_num + g_den z,   g_q = phi .* (g_phi - phi . g_phi)
// Writes g_q (fp32, into the dQ accumulator of the sparse backward), g_num /
// g_den rows (inputs of the dL/dC state build), a go (bf16, upstream gradient of
// the sparse branch) and the per-row alpha-logit gradient a (1 - a) go . (o_s - o_l).
// Two tile products per 64 rows: phi H (num) and g_num H^T (g_phi).
// --------------------------------------------------------------------------
struct BwdRowsArgs {
  RowPtr q, os, go;
  const float* C;
  const float* a_rows;
  float* gq;               // (B, L, H, 64) fp32 contiguous
  float* gnum;             // (B, L, H, 64) fp32 contiguous
  float* gden;             // (B, H, L)
  float* ga_row;           // (B, H, L)
  RowPtr gos;              // bf16 out
  int L, H, Mb, qblk;
};

__global__ void __launch_bounds__(256) lin_bwd_rows_kernel(const BwdRowsArgs a) {
  extern __shared__ __align__(16) float sm[];
  float* C = sm;                      // [64 d][LP]: H | z
  float* Ct = C + LSTATE;             // [64 e][LP]: H^T
  float* P = Ct + 64 * LP;            // phi rows
  float* G = P + 64 * LP;             // g_num rows
  float* S = G;                       // result tile of the products (G is dead at both times)
  __shared__ float Den[64], GD[64];
  const int m = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  load_state(C, a.C + (((int64_t)b * a.H + h) * a.Mb + m) * LSTATE, tid);
  __syncthreads();
  transpose_state(Ct, C, tid);
  const float z0 = C[(2 * lane) * LP + 64], z1 = C[(2 * lane + 1) * LP + 64];
  const int r0 = (tid >> 4) * 4, c0 = (tid & 15) * 4, tx = tid & 15;
  float zc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) zc[j] = C[(c0 + j) * LP + 64];
  for (int ch = 0; ch < a.qblk; ch += 64) {
    if (ch) __syncthreads();
    float2 qr[8];                   // this warp's eight rows: loads first, then the softmaxes
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = m * a.qblk + ch + warp + 8 * i;
      qr[i] = row < a.L ? ld_bf16x2(a.q, b, row, h, 2 * lane) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = warp + 8 * i;
      float2 phi = make_float2(0.f, 0.f);
      if (m * a.qblk + ch + rr < a.L) softmax_row(qr[i], phi);
      *reinterpret_cast<float2*>(P + rr * LP + 2 * lane) = phi;
      const float den = warp_sum(fmaf(phi.x, z0, phi.y * z1));
      if (lane == 0) Den[rr] = den + LIN_EPS;
    }
    __syncthreads();                  // also orders the writes of Ct before its first use
    float num[4][4] = {};
    const MmaPos mp(tid);
    {
      float fr[4][4] = {};
      warp_mm_tf32<false>(P, C, mp.mr, mp.nc, mp.g, mp.t, fr);
      frags_to_blocks(fr, S, mp.mr, mp.nc, mp.g, mp.t, r0, c0, num);
      __syncthreads();              // S (= G) has been read: the g_num rows may go in
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = m * a.qblk + ch + r0 + i;
      const bool live = row < a.L;    // no early exit: the shuffles below need every lane
      const float inv = 1.f / Den[r0 + i];
      float gn[4] = {0.f, 0.f, 0.f, 0.f};
      float uo = 0.f, ga = 0.f, al = 0.f;
      if (live) {
        al = a.a_rows[(int64_t)h * a.L + row];
        float g[4], s[4];
        ld_bf16x4(row_at(a.go, b, row, h) + c0, g);
        ld_bf16x4(row_at(a.os, b, row, h) + c0, s);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float ol = num[i][j] * inv;
          const float u = (1.f - al) * g[j];
          uo = fmaf(u, ol, uo);
          ga = fmaf(g[j], s[j] - ol, ga);
          gn[j] = u * inv;
        }
        st_bf16x4(row_at(a.gos, b, row, h) + c0, al * g[0], al * g[1], al * g[2], al * g[3]);
        *reinterpret_cast<float4*>(a.gnum + (((int64_t)b * a.L + row) * a.H + h) * 64 + c0) =
            make_float4(gn[0], gn[1], gn[2], gn[3]);
      }
      *reinterpret_cast<float4*>(G + (r0 + i) * LP + c0) = make_float4(gn[0], gn[1], gn[2], gn[3]);
      uo = half_warp_sum(uo);
      ga = half_warp_sum(ga);
      if (tx == 0) {
        const float g_den = -uo * inv;
        GD[r0 + i] = g_den;
        if (live) {
          const int64_t so = ((int64_t)b * a.H + h) * a.L + row;
          a.gden[so] = g_den;
          a.ga_row[so] = al * (1.f - al) * ga;
        }
      }
    }
    __syncthreads();
    float gp[4][4] = {};
    {
      float fr[4][4] = {};
      warp_mm_tf32<false>(G, Ct, mp.mr, mp.nc, mp.g, mp.t, fr);       // columns are d here
      frags_to_blocks(fr, S, mp.mr, mp.nc, mp.g, mp.t, r0, c0, gp);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = m * a.qblk + ch + r0 + i;
      const float g_den = GD[r0 + i];
      const float4 p4 = *reinterpret_cast<const float4*>(P + (r0 + i) * LP + c0);
      const float ps[4] = {p4.x, p4.y, p4.z, p4.w};
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gp[i][j] = fmaf(g_den, zc[j], gp[i][j]);
        dot = fmaf(ps[j], gp[i][j], dot);
      }
      dot = half_warp_sum(dot);
      if (row < a.L)
        *reinterpret_cast<float4*>(a.gq + (((int64_t)b * a.L + row) * a.H + h) * 64 + c0) =
            make_float4(ps[0] * (gp[i][0] - dot), ps[1] * (gp[i][1] - dot),
                        ps[2] * (gp[i][2] - dot), ps[3] * (gp[i][3] - dot));
    }
  }
}

// --------------------------------------------------------------------------
// Reverse mode, key side.  Per key block with gS = [gH | gz]:
//   g_phi = gH v + gz,  g_k = phi .* (g_phi - phi . g_phi),  g_v = phi gH
// added to the sparse branch's dK / dV (bf16) and written as the final dK / dV.
// --------------------------------------------------------------------------
struct BwdKvArgs {
  RowPtr k, v, gks, gvs, gk, gv;
  const float* gS;          // [(b, h)][Nb][LSTATE]
  int L, H, Nb, lim;
};

__global__ void __launch_bounds__(256) lin_bwd_kv_kernel(const BwdKvArgs a) {
  extern __shared__ __align__(16) float sm[];
  float* C = sm;                      // [64 d][LP]: gH | gz
  float* Ct = C + LSTATE;             // [64 e][LP]: gH^T
  float* P = Ct + 64 * LP;            // phi(k) rows
  float* V = P + 64 * LP;             // v rows
  float* S = V;                       // result tile of the products (V is dead by then)
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  load_state(C, a.gS + (((int64_t)b * a.H + h) * a.Nb + n) * LSTATE, tid);
  {
    float2 kr[8], vr[8];              // this warp's eight rows: loads first, then the softmaxes
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = n * 64 + warp + 8 * i;
      kr[i] = vr[i] = make_float2(0.f, 0.f);
      if (row < a.lim) {
        kr[i] = ld_bf16x2(a.k, b, row, h, 2 * lane);
        vr[i] = ld_bf16x2(a.v, b, row, h, 2 * lane);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = warp + 8 * i;
      float2 phi = make_float2(0.f, 0.f);
      if (n * 64 + rr < a.lim) softmax_row(kr[i], phi);
      *reinterpret_cast<float2*>(P + rr * LP + 2 * lane) = phi;
      *reinterpret_cast<float2*>(V + rr * LP + 2 * lane) = vr[i];
    }
  }
  __syncthreads();
  transpose_state(Ct, C, tid);
  const int r0 = (tid >> 4) * 4, c0 = (tid & 15) * 4;
  float gv[4][4] = {}, gp[4][4] = {};
  {
    const MmaPos mp(tid);
    float f1[4][4] = {}, f2[4][4] = {};
    __syncthreads();                  // Ct is complete
    warp_mm_tf32<false>(P, C, mp.mr, mp.nc, mp.g, mp.t, f1);     // g_v, columns e
    warp_mm_tf32<false>(V, Ct, mp.mr, mp.nc, mp.g, mp.t, f2);    // g_phi, columns d
    frags_to_blocks(f1, S, mp.mr, mp.nc, mp.g, mp.t, r0, c0, gv);
    frags_to_blocks(f2, S, mp.mr, mp.nc, mp.g, mp.t, r0, c0, gp);
  }
  float gz[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) gz[j] = C[(c0 + j) * LP + 64];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = n * 64 + r0 + i;
    const float4 p4 = *reinterpret_cast<const float4*>(P + (r0 + i) * LP + c0);
    const float ps[4] = {p4.x, p4.y, p4.z, p4.w};
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      gp[i][j] += gz[j];
      dot = fmaf(ps[j], gp[i][j], dot);
    }
    dot = half_warp_sum(dot);         // every lane takes part; rows past L only skip the stores
    if (row >= a.L) continue;
    float s[4];
    ld_bf16x4(row_at(a.gvs, b, row, h) + c0, s);
    st_bf16x4(row_at(a.gv, b, row, h) + c0, s[0] + gv[i][0], s[1] + gv[i][1], s[2] + gv[i][2],
              s[3] + gv[i][3]);
    ld_bf16x4(row_at(a.gks, b, row, h) + c0, s);
    st_bf16x4(row_at(a.gk, b, row, h) + c0, s[0] + ps[0] * (gp[i][0] - dot),
              s[1] + ps[1] * (gp[i][1] - dot), s[2] + ps[2] * (gp[i][2] - dot),
              s[3] + ps[3] * (gp[i][3] - dot));
  }
}


// 8-byte accesses of four bf16: base pointers 8-byte aligned, strides multiples of 4 elements
static bool rows_vec4_ok(const void* const* ptrs, int n, const int64_t* strides) {
  for (int i = 0; i < n; ++i) {
    if (!ptrs[i]) continue;
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 7) return false;
    for (int j = 0; j < 3; ++j)
      if (strides[3 * i + j] & 3) return false;
  }
  return true;
}

// --------------------------------------------------------------------------
// 0/1 complement masks of the selection, duplicated for the (hi, lo) halves of
// the states: cm[(b,h)][m][n] = cm[(b,h)][m][cp + n] = 1 unless key block n is
// selected by query block m (n < Nb; pads are 0).  `transposed` writes the
// [(b,h)][n][2 * pad4(Mb)] form instead, in two launches (fill, then clear).
// --------------------------------------------------------------------------
__global__ void comp_mask_rows_kernel(const int* __restrict__ sel, __nv_bfloat16* __restrict__ cm,
                                      int Mb, int Nb, int T, int cp) {
  const int m = blockIdx.x;
  const size_t bh = blockIdx.y;
  __nv_bfloat16* row = cm + (bh * Mb + m) * (size_t)(2 * cp);
  const __nv_bfloat16 one = __float2bfloat16(1.f), zero = __float2bfloat16(0.f);
  for (int i = threadIdx.x; i < 2 * cp; i += blockDim.x) {
    const int n = i < cp ? i : i - cp;
    row[i] = n < Nb ? one : zero;
  }
  __syncthreads();
  const int* s = sel + (bh * Mb + m) * (size_t)T;
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    const int n = s[t];
    if (n >= 0 && n < Nb) {
      row[n] = zero;
      row[cp + n] = zero;
    }
  }
}

__global__ void comp_mask_fill_t_kernel(__nv_bfloat16* __restrict__ cm, int Mb, int cp) {
  const size_t rowi = (size_t)blockIdx.y * gridDim.x + blockIdx.x;     // (bh, n)
  __nv_bfloat16* row = cm + rowi * (size_t)(2 * cp);
  const __nv_bfloat16 one = __float2bfloat16(1.f), zero = __float2bfloat16(0.f);
  for (int i = threadIdx.x; i < 2 * cp; i += blockDim.x) {
    const int m = i < cp ? i : i - cp;
    row[i] = m < Mb ? one : zero;
  }
}

__global__ void comp_mask_clear_t_kernel(const int* __restrict__ sel,
                                         __nv_bfloat16* __restrict__ cm, int Mb, int Nb, int T,
                                         int cp) {
  const int m = blockIdx.x;
  const size_t bh = blockIdx.y;
  const int* s = sel + (bh * Mb + m) * (size_t)T;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    const int n = s[t];
    if (n >= 0 && n < Nb) {
      __nv_bfloat16* row = cm + (bh * Nb + n) * (size_t)(2 * cp);
      row[m] = zero;
      row[cp + m] = zero;
    }
  }
}

static RowPtr row_ptr(const void* p, const int64_t* st) {
  RowPtr r;
  r.p = p;
  r.sb = st[0];
  r.sl = st[1];
  r.sh = st[2];
  return r;
}

template <typename K>
static int set_smem(K kern, size_t bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) ==
                 cudaSuccess
             ? 0
             : -3;
}

}  // namespace imf

using namespace imf;

extern "C" int imf_lin_state_elems() { return LSTATE; }

// sel (BH, Mb, T) int32 -> cm (BH, Mb, 2 * pad4(Nb)) bf16, or with `transposed`
// (BH, Nb, 2 * pad4(Mb)).
extern "C" int imf_comp_mask(const int* sel, void* cm, int BH, int Mb, int Nb, int T,
                             int transposed, void* stream) {
  if (BH <= 0 || Mb <= 0 || Nb <= 0 || T <= 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(cm);
  if (!transposed) {
    comp_mask_rows_kernel<<<dim3(Mb, BH), 128, 0, st>>>(sel, out, Mb, Nb, T, (Nb + 3) / 4 * 4);
  } else {
    const int cp = (Mb + 3) / 4 * 4;
    comp_mask_fill_t_kernel<<<dim3(Nb, BH), 128, 0, st>>>(out, Mb, cp);
    comp_mask_clear_t_kernel<<<dim3(Mb, BH), 64, 0, st>>>(sel, out, Mb, Nb, T, cp);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// strides: x(3), dx(3), y(3), dy(3) element strides (batch, row, head).
extern "C" int imf_lin_states(const void* x, const void* dx, const void* y, const void* dy,
                              const float* w, void* out, void* dout, int B, int L, int H, int bs,
                              int nblk, int nblk_pad, int lim, int y_fp32, const int64_t* strides,
                              void* stream) {
  if (bs % 64 || nblk_pad < nblk || B <= 0 || L <= 0 || H <= 0) return -1;
  StatesArgs a;
  a.x = row_ptr(x, strides);
  a.dx = row_ptr(dx, strides + 3);
  a.y = row_ptr(y, strides + 6);
  a.dy = row_ptr(dy, strides + 9);
  a.w = w;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.dout = static_cast<__nv_bfloat16*>(dout);
  a.L = L; a.H = H; a.bs = bs; a.nblk_pad = nblk_pad; a.lim = lim < L ? lim : L; a.y_fp32 = y_fp32;
  a.tangent = dx != nullptr;
  const dim3 grid(nblk, H, B);
  const size_t tile = (size_t)64 * LP * sizeof(float);      // X, Y (+ dX, dY with a tangent)
  if (dx) {
    if (set_smem(lin_states_kernel<true>, 4 * tile)) return -3;
    lin_states_kernel<true><<<grid, 256, 4 * tile, (cudaStream_t)stream>>>(a);
  } else {
    lin_states_kernel<false><<<grid, 256, 2 * tile, (cudaStream_t)stream>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// strides: q(3), dq(3), os(3), dos(3), o(3), dout(3).
extern "C" int imf_lin_apply(const void* q, const void* dq, const void* os, const void* dos,
                             const float* C, const float* dC, const float* a_rows, void* o,
                             void* dout, int B, int L, int H, int Mb, int qblk,
                             const int64_t* strides, void* stream) {
  if (qblk % 64 || B <= 0) return -1;
  const void* ptrs[6] = {q, dq, os, dos, o, dout};
  if (!rows_vec4_ok(ptrs, 6, strides)) return -2;
  ApplyArgs a;
  a.q = row_ptr(q, strides);
  a.dq = row_ptr(dq, strides + 3);
  a.os = row_ptr(os, strides + 6);
  a.dos = row_ptr(dos, strides + 9);
  a.o = row_ptr(o, strides + 12);
  a.dout = row_ptr(dout, strides + 15);
  a.C = C; a.dC = dC; a.a_rows = a_rows;
  a.L = L; a.H = H; a.Mb = Mb; a.qblk = qblk;
  const dim3 grid(Mb, H, B);
  const size_t base = (size_t)(LSTATE + 64 * LP) * sizeof(float);
  if (dq) {
    if (set_smem(lin_apply_kernel<true>, 2 * base)) return -3;
    lin_apply_kernel<true><<<grid, 256, 2 * base, (cudaStream_t)stream>>>(a);
  } else {
    lin_apply_kernel<false><<<grid, 256, base, (cudaStream_t)stream>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// strides: q(3), os(3), go(3), gos(3).  gq / gnum: (B, L, H, 64) fp32 contiguous.
extern "C" int imf_lin_bwd_rows(const void* q, const void* os, const void* go, const float* C,
                                const float* a_rows, float* gq, float* gnum, float* gden,
                                float* ga_row, void* gos, int B, int L, int H, int Mb, int qblk,
                                const int64_t* strides, void* stream) {
  if (qblk % 64 || B <= 0) return -1;
  const void* ptrs[4] = {q, os, go, gos};
  if (!rows_vec4_ok(ptrs, 4, strides)) return -2;
  BwdRowsArgs a;
  a.q = row_ptr(q, strides);
  a.os = row_ptr(os, strides + 3);
  a.go = row_ptr(go, strides + 6);
  a.gos = row_ptr(gos, strides + 9);
  a.C = C; a.a_rows = a_rows; a.gq = gq; a.gnum = gnum; a.gden = gden; a.ga_row = ga_row;
  a.L = L; a.H = H; a.Mb = Mb; a.qblk = qblk;
  const size_t smem = (size_t)(LSTATE + 3 * 64 * LP) * sizeof(float);
  if (set_smem(lin_bwd_rows_kernel, smem)) return -3;
  lin_bwd_rows_kernel<<<dim3(Mb, H, B), 256, smem, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// strides: k(3), v(3), gks(3), gvs(3), gk(3), gv(3).
extern "C" int imf_lin_bwd_kv(const void* k, const void* v, const void* gks, const void* gvs,
                              const float* gS, void* gk, void* gv, int B, int L, int H, int Nb,
                              int lim, const int64_t* strides, void* stream) {
  if (B <= 0) return -1;
  const void* ptrs[6] = {k, v, gks, gvs, gk, gv};
  if (!rows_vec4_ok(ptrs, 6, strides)) return -2;
  BwdKvArgs a;
  a.k = row_ptr(k, strides);
  a.v = row_ptr(v, strides + 3);
  a.gks = row_ptr(gks, strides + 6);
  a.gvs = row_ptr(gvs, strides + 9);
  a.gk = row_ptr(gk, strides + 12);
  a.gv = row_ptr(gv, strides + 15);
  a.gS = gS; a.L = L; a.H = H; a.Nb = Nb; a.lim = lim < L ? lim : L;
  const size_t smem = (size_t)(LSTATE + 3 * 64 * LP) * sizeof(float);
  if (set_smem(lin_bwd_kv_kernel, smem)) return -3;
  lin_bwd_kv_kernel<<<dim3(Nb, H, B), 256, smem, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
