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
// (phi(q), dL/dnum | dL/dden) to get dL/dC).  Every reduction has a fixed
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
  extern __shared__ float sm[];
  float* X = sm;                     // [64][64]
  float* Y = X + 64 * 64;            // [64][68]
  float* dX = Y + 64 * LW;           // tangent only
  float* dY = dX + 64 * 64;
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int d0 = (tid >> 4) * 4, e0 = (tid & 15) * 4;
  float acc[4][4] = {}, dacc[4][4] = {};
  float zacc = 0.f, dzacc = 0.f;
  for (int c0 = 0; c0 < a.bs; c0 += 64) {
    for (int rr = warp; rr < 64; rr += 8) {
      const int row = n * a.bs + c0 + rr;
      const bool valid = row < a.lim;
      float2 phi = make_float2(0.f, 0.f), dphi = phi, yv = phi, dyv = phi;
      float wv = 0.f;
      if (valid) {
        softmax_row(ld_bf16x2(a.x, b, row, h, 2 * lane), phi);
        yv = a.y_fp32 ? ld_f32x2(a.y, b, row, h, 2 * lane) : ld_bf16x2(a.y, b, row, h, 2 * lane);
        wv = a.w ? a.w[((int64_t)b * a.H + h) * a.L + row] : 1.f;
        if (TANGENT) {
          softmax_row_jvp(phi, ld_bf16x2(a.dx, b, row, h, 2 * lane), dphi);
          dyv = ld_bf16x2(a.dy, b, row, h, 2 * lane);
        }
      }
      *reinterpret_cast<float2*>(X + rr * 64 + 2 * lane) = phi;
      *reinterpret_cast<float2*>(Y + rr * LW + 2 * lane) = yv;
      if (lane == 0) Y[rr * LW + 64] = wv;
      if (TANGENT) {
        *reinterpret_cast<float2*>(dX + rr * 64 + 2 * lane) = dphi;
        *reinterpret_cast<float2*>(dY + rr * LW + 2 * lane) = dyv;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int rr = 0; rr < 64; ++rr) {
      const float4 xa = *reinterpret_cast<const float4*>(X + rr * 64 + d0);
      const float4 yb = *reinterpret_cast<const float4*>(Y + rr * LW + e0);
      const float xs[4] = {xa.x, xa.y, xa.z, xa.w}, ys[4] = {yb.x, yb.y, yb.z, yb.w};
      float dxs[4], dys[4];
      if (TANGENT) {
        const float4 da = *reinterpret_cast<const float4*>(dX + rr * 64 + d0);
        const float4 db = *reinterpret_cast<const float4*>(dY + rr * LW + e0);
        dxs[0] = da.x; dxs[1] = da.y; dxs[2] = da.z; dxs[3] = da.w;
        dys[0] = db.x; dys[1] = db.y; dys[2] = db.z; dys[3] = db.w;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(xs[i], ys[j], acc[i][j]);
          if (TANGENT) dacc[i][j] = fmaf(dxs[i], ys[j], fmaf(xs[i], dys[j], dacc[i][j]));
        }
      if (tid < 64) {
        const float wv = Y[rr * LW + 64];
        zacc = fmaf(X[rr * 64 + tid], wv, zacc);
        if (TANGENT) dzacc = fmaf(dX[rr * 64 + tid], wv, dzacc);
      }
    }
    __syncthreads();
  }
  const int64_t base = ((int64_t)b * a.H + h) * 2 * a.nblk_pad * LSTATE + (int64_t)n * LSTATE;
  const int64_t lo_off = (int64_t)a.nblk_pad * LSTATE;
  auto put = [&](__nv_bfloat16* dst, int d, int e, float v) {
    const __nv_bfloat16 hi = __float2bfloat16(v);
    dst[base + d * LW + e] = hi;
    dst[base + lo_off + d * LW + e] = __float2bfloat16(v - __bfloat162float(hi));
  };
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      put(a.out, d0 + i, e0 + j, acc[i][j]);
      if (TANGENT) put(a.dout, d0 + i, e0 + j, dacc[i][j]);
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

__device__ __forceinline__ void load_state(float* dst, const float* src, int tid) {
  for (int i = tid * 4; i < LSTATE; i += 256 * 4)
    *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
}

template <bool TANGENT>
__global__ void __launch_bounds__(256) lin_apply_kernel(const ApplyArgs a) {
  extern __shared__ float sm[];
  float* C = sm;                      // [64][68]
  float* P = C + LSTATE;              // phi rows [64][65]
  float* dC = P + 64 * 65;
  float* dP = dC + LSTATE;
  const int m = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t sidx = (((int64_t)b * a.H + h) * a.Mb + m) * LSTATE;
  load_state(C, a.C + sidx, tid);
  if (TANGENT) load_state(dC, a.dC + sidx, tid);
  const int r = tid >> 2, e0 = (tid & 3) * 16;
  for (int c0 = 0; c0 < a.qblk; c0 += 64) {
    __syncthreads();
    for (int rr = warp; rr < 64; rr += 8) {
      const int row = m * a.qblk + c0 + rr;
      float2 phi = make_float2(0.f, 0.f), dphi = phi;
      if (row < a.L) {
        softmax_row(ld_bf16x2(a.q, b, row, h, 2 * lane), phi);
        if (TANGENT) softmax_row_jvp(phi, ld_bf16x2(a.dq, b, row, h, 2 * lane), dphi);
      }
      P[rr * 65 + 2 * lane] = phi.x;
      P[rr * 65 + 2 * lane + 1] = phi.y;
      if (TANGENT) {
        dP[rr * 65 + 2 * lane] = dphi.x;
        dP[rr * 65 + 2 * lane + 1] = dphi.y;
      }
    }
    __syncthreads();
    const int row = m * a.qblk + c0 + r;
    float num[16] = {}, dnum[16] = {};
    float den = LIN_EPS, dden = 0.f;
#pragma unroll 2
    for (int d = 0; d < 64; ++d) {
      const float f = P[r * 65 + d];
      const float df = TANGENT ? dP[r * 65 + d] : 0.f;
      den = fmaf(f, C[d * LW + 64], den);
      if (TANGENT) dden = fmaf(df, C[d * LW + 64], fmaf(f, dC[d * LW + 64], dden));
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 c4 = *reinterpret_cast<const float4*>(C + d * LW + e0 + j);
        num[j] = fmaf(f, c4.x, num[j]);
        num[j + 1] = fmaf(f, c4.y, num[j + 1]);
        num[j + 2] = fmaf(f, c4.z, num[j + 2]);
        num[j + 3] = fmaf(f, c4.w, num[j + 3]);
        if (TANGENT) {
          const float4 t4 = *reinterpret_cast<const float4*>(dC + d * LW + e0 + j);
          dnum[j] = fmaf(df, c4.x, fmaf(f, t4.x, dnum[j]));
          dnum[j + 1] = fmaf(df, c4.y, fmaf(f, t4.y, dnum[j + 1]));
          dnum[j + 2] = fmaf(df, c4.z, fmaf(f, t4.z, dnum[j + 2]));
          dnum[j + 3] = fmaf(df, c4.w, fmaf(f, t4.w, dnum[j + 3]));
        }
      }
    }
    if (row < a.L) {
      const float inv = 1.f / den;
      const float al = a.a_rows[(int64_t)h * a.L + row], bl = 1.f - al;
      const __nv_bfloat16* os = static_cast<const __nv_bfloat16*>(a.os.p) + b * a.os.sb +
                                (int64_t)row * a.os.sl + h * a.os.sh + e0;
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(const_cast<void*>(a.o.p)) + b * a.o.sb +
                         (int64_t)row * a.o.sl + h * a.o.sh + e0;
      const __nv_bfloat16* dos = nullptr;
      __nv_bfloat16* dout = nullptr;
      if (TANGENT) {
        dos = static_cast<const __nv_bfloat16*>(a.dos.p) + b * a.dos.sb + (int64_t)row * a.dos.sl +
              h * a.dos.sh + e0;
        dout = static_cast<__nv_bfloat16*>(const_cast<void*>(a.dout.p)) + b * a.dout.sb +
               (int64_t)row * a.dout.sl + h * a.dout.sh + e0;
      }
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const float2 s2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(os + j));
        const float l0 = num[j] * inv, l1 = num[j + 1] * inv;
        *reinterpret_cast<__nv_bfloat162*>(o + j) =
            __floats2bfloat162_rn(al * s2.x + bl * l0, al * s2.y + bl * l1);
        if (TANGENT) {
          const float2 t2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dos + j));
          const float g0 = (dnum[j] - l0 * dden) * inv, g1 = (dnum[j + 1] - l1 * dden) * inv;
          *reinterpret_cast<__nv_bfloat162*>(dout + j) =
              __floats2bfloat162_rn(al * t2.x + bl * g0, al * t2.y + bl * g1);
        }
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
  extern __shared__ float sm[];
  float* C = sm;                      // [64][69]: odd pitch, rows are read with stride 4 below
  float* P = C + 64 * 69;             // phi rows [64][65]
  float* G = P + 64 * 65;             // g_num rows [64][65]
  const int m = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* src = a.C + (((int64_t)b * a.H + h) * a.Mb + m) * LSTATE;
  for (int i = tid; i < 64 * LW; i += 256) {
    const int d = i / LW, e = i - d * LW;
    C[d * 69 + e] = src[i];
  }
  const int r = tid >> 2, qd = tid & 3, e0 = qd * 16;
  for (int c0 = 0; c0 < a.qblk; c0 += 64) {
    __syncthreads();
    for (int rr = warp; rr < 64; rr += 8) {
      const int row = m * a.qblk + c0 + rr;
      float2 phi = make_float2(0.f, 0.f);
      if (row < a.L) softmax_row(ld_bf16x2(a.q, b, row, h, 2 * lane), phi);
      P[rr * 65 + 2 * lane] = phi.x;
      P[rr * 65 + 2 * lane + 1] = phi.y;
    }
    __syncthreads();
    const int row = m * a.qblk + c0 + r;
    const bool live = row < a.L;
    float num[16] = {};
    float den = LIN_EPS;
    for (int d = 0; d < 64; ++d) {
      const float f = P[r * 65 + d];
      den = fmaf(f, C[d * 69 + 64], den);
#pragma unroll
      for (int j = 0; j < 16; ++j) num[j] = fmaf(f, C[d * 69 + e0 + j], num[j]);
    }
    const float inv = 1.f / den;
    float al = 0.f, uo = 0.f, ga = 0.f;
    float gn[16];
    const int64_t roff = (((int64_t)b * a.L + row) * a.H + h) * 64 + e0;
    if (live) {
      al = a.a_rows[(int64_t)h * a.L + row];
      const __nv_bfloat16* go = static_cast<const __nv_bfloat16*>(a.go.p) + b * a.go.sb +
                                (int64_t)row * a.go.sl + h * a.go.sh + e0;
      const __nv_bfloat16* os = static_cast<const __nv_bfloat16*>(a.os.p) + b * a.os.sb +
                                (int64_t)row * a.os.sl + h * a.os.sh + e0;
      __nv_bfloat16* gos = static_cast<__nv_bfloat16*>(const_cast<void*>(a.gos.p)) + b * a.gos.sb +
                           (int64_t)row * a.gos.sl + h * a.gos.sh + e0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float g = __bfloat162float(go[j]);
        const float ol = num[j] * inv;
        const float u = (1.f - al) * g;
        uo = fmaf(u, ol, uo);
        ga = fmaf(g, __bfloat162float(os[j]) - ol, ga);
        gn[j] = u * inv;
        gos[j] = __float2bfloat16(al * g);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) gn[j] = 0.f;
    }
    // the four threads of a row hold 16 columns each
    uo += __shfl_xor_sync(0xffffffffu, uo, 1);
    uo += __shfl_xor_sync(0xffffffffu, uo, 2);
    ga += __shfl_xor_sync(0xffffffffu, ga, 1);
    ga += __shfl_xor_sync(0xffffffffu, ga, 2);
    const float g_den = -uo * inv;
#pragma unroll
    for (int j = 0; j < 16; ++j) G[r * 65 + e0 + j] = gn[j];
    if (live) {
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(a.gnum + roff + j) = make_float4(gn[j], gn[j + 1], gn[j + 2], gn[j + 3]);
      if (qd == 0) {
        const int64_t so = ((int64_t)b * a.H + h) * a.L + row;
        a.gden[so] = g_den;
        a.ga_row[so] = al * (1.f - al) * ga;
      }
    }
    __syncthreads();
    // g_phi for d = qd + 4 i
    float gp[16];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = qd + 4 * i;
      float acc = g_den * C[d * 69 + 64];
      for (int e = 0; e < 64; ++e) acc = fmaf(C[d * 69 + e], G[r * 65 + e], acc);
      gp[i] = acc;
      dot = fmaf(P[r * 65 + d], acc, dot);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    if (live) {
      float* gq = a.gq + (((int64_t)b * a.L + row) * a.H + h) * 64;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int d = qd + 4 * i;
        gq[d] = P[r * 65 + d] * (gp[i] - dot);
      }
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
  extern __shared__ float sm[];
  float* C = sm;                      // [64][69]
  float* P = C + 64 * 69;             // phi(k) rows [64][65]
  float* V = P + 64 * 65;             // v rows [64][65]
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* src = a.gS + (((int64_t)b * a.H + h) * a.Nb + n) * LSTATE;
  for (int i = tid; i < 64 * LW; i += 256) {
    const int d = i / LW, e = i - d * LW;
    C[d * 69 + e] = src[i];
  }
  for (int rr = warp; rr < 64; rr += 8) {
    const int row = n * 64 + rr;
    float2 phi = make_float2(0.f, 0.f), vv = phi;
    if (row < a.lim) {
      softmax_row(ld_bf16x2(a.k, b, row, h, 2 * lane), phi);
      vv = ld_bf16x2(a.v, b, row, h, 2 * lane);
    }
    P[rr * 65 + 2 * lane] = phi.x;
    P[rr * 65 + 2 * lane + 1] = phi.y;
    V[rr * 65 + 2 * lane] = vv.x;
    V[rr * 65 + 2 * lane + 1] = vv.y;
  }
  __syncthreads();
  const int r = tid >> 2, qd = tid & 3, e0 = qd * 16;
  const int row = n * 64 + r;
  const bool live = row < a.L;       // no early return: the shuffles below need every lane
  // g_v for columns e0 .. e0 + 15
  float gv[16] = {};
  for (int d = 0; d < 64; ++d) {
    const float f = P[r * 65 + d];
#pragma unroll
    for (int j = 0; j < 16; ++j) gv[j] = fmaf(f, C[d * 69 + e0 + j], gv[j]);
  }
  // g_phi for d = qd + 4 i
  float gp[16];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = qd + 4 * i;
    float acc = C[d * 69 + 64];
    for (int e = 0; e < 64; ++e) acc = fmaf(C[d * 69 + e], V[r * 65 + e], acc);
    gp[i] = acc;
    dot = fmaf(P[r * 65 + d], acc, dot);
  }
  dot += __shfl_xor_sync(0xffffffffu, dot, 1);
  dot += __shfl_xor_sync(0xffffffffu, dot, 2);
  if (!live) return;
  auto at = [&](const RowPtr& t) {
    return static_cast<__nv_bfloat16*>(const_cast<void*>(t.p)) + b * t.sb + (int64_t)row * t.sl +
           h * t.sh;
  };
  const __nv_bfloat16 *gks = at(a.gks), *gvs = at(a.gvs);
  __nv_bfloat16 *gk = at(a.gk), *gvo = at(a.gv);
#pragma unroll
  for (int j = 0; j < 16; ++j)
    gvo[e0 + j] = __float2bfloat16(__bfloat162float(gvs[e0 + j]) + gv[j]);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = qd + 4 * i;
    gk[d] = __float2bfloat16(__bfloat162float(gks[d]) + P[r * 65 + d] * (gp[i] - dot));
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
  const size_t base = (size_t)(64 * 64 + 64 * LW) * sizeof(float);
  if (dx) {
    if (set_smem(lin_states_kernel<true>, 2 * base)) return -3;
    lin_states_kernel<true><<<grid, 256, 2 * base, (cudaStream_t)stream>>>(a);
  } else {
    lin_states_kernel<false><<<grid, 256, base, (cudaStream_t)stream>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// strides: q(3), dq(3), os(3), dos(3), o(3), dout(3).
extern "C" int imf_lin_apply(const void* q, const void* dq, const void* os, const void* dos,
                             const float* C, const float* dC, const float* a_rows, void* o,
                             void* dout, int B, int L, int H, int Mb, int qblk,
                             const int64_t* strides, void* stream) {
  if (qblk % 64 || B <= 0) return -1;
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
  const size_t base = (size_t)(LSTATE + 64 * 65) * sizeof(float);
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
  BwdRowsArgs a;
  a.q = row_ptr(q, strides);
  a.os = row_ptr(os, strides + 3);
  a.go = row_ptr(go, strides + 6);
  a.gos = row_ptr(gos, strides + 9);
  a.C = C; a.a_rows = a_rows; a.gq = gq; a.gnum = gnum; a.gden = gden; a.ga_row = ga_row;
  a.L = L; a.H = H; a.Mb = Mb; a.qblk = qblk;
  const size_t smem = (size_t)(64 * 69 + 2 * 64 * 65) * sizeof(float);
  if (set_smem(lin_bwd_rows_kernel, smem)) return -3;
  lin_bwd_rows_kernel<<<dim3(Mb, H, B), 256, smem, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// strides: k(3), v(3), gks(3), gvs(3), gk(3), gv(3).
extern "C" int imf_lin_bwd_kv(const void* k, const void* v, const void* gks, const void* gvs,
                              const float* gS, void* gk, void* gv, int B, int L, int H, int Nb,
                              int lim, const int64_t* strides, void* stream) {
  if (B <= 0) return -1;
  BwdKvArgs a;
  a.k = row_ptr(k, strides);
  a.v = row_ptr(v, strides + 3);
  a.gks = row_ptr(gks, strides + 6);
  a.gvs = row_ptr(gvs, strides + 9);
  a.gk = row_ptr(gk, strides + 12);
  a.gv = row_ptr(gv, strides + 15);
  a.gS = gS; a.L = L; a.H = H; a.Nb = Nb; a.lim = lim < L ? lim : L;
  const size_t smem = (size_t)(64 * 69 + 2 * 64 * 65) * sizeof(float);
  if (set_smem(lin_bwd_kv_kernel, smem)) return -3;
  lin_bwd_kv_kernel<<<dim3(Nb, H, B), 256, smem, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
