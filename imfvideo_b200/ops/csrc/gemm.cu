// bf16 GEMM on tcgen05 tensor cores with TMEM accumulators, fed by TMA.
//
//   C[M, N] = op(A) * op(B)^T (+ bias on the first `bias_rows` rows)
//
// A is either K-major ([M, K], K contiguous) or MN-major ([K, M], M
// contiguous); likewise B ([N, K] or [K, N]).  All four combinations map to
// UMMA shared-memory descriptors directly, so forward (X W^T), data-gradient
// (dY W) and weight-gradient (dY^T X) products need no transposed copies.
// The dual-number forward stacks primal and tangent rows into one launch.
//
// Persistent grid: one CTA per SM walks over the 128 x BN output tiles (n
// fastest, so neighbouring CTAs share the A tile in L2).  Warps 0-3: epilogue,
// warp 4: TMA producer, warp 5: MMA issuer.  STAGES-deep mbarrier ring for the
// operands and TWO accumulator buffers in TMEM, so the MMAs of the next tile
// run while the previous tile is drained.  The epilogue converts the
// accumulator in registers, stages the tile in shared memory in the swizzled
// TMA layout (conflict-free 16-byte stores) and writes it with one TMA store
// per 128-byte-wide panel; when C cannot be described by a tensor map (odd
// pitch or base) it falls back to direct stores.  Replaces the reference's
// `_mm16_kernel` / cuBLAS / `_scaled_mm` calls on the JVP path (reference
// models/triton_mla_block_jvp.py:89-148).
#include "common.cuh"
#include "host_util.h"

namespace imf {

#ifndef IMF_GEMM_WIDE_N
#define IMF_GEMM_WIDE_N 1024
#endif
#ifndef IMF_GEMM_WIDE_K
#define IMF_GEMM_WIDE_K 512
#endif
constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN, int STAGES, typename OutT>
struct GemmSmem {
  alignas(1024) uint8_t a[STAGES][GEMM_BM * GEMM_BK * 2];
  alignas(1024) uint8_t b[STAGES][BN * GEMM_BK * 2];
  alignas(1024) uint8_t c[GEMM_BM * BN * sizeof(OutT)];   // panels of [128 rows][128 bytes]
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct GemmTiles {
  int n_m, n_n, total;     // tiles along M, N; total = n_m * n_n * batch * splits
  int splits, kb_per;      // split-K: slice z of the K loop covers k-blocks [z kb_per, (z+1) kb_per)
                           // and writes plane z of C (batch must be 1 then)
  int sym;                 // the product is symmetric (X X^T, A A with A symmetric): only the tiles
                           // on and above the diagonal are computed (n_m (n_m + 1) / 2 per
                           // batch entry) and the epilogue writes each one's mirror image too
};

// FP8: operands are e4m3 bytes (K-major only); a 128-byte shared-memory row then holds 128
// K elements and one instruction covers 32 of them, so the byte geometry of the pipeline is
// the one of the bf16 kernel.  `alpha_dev` (optional): two device floats whose product scales
// the result (the de-quantisation scales of the two fp8 operands).
template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT, bool FP8 = false>
__global__ void __launch_bounds__(GEMM_THREADS, 2)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_c, OutT* __restrict__ Cbase,
            const float* __restrict__ bias, int M, int N, int K, int64_t ldc, int bias_rows,
            float alpha, int accumulate_out, int* status, const OutT* __restrict__ Cin_base,
            float beta, int64_t batch_stride_c, GemmTiles tiles, int tma_store,
            const float* __restrict__ alpha_dev = nullptr) {
  static_assert(!FP8 || (!A_MN && !B_MN), "fp8 operands are K-major");
  constexpr int KB_ELEMS = FP8 ? 2 * GEMM_BK : GEMM_BK;      // K elements per 128-byte row
  if (alpha_dev) alpha *= alpha_dev[0] * alpha_dev[1];
  extern __shared__ uint8_t smem_raw[];
  auto& s = *reinterpret_cast<GemmSmem<BN, STAGES, OutT>*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + KB_ELEMS - 1) / KB_ELEMS;
  constexpr int PANEL_COLS = 128 / (int)sizeof(OutT);      // 64 bf16 or 32 fp32 columns

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);     // one arrival per epilogue warp
    }
    s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(&s.tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;
  // bz: batch index of the operands; cz: plane of C (batch index, or K slice under split-K)
  auto tile_coords = [&](int tile, int& n0, int& m0, int& bz, int& cz, int& kb0, int& kb1) {
    if (tiles.sym) {
      const int per = tiles.n_m * (tiles.n_m + 1) / 2;
      cz = tile / per;
      int u = tile % per, tm = 0, len = tiles.n_m;       // row tm holds the tiles tn = tm .. n_m - 1
      while (u >= len) { u -= len; --len; ++tm; }
      m0 = tm * GEMM_BM;
      n0 = (tm + u) * BN;
    } else {
      n0 = (tile % tiles.n_n) * BN;
      m0 = ((tile / tiles.n_n) % tiles.n_m) * GEMM_BM;
      cz = tile / (tiles.n_n * tiles.n_m);
    }
    if (tiles.splits > 1) {
      bz = 0;
      kb0 = cz * tiles.kb_per;
      kb1 = kb0 + tiles.kb_per < num_kb ? kb0 + tiles.kb_per : num_kb;
    } else {
      bz = cz;
      kb0 = 0;
      kb1 = num_kb;
    }
  };

  if (warp == 4) {
    // ------------------------------------------------------ TMA producer --
    if (elect_one()) {
      prefetch_tmap(&tm_a);
      prefetch_tmap(&tm_b);
      constexpr uint32_t bytes = (GEMM_BM + BN) * GEMM_BK * 2;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles.total && ok; tile += gridDim.x) {
        int n0, m0, bz, cz, kb0, kb1;
        tile_coords(tile, n0, m0, bz, cz, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int st = it % STAGES;
          if (it >= STAGES && !mbar_wait(&s.empty[st], ((it / STAGES) & 1) ^ 1, abort_flag, status,
                                         STATUS_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&s.full[st], bytes);
          const int k0 = kb * KB_ELEMS;
          if (!A_MN) {
            tma_load_3d(s.a[st], &tm_a, &s.full[st], k0, m0, bz);
          } else {
            tma_load_3d(s.a[st], &tm_a, &s.full[st], m0, k0, bz);
            tma_load_3d(s.a[st] + 64 * 128, &tm_a, &s.full[st], m0 + 64, k0, bz);
          }
          if (!B_MN) {
            tma_load_3d(s.b[st], &tm_b, &s.full[st], k0, n0, bz);
          } else {
#pragma unroll
            for (int p = 0; p < BN / 64; ++p)
              tma_load_3d(s.b[st] + p * 64 * 128, &tm_b, &s.full[st], n0 + p * 64, k0, bz);
          }
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------- MMA issuer --
    if (elect_one()) {
      constexpr uint32_t idesc = FP8 ? make_idesc(GEMM_BM, BN, FMT_E4M3, FMT_E4M3, 1, 0, 0)
                                     : idesc_bf16(GEMM_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, tn = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles.total && ok; tile += gridDim.x, ++tn) {
        const uint32_t buf = tn & 1;
        if (tn >= 2)     // the epilogue has drained this accumulator buffer
          ok = mbar_wait(&s.acc_empty[buf], ((tn >> 1) - 1) & 1, abort_flag, status,
                         STATUS_TIMEOUT_SOFTMAX);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem + buf * BN;
        int n0_, m0_, bz_, cz_, kb0, kb1;
        tile_coords(tile, n0_, m0_, bz_, cz_, kb0, kb1);
        for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
          const int st = it % STAGES;
          ok = mbar_wait(&s.full[st], (it / STAGES) & 1, abort_flag, status, STATUS_TIMEOUT_TMA);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(s.a[st]), b_base = smem_u32(s.b[st]);
#pragma unroll
          for (int ks = 0; ks < GEMM_BK / 16; ++ks) {
            const uint64_t da = A_MN ? sdesc_mnmajor(a_base + ks * 2048, 64 * 128)
                                     : sdesc_kmajor(a_base + ks * 32);
            const uint64_t db = B_MN ? sdesc_mnmajor(b_base + ks * 2048, 64 * 128)
                                     : sdesc_kmajor(b_base + ks * 32);
            if (FP8) mma_ss_f8(acc, da, db, idesc, kb != kb0 || ks != 0);
            else mma_ss(acc, da, db, idesc, kb != kb0 || ks != 0);
          }
          tc_commit(&s.empty[st]);
        }
        tc_commit(&s.acc_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue --
    uint32_t tn = 0;
    bool dead = false;     // a wait gave up: keep walking (the named barriers below are
                           // counted per tile by all four warps) but touch nothing
    for (int tile = blockIdx.x; tile < tiles.total; tile += gridDim.x, ++tn) {
      int n0, m0, bz, cz, kb0_, kb1_;
      tile_coords(tile, n0, m0, bz, cz, kb0_, kb1_);
      const uint32_t buf = tn & 1;
      OutT* C = Cbase + (int64_t)cz * batch_stride_c;
      const OutT* Cin = Cin_base ? Cin_base + (int64_t)cz * batch_stride_c : nullptr;
      if (!dead)
        dead = !__all_sync(0xffffffffu, mbar_wait(&s.acc_full[buf], (tn >> 1) & 1, abort_flag,
                                                  status, STATUS_TIMEOUT_MMA));
      tc_fence_after();
      const int r_in = warp * 32 + lane;
      const int row = m0 + r_in;
      const bool full_tile = tma_store && !accumulate_out;
      if (full_tile && tn > 0) {
        // the previous tile's TMA store has finished reading the staging buffer
        if (threadIdx.x == 0) tma_store_wait_read();
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (!dead) {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tmem + buf * BN, warp * 32, c), r);
        tc_wait_ld();
        const bool add_bias = bias != nullptr && row < bias_rows;
        if (full_tile) {
          // convert and stage: 16-byte chunk k of row r goes to chunk k ^ (r % 8) of the
          // row's 128-byte line in its panel (SWIZZLE_128B)
          if constexpr (sizeof(OutT) == 2) {
            uint32_t o[16];
            uint32_t cv[16];
            const bool have_cin =
                Cin && row < M && n0 + c + 32 <= N &&
                (reinterpret_cast<uintptr_t>(Cin + (int64_t)row * ldc + n0 + c) & 15u) == 0;
            if (have_cin) {
              const uint4* c4 = reinterpret_cast<const uint4*>(Cin + (int64_t)row * ldc + n0 + c);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint4 t = c4[i];
                cv[4 * i] = t.x; cv[4 * i + 1] = t.y; cv[4 * i + 2] = t.z; cv[4 * i + 3] = t.w;
              }
            }
            if (!Cin && !add_bias) {        // plain product: nothing to read, nothing to test
#pragma unroll
              for (int i = 0; i < 16; ++i)
                o[i] = pack_bf16(__uint_as_float(r[2 * i]) * alpha,
                                 __uint_as_float(r[2 * i + 1]) * alpha);
            } else
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float x = __uint_as_float(r[2 * i]) * alpha;
              float y = __uint_as_float(r[2 * i + 1]) * alpha;
              if (have_cin) {
                x += beta * bf16_lo(cv[i]);
                y += beta * bf16_hi(cv[i]);
              } else if (Cin && row < M) {
                if (n0 + c + 2 * i < N) x += beta * __bfloat162float(Cin[(int64_t)row * ldc + n0 + c + 2 * i]);
                if (n0 + c + 2 * i + 1 < N) y += beta * __bfloat162float(Cin[(int64_t)row * ldc + n0 + c + 2 * i + 1]);
              }
              if (add_bias) {
                if (n0 + c + 2 * i < N) x += bias[n0 + c + 2 * i];
                if (n0 + c + 2 * i + 1 < N) y += bias[n0 + c + 2 * i + 1];
              }
              o[i] = pack_bf16(x, y);
            }
            if (tiles.sym && m0 != n0 && row < M) {
              // mirror image of an off-diagonal tile: element (row, col) also goes to (col, row);
              // for a fixed column the 32 lanes write 32 consecutive bf16 of one row of C
              uint16_t* Ct = reinterpret_cast<uint16_t*>(C);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int col = n0 + c + 2 * i;
                if (col < N) Ct[(int64_t)col * ldc + row] = (uint16_t)(o[i] & 0xffffu);
                if (col + 1 < N) Ct[(int64_t)(col + 1) * ldc + row] = (uint16_t)(o[i] >> 16);
              }
            }
            uint8_t* panel = s.c + (c / PANEL_COLS) * (GEMM_BM * 128) + r_in * 128;
            const int k0 = (c % PANEL_COLS) / 8;          // first 16-byte chunk of this group
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(panel + (((k0 + i) ^ (r_in & 7)) << 4)) =
                  make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          } else {
            uint8_t* panel = s.c + (c / PANEL_COLS) * (GEMM_BM * 128) + r_in * 128;
            if (!Cin && !add_bias) {        // plain product
#pragma unroll
              for (int i = 0; i < 8; ++i)
                *reinterpret_cast<float4*>(panel + ((i ^ (r_in & 7)) << 4)) =
                    make_float4(__uint_as_float(r[4 * i]) * alpha, __uint_as_float(r[4 * i + 1]) * alpha,
                                __uint_as_float(r[4 * i + 2]) * alpha, __uint_as_float(r[4 * i + 3]) * alpha);
            } else
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 v;
              v.x = __uint_as_float(r[4 * i]) * alpha;
              v.y = __uint_as_float(r[4 * i + 1]) * alpha;
              v.z = __uint_as_float(r[4 * i + 2]) * alpha;
              v.w = __uint_as_float(r[4 * i + 3]) * alpha;
              const int col = n0 + c + 4 * i;
              if (Cin && row < M) {
                const float* ci = reinterpret_cast<const float*>(Cin) + (int64_t)row * ldc + col;
                if (col < N) v.x += beta * ci[0];
                if (col + 1 < N) v.y += beta * ci[1];
                if (col + 2 < N) v.z += beta * ci[2];
                if (col + 3 < N) v.w += beta * ci[3];
              }
              if (add_bias) {
                if (col < N) v.x += bias[col];
                if (col + 1 < N) v.y += bias[col + 1];
                if (col + 2 < N) v.z += bias[col + 2];
                if (col + 3 < N) v.w += bias[col + 3];
              }
              *reinterpret_cast<float4*>(panel + ((i ^ (r_in & 7)) << 4)) = v;
            }
          }
        } else if (row < M) {
          OutT* dst = C + (int64_t)row * ldc + n0 + c;
          for (int i = 0; i < 32; ++i) {
            const int col = n0 + c + i;
            if (col < N) {
              float x = __uint_as_float(r[i]) * alpha;
              if (add_bias) x += bias[col];
              if (accumulate_out) x += static_cast<float>(dst[i]);
              if (Cin) x += beta * static_cast<float>(Cin[(int64_t)row * ldc + col]);
              dst[i] = static_cast<OutT>(x);
            }
          }
        }
      }
      // the accumulator buffer is free again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
      }
      if (full_tile) {
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 0 && !dead) {
#pragma unroll
          for (int pn = 0; pn < BN / PANEL_COLS; ++pn)
            if (n0 + pn * PANEL_COLS < N)
              tma_store_3d(&tm_c, s.c + pn * (GEMM_BM * 128), n0 + pn * PANEL_COLS, m0, cz);
          tma_store_commit();
        }
      }
    }
    if (threadIdx.x == 0) tma_store_wait_all();
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 2 * BN);
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT, bool FP8 = false>
static int launch_gemm(const void* A, const void* B, void* C, const float* bias, int M, int N,
                       int K, int64_t lda, int64_t ldb, int64_t ldc, int bias_rows, float alpha,
                       int accumulate_out, int* status, cudaStream_t stream, int batch = 1,
                       int64_t sa = 0, int64_t sb = 0, int64_t sc = 0, const void* Cin = nullptr,
                       float beta = 0.f, int splits = 1, const float* alpha_dev = nullptr,
                       int sym = 0) {
  constexpr int OES = FP8 ? 1 : 2;                      // operand element size
  constexpr CUtensorMapDataType ODT =
      FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  constexpr uint32_t KBOX = FP8 ? 128u : 64u;           // K elements of one 128-byte row
  CUtensorMap ta, tb, tc;
  int rc;
  if (splits > 1 && batch != 1) return IMF_ERR_ARG;
  const int c_planes = splits > 1 ? splits : batch;
  {
    // K-major: dims (K, M), box (64, 128).  MN-major: dims (M, K), box (64, 64).
    uint64_t dims[3] = {A_MN ? (uint64_t)M : (uint64_t)K, A_MN ? (uint64_t)K : (uint64_t)M,
                        (uint64_t)batch};
    uint64_t str[3] = {OES, (uint64_t)lda * OES, (uint64_t)(batch > 1 ? sa : (int64_t)lda) * OES};
    uint32_t box[3] = {A_MN ? 64u : KBOX, A_MN ? 64u : (uint32_t)GEMM_BM, 1};
    rc = make_tmap(&ta, ODT, 3, const_cast<void*>(A), dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {B_MN ? (uint64_t)N : (uint64_t)K, B_MN ? (uint64_t)K : (uint64_t)N,
                        (uint64_t)batch};
    uint64_t str[3] = {OES, (uint64_t)ldb * OES, (uint64_t)(batch > 1 ? sb : (int64_t)ldb) * OES};
    uint32_t box[3] = {B_MN ? 64u : KBOX, B_MN ? 64u : (uint32_t)BN, 1};
    rc = make_tmap(&tb, ODT, 3, const_cast<void*>(B), dims, str, box);
    if (rc) return rc;
  }
  // C through TMA when its pitch, batch stride and base are 16-byte multiples
  constexpr int ES = (int)sizeof(OutT);
  int tma_store = ((ldc * ES) % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15u) == 0) &&
                  (c_planes == 1 || (sc * ES) % 16 == 0) && !accumulate_out;
  tc = ta;
  if (tma_store) {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)c_planes};
    uint64_t str[3] = {(uint64_t)ES, (uint64_t)ldc * ES,
                       (uint64_t)(c_planes > 1 ? sc : ldc * (int64_t)M) * ES};
    uint32_t box[3] = {(uint32_t)(128 / ES), (uint32_t)GEMM_BM, 1};
    if (make_tmap(&tc, ES == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                        3, C, dims, str, box))
      tma_store = 0;
  }
  auto kern = gemm_kernel<BN, STAGES, A_MN, B_MN, OutT, FP8>;
  const size_t smem = sizeof(GemmSmem<BN, STAGES, OutT>) + 1024;
  // per device (the attribute belongs to the device's copy of the kernel)
  constexpr int MAX_DEVICES = 64;
  static bool attr_set[MAX_DEVICES] = {false};
  static int sms_of[MAX_DEVICES] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  const int di = (dev >= 0 && dev < MAX_DEVICES) ? dev : 0;
  if (!attr_set[di]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return IMF_ERR_LAUNCH;
    attr_set[di] = true;
  }
  GemmTiles tiles;
  tiles.n_n = (N + BN - 1) / BN;
  tiles.n_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int num_kb = (K + (int)KBOX - 1) / (int)KBOX;
  tiles.kb_per = splits > 1 ? (num_kb + splits - 1) / splits : num_kb;
  tiles.splits = splits > 1 ? (num_kb + tiles.kb_per - 1) / tiles.kb_per : 1;   // no empty slice
  if (splits > 1 && tiles.splits != splits) return IMF_ERR_ARG;
  tiles.total = tiles.n_n * tiles.n_m * (splits > 1 ? tiles.splits : batch);
  tiles.sym = sym;
  if (sym) {
    // square bf16 result through the staged (TMA store) epilogue, square tiles, no split-K
    if (M != N || BN != GEMM_BM || ES != 2 || !tma_store || splits > 1 || bias) return IMF_ERR_ARG;
    tiles.total = tiles.n_m * (tiles.n_m + 1) / 2 * batch;
  }
  int sms = sms_of[di];
  if (!sms) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    sms_of[di] = sms;
  }
  // two persistent CTAs per SM when their shared memory allows it (256 TMEM columns each)
  const int per_sm = (2 * (smem + 1024) <= 233472) ? 2 : 1;
  const int grid = tiles.total < sms * per_sm ? tiles.total : sms * per_sm;
  kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, tc, static_cast<OutT*>(C), bias, M, N, K, ldc,
                                             bias_rows, alpha, accumulate_out, status,
                                             static_cast<const OutT*>(Cin), beta, sc, tiles,
                                             tma_store, alpha_dev);
  return cudaGetLastError() == cudaSuccess ? IMF_OK : IMF_ERR_LAUNCH;
}

}  // namespace imf

// C = alpha * op(A) op(B)^T (+bias) ; bf16 operands.
//   a_mn / b_mn: 0 = K-major ([rows, K]), 1 = MN-major ([K, rows]).
//   out_fp32: 0 = bf16 output, 1 = fp32 output.  lda/ldb/ldc in elements.
//   accumulate_out: C += result (fp32 read-modify-write, for split products).
extern "C" int imf_gemm_bf16(const void* A, const void* B, void* C, const float* bias, int M,
                             int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_mn,
                             int b_mn, int out_fp32, int bias_rows, float alpha,
                             int accumulate_out, int* status, void* stream) {
  using namespace imf;
  if (M <= 0 || N <= 0 || K <= 0) return IMF_ERR_ARG;
  if ((lda & 7) || (ldb & 7)) return IMF_ERR_ARG;  // TMA strides are multiples of 16 B
  cudaStream_t st = static_cast<cudaStream_t>(stream);
// fp32 output: the 64 KB staging tile leaves room for one CTA per SM only, so the operand
// pipeline is four stages deep there; bf16 output: see IMF_GEMM_DEEP below (two CTAs per SM
// with two stages each only for the MN-major-A instances).
#define IMF_GEMM_STAGES(OT) (sizeof(OT) == 4 ? 4 : 2)
#define IMF_GEMM_CASE(AM, BM_, OT)                                                          \
  return launch_gemm<128, IMF_GEMM_STAGES(OT), AM, BM_, OT>(                                \
      A, B, C, bias, M, N, K, lda, ldb, ldc, bias_rows, alpha, accumulate_out, status, st)
  if (out_fp32) {
    if (!a_mn && !b_mn) IMF_GEMM_CASE(false, false, float);
    if (!a_mn && b_mn) IMF_GEMM_CASE(false, true, float);
    if (a_mn && !b_mn) IMF_GEMM_CASE(true, false, float);
    IMF_GEMM_CASE(true, true, float);
  } else {
    // wide, deep products: 128 x 256 tiles (one CTA per SM, three operand stages) halve the
    // bytes of the A panel per flop.  An SM reads 64 B per clock from L2, which is what bounds
    // these kernels: 65,560 x 5,472 x 1,024 runs at 1,265 TFLOP/s with the wide tile, 1,174
    // with 128 x 128 tiles and six stages.  Short-K or narrow products keep 128 x 128 tiles
    if (N >= IMF_GEMM_WIDE_N && K >= IMF_GEMM_WIDE_K) {
#define IMF_GEMM_WIDE(AM, BM_)                                                              \
  return launch_gemm<256, 3, AM, BM_, __nv_bfloat16>(                                       \
      A, B, C, bias, M, N, K, lda, ldb, ldc, bias_rows, alpha, accumulate_out, status, st)
      if (!a_mn && !b_mn) IMF_GEMM_WIDE(false, false);
      if (!a_mn && b_mn) IMF_GEMM_WIDE(false, true);
#undef IMF_GEMM_WIDE
    }
    // One CTA per SM with a deep operand ring beats two CTAs with two stages each (a k-block
    // takes about 1,450 cycles to land, so two stages cap a CTA at two k-blocks per 2,000
    // cycles): four stages for short K (58,280 x 1,024 x 256: 51.8 -> 47.5 us), six from
    // K = 512 on (65,560 x 5,472 x 1,024: 693 -> 624 us, 1,178 TFLOP/s).
#define IMF_GEMM_DEEP(AM, BM_)                                                              \
  {                                                                                         \
    if (K >= 512)                                                                           \
      return launch_gemm<128, 6, AM, BM_, __nv_bfloat16>(A, B, C, bias, M, N, K, lda, ldb,   \
                                                        ldc, bias_rows, alpha,              \
                                                        accumulate_out, status, st);        \
    return launch_gemm<128, 4, AM, BM_, __nv_bfloat16>(A, B, C, bias, M, N, K, lda, ldb, ldc, \
                                                      bias_rows, alpha, accumulate_out,     \
                                                      status, st);                          \
  }
    if (!a_mn && !b_mn) IMF_GEMM_DEEP(false, false);
    if (!a_mn && b_mn) IMF_GEMM_DEEP(false, true);
#undef IMF_GEMM_DEEP
    if (a_mn && !b_mn) IMF_GEMM_CASE(true, false, __nv_bfloat16);
    IMF_GEMM_CASE(true, true, __nv_bfloat16);
  }
#undef IMF_GEMM_CASE
}

// fp8 (e4m3) operands, both K-major ([M, K] and [N, K] bytes, row pitches multiples of 16):
// C = alpha * scales[0] * scales[1] * A B^T (+ bias), bf16 or fp32 output.  `scales`: two device
// floats (the operands' de-quantisation scales, see imf_quantize_fp8) or null.  The B200 form
// of the reference's `_fp8_mm` (reference models/triton_block_jvp.py:80-86).
extern "C" int imf_gemm_fp8(const void* A, const void* B, void* C, const float* bias, int M, int N,
                            int K, int64_t lda, int64_t ldb, int64_t ldc, int out_fp32,
                            int bias_rows, float alpha, const float* scales, int* status,
                            void* stream) {
  using namespace imf;
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 15) || (ldb & 15)) return IMF_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_fp32)
    return launch_gemm<128, 4, false, false, float, true>(A, B, C, bias, M, N, K, lda, ldb, ldc,
                                                          bias_rows, alpha, 0, status, st, 1, 0, 0,
                                                          0, nullptr, 0.f, 1, scales);
  return launch_gemm<128, 2, false, false, __nv_bfloat16, true>(
      A, B, C, bias, M, N, K, lda, ldb, ldc, bias_rows, alpha, 0, status, st, 1, 0, 0, 0, nullptr,
      0.f, 1, scales);
}

// Split-K product for long-K / small-output shapes (weight gradients dY^T X with K = tokens):
// slice z of `splits` equal K ranges writes plane z of `partial` ([splits][M][N] fp32); the
// slices are summed in a fixed order by imf_splitk_reduce, so the result does not depend on
// which CTA finishes first.  `splits` must satisfy ceil(nkb / ceil(nkb / splits)) == splits for
// nkb = ceil(K / 64) (imf_gemm_splitk_count returns such a value).
extern "C" int imf_gemm_splitk_count(int M, int N, int K, int target_tiles) {
  const int tiles_mn = ((M + 127) / 128) * ((N + 127) / 128);
  const int nkb = (K + imf::GEMM_BK - 1) / imf::GEMM_BK;
  int want = (target_tiles + tiles_mn - 1) / tiles_mn;
  if (want > nkb / 4) want = nkb / 4;          // at least four k-blocks per slice
  if (want < 1) want = 1;
  const int per = (nkb + want - 1) / want;
  return (nkb + per - 1) / per;
}

extern "C" int imf_gemm_bf16_splitk(const void* A, const void* B, float* partial, int M, int N,
                                    int K, int64_t lda, int64_t ldb, int a_mn, int b_mn,
                                    int splits, int* status, void* stream) {
  using namespace imf;
  if (M <= 0 || N <= 0 || K <= 0 || splits < 2) return IMF_ERR_ARG;
  if ((lda & 7) || (ldb & 7)) return IMF_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t plane = (int64_t)M * N;
#define IMF_GEMM_CASE(AM, BM_)                                                                  \
  return launch_gemm<128, 4, AM, BM_, float>(A, B, partial, nullptr, M, N, K, lda, ldb, N, 0,   \
                                             1.f, 0, status, st, 1, 0, 0, plane, nullptr, 0.f,  \
                                             splits)
  if (!a_mn && !b_mn) IMF_GEMM_CASE(false, false);
  if (!a_mn && b_mn) IMF_GEMM_CASE(false, true);
  if (a_mn && !b_mn) IMF_GEMM_CASE(true, false);
  IMF_GEMM_CASE(true, true);
#undef IMF_GEMM_CASE
}

namespace imf {
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, long plane,
                                     int N, float* __restrict__ out, int64_t ldo, float alpha,
                                     int accumulate) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= plane) return;
  float acc = 0.f;
  for (int z = 0; z < splits; ++z) acc += partial[z * plane + i];     // fixed order
  float* dst = out + (i / N) * ldo + (i % N);
  *dst = accumulate ? *dst + alpha * acc : alpha * acc;
}
}  // namespace imf

// out[M, N] (row pitch ldo) (+)= alpha * sum_z partial[z]
extern "C" int imf_splitk_reduce(const float* partial, int splits, int M, int N, float* out,
                                 int64_t ldo, float alpha, int accumulate, void* stream) {
  if (splits < 1 || M <= 0 || N <= 0) return imf::IMF_ERR_ARG;
  const long plane = (long)M * N;
  imf::splitk_reduce_kernel<<<(unsigned)((plane + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      partial, splits, plane, N, out, ldo, alpha, accumulate);
  return cudaGetLastError() == cudaSuccess ? imf::IMF_OK : imf::IMF_ERR_LAUNCH;
}

// Batched form with an additive source: C[z] = alpha * op(A[z]) op(B[z])^T + beta * Cin[z].
// sa/sb/sc: batch strides in elements (multiples of 8 for A, B).  Used by the
// Newton-Schulz iteration (X X^T, b A + c A A, a X + B X as three launches).
extern "C" int imf_gemm_bf16_batched(const void* A, const void* B, void* C, const void* Cin, int M,
                                     int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                                     int batch, int64_t sa, int64_t sb, int64_t sc, int a_mn,
                                     int b_mn, int out_fp32, float alpha, float beta, int* status,
                                     void* stream) {
  using namespace imf;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return IMF_ERR_ARG;
  if ((lda & 7) || (ldb & 7) || (batch > 1 && ((sa & 7) || (sb & 7)))) return IMF_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define IMF_GEMM_CASE(AM, BM_, OT)                                                              \
  return launch_gemm<128, IMF_GEMM_STAGES(OT), AM, BM_, OT>(                                    \
      A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, alpha, 0, status, st, batch, sa, sb, sc, Cin, beta)
  if (out_fp32) {
    if (!a_mn && !b_mn) IMF_GEMM_CASE(false, false, float);
    if (!a_mn && b_mn) IMF_GEMM_CASE(false, true, float);
    if (a_mn && !b_mn) IMF_GEMM_CASE(true, false, float);
    IMF_GEMM_CASE(true, true, float);
  } else {
    if (!a_mn && !b_mn) IMF_GEMM_CASE(false, false, __nv_bfloat16);
    if (!a_mn && b_mn) IMF_GEMM_CASE(false, true, __nv_bfloat16);
    if (a_mn && !b_mn) IMF_GEMM_CASE(true, false, __nv_bfloat16);
    IMF_GEMM_CASE(true, true, __nv_bfloat16);
  }
#undef IMF_GEMM_CASE
}

// The same for a product that is known to be symmetric (M = N; X X^T, X^T X, or A A with A
// symmetric; Cin symmetric too): computes the tiles on and above the diagonal only and writes
// their mirror images from the epilogue.  bf16 output, ldc a multiple of 8.
extern "C" int imf_gemm_bf16_batched_sym(const void* A, const void* B, void* C, const void* Cin,
                                         int M, int K, int64_t lda, int64_t ldb, int64_t ldc,
                                         int batch, int64_t sa, int64_t sb, int64_t sc, int mn,
                                         float alpha, float beta, int* status, void* stream) {
  using namespace imf;
  if (M <= 0 || K <= 0 || batch <= 0) return IMF_ERR_ARG;
  if ((lda & 7) || (ldb & 7) || (batch > 1 && ((sa & 7) || (sb & 7)))) return IMF_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  using OT = __nv_bfloat16;
  if (mn)      // both operands MN-major ([K, M]): X^T X
    return launch_gemm<128, IMF_GEMM_STAGES(OT), true, true, OT>(
        A, B, C, nullptr, M, M, K, lda, ldb, ldc, 0, alpha, 0, status, st, batch, sa, sb, sc, Cin,
        beta, 1, nullptr, 1);
  return launch_gemm<128, IMF_GEMM_STAGES(OT), false, false, OT>(
      A, B, C, nullptr, M, M, K, lda, ldb, ldc, 0, alpha, 0, status, st, batch, sa, sb, sc, Cin,
      beta, 1, nullptr, 1);
}

// ---------------------------------------------------------------------------
// Per-tensor fp8 (e4m3) quantisation of a bf16 matrix for imf_gemm_fp8: x8 = round(x / s),
// s = amax(|x|) / 448 (the largest e4m3 value), two launches; `scale_out` receives s.
// ---------------------------------------------------------------------------
#include <cuda_fp8.h>
namespace imf {
__global__ void fp8_amax_kernel(const __nv_bfloat16* __restrict__ x, long rows, int cols,
                                int64_t ld, unsigned int* __restrict__ amax_bits) {
  float m = 0.f;
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(__bfloat162float(x[(i / cols) * ld + i % cols])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));   // m >= 0: bits order
}
__global__ void fp8_cast_kernel(const __nv_bfloat16* __restrict__ x, long rows, int cols, int64_t ld,
                                uint8_t* __restrict__ out, int64_t ldo,
                                const unsigned int* __restrict__ amax_bits,
                                float* __restrict__ scale_out) {
  const float amax = __uint_as_float(*amax_bits);
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / s;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = s;
  const long n = rows * ldo;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / ldo;
    const int c = (int)(i % ldo);
    const float v = c < cols ? __bfloat162float(x[r * ld + c]) * inv : 0.f;   // pad columns: 0
    out[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  }
}
}  // namespace imf

// x: (rows, cols) bf16 with row pitch ld; out: (rows, ldo) bytes, ldo >= cols and a multiple
// of 16 (columns cols..ldo-1 are written as zero); amax_scratch: one zeroed device word.
extern "C" int imf_quantize_fp8(const void* x, long rows, int cols, int64_t ld, void* out,
                                int64_t ldo, unsigned int* amax_scratch, float* scale_out,
                                void* stream) {
  if (rows <= 0 || cols <= 0 || ldo < cols || (ldo & 15)) return imf::IMF_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  long blocks = (rows * cols + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  imf::fp8_amax_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows,
                                                         cols, ld, amax_scratch);
  imf::fp8_cast_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows,
                                                         cols, ld, static_cast<uint8_t*>(out), ldo,
                                                         amax_scratch, scale_out);
  return cudaGetLastError() == cudaSuccess ? imf::IMF_OK : imf::IMF_ERR_LAUNCH;
}

