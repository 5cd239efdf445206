// Host-side helpers shared by the launchers: tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), a per-device
// status word that kernels write when a bounded wait runs out, and argument
// checks that return error codes instead of launching.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace imf {

// error codes returned by every extern "C" launcher (0 = launched)
enum : int {
  IMF_OK = 0,
  IMF_ERR_ARG = -1,       // bad shape / stride / alignment
  IMF_ERR_DRIVER = -2,    // tensor-map encode or driver entry point failed
  IMF_ERR_LAUNCH = -3,    // cudaLaunch error (see cudaGetLastError)
  IMF_ERR_TOO_LARGE = -4,
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rank-N (<= 5) tiled map with 128-byte swizzle.  dims/strides innermost
// first; strides[0] is implied (element size); strides in BYTES.
inline int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, void* base,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return IMF_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return IMF_ERR_ARG;
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) {
      if (strides_bytes[i] & 15u) return IMF_ERR_ARG;
      gs[i - 1] = strides_bytes[i];
    }
  }
  CUresult r = fn(out, dt, rank, base, gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "imf_b200: cuTensorMapEncodeTiled failed (%d)\n", (int)r);
    return IMF_ERR_DRIVER;
  }
  return IMF_OK;
}

}  // namespace imf
