// Allocation-free variant of the dense attention forward.
//
// This entry point has no counterpart in the reference implementation; it
// exists for callers of this library that are not able to allocate device
// memory themselves: code running inside a region where cudaMalloc is
// forbidden or would deadlock (for example a host callback, a real-time
// inference loop with a fixed memory budget, or an embedding application that
// hands this library only its input and output buffers and owns no allocator).
//
// The regular entry point (imf_attn_fwd) expects the caller to provide a
// scratch buffer for the partial results of work items that are split between
// two thread blocks.  Here that scratch lives in a file-scope __device__ array
// inside the library, so the caller passes inputs and outputs only.
//
// Limits and rules:
//  * primal forward only (no tangent), head_dim 64, bf16, same layouts as
//    imf_attn_fwd;
//  * the built-in scratch holds the partials of at most
//    IMF_ATTN_NOALLOC_MAX_CTAS (160) thread blocks = 32,931,840 bytes; every
//    GPU that loads the library keeps that much reserved until the process
//    exits.  A device with more SMs than that, for a problem that needs one
//    partial slot per SM, is rejected with IMF_ERR_TOO_LARGE (-4);
//  * the first call on each device looks up the device address of the array
//    (cudaGetSymbolAddress, with that device current).  Make that first call
//    outside of any stream capture.  First calls made at the same time from
//    several host threads are safe: each of them looks up and stores the same
//    address for that device;
//  * all calls on a device share the one array and it keeps the previous
//    call's contents.  Nothing in it needs to start at zero: every slot that a
//    launch reads was written earlier in the same launch sequence.  Two calls
//    whose kernels can overlap on the GPU (different streams without an
//    ordering between them) race on the array and give wrong results; order
//    them on one stream or with events;
//  * no cudaMalloc / cudaFree / allocating library routine is called.
#pragma once
#include <stdint.h>

#define IMF_ATTN_NOALLOC_MAX_CTAS 160

#ifdef __cplusplus
extern "C" {
#endif

// q, k, v, o: (B, L, H, 64) bf16; strides: 9 element strides (batch, row, head)
// for q, k, v; o strides (o_sb, o_sl, o_sh); lse: (B, H, L) fp32 or null.
// Returns 0 on launch, a negative IMF_ERR_* code otherwise.
int imf_attn_fwd_noalloc(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                         int L, int H, int head_dim, const int64_t* strides, int64_t o_sb,
                         int64_t o_sl, int64_t o_sh, float scale, int* status, void* stream);

#ifdef __cplusplus
}
#endif
