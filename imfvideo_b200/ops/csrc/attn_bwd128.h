// Host-side interface of the head_dim-128 attention backward (attn_bwd128.cu); the public
// entry point imf_attn_bwd (attn_bwd.cu) dispatches here when head_dim is 128.
#pragma once
#include <stdint.h>

namespace imf {

struct Bwd128Args {
  const void *q, *k, *v, *o, *d_o;        // (B, L, H, 128) bf16
  const float* lse;                       // (B, H, L) from the forward
  void *dq, *dk, *dv;                     // dq contiguous; dk / dv with their own strides
  int B, L, H;
  const int64_t* strides;                 // (batch, row, head) element strides of q, k, v, d_o
  const int64_t* o_strides;
  const int64_t* dk_strides;
  const int64_t* dv_strides;
  float scale;
  void* scratch;
  long scratch_bytes;
  int* status;
  void* stream;
  bool fixed_order;                       // dQ adds in a fixed order (needs `status`)
};

long attn_bwd128_scratch_bytes(int B, int L, int H);
int attn_bwd128_launch(const Bwd128Args& a);

}  // namespace imf
