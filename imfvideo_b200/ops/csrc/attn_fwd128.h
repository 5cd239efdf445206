// Host-side interface of the head_dim-128 attention forward (attn_fwd128.cu); the public
// entry point imf_attn_fwd (attn_fwd.cu) dispatches here when head_dim is 128.
#pragma once
#include <stdint.h>

namespace imf {

struct Fwd128Args {
  const void *q, *k, *v, *dq, *dk, *dv;   // (B, L, H, 128) bf16; dq/dk/dv null = primal only
  void *o, *dout;                         // outputs, contiguous in the last dimension
  float* lse;                             // (B, H, L) or null
  int B, L, H;
  const int64_t* strides;                 // (batch, row, head) element strides of q, k, v (, dq, dk, dv)
  int64_t o_sb, o_sl, o_sh;
  float scale;
  void* scratch;
  long scratch_bytes;
  int* status;
  void* stream;
};

long attn_fwd128_scratch_bytes(int B, int L, int H, int tangent);
int attn_fwd128_launch(const Fwd128Args& a);

}  // namespace imf
