// Shared between the two prefill attention kernels (attention.cu: mma.sync; attn_prefill_tc5.cu: tcgen05).
#pragma once
#include "common.cuh"

namespace b200 {

struct PrefillParams {
  const void* q; const void* k; const void* v; const void* mask; void* out;
  int64_t B, T, S;
  int Hq, Hkv;
  int64_t qs[3], ks[3], vs[3];
  int64_t mask_b, mask_t;
  float scale;
  int mask_dtype;
  int mask_staged;   // the mask can travel through shared memory (activation dtype, 16-byte-aligned rows)
};

// Prefill attention on the tcgen05 path (head_dim 128, 16-bit types, 16-byte aligned strides, mask absent or
// in the activation type).  Returns B200_ENOTSUP for anything else; the caller then uses the mma.sync kernel.
int attn_prefill_tc5(const PrefillParams& p, int dtype, cudaStream_t stream);
// code left by a bounded wait of that kernel that ran out (0 = none); optionally cleared
int attn_prefill_tc5_error(bool clear);

}  // namespace b200
