// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library have no allocator to offer: a runtime that owns all device
// memory and hands out none, a plug-in called from inside somebody else's stream capture,
// or FFI glue that can pass pointers it was given but cannot call cudaMalloc.  For them the
// split-KV partials of the decode attention kernel live in a fixed array inside the library
// image instead of a caller-provided workspace.
#include "common.cuh"

#define B200_ATTN_DECODE_STATIC_SCRATCH_BYTES (8ll << 20)

// Every GPU that loads the library keeps these 8 MiB until the process exits.
static __device__ __align__(256) unsigned char g_attn_decode_scratch[B200_ATTN_DECODE_STATIC_SCRATCH_BYTES];

extern "C" int b200_attn_decode_noalloc(const void* q, const void* k, const void* v, const void* mask, void* out, int64_t B,
                                        int Hq, int Hkv, int64_t S, int D, int64_t q_batch_stride, int64_t kv_batch_stride,
                                        int64_t kv_head_stride, int64_t mask_batch_stride, float scale, int dtype,
                                        void* stream) {
  const int64_t need = b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D);
  if (need > B200_ATTN_DECODE_STATIC_SCRATCH_BYTES)
    B200_FAIL(B200_ELIMIT,
              "b200_attn_decode_noalloc: B=%lld, Hq=%d, Hkv=%d, S=%lld needs %lld bytes of split-KV scratch, the built-in array "
              "holds %lld; use b200_attn_decode with a caller-provided workspace",
              (long long)B, Hq, Hkv, (long long)S, (long long)need, (long long)B200_ATTN_DECODE_STATIC_SCRATCH_BYTES);
  // In host code the array's name is only a handle; its device address is looked up once
  // per device (with that device current) and cached.
  static void* scratch_of_device[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) B200_FAIL(B200_ELAUNCH, "b200_attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (scratch_of_device[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_decode_scratch);
    if (e != cudaSuccess || p == nullptr) B200_FAIL(B200_ELAUNCH, "b200_attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    scratch_of_device[dev] = p;
  }
  return b200_attn_decode(q, k, v, mask, out, B, Hq, Hkv, S, D, q_batch_stride, kv_batch_stride, kv_head_stride, mask_batch_stride,
                          scale, dtype, scratch_of_device[dev], B200_ATTN_DECODE_STATIC_SCRATCH_BYTES, stream);
}
