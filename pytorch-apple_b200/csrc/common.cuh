// Shared helpers for the b200nn kernels: error reporting, dtype dispatch,
// 128-bit vector access and warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200nn.h"

namespace b200 {

// ---- host-side error plumbing ------------------------------------------------
void set_error(const char* fmt, ...);
int sm_count();  // SM count of the current device (cached per device)
bool pdl_enabled();  // programmatic dependent launch for the decode-path kernels (B200NN_PDL=0 turns it off)

// ---- programmatic dependent launch ---------------------------------------------
// A kernel launched through launch_pdl may start while its predecessor in the stream is
// still draining; it must execute pdl_wait() before it touches memory the predecessor
// writes (the wait returns once the predecessor grid has completed and flushed).
// pdl_trigger() lets the successor's blocks be scheduled early.  Both are no-ops for a
// plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  if (pdl_enabled()) {
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define B200_FAIL(code, ...)        \
  do {                              \
    ::b200::set_error(__VA_ARGS__); \
    return (code);                  \
  } while (0)

#define B200_CHECK_ARG(cond, ...) \
  do {                            \
    if (!(cond)) B200_FAIL(B200_EINVAL, __VA_ARGS__); \
  } while (0)

#define B200_CHECK_LAUNCH(name)                                                         \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess) B200_FAIL(B200_ELAUNCH, "%s: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// Function attributes and occupancy answers belong to one device; a cache of them is indexed by the
// device current at the call.  slot() is nullptr when the device cannot be read or lies outside the table.
constexpr int B200_MAX_DEVICES = 64;
template <typename V> struct PerDevice {
  V v[B200_MAX_DEVICES] = {};
  V* slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= B200_MAX_DEVICES) return nullptr;
    return &v[dev];
  }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int dtype_size(int dt) {
  switch (dt) {
    case B200_F32: case B200_I32: return 4;
    case B200_F16: case B200_BF16: return 2;
    case B200_I64: return 8;
    case B200_U8: return 1;
  }
  return 0;
}

// ---- device-side scalar conversion ---------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// round a float to the precision of dtype code `dt`, keep it as float
__device__ __forceinline__ float round_to(float v, int dt) {
  if (dt == B200_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dt == B200_F16) return __half2float(__float2half_rn(v));
  return v;
}
template <typename T> __device__ __forceinline__ float round_as(float v) { return to_f32<T>(from_f32<T>(v)); }

// x * sigmoid(x) on the special-function units, branch-free (the IEEE division and expf
// carry slow-path branches that keep the compiler from interleaving independent elements).
// The result feeds a 16-bit rounding, which absorbs the ~2^-21 relative error.
__device__ __forceinline__ float silu_f32(float x) { return __fdividef(x, 1.f + __expf(-x)); }

__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dt) {
  switch (dt) {
    case B200_F32: return static_cast<const float*>(p)[i];
    case B200_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case B200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    case B200_I32: return static_cast<float>(static_cast<const int32_t*>(p)[i]);
    case B200_I64: return static_cast<float>(static_cast<const int64_t*>(p)[i]);
    case B200_U8: return static_cast<float>(static_cast<const uint8_t*>(p)[i]);
  }
  return 0.f;
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, int dt, float v) {
  switch (dt) {
    case B200_F32: static_cast<float*>(p)[i] = v; break;
    case B200_F16: static_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case B200_BF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    case B200_I32: static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
    case B200_I64: static_cast<int64_t*>(p)[i] = static_cast<int64_t>(v); break;
    case B200_U8: static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(v); break;
  }
}
__device__ __forceinline__ int64_t load_index(const void* p, int64_t i, int dt) {
  return dt == B200_I64 ? static_cast<const int64_t*>(p)[i] : static_cast<int64_t>(static_cast<const int32_t*>(p)[i]);
}

// ---- 128-bit packs of 16-bit floats -------------------------------------------
template <typename T> struct Pack8 { uint4 raw; };  // 8 x 16-bit

// Conversions run at a quarter of the ALU rate, so pairs go through the packed forms: one
// cvt.rn.{f16x2,bf16x2}.f32 per two values on the way out; bf16 -> f32 is a shift / mask.
template <typename T> __device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& raw, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x; f[2 * i + 1] = v.y;
  }
}
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float (&f)[8]);
template <> __device__ __forceinline__ uint4 pack8<__half>(const float (&f)[8]) {
  uint4 raw;
  __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}
template <> __device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}
// round two values to T and back (what storing them as T and reloading would give)
template <typename T> __device__ __forceinline__ void round2(float& a, float& b);
template <> __device__ __forceinline__ void round2<__half>(float& a, float& b) {
  const float2 v = __half22float2(__floats2half2_rn(a, b));
  a = v.x; b = v.y;
}
template <> __device__ __forceinline__ void round2<__nv_bfloat16>(float& a, float& b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xffff0000u);
}

__device__ __forceinline__ uint4 ld_global_nc_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// ---- reductions --------------------------------------------------------------
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
// Block-wide reductions; `scratch` holds >= 33 floats.  Every thread gets the result.
template <bool IS_MAX> __device__ __forceinline__ float block_reduce(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : (IS_MAX ? -INFINITY : 0.f);
    t = IS_MAX ? warp_max(t) : warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Dispatch a 16-bit float dtype code to a template parameter.
#define B200_DISPATCH_HALF(dt, T, ...)                              \
  if ((dt) == B200_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if ((dt) == B200_F16) { using T = __half; __VA_ARGS__; }     \
  else B200_FAIL(B200_ENOTSUP, "%s: dtype %d is not f16/bf16", __func__, (int)(dt))

#define B200_DISPATCH_FLOAT(dt, T, ...)                             \
  if ((dt) == B200_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if ((dt) == B200_F16) { using T = __half; __VA_ARGS__; }     \
  else if ((dt) == B200_F32) { using T = float; __VA_ARGS__; }      \
  else B200_FAIL(B200_ENOTSUP, "%s: dtype %d is not a float type", __func__, (int)(dt))

}  // namespace b200
