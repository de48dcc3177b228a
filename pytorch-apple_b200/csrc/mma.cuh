// Warp-level tensor-core primitives shared by the GEMM and attention kernels:
// m16n8k16 MMA with fp32 accumulation for f16 / bf16, ldmatrix, cp.async.
#pragma once
#include "common.cuh"

namespace b200 {

template <typename T> struct MmaType;
template <> struct MmaType<__half> {
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};
template <> struct MmaType<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
// Transpose an 8x8 matrix of 16-bit values held one row pair per thread (the ldmatrix layout).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
// 2^x, flushing denormals; -inf -> 0
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 16-byte async copy global -> shared; bytes beyond `src_bytes` (0 or 16) are zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// pack two floats into one 32-bit register of 16-bit values (lo = first)
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Packed 16-bit pair arithmetic on raw registers.  a + b rounds the exact sum once, which is
// what adding two 16-bit tensors in fp32 and rounding the result gives; max is maxNum.
template <typename T> __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t add2<__half>(uint32_t a, uint32_t b) {
  const __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t add2<__nv_bfloat16>(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T> __device__ __forceinline__ uint32_t relu2(uint32_t a);
template <> __device__ __forceinline__ uint32_t relu2<__half>(uint32_t a) {
  const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), __float2half2_rn(0.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t relu2<__nv_bfloat16>(uint32_t a) {
  const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), __float2bfloat162_rn(0.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// inverse of pack2
template <typename T> __device__ __forceinline__ void unpack2(uint32_t raw, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t raw, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw));
  lo = f.x; hi = f.y;
}
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t raw, float& lo, float& hi) {
  lo = __uint_as_float(raw << 16);
  hi = __uint_as_float(raw & 0xffff0000u);
}

}  // namespace b200
