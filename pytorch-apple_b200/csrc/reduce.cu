// Row reductions: RMSNorm, (masked) softmax, mean over the last axis, arg-max.
// All are bandwidth kernels: 128-bit loads, the row held in registers between the
// reduction and the write, warp-shuffle reductions, fp32 arithmetic.
#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// RMSNorm.  One warp per row while the row fits in registers (cols <= 2048),
// otherwise one block per row with a second read that hits L1/L2.
// ---------------------------------------------------------------------------
template <typename T, int MAXP>  // MAXP = 16-byte packs per lane
__global__ void __launch_bounds__(128) rmsnorm_warp_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                                           int64_t rows, int cols, int64_t xs, int64_t ys, float eps,
                                                           int round_mid) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_wait();
  pdl_trigger();
  if (row >= rows) return;
  const int npack = cols >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * xs);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4 raw[MAXP], gain[MAXP];
  // every load of the row and of the gains is in flight before anything waits: the kernel lives for
  // about two memory round trips, and asking for the gains only after the reduction made it three
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int pk = lane + 32 * i;
    if (pk < npack) raw[i] = ld_global_nc_v4(xr + pk);
  }
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int pk = lane + 32 * i;
    if (pk < npack) gain[i] = __ldg(wv + pk);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int pk = lane + 32 * i;
    if (pk < npack) {
      float f[8];
      unpack8<T>(raw[i], f);
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
    }
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ys);
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int pk = lane + 32 * i;
    if (pk < npack) {
      float f[8], g[8];
      unpack8<T>(raw[i], f);
      unpack8<T>(gain[i], g);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float n = f[k] * r;
        if (round_mid) n = round_as<T>(n);
        f[k] = n * g[k];
      }
      yr[pk] = pack8<T>(f);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_block_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                                            int64_t cols, int64_t xs, int64_t ys, float eps, int round_mid) {
  __shared__ float scratch[33];
  const T* xr = x + static_cast<int64_t>(blockIdx.x) * xs;
  T* yr = y + static_cast<int64_t>(blockIdx.x) * ys;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32<T>(xr[c]);
    ss += v * v;
  }
  ss = block_reduce<false>(ss, scratch);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float n = to_f32<T>(xr[c]) * r;
    if (round_mid) n = round_as<T>(n);
    yr[c] = from_f32<T>(n * to_f32<T>(w[c]));
  }
}

// ---------------------------------------------------------------------------
// Softmax over the last axis with optional scale and broadcast additive mask.
// ---------------------------------------------------------------------------
struct SoftmaxParams {
  const void* x;
  const void* mask;
  void* y;
  int64_t d1, d2, cols;
  int64_t ms0, ms1, ms2;
  float scale;
  int round_steps;
  int mask_dtype;
  int d1_inner;   // walk d1 fastest: blocks that share a mask row (mask broadcast over d1) run back to back
};

__device__ __forceinline__ float fast_exp(float x) { return exp2f(x * 1.4426950408889634f); }
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// True when rounding a and b to T would not change them (cheap test, may say false for
// values that are in fact representable).  bf16 is the upper half of an fp32.
template <typename T> __device__ __forceinline__ bool exact_in(const float (&f)[8]) { return false; }
template <> __device__ __forceinline__ bool exact_in<__nv_bfloat16>(const float (&f)[8]) {
  uint32_t low = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) low |= __float_as_uint(f[k]);
  return (low & 0xffffu) == 0;
}

// Block reduction with one barrier: every warp leaves its partial in `slot` and every
// thread combines all partials itself.  Consecutive calls must alternate between two slots.
template <bool IS_MAX, int BLOCK> __device__ __forceinline__ float block_combine(float v, float* slot) {
  constexpr int NW = BLOCK / 32;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (NW == 1) return v;
  if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
  __syncthreads();
  if (NW <= 8) {
    float t = slot[0];
#pragma unroll
    for (int i = 1; i < NW; ++i) t = IS_MAX ? fmaxf(t, slot[i]) : t + slot[i];
    return t;
  }
  const float t = slot[threadIdx.x & 31];  // NW == 32
  return IS_MAX ? warp_max(t) : warp_sum(t);
}

// BLOCK threads cooperate on one row (one block per row); each holds up to 4 packs of 8
// elements.  The special function unit that computes ex2 also does the float conversions, and
// it is the unit this kernel can saturate before the memory system: values are rounded in pairs
// (one packed conversion per two elements), and the rounding after the mask is added is skipped
// for a pack whose sums are already representable (always so for masks of 0 / -inf).
// (A persistent variant that prefetched its next row into registers ran 40 % slower: 80
// registers instead of 56 cost more in resident threads than the prefetch gained.)
template <typename TI, typename TO, int BLOCK>
__global__ void __launch_bounds__(BLOCK) softmax_row_kernel(const __grid_constant__ SoftmaxParams p) {
  __shared__ float scratch[2][32];
  constexpr int MAXP = 4;
  constexpr float LOG2E = 1.4426950408889634f;
  const int npack = static_cast<int>(p.cols >> 3);
  const bool scaled = p.scale != 1.f, rounded = p.round_steps != 0;
  const bool mask16 = p.mask && p.mask_dtype != B200_F32;
  uint4 raw[MAXP], mraw[MAXP];
  // row index and mask offset of work item `idx`
  auto locate = [&](int64_t idx, int64_t& row, int64_t& moff) {
    int64_t i0, i1, i2;
    if (p.d1_inner) {   // a mask row is then read from DRAM once and found in L2 by the other d1 - 1 blocks
      i1 = idx % p.d1; i2 = (idx / p.d1) % p.d2; i0 = idx / (p.d2 * p.d1);
    } else {
      i2 = idx % p.d2; i1 = (idx / p.d2) % p.d1; i0 = idx / (p.d2 * p.d1);
    }
    row = (i0 * p.d1 + i1) * p.d2 + i2;
    moff = i0 * p.ms0 + i1 * p.ms1 + i2 * p.ms2;
  };
  auto issue = [&](int64_t row, int64_t moff) {
    const uint4* xr = reinterpret_cast<const uint4*>(static_cast<const TI*>(p.x) + row * p.cols);
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pk = threadIdx.x + BLOCK * i;
      if (pk < npack) {
        raw[i] = ld_global_nc_v4(xr + pk);
        if (mask16) mraw[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const TI*>(p.mask) + moff) + pk);
      }
    }
  };
  int64_t row, moff;
  locate(blockIdx.x, row, moff);
  issue(row, moff);
  {
    float v[MAXP][8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pk = threadIdx.x + BLOCK * i;
      if (pk < npack) {
        unpack8<TI>(raw[i], v[i]);
        if (scaled) {
#pragma unroll
          for (int k = 0; k < 8; k += 2) {
            v[i][k] *= p.scale; v[i][k + 1] *= p.scale;
            if (rounded) round2<TI>(v[i][k], v[i][k + 1]);
          }
        }
        if (p.mask) {
          float m[8];
          if (mask16) {
            unpack8<TI>(mraw[i], m);
          } else {
            const float4* mp = reinterpret_cast<const float4*>(static_cast<const float*>(p.mask) + moff) + 2 * pk;
            const float4 a = __ldg(mp), b = __ldg(mp + 1);
            m[0] = a.x; m[1] = a.y; m[2] = a.z; m[3] = a.w; m[4] = b.x; m[5] = b.y; m[6] = b.z; m[7] = b.w;
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) v[i][k] += m[k];
          if (rounded && !exact_in<TI>(v[i])) {
#pragma unroll
            for (int k = 0; k < 8; k += 2) round2<TI>(v[i][k], v[i][k + 1]);
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) mx = fmaxf(mx, v[i][k]);
      }
    }
    TO* yr = static_cast<TO*>(p.y) + row * p.cols;
    mx = block_combine<true, BLOCK>(mx, scratch[0]);
    if (mx == -INFINITY) mx = 0.f;  // fully -inf row: every exp is 0, the row becomes 0 * inf = NaN as in ATen
    const float mxl = mx * LOG2E;
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pk = threadIdx.x + BLOCK * i;
      if (pk < npack) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { v[i][k] = ex2_ftz(fmaf(v[i][k], LOG2E, -mxl)); sum += v[i][k]; }
      }
    }
    sum = block_combine<false, BLOCK>(sum, scratch[1]);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pk = threadIdx.x + BLOCK * i;
      if (pk < npack) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] *= inv;
        if (sizeof(TO) == 2) {
          reinterpret_cast<uint4*>(yr)[pk] = pack8<TO>(v[i]);
        } else {
          float4* o = reinterpret_cast<float4*>(yr) + 2 * pk;
          o[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          o[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
      }
    }
  }
}

// Any cols / alignment: three passes, the row re-read from cache.
__global__ void __launch_bounds__(256) softmax_generic_kernel(const __grid_constant__ SoftmaxParams p, int in_dtype, int out_dtype) {
  __shared__ float scratch[33];
  const int64_t row = blockIdx.x;
  const int64_t i2 = row % p.d2, i1 = (row / p.d2) % p.d1, i0 = row / (p.d2 * p.d1);
  const int64_t base = row * p.cols;
  const int64_t moff = i0 * p.ms0 + i1 * p.ms1 + i2 * p.ms2;
  auto value = [&](int64_t c) {
    float t = load_as_f32(p.x, base + c, in_dtype);
    if (p.scale != 1.f) { t *= p.scale; if (p.round_steps) t = round_to(t, in_dtype); }
    if (p.mask) { t += load_as_f32(p.mask, moff + c, p.mask_dtype); if (p.round_steps) t = round_to(t, in_dtype); }
    return t;
  };
  float mx = -INFINITY;
  for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x) mx = fmaxf(mx, value(c));
  mx = block_reduce<true>(mx, scratch);
  if (mx == -INFINITY) mx = 0.f;
  float sum = 0.f;
  for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x) sum += fast_exp(value(c) - mx);
  sum = block_reduce<false>(sum, scratch);
  const float inv = 1.f / sum;
  for (int64_t c = threadIdx.x; c < p.cols; c += blockDim.x)
    store_from_f32(p.y, base + c, out_dtype, fast_exp(value(c) - mx) * inv);
}

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) mean_last_dim_kernel(const void* x, void* y, int64_t rows, int64_t cols, int in_dtype,
                                                            int out_dtype) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float s = 0.f;
  for (int64_t c = lane; c < cols; c += 32) s += load_as_f32(x, row * cols + c, in_dtype);
  s = warp_sum(s);
  if (lane == 0) store_from_f32(y, row, out_dtype, s / static_cast<float>(cols));
}

// ---------------------------------------------------------------------------
// Arg-max per row (greedy sampling).  One block per row; ties -> lowest index.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const T* __restrict__ x, int64_t* __restrict__ out, int64_t cols,
                                                           int64_t row_stride) {
  __shared__ float s_val[32];
  __shared__ int64_t s_idx[32];
  pdl_wait();
  pdl_trigger();
  const T* xr = x + static_cast<int64_t>(blockIdx.x) * row_stride;
  float best = -INFINITY;
  int64_t bidx = INT64_MAX;
  const bool vec = sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(xr) & 15u) == 0;
  const int64_t npack = vec ? (cols >> 3) : 0;
  for (int64_t pk = threadIdx.x; pk < npack; pk += blockDim.x) {
    float f[8];
    unpack8<T>(ld_global_nc_v4(reinterpret_cast<const uint4*>(xr) + pk), f);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (f[k] > best) { best = f[k]; bidx = pk * 8 + k; }
  }
  for (int64_t c = npack * 8 + threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32<T>(xr[c]);
    if (v > best || (v == best && c < bidx)) { best = v; bidx = c; }
  }
  auto better = [](float v, int64_t i, float bv, int64_t bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, bidx, o);
    if (better(ov, oi, best, bidx)) { best = ov; bidx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = bidx; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? s_val[lane] : -INFINITY;
    bidx = lane < nw ? s_idx[lane] : INT64_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (better(ov, oi, best, bidx)) { best = ov; bidx = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bidx == INT64_MAX ? 0 : bidx;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rmsnorm(const void* x, const void* w, void* y, int64_t rows, int64_t cols, int64_t x_row_stride,
                            int64_t y_row_stride, float eps, int dtype, int round_mid, void* stream) {
  B200_CHECK_ARG(x && w && y && rows >= 0 && cols > 0, "b200_rmsnorm: bad arguments");
  if (rows == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = cols % 8 == 0 && cols <= 2048 && x_row_stride % 8 == 0 && y_row_stride % 8 == 0 && aligned16(x) &&
                   aligned16(w) && aligned16(y);
  B200_DISPATCH_HALF(dtype, T, {
    const T* xp = static_cast<const T*>(x);
    const T* wp = static_cast<const T*>(w);
    T* yp = static_cast<T*>(y);
    if (vec) {
      const int grid = static_cast<int>(ceil_div(rows, 4));
      if (cols <= 1024)
        launch_pdl(rmsnorm_warp_kernel<T, 4>, dim3(grid), dim3(128), 0, st, xp, wp, yp, rows, (int)cols, x_row_stride, y_row_stride, eps, round_mid);
      else
        launch_pdl(rmsnorm_warp_kernel<T, 8>, dim3(grid), dim3(128), 0, st, xp, wp, yp, rows, (int)cols, x_row_stride, y_row_stride, eps, round_mid);
    } else {
      rmsnorm_block_kernel<T><<<static_cast<int>(rows), 256, 0, st>>>(xp, wp, yp, cols, x_row_stride, y_row_stride, eps, round_mid);
    }
  });
  B200_CHECK_LAUNCH("rmsnorm_kernel");
  return B200_OK;
}

template <typename TI, typename TO, int BLOCK>
static void launch_softmax_block(const SoftmaxParams& p, int64_t rows, cudaStream_t st) {
  softmax_row_kernel<TI, TO, BLOCK><<<static_cast<int>(rows), BLOCK, 0, st>>>(p);
}

template <typename TI, typename TO>
static void launch_softmax_rows(const SoftmaxParams& p, int64_t rows, cudaStream_t st) {
  if (p.cols <= 1024) launch_softmax_block<TI, TO, 32>(p, rows, st);
  else if (p.cols <= 2048) launch_softmax_block<TI, TO, 64>(p, rows, st);
  else if (p.cols <= 4096) launch_softmax_block<TI, TO, 128>(p, rows, st);
  else if (p.cols <= 8192) launch_softmax_block<TI, TO, 256>(p, rows, st);
  else launch_softmax_block<TI, TO, 1024>(p, rows, st);
}

extern "C" int b200_softmax(const void* x, const void* mask, void* y, int64_t d0, int64_t d1, int64_t d2, int64_t cols,
                            int64_t ms0, int64_t ms1, int64_t ms2, float scale, int in_dtype, int mask_dtype,
                            int out_dtype, int round_steps, void* stream) {
  B200_CHECK_ARG(x && y && d0 >= 0 && d1 >= 0 && d2 >= 0 && cols > 0, "b200_softmax: bad arguments");
  const int64_t rows = d0 * d1 * d2;
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(rows < (1ll << 31), "b200_softmax: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SoftmaxParams p{x, mask, y, d1, d2, cols, ms0, ms1, ms2, scale, round_steps, mask_dtype, (mask && ms1 == 0 && d1 > 1) ? 1 : 0};
  const bool half_in = in_dtype == B200_BF16 || in_dtype == B200_F16;
  bool vec = half_in && cols % 8 == 0 && cols <= 32768 && aligned16(x) && aligned16(y) &&
             (out_dtype == in_dtype || out_dtype == B200_F32);
  if (vec && mask)
    vec = (mask_dtype == in_dtype || mask_dtype == B200_F32) && aligned16(mask) && ms0 % 8 == 0 && ms1 % 8 == 0 && ms2 % 8 == 0;
  if (vec) {
    if (in_dtype == B200_BF16) {
      if (out_dtype == B200_F32) launch_softmax_rows<__nv_bfloat16, float>(p, rows, st);
      else launch_softmax_rows<__nv_bfloat16, __nv_bfloat16>(p, rows, st);
    } else {
      if (out_dtype == B200_F32) launch_softmax_rows<__half, float>(p, rows, st);
      else launch_softmax_rows<__half, __half>(p, rows, st);
    }
  } else {
    softmax_generic_kernel<<<static_cast<int>(rows), 256, 0, st>>>(p, in_dtype, out_dtype);
  }
  B200_CHECK_LAUNCH("softmax_kernel");
  return B200_OK;
}

extern "C" int b200_mean_last_dim(const void* x, void* y, int64_t rows, int64_t cols, int in_dtype, int out_dtype,
                                  void* stream) {
  B200_CHECK_ARG(x && y && rows >= 0 && cols > 0, "b200_mean_last_dim: bad arguments");
  if (rows == 0) return B200_OK;
  mean_last_dim_kernel<<<static_cast<int>(ceil_div(rows, 4)), 128, 0, static_cast<cudaStream_t>(stream)>>>(x, y, rows, cols,
                                                                                                           in_dtype, out_dtype);
  B200_CHECK_LAUNCH("mean_last_dim_kernel");
  return B200_OK;
}

extern "C" int b200_argmax_rows(const void* x, int64_t* out, int64_t rows, int64_t cols, int64_t row_stride, int dtype,
                                void* stream) {
  B200_CHECK_ARG(x && out && rows >= 0 && cols > 0, "b200_argmax_rows: bad arguments");
  if (rows == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_FLOAT(dtype, T, {
    launch_pdl(argmax_rows_kernel<T>, dim3(static_cast<unsigned>(rows)), dim3(1024), 0, st, static_cast<const T*>(x), out, cols, row_stride);
  });
  B200_CHECK_LAUNCH("argmax_rows_kernel");
  return B200_OK;
}
