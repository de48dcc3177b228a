// Dense contractions on the warp-level tensor-core path:
//   * gemm_tile_kernel  - 128x128 / 64x128 tiles, 4-stage cp.async pipeline, swizzled
//                         shared memory, ldmatrix + m16n8k16; serves linear layers with
//                         large M and, with the im2col gather switched on, NHWC convolution;
//   * gemm_skinny_kernel - M <= 64 (decode): weights streamed once from HBM straight into
//                         MMA fragments (no shared memory), split-K across CTAs;
//   * matmul_strided_kernel - fully strided batched fallback on CUDA cores.
#include "gemm_tc5.cuh"
#include "mma.cuh"

#include <stdlib.h>

namespace b200 {

// ===========================================================================
// Tiled GEMM / implicit-GEMM convolution.
//   out[m, n] = epi( sum_k A[m, k] * W[n, k] + bias[n] + residual[m, n] )
// ===========================================================================
struct ConvGeom {
  int H, W, C, KH, KW, sh, sw, ph, pw, Ho, Wo;
};

struct GemmParams {
  const void* A;
  const void* W;
  const void* bias;      // may be null
  const void* residual;  // may be null
  const void* aux;       // may be null (silu_mul)
  void* out;
  int64_t M, N, K;
  int64_t lda, ldw, ldo, ldr, ldaux;
  int bias_dtype;
  int epilogue;
  ConvGeom g;
};

constexpr int BN = 128, BK = 32, STAGES = 4;

// byte offset of 16-byte chunk `c` (0..3) of row `r` in a [rows][32] 16-bit tile
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return static_cast<uint32_t>(r * 64 + ((c ^ ((r >> 1) & 3)) << 4)); }

template <typename T, int MT, bool IS_CONV>  // MT = 16-row MMA tiles per warp along M (4 -> BM 128, 2 -> BM 64)
__global__ void __launch_bounds__(256) gemm_tile_kernel(const __grid_constant__ GemmParams p) {
  constexpr int BM = MT * 32;
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_base = smem_u32(smem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int warp_m = warp >> 2, warp_n = warp & 3;  // 2 x 4 warps
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
  const T* __restrict__ A = static_cast<const T*>(p.A);
  const T* __restrict__ Wt = static_cast<const T*>(p.W);

  // ---- per-thread load assignment: chunk ids tid + 256*i ---------------------
  constexpr int A_ITERS = BM * 4 / 256, B_ITERS = BN * 4 / 256;
  const int ld_c = tid & 3;  // same 16-byte column for all of this thread's chunks
  const T* a_ptr[A_ITERS];
  bool a_ok[A_ITERS];
  int a_ih0[A_ITERS], a_iw0[A_ITERS];
#pragma unroll
  for (int i = 0; i < A_ITERS; ++i) {
    const int64_t m = m0 + (tid >> 2) + 64 * i;
    a_ok[i] = m < p.M;
    if (IS_CONV) {
      const int64_t mm = a_ok[i] ? m : 0;
      const int ow = static_cast<int>(mm % p.g.Wo);
      const int oh = static_cast<int>((mm / p.g.Wo) % p.g.Ho);
      const int64_t n = mm / (static_cast<int64_t>(p.g.Wo) * p.g.Ho);
      a_ih0[i] = oh * p.g.sh - p.g.ph;
      a_iw0[i] = ow * p.g.sw - p.g.pw;
      a_ptr[i] = A + n * p.g.H * p.g.W * p.g.C;
    } else {
      a_ptr[i] = A + (a_ok[i] ? m : 0) * p.lda;
      a_ih0[i] = a_iw0[i] = 0;
    }
  }
  const T* b_ptr[B_ITERS];
  bool b_ok[B_ITERS];
#pragma unroll
  for (int i = 0; i < B_ITERS; ++i) {
    const int64_t n = n0 + (tid >> 2) + 64 * i;
    b_ok[i] = n < p.N;
    b_ptr[i] = Wt + (b_ok[i] ? n : 0) * p.ldw;
  }

  auto load_tile = [&](int stage, int64_t k0) {
    const uint32_t sA = smem_base + stage * STAGE_BYTES, sB = sA + A_BYTES;
    const int64_t k = k0 + ld_c * 8;
    const bool k_ok = k < p.K;
    int r = 0, s = 0, c = 0;
    if (IS_CONV && k_ok) {
      const int rs = static_cast<int>(k / p.g.C);
      c = static_cast<int>(k - static_cast<int64_t>(rs) * p.g.C);
      r = rs / p.g.KW;
      s = rs - r * p.g.KW;
    }
#pragma unroll
    for (int i = 0; i < A_ITERS; ++i) {
      const int row = (tid >> 2) + 64 * i;
      const T* src = a_ptr[i];
      bool ok = a_ok[i] && k_ok;
      if (IS_CONV) {
        const int ih = a_ih0[i] + r, iw = a_iw0[i] + s;
        ok = ok && ih >= 0 && ih < p.g.H && iw >= 0 && iw < p.g.W;
        if (ok) src += (static_cast<int64_t>(ih) * p.g.W + iw) * p.g.C + c;
      } else if (ok) {
        src += k;
      }
      cp_async16(sA + tile_off(row, ld_c), ok ? src : static_cast<const void*>(A), ok ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < B_ITERS; ++i) {
      const int row = (tid >> 2) + 64 * i;
      const bool ok = b_ok[i] && k_ok;
      cp_async16(sB + tile_off(row, ld_c), ok ? static_cast<const void*>(b_ptr[i] + k) : static_cast<const void*>(Wt), ok ? 16 : 0);
    }
  };

  float acc[MT][4][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  const int64_t KT = (p.K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) load_tile(s, static_cast<int64_t>(s) * BK);
    cp_async_commit();
  }

  // ldmatrix lane addressing (see mma.cuh): A x4 = (rows 0-7,k lo),(rows 8-15,k lo),(rows 0-7,k hi),(rows 8-15,k hi)
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_kc = lane >> 4;
  // B x4 = (n 0-7,k lo),(n 0-7,k hi),(n 8-15,k lo),(n 8-15,k hi)
  const int b_row = (lane & 7) + ((lane >> 4) & 1) * 8, b_kc = (lane >> 3) & 1;

  for (int64_t kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int64_t nk = kt + STAGES - 1;
      if (nk < KT) load_tile(static_cast<int>(nk % STAGES), nk * BK);
      cp_async_commit();
    }
    const uint32_t sA = smem_base + static_cast<int>(kt % STAGES) * STAGE_BYTES, sB = sA + A_BYTES;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t af[MT][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < MT; ++i) ldmatrix_x4(af[i], sA + tile_off(warp_m * (MT * 16) + i * 16 + a_row, ks * 2 + a_kc));
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t r[4];
        ldmatrix_x4(r, sB + tile_off(warp_n * 32 + j * 16 + b_row, ks * 2 + b_kc));
        bf[2 * j][0] = r[0]; bf[2 * j][1] = r[1]; bf[2 * j + 1][0] = r[2]; bf[2 * j + 1][1] = r[3];
      }
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) MmaType<T>::mma(acc[i][j], af[i], bf[j]);
    }
  }
  cp_async_wait<0>();

  // ---- epilogue --------------------------------------------------------------
  const int g = lane >> 2, t = lane & 3;
  T* __restrict__ out = static_cast<T*>(p.out);
  const T* __restrict__ res = static_cast<const T*>(p.residual);
  const T* __restrict__ aux = static_cast<const T*>(p.aux);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int64_t n = n0 + warp_n * 32 + j * 8 + 2 * t;
    if (n >= p.N) continue;
    const bool n1 = n + 1 < p.N;
    float b0 = 0.f, b1 = 0.f;
    if (p.bias) {
      b0 = load_as_f32(p.bias, n, p.bias_dtype);
      if (n1) b1 = load_as_f32(p.bias, n + 1, p.bias_dtype);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t m = m0 + warp_m * (MT * 16) + i * 16 + g + 8 * h;
        if (m >= p.M) continue;
        float v0 = acc[i][j][2 * h] + b0, v1 = acc[i][j][2 * h + 1] + b1;
        if (res) {
          // the unfused graph rounds the linear's output before the residual add
          v0 = round_as<T>(v0) + to_f32<T>(res[m * p.ldr + n]);
          if (n1) v1 = round_as<T>(v1) + to_f32<T>(res[m * p.ldr + n + 1]);
        }
        if (p.epilogue & B200_EPI_RELU) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
        if (p.epilogue & B200_EPI_SILU_MUL) {
          const float s0 = round_as<T>(v0), s1 = round_as<T>(v1);
          v0 = round_as<T>(silu_f32(s0)) * to_f32<T>(aux[m * p.ldaux + n]);
          if (n1) v1 = round_as<T>(silu_f32(s1)) * to_f32<T>(aux[m * p.ldaux + n + 1]);
        }
        T* o = out + m * p.ldo + n;
        if (n1 && ((reinterpret_cast<uintptr_t>(o) & 3u) == 0)) {
          *reinterpret_cast<uint32_t*>(o) = pack2<T>(v0, v1);
        } else {
          o[0] = from_f32<T>(v0);
          if (n1) o[1] = from_f32<T>(v1);
        }
      }
  }
}

// ===========================================================================
// Skinny-M weight-streaming GEMM (decode).
//
// The weight matrix is the MMA "A" operand (16 output features x 16 k) and the
// activations are the "B" operand (k x 8 batch rows).  Both fragments are filled by
// plain 16-byte global loads: within a 32-wide k chunk, thread t of a quad owns
// k = 8t..8t+7 of its row for BOTH operands, which is a consistent permutation of
// the k index and so leaves the dot product unchanged.  Weights therefore go
// HBM -> registers -> tensor core exactly once; activations are re-read from L1/L2.
// ===========================================================================
struct SkinnyParams {
  const void* X;  // [M, K]
  const void* W;  // [N, K]
  const void* bias;
  const void* residual;
  const void* aux;
  void* out;
  float* ws;           // fp32 [N][MPAD] partial sums (zero on entry, zero on exit)
  unsigned int* ctr;   // one arrival counter per row block (zero on entry and exit)
  int64_t M, N, K;
  int64_t ldx, ldw, ldo, ldr, ldaux;
  int bias_dtype, epilogue;
  int splits;          // CTAs along K
  int64_t k_per_split; // multiple of 32
};

constexpr int SK_ROWS = 128;  // output features per CTA (4 warps x 2 x 16)

__device__ __forceinline__ void red_add_v2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

template <typename T, int NT>  // NT = 8-row batch tiles (MPAD = 8*NT)
__global__ void __launch_bounds__(128) gemm_skinny_kernel(const __grid_constant__ SkinnyParams p) {
  constexpr int MPAD = NT * 8;
  __shared__ float stage[SK_ROWS][MPAD + 1];
  __shared__ int is_last;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  pdl_trigger();
  pdl_wait();
  const int64_t n_blk = static_cast<int64_t>(blockIdx.x) * SK_ROWS;
  const int64_t k_begin = static_cast<int64_t>(blockIdx.y) * p.k_per_split;
  const int64_t k_end = min(p.K, k_begin + p.k_per_split);
  const T* __restrict__ Wt = static_cast<const T*>(p.W);
  const T* __restrict__ X = static_cast<const T*>(p.X);

  // rows of W this thread feeds: two 16-row tiles, rows g and g+8 of each
  const T* w_row[2][2];
  bool w_ok[2][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t n = n_blk + warp * 32 + i * 16 + g + 8 * h;
      w_ok[i][h] = n < p.N;
      w_row[i][h] = Wt + (w_ok[i][h] ? n : 0) * p.ldw;
    }
  const T* x_row[NT];
  bool x_ok[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int64_t m = j * 8 + g;
    x_ok[j] = m < p.M;
    x_row[j] = X + (x_ok[j] ? m : 0) * p.ldx;
  }

  float acc[2][NT][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  // Weight fragments are double-buffered in registers: [tile][row half].
  auto load_w = [&](uint4 (&wf)[2][2], int64_t k) {
    const bool k_ok = k + 8 * t < k_end;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        wf[i][h] = (k_ok && w_ok[i][h]) ? ld_global_nc_v4(w_row[i][h] + k + 8 * t) : zero4;
  };
  auto compute = [&](const uint4 (&wf)[2][2], int64_t k) {
    const bool k_ok = k + 8 * t < k_end;
    uint4 xf[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j)
      xf[j] = (k_ok && x_ok[j]) ? __ldg(reinterpret_cast<const uint4*>(x_row[j] + k + 8 * t)) : zero4;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t a1[4] = {wf[i][0].x, wf[i][1].x, wf[i][0].y, wf[i][1].y};
      const uint32_t a2[4] = {wf[i][0].z, wf[i][1].z, wf[i][0].w, wf[i][1].w};
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint32_t b1[2] = {xf[j].x, xf[j].y};
        const uint32_t b2[2] = {xf[j].z, xf[j].w};
        MmaType<T>::mma(acc[i][j], a1, b1);
        MmaType<T>::mma(acc[i][j], a2, b2);
      }
    }
  };

  uint4 w0[2][2], w1[2][2];
  load_w(w0, k_begin);
  for (int64_t k = k_begin; k < k_end; k += 64) {
    load_w(w1, k + 32);   // loads past k_end return zeros
    compute(w0, k);
    load_w(w0, k + 64);
    compute(w1, k + 32);
  }

  // acc[i][j][2h+e] = partial out[m = 8j + 2t + e][n = n_blk + warp*32 + 16i + g + 8h]
  bool finish = true;
  if (p.splits > 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t n = n_blk + warp * 32 + i * 16 + g + 8 * h;
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < NT; ++j) red_add_v2(p.ws + n * MPAD + j * 8 + 2 * t, acc[i][j][2 * h], acc[i][j][2 * h + 1]);
        }
      }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int ticket = atomicAdd(p.ctr + blockIdx.x, 1u);
      is_last = ticket == static_cast<unsigned int>(p.splits) - 1u;
    }
    __syncthreads();
    finish = is_last != 0;
    if (finish) {
      __threadfence();
      // pull the summed tile from L2 and leave the workspace zeroed for the next launch
      for (int idx = threadIdx.x; idx < SK_ROWS * MPAD; idx += 128) {
        const int r = idx / MPAD, m = idx % MPAD;
        const int64_t n = n_blk + r;
        float v = 0.f;
        if (n < p.N) {
          float* a = p.ws + n * MPAD + m;
          v = __ldcg(a);
          __stcg(a, 0.f);
        }
        stage[r][m] = v;
      }
      if (threadIdx.x == 0) p.ctr[blockIdx.x] = 0u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int r = warp * 32 + i * 16 + g + 8 * h;
          stage[r][j * 8 + 2 * t] = acc[i][j][2 * h];
          stage[r][j * 8 + 2 * t + 1] = acc[i][j][2 * h + 1];
        }
  }
  if (!finish) return;
  __syncthreads();

  if (p.epilogue & B200_EPI_GLU) {
    // rows 0..63 of this block are gate features, rows 64..127 the matching up features
    if (threadIdx.x >= 64) return;
    const int64_t ng = n_blk + threadIdx.x, no = static_cast<int64_t>(blockIdx.x) * 64 + threadIdx.x;
    const float bg = p.bias ? load_as_f32(p.bias, ng, p.bias_dtype) : 0.f;
    const float bu = p.bias ? load_as_f32(p.bias, ng + 64, p.bias_dtype) : 0.f;
    T* __restrict__ og = static_cast<T*>(p.out);
    for (int64_t m = 0; m < p.M; ++m) {
      const float s = round_as<T>(stage[threadIdx.x][m] + bg);
      og[m * p.ldo + no] = from_f32<T>(round_as<T>(silu_f32(s)) * round_as<T>(stage[threadIdx.x + 64][m] + bu));
    }
    return;
  }
  // epilogue: thread r owns output feature n_blk + r, walks the batch rows
  const int64_t n = n_blk + threadIdx.x;
  if (n >= p.N) return;
  const float b = p.bias ? load_as_f32(p.bias, n, p.bias_dtype) : 0.f;
  T* __restrict__ out = static_cast<T*>(p.out);
  const T* __restrict__ res = static_cast<const T*>(p.residual);
  const T* __restrict__ aux = static_cast<const T*>(p.aux);
  for (int64_t m = 0; m < p.M; ++m) {
    float v = stage[threadIdx.x][m] + b;
    if (res) v = round_as<T>(v) + to_f32<T>(res[m * p.ldr + n]);
    if (p.epilogue & B200_EPI_RELU) v = fmaxf(v, 0.f);
    if (p.epilogue & B200_EPI_SILU_MUL) {
      const float s = round_as<T>(v);
      v = round_as<T>(silu_f32(s)) * to_f32<T>(aux[m * p.ldaux + n]);
    }
    out[m * p.ldo + n] = from_f32<T>(v);
  }
}

// ===========================================================================
// Fully strided batched matmul on CUDA cores (fallback for unfused graph matmuls).
// ===========================================================================
struct StridedMM {
  const void* A; const void* B; void* out;
  int64_t b1, b2, M, N, K;
  int64_t as[4], bs[4], os[4];  // (b1, b2, row, col) strides; A:(.,.,m,k) B:(.,.,k,n) out:(.,.,m,n)
};

template <typename T>
__global__ void __launch_bounds__(256) matmul_strided_kernel(const __grid_constant__ StridedMM p) {
  __shared__ float sa[16][17], sb[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t batch = blockIdx.z, i1 = batch / p.b2, i2 = batch % p.b2;
  const T* A = static_cast<const T*>(p.A) + i1 * p.as[0] + i2 * p.as[1];
  const T* B = static_cast<const T*>(p.B) + i1 * p.bs[0] + i2 * p.bs[1];
  T* O = static_cast<T*>(p.out) + i1 * p.os[0] + i2 * p.os[1];
  const int64_t m = static_cast<int64_t>(blockIdx.y) * 16 + ty, n = static_cast<int64_t>(blockIdx.x) * 16 + tx;
  float acc = 0.f;
  for (int64_t k0 = 0; k0 < p.K; k0 += 16) {
    const int64_t ka = k0 + tx, kb = k0 + ty;
    sa[ty][tx] = (m < p.M && ka < p.K) ? to_f32<T>(A[m * p.as[2] + ka * p.as[3]]) : 0.f;
    sb[ty][tx] = (kb < p.K && n < p.N) ? to_f32<T>(B[kb * p.bs[2] + n * p.bs[3]]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc += sa[ty][k] * sb[k][tx];
    __syncthreads();
  }
  if (m < p.M && n < p.N) O[m * p.os[2] + n * p.os[3]] = from_f32<T>(acc);
}

// ---------------------------------------------------------------------------
template <typename T, int MT, bool IS_CONV> static int launch_tile(const GemmParams& p, cudaStream_t st) {
  constexpr int BM = MT * 32;
  constexpr int SMEM = STAGES * (BM * BK * 2 + BN * BK * 2);
  static PerDevice<bool> configured_on;  // per instantiation and device
  bool* configured = configured_on.slot();
  if (!configured) B200_FAIL(B200_ELAUNCH, "gemm_tile_kernel: no current device");
  if (!*configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tile_kernel<T, MT, IS_CONV>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "gemm_tile_kernel attribute: %s", cudaGetErrorString(e));
    *configured = true;
  }
  dim3 grid(static_cast<unsigned>(ceil_div(p.N, BN)), static_cast<unsigned>(ceil_div(p.M, BM)));
  gemm_tile_kernel<T, MT, IS_CONV><<<grid, 256, SMEM, st>>>(p);
  B200_CHECK_LAUNCH("gemm_tile_kernel");
  return B200_OK;
}

template <typename T, bool IS_CONV> static int launch_tile_auto(const GemmParams& p, cudaStream_t st) {
  // prefer 128-row tiles unless they leave most SMs idle
  const int64_t ctas128 = ceil_div(p.N, BN) * ceil_div(p.M, 128);
  if (p.M <= 64 || ctas128 < sm_count()) return launch_tile<T, 2, IS_CONV>(p, st);
  return launch_tile<T, 4, IS_CONV>(p, st);
}

struct SkinnyPlan { int splits; int64_t k_per_split; int64_t row_blocks; int mpad; };

static SkinnyPlan plan_skinny(int64_t M, int64_t N, int64_t K) {
  SkinnyPlan s;
  s.mpad = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
  s.row_blocks = ceil_div(N, SK_ROWS);
  const int64_t ksteps = ceil_div(K, 32);
  const int64_t target = 4 * 148;  // CTAs wanted in flight (fixed, so that plans do not depend on the device)
  int64_t splits = target / s.row_blocks;
  if (splits < 1) splits = 1;
  const int64_t max_splits = ksteps / 4 > 0 ? ksteps / 4 : 1;  // at least 4 k-steps (128 k) per CTA
  if (splits > max_splits) splits = max_splits;
  const int64_t steps_per = ceil_div(ksteps, splits);
  s.k_per_split = steps_per * 32;
  s.splits = static_cast<int>(ceil_div(ksteps, steps_per));
  return s;
}

}  // namespace b200

using namespace b200;

static int64_t skinny_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M > 64 || M <= 0) return 0;
  const SkinnyPlan s = plan_skinny(M, N, K);
  if (s.splits <= 1) return 0;
  return s.row_blocks * SK_ROWS * s.mpad * 4 + s.row_blocks * 4 + 256;
}

extern "C" int64_t b200_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const int64_t a = skinny_workspace_bytes(M, N, K), b = linear_tc5_workspace_bytes(M, N, K);
  return a > b ? a : b;
}

extern "C" int b200_linear_norm(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M,
                                int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldo, int64_t ldr, int dtype,
                                int bias_dtype, int epilogue, float norm_eps, const float* sumsq_in, int sumsq_in_cols,
                                float* sumsq_out, void* stream) {
  B200_CHECK_ARG(A && W && out && M >= 0 && N > 0 && K > 0, "b200_linear_norm: bad arguments");
  B200_CHECK_ARG(!(epilogue & B200_EPI_SILU_MUL), "b200_linear_norm: the silu_mul epilogue is not available here");
  B200_CHECK_ARG(!(epilogue & B200_EPI_GLU) || (N % 128 == 0 && !residual && !sumsq_out), "b200_linear_norm: the gated epilogue needs N %% 128 == 0 and excludes residual / sumsq_out");
  B200_CHECK_ARG(!sumsq_in || sumsq_in_cols > 0, "b200_linear_norm: sumsq_in needs its column count");
  if (M == 0) return B200_OK;
  if (M > 64) B200_FAIL(B200_ENOTSUP, "b200_linear_norm: M = %lld; the fused forms exist for decode shapes (M <= 64) only", (long long)M);
  if (!(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && aligned16(A) && aligned16(W)))
    B200_FAIL(B200_EALIGN, "b200_linear_norm: K, lda, ldw must be multiples of 8 and A, W 16-byte aligned");
  Tc5Args t{A, W, bias, residual, nullptr, out, M, N, K, lda, ldw, ldo, ldr, 0, dtype, bias_dtype, epilogue, nullptr, 0};
  t.norm_eps = norm_eps; t.sumsq_in = sumsq_in; t.sumsq_in_cols = sumsq_in_cols; t.sumsq_out = sumsq_out;
  const int rc = linear_tc5(t, static_cast<cudaStream_t>(stream));
  if (rc == B200_ENOTSUP)
    B200_FAIL(B200_ENOTSUP, "b200_linear_norm: operands outside the fused kernel's rules (sumsq_in: at most 32 partials per row; "
                            "sumsq_out: N %% 64 == 0, 8-byte aligned rows of out / residual, bias in fp32 or the activation type)");
  return rc;
}

extern "C" int b200_linear(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M,
                           int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldo, int64_t ldr, int dtype,
                           int bias_dtype, int epilogue, const void* aux, int64_t ldaux, void* workspace,
                           int64_t workspace_bytes, void* stream) {
  B200_CHECK_ARG(A && W && out && M >= 0 && N > 0 && K > 0, "b200_linear: bad arguments");
  B200_CHECK_ARG(!(epilogue & B200_EPI_SILU_MUL) || aux, "b200_linear: silu_mul epilogue needs aux");
  B200_CHECK_ARG(!(epilogue & B200_EPI_GLU) || (N % 128 == 0 && !residual && !(epilogue & ~(B200_EPI_GLU | B200_EPI_W_STATIC))),
                 "b200_linear: the gated epilogue needs N %% 128 == 0 and excludes residual / other epilogues");
  if (M == 0) return B200_OK;
  if (!(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && aligned16(A) && aligned16(W)))
    B200_FAIL(B200_EALIGN, "b200_linear: K, lda, ldw must be multiples of 8 and A, W 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {   // the tcgen05 kernels first (measured faster for every batch size); what follows are the fallbacks for operands they cannot take
    Tc5Args t{A, W, bias, residual, aux, out, M, N, K, lda, ldw, ldo, ldr, ldaux, dtype, bias_dtype, epilogue, workspace, workspace_bytes};
    const int rc = linear_tc5(t, st);
    if (rc != B200_ENOTSUP) return rc;
  }
  if (M <= 64) {
    const SkinnyPlan s = plan_skinny(M, N, K);
    SkinnyParams p;
    p.X = A; p.W = W; p.bias = bias; p.residual = residual; p.aux = aux; p.out = out;
    p.M = M; p.N = N; p.K = K; p.ldx = lda; p.ldw = ldw; p.ldo = ldo; p.ldr = ldr; p.ldaux = ldaux;
    p.bias_dtype = bias_dtype; p.epilogue = epilogue; p.splits = s.splits; p.k_per_split = s.k_per_split;
    p.ws = nullptr; p.ctr = nullptr;
    if (s.splits > 1) {
      const int64_t need = skinny_workspace_bytes(M, N, K);
      if (!workspace || workspace_bytes < need || !aligned16(workspace))
        B200_FAIL(B200_EINVAL, "b200_linear: workspace of %lld bytes required (got %lld)", (long long)need, (long long)workspace_bytes);
      p.ws = static_cast<float*>(workspace);
      p.ctr = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(workspace) + s.row_blocks * SK_ROWS * s.mpad * 4);
    }
    dim3 grid(static_cast<unsigned>(s.row_blocks), static_cast<unsigned>(s.splits));
    B200_DISPATCH_HALF(dtype, T, {
      switch (s.mpad) {
        case 8: launch_pdl(gemm_skinny_kernel<T, 1>, grid, dim3(128), 0, st, p); break;
        case 16: launch_pdl(gemm_skinny_kernel<T, 2>, grid, dim3(128), 0, st, p); break;
        case 32: launch_pdl(gemm_skinny_kernel<T, 4>, grid, dim3(128), 0, st, p); break;
        default: launch_pdl(gemm_skinny_kernel<T, 8>, grid, dim3(128), 0, st, p); break;
      }
    });
    B200_CHECK_LAUNCH("gemm_skinny_kernel");
    return B200_OK;
  }
  if (epilogue & B200_EPI_GLU) B200_FAIL(B200_ENOTSUP, "b200_linear: the gated epilogue needs the tcgen05 path (operands aligned, B200NN_DISABLE_TC5 unset)");
  GemmParams p;
  p.A = A; p.W = W; p.bias = bias; p.residual = residual; p.aux = aux; p.out = out;
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldw = ldw; p.ldo = ldo; p.ldr = ldr; p.ldaux = ldaux;
  p.bias_dtype = bias_dtype; p.epilogue = epilogue;
  p.g = ConvGeom{};
  B200_DISPATCH_HALF(dtype, T, { return launch_tile_auto<T, false>(p, st); });
  return B200_OK;
}

extern "C" int b200_linear_rmsnorm(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M,
                                   int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldo, int64_t ldr, int dtype,
                                   int bias_dtype, int epilogue, void* workspace, int64_t workspace_bytes, const void* norm_weight,
                                   void* norm_out, int64_t ldn, float norm_eps, int round_mid, void* stream) {
  B200_CHECK_ARG(A && W && out && norm_weight && norm_out && M >= 0 && N > 0 && K > 0, "b200_linear_rmsnorm: bad arguments");
  B200_CHECK_ARG(!(epilogue & (B200_EPI_SILU_MUL | B200_EPI_GLU)), "b200_linear_rmsnorm: gated epilogues are not supported");
  if (M == 0) return B200_OK;
  int done = 0;
  int rc = B200_ENOTSUP;
  if (K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && aligned16(A) && aligned16(W)) {
    Tc5Args t{A, W, bias, residual, nullptr, out, M, N, K, lda, ldw, ldo, ldr, 0, dtype, bias_dtype, epilogue, workspace, workspace_bytes};
    t.norm_tail.gain = norm_weight; t.norm_tail.out = norm_out; t.norm_tail.ld = ldn; t.norm_tail.eps = norm_eps;
    t.norm_tail.round_mid = round_mid; t.norm_tail.done = &done;
    rc = linear_tc5(t, static_cast<cudaStream_t>(stream));
  }
  if (rc == B200_ENOTSUP)
    rc = b200_linear(A, W, bias, residual, out, M, N, K, lda, ldw, ldo, ldr, dtype, bias_dtype, epilogue, nullptr, 0, workspace, workspace_bytes, stream);
  if (rc != B200_OK || done) return rc;
  return b200_rmsnorm(out, norm_weight, norm_out, M, N, ldo, ldn, norm_eps, dtype, round_mid, stream);
}

extern "C" int b200_conv2d_nhwc(const void* x, const void* w, const float* bias, const void* residual, void* y, int N, int H,
                                int W, int C, int C_pad, int O, int KH, int KW, int sh, int sw, int ph, int pw, int Ho, int Wo,
                                int dtype, int epilogue, void* stream) {
  B200_CHECK_ARG(x && w && y && N >= 0 && H > 0 && W > 0 && C > 0 && O > 0 && KH > 0 && KW > 0 && sh > 0 && sw > 0 && Ho > 0 && Wo > 0,
                 "b200_conv2d_nhwc: bad arguments");
  B200_CHECK_ARG(C == C_pad && C % 8 == 0, "b200_conv2d_nhwc: channels must be padded to a multiple of 8 (C=%d, C_pad=%d)", C, C_pad);
  B200_CHECK_ARG(!(epilogue & B200_EPI_SILU_MUL), "b200_conv2d_nhwc: unsupported epilogue");
  if (!(aligned16(x) && aligned16(w))) B200_FAIL(B200_EALIGN, "b200_conv2d_nhwc: x and w must be 16-byte aligned");
  if (N == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (KH == 1 && KW == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0 && static_cast<int64_t>(N) * Ho * Wo > 64) {
    // a 1x1 stride-1 convolution over channels-last data is a plain GEMM over [N*H*W, C]
    const int64_t rows = static_cast<int64_t>(N) * Ho * Wo;
    Tc5Args t{x, w, bias, residual, nullptr, y, rows, O, C, C, C, O, O, 0, dtype, B200_F32, epilogue | B200_EPI_W_STATIC, nullptr, 0};
    const int rc = linear_tc5(t, st);
    if (rc != B200_ENOTSUP) return rc;
  }
  if (C % 64 == 0 || C == 8) {
    // implicit GEMM on the tcgen05 path: A rows fetched by the kernel itself
    const int64_t rows = static_cast<int64_t>(N) * Ho * Wo, K = static_cast<int64_t>(KH) * KW * C;
    Tc5Args t{x, w, bias, residual, nullptr, y, rows, O, K, 0, K, O, O, 0, dtype, B200_F32, epilogue, nullptr, 0};
    Tc5Conv g{H, W, C, KH, KW, sh, sw, ph, pw, Ho, Wo};
    g.batch = N;
    const int rc = conv_tc5(t, g, st);
    if (rc != B200_ENOTSUP) return rc;
  }
  GemmParams p;
  p.A = x; p.W = w; p.bias = bias; p.residual = residual; p.aux = nullptr; p.out = y;
  p.M = static_cast<int64_t>(N) * Ho * Wo; p.N = O; p.K = static_cast<int64_t>(KH) * KW * C;
  p.lda = 0; p.ldw = p.K; p.ldo = O; p.ldr = O; p.ldaux = 0;
  p.bias_dtype = B200_F32; p.epilogue = epilogue;
  p.g = ConvGeom{H, W, C, KH, KW, sh, sw, ph, pw, Ho, Wo};
  B200_DISPATCH_HALF(dtype, T, { return launch_tile_auto<T, true>(p, st); });
  return B200_OK;
}

extern "C" int b200_linear_qkv_rope(const void* A, const void* W, const void* bias, int64_t M, int64_t N, int64_t K, int64_t lda,
                                    int64_t ldw, int dtype, int bias_dtype, int epilogue, float norm_eps, const float* sumsq_in,
                                    int sumsq_in_cols, const void* cos_t, const void* sin_t, void* q_out, void* k_cache,
                                    void* v_cache, const void* cache_pos, int64_t cache_len, int pos_dtype, int Hq, int Hkv,
                                    void* stream) {
  B200_CHECK_ARG(A && W && cos_t && sin_t && q_out && k_cache && v_cache && cache_pos && M >= 0 && N > 0 && K > 0 && Hq > 0 && Hkv > 0 &&
                 cache_len > 0, "b200_linear_qkv_rope: bad arguments");
  B200_CHECK_ARG(N == static_cast<int64_t>(Hq + 2 * Hkv) * 128, "b200_linear_qkv_rope: N must be (Hq + 2 Hkv) * 128 (head dimension 128)");
  B200_CHECK_ARG(!(epilogue & ~B200_EPI_W_STATIC), "b200_linear_qkv_rope: no epilogue terms besides the bias");
  B200_CHECK_ARG(!sumsq_in || sumsq_in_cols > 0, "b200_linear_qkv_rope: sumsq_in needs its column count");
  if (M == 0) return B200_OK;
  if (M > 64) B200_FAIL(B200_ENOTSUP, "b200_linear_qkv_rope: M = %lld; one token per sequence and at most 64 sequences", (long long)M);
  if (!(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && aligned16(A) && aligned16(W)))
    B200_FAIL(B200_EALIGN, "b200_linear_qkv_rope: K, lda, ldw must be multiples of 8 and A, W 16-byte aligned");
  Tc5Args t{A, W, bias, nullptr, nullptr, nullptr, M, N, K, lda, ldw, 0, 0, 0, dtype, bias_dtype, epilogue, nullptr, 0};
  t.norm_eps = norm_eps; t.sumsq_in = sumsq_in; t.sumsq_in_cols = sumsq_in_cols;
  t.rope.cos = cos_t; t.rope.sin = sin_t; t.rope.q_out = q_out; t.rope.k_cache = k_cache; t.rope.v_cache = v_cache;
  t.rope.cache_pos = cache_pos; t.rope.cache_len = cache_len; t.rope.Hq = Hq; t.rope.Hkv = Hkv; t.rope.pos_dtype = pos_dtype;
  const int rc = linear_tc5(t, static_cast<cudaStream_t>(stream));
  if (rc == B200_ENOTSUP)
    B200_FAIL(B200_ENOTSUP, "b200_linear_qkv_rope: operands outside the fused kernel's rules (16-byte aligned tables and destinations, "
                            "int32 / int64 position, at most 32 sum-of-squares partials per row)");
  return rc;
}

extern "C" int b200_matmul_strided(const void* A, const void* B, void* out, int64_t b1, int64_t b2, int64_t M, int64_t N,
                                   int64_t K, const int64_t a_strides[4], const int64_t b_strides[4],
                                   const int64_t o_strides[4], int dtype, void* stream) {
  B200_CHECK_ARG(A && B && out && b1 >= 0 && b2 >= 0 && M >= 0 && N >= 0 && K >= 0 && a_strides && b_strides && o_strides,
                 "b200_matmul_strided: bad arguments");
  if (b1 * b2 * M * N == 0) return B200_OK;
  B200_CHECK_ARG(b1 * b2 <= 65535, "b200_matmul_strided: batch %lld too large", (long long)(b1 * b2));
  StridedMM p;
  p.A = A; p.B = B; p.out = out; p.b1 = b1; p.b2 = b2; p.M = M; p.N = N; p.K = K;
  for (int i = 0; i < 4; ++i) { p.as[i] = a_strides[i]; p.bs[i] = b_strides[i]; p.os[i] = o_strides[i]; }
  dim3 grid(static_cast<unsigned>(ceil_div(N, 16)), static_cast<unsigned>(ceil_div(M, 16)), static_cast<unsigned>(b1 * b2));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_FLOAT(dtype, T, { matmul_strided_kernel<T><<<grid, 256, 0, st>>>(p); });
  B200_CHECK_LAUNCH("matmul_strided_kernel");
  return B200_OK;
}
