// tcgen05 GEMM for large M:  out[M,N] = epi(A[M,K] * W[N,K]^T + bias + residual).
//
// One CTA computes a 128 x BN tile.  Warp 0 streams 128x64 (A) and BNx64 (W) tiles
// through a ring of shared-memory stages with TMA (128-byte swizzle, no multicast);
// warp 1 issues tcgen05.mma (M=128, N=BN, K=16) from shared-memory descriptors into a
// tensor-memory accumulator and releases stages with tcgen05.commit; warps 2-5 read the
// accumulator back with tcgen05.ld (each warp owns the 32 TMEM lanes of its quarter),
// apply the epilogue in fp32 and store.  Every barrier wait is bounded: on a timeout the
// CTA records an error code in `g_tc5_error`, drains its own copies and exits.
#include "gemm_tc5.cuh"
#include "tc5.cuh"

#include <stdlib.h>

namespace b200 {

__device__ int g_tc5_error = 0;

namespace {

constexpr int BM = 128, BK = 64;
// Kernel modes.
//   0  compute-bound shapes (several row tiles): two CTAs per SM with a short ring, so that
//      one CTA's epilogue overlaps the other's main loop;
//   1  a single row tile with 64 < M <= 128: pure weight streaming, one CTA per SM, deep ring;
//   2  M <= 64 (decode): the activation tile is loaded 64 rows high (the MMA still reads 128
//      rows; the upper half is whatever follows in shared memory and only feeds accumulator
//      rows that are never stored), which halves the stage size: two CTAs per SM, so the
//      next GEMM in the stream can already sit on the SM and prefetch its weights.
//   3  as 2, but one CTA per SM with a ring twice as deep (more bytes in flight per CTA).
template <int BN, int MODE> struct Cfg {
  static constexpr int AROWS = MODE >= 2 ? 64 : 128;
  static constexpr int A_STAGE = AROWS * BK * 2;
  static constexpr int ST = MODE == 0 ? (BN == 128 ? 3 : 4) : MODE == 1 ? (BN == 128 ? 6 : 8) : MODE == 2 ? (BN == 128 ? 4 : 6) : (BN == 128 ? 8 : 12);
  static constexpr int CTAS = (MODE == 1 || MODE == 3) ? 1 : 2;
};

int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return e && e[0] ? atoi(e) : dflt;
}
// decode (M <= 64) tuning: ring depth / CTAs per SM, and how many CTAs split-K aims for
int decode_deep() { static int v = env_int("B200NN_TC5_DECODE_DEEP", 0); return v; }
int split_target() { static int v = env_int("B200NN_TC5_SPLIT_CTAS", 148); return v; }
int split_traffic_div() { static int v = env_int("B200NN_TC5_SPLIT_TRAFFIC", 8); return v; }
int split_min_kb() { static int v = env_int("B200NN_TC5_SPLIT_MIN_KB", 4); return v; }

struct Tc5Params {
  const void* bias; const void* residual; const void* aux; void* out;
  float* ws;            // split-K partial sums, fp32 [M][ws_pitch]; zero on entry, zero on exit
  unsigned int* ctr;    // one arrival counter per output tile; zero on entry and exit
  int64_t M, N, K, ldo, ldr, ldaux, ws_pitch;
  int bias_dtype, epilogue, splits, kb_per_split;
  const void* x;   // convolution input (implicit-GEMM mode only)
  Tc5Conv g;
};

template <typename T> struct AbFormat;
template <> struct AbFormat<__half> { static constexpr int value = 0; };
template <> struct AbFormat<__nv_bfloat16> { static constexpr int value = 1; };

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// bias / residual / activation on 32 consecutive outputs of row m starting at column n, then store
template <typename T>
__device__ __forceinline__ void finish_row(const Tc5Params& p, float (&v)[32], int64_t m, int64_t n) {
  const int cnt = static_cast<int>(p.N - n < 32 ? p.N - n : 32);
  const T* __restrict__ res = static_cast<const T*>(p.residual);
  const T* __restrict__ aux = static_cast<const T*>(p.aux);
  if (p.bias) {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < cnt) v[i] += load_as_f32(p.bias, n + i, p.bias_dtype);
  }
  if (res) {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < cnt) v[i] = round_as<T>(v[i]) + to_f32<T>(res[m * p.ldr + n + i]);
  }
  if (p.epilogue & B200_EPI_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
  }
  if (p.epilogue & B200_EPI_SILU_MUL) {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < cnt) {
      const float s = round_as<T>(v[i]);
      v[i] = round_as<T>(s / (1.f + expf(-s))) * to_f32<T>(aux[m * p.ldaux + n + i]);
    }
  }
  T* o = static_cast<T*>(p.out) + m * p.ldo + n;
  if (cnt == 32 && (reinterpret_cast<uintptr_t>(o) & 15u) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = v[8 * j + i];
      reinterpret_cast<uint4*>(o)[j] = pack8<T>(f);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < cnt) o[i] = from_f32<T>(v[i]);
  }
}

// gated-MLP epilogue: 32 gate accumulators and the 32 matching up accumulators of row m
template <typename T>
__device__ __forceinline__ void finish_glu(const Tc5Params& p, float (&vg)[32], float (&vu)[32], int64_t m, int64_t n_merged, int64_t n_out) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float g = vg[i], u = vu[i];
    if (p.bias) { g += load_as_f32(p.bias, n_merged + i, p.bias_dtype); u += load_as_f32(p.bias, n_merged + 64 + i, p.bias_dtype); }
    const float s = round_as<T>(g);
    v[i] = round_as<T>(s / (1.f + expf(-s))) * round_as<T>(u);
  }
  T* o = static_cast<T*>(p.out) + m * p.ldo + n_out;
  if ((reinterpret_cast<uintptr_t>(o) & 15u) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = v[8 * j + i];
      reinterpret_cast<uint4*>(o)[j] = pack8<T>(f);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = from_f32<T>(v[i]);
  }
}

__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_dst, const void* gptr, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gptr), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc5::smem_addr(bar)) : "memory");
}

// CONV = false: A tiles arrive by TMA.  CONV = true (implicit-GEMM convolution): the four
// epilogue warps, idle during the main loop, gather the A tile - one output pixel per
// thread, 128 bytes of channels per k-block - with zero-filling cp.async into the same
// 128-byte-swizzled layout TMA would produce, and signal the stage's barrier themselves.
template <typename T, int BN, bool CONV, int MODE>
__global__ void __launch_bounds__(192, Cfg<BN, MODE>::CTAS) gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_w, const Tc5Params p) {
  constexpr int ST = Cfg<BN, MODE>::ST, A_STAGE = Cfg<BN, MODE>::A_STAGE;
  constexpr int B_STAGE = BN * BK * 2, STAGE = A_STAGE + B_STAGE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[ST], empty_bar[ST], acc_bar;
  __shared__ uint32_t tmem_holder;
  __shared__ int failed, is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int KB = static_cast<int>((p.K + BK - 1) / BK);
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int nkb = min(KB, kb0 + p.kb_per_split) - kb0;   // >= 1 by construction of the grid

  if (threadIdx.x == 0) {
    failed = 0;
    is_last = 0;
    for (int s = 0; s < ST; ++s) { tc5::mbar_init(&full_bar[s], CONV ? 129 : 1); tc5::mbar_init(&empty_bar[s], 1); }
    tc5::mbar_init(&acc_bar, 1);
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&map_a);
    tc5::prefetch_tensormap(&map_w);
  }
  if (warp == 1) { tc5::tmem_alloc(&tmem_holder, BN); tc5::tmem_relinquish(); }
  tc5::tc_fence_before();
  __syncthreads();
  tc5::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_trigger();   // the next kernel in the stream may be scheduled (it waits for this one before reading)

  if (warp == 0) {
    if (lane == 0) {
      // Weights that no kernel of this stream writes can be fetched before the predecessor has
      // finished: fill the ring with weight tiles first, then wait, then add the activation tiles.
      int pre = 0;
      if (!CONV && (p.epilogue & B200_EPI_W_STATIC)) {
        pre = nkb < ST ? nkb : ST;
        for (int i = 0; i < pre; ++i) {
          tc5::mbar_arrive_expect_tx(&full_bar[i], STAGE);
          tc5::tma_load_2d(smem + i * STAGE + A_STAGE, &map_w, &full_bar[i], (kb0 + i) * BK, n0);
        }
      }
      pdl_wait();
      int issued = pre;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % ST;
        const uint32_t ph = (i / ST) & 1;
        if (i >= pre) {
          if (!tc5::mbar_wait(&empty_bar[s], ph ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 1); break; }
          if (*reinterpret_cast<volatile int*>(&failed)) break;
          tc5::mbar_arrive_expect_tx(&full_bar[s], CONV ? B_STAGE : STAGE);
          tc5::tma_load_2d(smem + s * STAGE + A_STAGE, &map_w, &full_bar[s], (kb0 + i) * BK, n0);
        }
        if (!CONV) tc5::tma_load_2d(smem + s * STAGE, &map_a, &full_bar[s], (kb0 + i) * BK, m0);
        if (i + 1 > issued) issued = i + 1;
      }
      if (*reinterpret_cast<volatile int*>(&failed)) {  // wait (bounded) for our own copies still in flight
        for (int i = issued > ST ? issued - ST : 0; i < issued; ++i) tc5::mbar_wait(&full_bar[i % ST], (i / ST) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::umma_idesc(BM, BN, AbFormat<T>::value);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % ST;
        const uint32_t ph = (i / ST) & 1;
        if (!tc5::mbar_wait(&full_bar[s], ph)) { failed = 1; atomicExch(&g_tc5_error, 2); break; }
        tc5::tc_fence_after();
        const uint32_t a_addr = tc5::smem_addr(smem + s * STAGE), b_addr = a_addr + A_STAGE;
        const uint64_t da = tc5::umma_desc_sw128(a_addr), db = tc5::umma_desc_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)  // 16 elements = 32 bytes = 2 descriptor address units
          tc5::umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
        tc5::umma_commit(&empty_bar[s]);
      }
      tc5::umma_commit(&acc_bar);
    }
  } else {
    pdl_wait();   // residual, bias, split-K scratch and convolution inputs come from earlier kernels
    const int q = warp & 3;  // warps 2,3,4,5 -> TMEM lane quarters 2,3,0,1
    if (CONV) {
      // ---- A-operand gather: this thread owns tile row q*32+lane (the pixel it will also finish) ----
      constexpr int LAG = 2;   // k-blocks of copies kept in flight per thread
      const int row = q * 32 + lane;
      const int64_t mrow = static_cast<int64_t>(m0) + row;
      const bool row_ok = mrow < p.M;
      const int64_t mm = row_ok ? mrow : 0;
      const int ow = static_cast<int>(mm % p.g.Wo), oh = static_cast<int>((mm / p.g.Wo) % p.g.Ho);
      const int64_t img = mm / (static_cast<int64_t>(p.g.Wo) * p.g.Ho);
      const int ih0 = oh * p.g.sh - p.g.ph, iw0 = ow * p.g.sw - p.g.pw;
      const T* xb = static_cast<const T*>(p.x) + img * p.g.H * p.g.W * p.g.C;
      const int cpb = p.g.C / BK;   // k-blocks per filter tap
      const uint32_t row_off = row * 128, swz = row & 7;
      bool alive = true;
      for (int i = 0; i < nkb + LAG; ++i) {
        if (i < nkb && alive) {
          const int s = i % ST;
          if (!tc5::mbar_wait(&empty_bar[s], ((i / ST) & 1) ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 4); alive = false; }
          if (alive) {
            const int kb = kb0 + i, tap = kb / cpb, c0 = (kb - tap * cpb) * BK;
            const int r = tap / p.g.KW, sx = tap - r * p.g.KW;
            const int ih = ih0 + r, iw = iw0 + sx;
            const bool in = row_ok && ih >= 0 && ih < p.g.H && iw >= 0 && iw < p.g.W;
            const T* src = in ? xb + (static_cast<int64_t>(ih) * p.g.W + iw) * p.g.C + c0 : static_cast<const T*>(p.x);
            const uint32_t dst = tc5::smem_addr(smem + s * STAGE) + row_off;
#pragma unroll
            for (int j = 0; j < 8; ++j) cp_async16_zfill(dst + ((j ^ swz) << 4), src + (in ? j * 8 : 0), in ? 16 : 0);
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (i >= LAG && alive) {
          asm volatile("cp.async.wait_group %0;" ::"n"(LAG) : "memory");
          tc5::fence_proxy_async();          // generic-proxy writes -> visible to the tensor core's async-proxy reads
          mbar_arrive(&full_bar[(i - LAG) % ST]);
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    bool ok = true;
    if (lane == 0) ok = tc5::mbar_wait(&acc_bar, 0);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok && lane == 0) { failed = 1; atomicExch(&g_tc5_error, 3); }
    ok = ok && !*reinterpret_cast<volatile int*>(&failed);
    ok = __all_sync(0xffffffffu, ok);
    const int64_t m = m0 + q * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const bool glu = (p.epilogue & B200_EPI_GLU) != 0;  // host guarantees BN == 128 and N % 128 == 0
    if (ok && glu && p.splits == 1) {
      tc5::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        float vg[32], vu[32];
        __syncwarp();
        tc5::tmem_ld_32x32(t_row + c * 32, vg);
        tc5::tmem_ld_32x32(t_row + 64 + c * 32, vu);
        if (m < p.M) finish_glu<T>(p, vg, vu, m, n0 + c * 32, n0 / 2 + c * 32);
      }
      tc5::tc_fence_before();
    } else if (ok) {
      tc5::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        __syncwarp();  // tcgen05.ld is warp-collective; lanes that skipped the stores rejoin here
        tc5::tmem_ld_32x32(t_row + c * 32, v);
        const int64_t n = n0 + c * 32;
        if (m >= p.M) continue;
        if (p.splits == 1) {
          if (n < p.N) finish_row<T>(p, v, m, n);
        } else {
          float* w = p.ws + m * p.ws_pitch + n;
#pragma unroll
          for (int j = 0; j < 8; ++j) red_add_v4(w + 4 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
      }
      tc5::tc_fence_before();
    }
    if (p.splits > 1) {  // uniform for the whole grid: the four epilogue warps meet on named barrier 1
      __threadfence();
      epilogue_bar();
      if (warp == 2 && lane == 0) {
        const unsigned int tile = blockIdx.y * gridDim.x + blockIdx.x;
        const unsigned int ticket = atomicAdd(p.ctr + tile, 1u);
        is_last = ticket == static_cast<unsigned int>(p.splits) - 1u;
        if (is_last) p.ctr[tile] = 0u;
      }
      epilogue_bar();
      auto take = [&](int64_t n, float (&v)[32]) {  // read 32 summed partials and leave zeros behind
        float4* w = reinterpret_cast<float4*>(p.ws + m * p.ws_pitch + n);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 t = __ldcg(w + j);
          __stcg(w + j, make_float4(0.f, 0.f, 0.f, 0.f));
          v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
        }
      };
      if (*reinterpret_cast<volatile int*>(&is_last) && m < p.M && glu) {
        __threadfence();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          float vg[32], vu[32];
          take(n0 + c * 32, vg);
          take(n0 + 64 + c * 32, vu);
          finish_glu<T>(p, vg, vu, m, n0 + c * 32, n0 / 2 + c * 32);
        }
      } else if (*reinterpret_cast<volatile int*>(&is_last) && m < p.M) {
        __threadfence();
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int64_t n = n0 + c * 32;
          float v[32];
          take(n, v);
          if (n < p.N) finish_row<T>(p, v, m, n);
        }
      }
    }
  }
  __syncthreads();
  if (warp == 1) { tc5::tc_fence_after(); tc5::tmem_dealloc(tmem_base, BN); }
}

// ===========================================================================================
// Persistent variant for compute-bound shapes (several row tiles, no split-K).
//
// One CTA per SM walks the tile list (tile = blockIdx.x, += gridDim.x; row tiles of one
// column tile are neighbours, so concurrently running CTAs share a weight tile in L2).  The
// shared-memory ring runs across tile boundaries, and the accumulator is double-buffered in
// tensor memory (2 x BN columns), so the four epilogue warps drain tile i while the MMA warp
// already works on tile i+1.  BN = 256 halves the shared-memory traffic per flop of the
// 128-wide tiles.  Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue, and
// for convolutions warps 6-9 gather the A tile (implicit GEMM) as in the kernel above.
// ===========================================================================================
template <int BN> struct PCfg {
  static constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2, STAGE = A_STAGE + B_STAGE;
  static constexpr int ST = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int SMEM = ST * STAGE + 1024;
};

template <typename T, int BN, bool CONV>
__global__ void __launch_bounds__(CONV ? 320 : 192, 1) gemm_tc5p_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                       const __grid_constant__ CUtensorMap map_w, const Tc5Params p,
                                                                       const int tiles_m, const int n_tiles) {
  constexpr int ST = PCfg<BN>::ST, A_STAGE = PCfg<BN>::A_STAGE, B_STAGE = PCfg<BN>::B_STAGE, STAGE = PCfg<BN>::STAGE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[ST], empty_bar[ST], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = static_cast<int>((p.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < ST; ++s) { tc5::mbar_init(&full_bar[s], CONV ? 129 : 1); tc5::mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { tc5::mbar_init(&acc_full[b], 1); tc5::mbar_init(&acc_empty[b], 4); }
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&map_a);
    tc5::prefetch_tensormap(&map_w);
  }
  if (warp == 1) { tc5::tmem_alloc(&tmem_holder, 2 * BN); tc5::tmem_relinquish(); }
  tc5::tc_fence_before();
  __syncthreads();
  tc5::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_trigger();
  auto dead = [&]() { return *reinterpret_cast<volatile int*>(&failed) != 0; };

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      int it = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !dead(); tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % ST;
          if (!tc5::mbar_wait(&empty_bar[s], ((it / ST) & 1) ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 11); break; }
          tc5::mbar_arrive_expect_tx(&full_bar[s], CONV ? B_STAGE : STAGE);
          if (!CONV) tc5::tma_load_2d(smem + s * STAGE, &map_a, &full_bar[s], kb * BK, m0);
          tc5::tma_load_2d(smem + s * STAGE + A_STAGE, &map_w, &full_bar[s], kb * BK, n0);
        }
      }
      if (dead()) {  // wait (bounded) for our own copies still in flight
        for (int i = it > ST ? it - ST : 0; i < it; ++i) tc5::mbar_wait(&full_bar[i % ST], (i / ST) & 1, 1u << 16);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::umma_idesc(BM, BN, AbFormat<T>::value);
      int it = 0, ti = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !dead(); tile += gridDim.x, ++ti) {
        const int b = ti & 1;
        if (!tc5::mbar_wait(&acc_empty[b], ((ti >> 1) & 1) ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 12); break; }
        tc5::tc_fence_after();
        const uint32_t acc = tmem_base + b * BN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % ST;
          if (!tc5::mbar_wait(&full_bar[s], (it / ST) & 1)) { failed = 1; atomicExch(&g_tc5_error, 13); break; }
          tc5::tc_fence_after();
          const uint32_t a_addr = tc5::smem_addr(smem + s * STAGE), b_addr = a_addr + A_STAGE;
          const uint64_t da = tc5::umma_desc_sw128(a_addr), db = tc5::umma_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) tc5::umma_f16(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          tc5::umma_commit(&empty_bar[s]);
        }
        if (dead()) break;
        tc5::umma_commit(&acc_full[b]);
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    pdl_wait();
    const bool glu = (p.epilogue & B200_EPI_GLU) != 0;
    int ti = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
      const int b = ti & 1;
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      bool ok = true;
      if (lane == 0) ok = tc5::mbar_wait(&acc_full[b], (ti >> 1) & 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) { failed = 1; atomicExch(&g_tc5_error, 14); }
      ok = __all_sync(0xffffffffu, ok && !dead());
      if (!ok) break;
      tc5::tc_fence_after();
      const int64_t m = static_cast<int64_t>(m0) + q * 32 + lane;
      const uint32_t t_row = tmem_base + b * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (glu) {
#pragma unroll 1
        for (int h = 0; h < BN / 128; ++h)
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            float vg[32], vu[32];
            __syncwarp();
            tc5::tmem_ld_32x32(t_row + h * 128 + c * 32, vg);
            tc5::tmem_ld_32x32(t_row + h * 128 + 64 + c * 32, vu);
            const int64_t nm = static_cast<int64_t>(n0) + h * 128 + c * 32;
            if (m < p.M && nm < p.N) finish_glu<T>(p, vg, vu, m, nm, (static_cast<int64_t>(n0) + h * 128) / 2 + c * 32);
          }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          __syncwarp();
          tc5::tmem_ld_32x32(t_row + c * 32, v);
          const int64_t n = static_cast<int64_t>(n0) + c * 32;
          if (m < p.M && n < p.N) finish_row<T>(p, v, m, n);
        }
      }
      tc5::tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);   // this warp has drained its quarter of the accumulator
    }
  } else if (CONV) {
    // ---- A-operand gather (warps 6-9): thread r owns tile row r, i.e. one output pixel per tile ----
    constexpr int LAG = 2;
    const int row = (warp - 6) * 32 + lane;
    const int cpb = p.g.C / BK;
    const uint32_t row_off = row * 128, swz = row & 7;
    pdl_wait();
    int it = 0;          // k-blocks issued
    int arrived = 0;     // k-blocks signalled
    bool alive = true;
    for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const int64_t mrow = static_cast<int64_t>(tile % tiles_m) * BM + row;
      const bool row_ok = mrow < p.M;
      const int64_t mm = row_ok ? mrow : 0;
      const int ow = static_cast<int>(mm % p.g.Wo), oh = static_cast<int>((mm / p.g.Wo) % p.g.Ho);
      const int64_t img = mm / (static_cast<int64_t>(p.g.Wo) * p.g.Ho);
      const int ih0 = oh * p.g.sh - p.g.ph, iw0 = ow * p.g.sw - p.g.pw;
      const T* xb = static_cast<const T*>(p.x) + img * p.g.H * p.g.W * p.g.C;
      for (int kb = 0; kb < KB && alive; ++kb, ++it) {
        const int s = it % ST;
        if (!tc5::mbar_wait(&empty_bar[s], ((it / ST) & 1) ^ 1) || dead()) { failed = 1; atomicExch(&g_tc5_error, 15); alive = false; break; }
        const int tap = kb / cpb, c0 = (kb - tap * cpb) * BK;
        const int r = tap / p.g.KW, sx = tap - r * p.g.KW;
        const int ih = ih0 + r, iw = iw0 + sx;
        const bool in = row_ok && ih >= 0 && ih < p.g.H && iw >= 0 && iw < p.g.W;
        const T* src = in ? xb + (static_cast<int64_t>(ih) * p.g.W + iw) * p.g.C + c0 : static_cast<const T*>(p.x);
        const uint32_t dst = tc5::smem_addr(smem + s * STAGE) + row_off;
#pragma unroll
        for (int j = 0; j < 8; ++j) cp_async16_zfill(dst + ((j ^ swz) << 4), src + (in ? j * 8 : 0), in ? 16 : 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (it - arrived >= LAG) {
          asm volatile("cp.async.wait_group %0;" ::"n"(LAG) : "memory");
          tc5::fence_proxy_async();
          mbar_arrive(&full_bar[arrived % ST]);
          ++arrived;
        }
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (alive) {
      tc5::fence_proxy_async();
      for (; arrived < it; ++arrived) mbar_arrive(&full_bar[arrived % ST]);
    }
  }
  __syncthreads();
  if (warp == 1) { tc5::tc_fence_after(); tc5::tmem_dealloc(tmem_base, 2 * BN); }
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, K] row-major with row stride `ld` elements -> map with a (64 x box_rows) box, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows, int dtype) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Tc5Plan { int bn, splits, kb_per_split; int64_t tiles_n, tiles_m, ws_pitch; };

Tc5Plan plan_tc5(int64_t M, int64_t N, int64_t K, bool glu = false) {
  Tc5Plan pl;
  const int64_t tm = ceil_div(M, BM);
  // 64-wide tiles whenever 128-wide ones would not give every SM a tile (148 SMs; fixed so that
  // the workspace size does not depend on the device the plan is made on)
  pl.bn = (!glu && ceil_div(N, 128) * tm < 148) ? 64 : 128;   // the gated epilogue pairs columns c and c+64 of a 128-wide tile
  pl.tiles_n = ceil_div(N, pl.bn);
  pl.tiles_m = tm;
  const int64_t tiles = pl.tiles_n * tm, KB = ceil_div(K, BK);
  int64_t splits = 1;
  if (tiles < 100) {
    splits = split_target() == 148 ? ceil_div(148, tiles) : split_target() / tiles;
    const int64_t by_traffic = K / (split_traffic_div() * (M < BM ? M : BM));   // partial sums stay below the weight bytes
    if (splits > by_traffic) splits = by_traffic;
    if (splits > KB / split_min_kb()) splits = KB / split_min_kb();             // at least this many k-blocks per CTA
    if (splits < 1) splits = 1;
  }
  pl.kb_per_split = static_cast<int>(ceil_div(KB, splits));
  pl.splits = static_cast<int>(ceil_div(KB, pl.kb_per_split));
  pl.ws_pitch = pl.tiles_n * pl.bn;
  return pl;
}

template <typename T, int BN, bool CONV, int MODE = 0>
int launch(const Tc5Args& a, const Tc5Plan& pl, cudaStream_t st, const Tc5Conv* g = nullptr) {
  constexpr int SMEM = Cfg<BN, MODE>::ST * (Cfg<BN, MODE>::A_STAGE + BN * BK * 2) + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc5_kernel<T, BN, CONV, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    configured = true;
  }
  CUtensorMap ma, mw;
  if (!make_map(&mw, a.W, a.N, a.K, a.ldw, BN, a.dtype)) return B200_ENOTSUP;
  if (CONV) ma = mw;   // unused in implicit-GEMM mode
  else if (!make_map(&ma, a.A, a.M, a.K, a.lda, Cfg<BN, MODE>::AROWS, a.dtype)) return B200_ENOTSUP;
  Tc5Params p;
  p.x = a.A;
  p.g = g ? *g : Tc5Conv{};
  p.bias = a.bias; p.residual = a.residual; p.aux = a.aux; p.out = a.out;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo; p.ldr = a.ldr; p.ldaux = a.ldaux; p.ws_pitch = pl.ws_pitch;
  p.bias_dtype = a.bias_dtype; p.epilogue = a.epilogue; p.splits = pl.splits; p.kb_per_split = pl.kb_per_split;
  p.ws = nullptr; p.ctr = nullptr;
  if (pl.splits > 1) {
    const int64_t need = a.M * pl.ws_pitch * 4 + pl.tiles_n * pl.tiles_m * 4 + 256;
    if (!a.workspace || a.workspace_bytes < need || !aligned16(a.workspace)) return B200_ENOTSUP;
    p.ws = static_cast<float*>(a.workspace);
    p.ctr = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(a.workspace) + a.M * pl.ws_pitch * 4);
  }
  dim3 grid(static_cast<unsigned>(pl.tiles_n), static_cast<unsigned>(pl.tiles_m), static_cast<unsigned>(pl.splits));
  launch_pdl(gemm_tc5_kernel<T, BN, CONV, MODE>, grid, dim3(192), SMEM, st, ma, mw, p);
  B200_CHECK_LAUNCH("gemm_tc5_kernel");
  return B200_OK;
}

template <typename T, int BN, bool CONV>
int launch_persistent(const Tc5Args& a, cudaStream_t st, const Tc5Conv* g = nullptr) {
  constexpr int SMEM = PCfg<BN>::SMEM;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc5p_kernel<T, BN, CONV>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    configured = true;
  }
  CUtensorMap ma, mw;
  if (!make_map(&mw, a.W, a.N, a.K, a.ldw, BN, a.dtype)) return B200_ENOTSUP;
  if (CONV) ma = mw;
  else if (!make_map(&ma, a.A, a.M, a.K, a.lda, BM, a.dtype)) return B200_ENOTSUP;
  Tc5Params p;
  p.bias = a.bias; p.residual = a.residual; p.aux = a.aux; p.out = a.out;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo; p.ldr = a.ldr; p.ldaux = a.ldaux; p.ws_pitch = 0;
  p.bias_dtype = a.bias_dtype; p.epilogue = a.epilogue; p.splits = 1; p.kb_per_split = static_cast<int>(ceil_div(a.K, BK));
  p.ws = nullptr; p.ctr = nullptr;
  p.x = a.A;
  p.g = g ? *g : Tc5Conv{};
  const int64_t tiles_m = ceil_div(a.M, BM), tiles = tiles_m * ceil_div(a.N, BN);
  if (tiles >= (1ll << 31)) return B200_ENOTSUP;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  launch_pdl(gemm_tc5p_kernel<T, BN, CONV>, dim3(grid), dim3(CONV ? 320 : 192), SMEM, st, ma, mw, p, static_cast<int>(tiles_m),
             static_cast<int>(tiles));
  B200_CHECK_LAUNCH("gemm_tc5p_kernel");
  return B200_OK;
}

// Tile width of the persistent kernel for a shape, or 0 when the shape should stay on the
// one-tile-per-CTA kernel (too few tiles to fill the SMs with wide tiles).
int persistent_bn(int64_t M, int64_t N, bool glu) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("B200NN_TC5_PERSISTENT");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  const int64_t tm = ceil_div(M, BM);
  if (!enabled || tm < 2) return 0;
  if (ceil_div(N, 256) * tm >= 2 * 148) return 256;
  if (ceil_div(N, 128) * tm >= 148) return 128;
  if (!glu && ceil_div(N, 64) * tm >= 148) return 64;
  return 0;
}

template <bool CONV> int dispatch_persistent(int bn, const Tc5Args& a, cudaStream_t st, const Tc5Conv* g) {
  if (a.dtype == B200_BF16) {
    if (bn == 256) return launch_persistent<__nv_bfloat16, 256, CONV>(a, st, g);
    if (bn == 128) return launch_persistent<__nv_bfloat16, 128, CONV>(a, st, g);
    return launch_persistent<__nv_bfloat16, 64, CONV>(a, st, g);
  }
  if (bn == 256) return launch_persistent<__half, 256, CONV>(a, st, g);
  if (bn == 128) return launch_persistent<__half, 128, CONV>(a, st, g);
  return launch_persistent<__half, 64, CONV>(a, st, g);
}

}  // namespace

bool tc5_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* e = getenv("B200NN_DISABLE_TC5");
    state = (e && e[0] == '1') ? 0 : 1;
  }
  return state == 1;
}

int64_t linear_tc5_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int64_t need = 0;
  for (int glu = 0; glu < 2; ++glu) {  // the caller does not say which epilogue it will ask for
    if (glu && N % 128) continue;
    const Tc5Plan pl = plan_tc5(M, N, K, glu != 0);
    if (pl.splits <= 1) continue;
    const int64_t b = M * pl.ws_pitch * 4 + pl.tiles_n * pl.tiles_m * 4 + 256;
    need = b > need ? b : need;
  }
  return need;
}

int linear_tc5(const Tc5Args& a, cudaStream_t st) {
  if (!tc5_enabled()) return B200_ENOTSUP;
  if (a.dtype != B200_BF16 && a.dtype != B200_F16) return B200_ENOTSUP;
  if (a.K % 8 || a.lda % 8 || a.ldw % 8 || !aligned16(a.A) || !aligned16(a.W)) return B200_ENOTSUP;
  if (a.M >= (1ll << 31) || a.N >= (1ll << 31) || a.K >= (1ll << 31)) return B200_ENOTSUP;
  const bool glu = (a.epilogue & B200_EPI_GLU) != 0;
  if (glu && (a.N % 128 || (a.epilogue & ~(B200_EPI_GLU | B200_EPI_W_STATIC)) || a.residual)) return B200_ENOTSUP;
  if (const int bn = persistent_bn(a.M, a.N, glu)) return dispatch_persistent<false>(bn, a, st, nullptr);
  const Tc5Plan pl = plan_tc5(a.M, a.N, a.K, glu);
  if (pl.tiles_m > 65535 || pl.splits > 65535) return B200_ENOTSUP;
  if (pl.tiles_m == 1 && a.M <= 64 && decode_deep()) {
    if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false, 3>(a, pl, st) : launch<__nv_bfloat16, 128, false, 3>(a, pl, st);
    return pl.bn == 64 ? launch<__half, 64, false, 3>(a, pl, st) : launch<__half, 128, false, 3>(a, pl, st);
  }
  if (pl.tiles_m == 1 && a.M <= 64) {
    if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false, 2>(a, pl, st) : launch<__nv_bfloat16, 128, false, 2>(a, pl, st);
    return pl.bn == 64 ? launch<__half, 64, false, 2>(a, pl, st) : launch<__half, 128, false, 2>(a, pl, st);
  }
  if (pl.tiles_m == 1) {
    if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false, 1>(a, pl, st) : launch<__nv_bfloat16, 128, false, 1>(a, pl, st);
    return pl.bn == 64 ? launch<__half, 64, false, 1>(a, pl, st) : launch<__half, 128, false, 1>(a, pl, st);
  }
  if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false>(a, pl, st) : launch<__nv_bfloat16, 128, false>(a, pl, st);
  return pl.bn == 64 ? launch<__half, 64, false>(a, pl, st) : launch<__half, 128, false>(a, pl, st);
}

int conv_tc5(const Tc5Args& a, const Tc5Conv& g, cudaStream_t st) {
  if (!tc5_enabled()) return B200_ENOTSUP;
  if (a.dtype != B200_BF16 && a.dtype != B200_F16) return B200_ENOTSUP;
  if (g.C % BK || a.K != static_cast<int64_t>(g.KH) * g.KW * g.C || a.ldw % 8 || !aligned16(a.A) || !aligned16(a.W)) return B200_ENOTSUP;
  if (a.M >= (1ll << 31) || a.N >= (1ll << 31) || (a.epilogue & ~(B200_EPI_RELU | B200_EPI_W_STATIC))) return B200_ENOTSUP;
  if (const int bn = persistent_bn(a.M, a.N, false)) return dispatch_persistent<true>(bn, a, st, &g);
  Tc5Plan pl;
  pl.bn = a.N >= 128 ? 128 : 64;
  pl.tiles_n = ceil_div(a.N, pl.bn);
  pl.tiles_m = ceil_div(a.M, BM);
  pl.splits = 1;
  pl.kb_per_split = static_cast<int>(a.K / BK);
  pl.ws_pitch = pl.tiles_n * pl.bn;
  if (pl.tiles_m > 65535) return B200_ENOTSUP;
  if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, true, 0>(a, pl, st, &g) : launch<__nv_bfloat16, 128, true, 0>(a, pl, st, &g);
  return pl.bn == 64 ? launch<__half, 64, true, 0>(a, pl, st, &g) : launch<__half, 128, true, 0>(a, pl, st, &g);
}

}  // namespace b200

extern "C" int b200_debug_device_error(int* code, int clear) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, b200::g_tc5_error, sizeof(int));
  if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "b200_debug_device_error: %s", cudaGetErrorString(e));
  if (code) *code = v;
  if (clear && v) {
    v = 0;
    cudaMemcpyToSymbol(b200::g_tc5_error, &v, sizeof(int));
  }
  return B200_OK;
}
