// tcgen05 GEMM and implicit-GEMM convolution:  out[M,N] = epi(A[M,K] * W[N,K]^T + bias + residual).
//
// Two kernels share the building blocks: gemm_tc5_kernel computes one 128 x BN tile per CTA
// (decode weight streaming with split-K inside a thread-block cluster, small and mid-size
// shapes); gemm_tc5p_kernel is persistent (one CTA per SM walks the tile list, accumulator
// double-buffered in tensor memory, optional bulk-copy epilogue).  In both, per tile:  Warp 0 streams 128x64 (A) and BNx64 (W) tiles
// through a ring of shared-memory stages with TMA (128-byte swizzle, no multicast);
// warp 1 issues tcgen05.mma (M=128, N=BN, K=16) from shared-memory descriptors into a
// tensor-memory accumulator and releases stages with tcgen05.commit; warps 2-5 read the
// accumulator back with tcgen05.ld (each warp owns the 32 TMEM lanes of its quarter),
// apply the epilogue in fp32 and store.  Every barrier wait is bounded: on a timeout the
// CTA records an error code in `g_tc5_error`, drains its own copies and exits.
#include "attention.cuh"
#include "gemm_tc5.cuh"
#include "mma.cuh"
#include "tc5.cuh"

#include <stdlib.h>

namespace b200 {

__device__ int g_tc5_error = 0;

namespace {

constexpr int BM = 128, BK = 64;
constexpr int NORM_MAX_PARTS = 32;   // row scaling: at most this many sum-of-squares partials per row
// Kernel modes.
//   0  compute-bound shapes (several row tiles): two CTAs per SM with a short ring, so that
//      one CTA's epilogue overlaps the other's main loop;
//   1  a single row tile with 64 < M <= 128: pure weight streaming, one CTA per SM, deep ring;
//   2  M <= 64 (decode): the activation tile is loaded 64 rows high (the MMA still reads 128
//      rows; the upper half is whatever follows in shared memory and only feeds accumulator
//      rows that are never stored), which halves the stage size; one CTA per SM with a ring of
//      7 (128-wide tiles) or 12 (64-wide) stages - weight streaming is bound by the bytes a
//      CTA keeps in flight (two CTAs per SM with rings half as deep measured 4 % slower).
template <int BN, int MODE> struct Cfg {
  static constexpr int AROWS = MODE >= 2 ? 64 : 128;
  static constexpr int A_STAGE = AROWS * BK * 2;
  // k-blocks per ring stage: the linear shapes with staged epilogues pair them (one barrier hand-off per two
  // k-blocks of MMAs; decode step 2.83 -> 2.76 ms, projections of a 512-token prompt 11.2 -> 10.7 us)
  static constexpr int KPS = MODE >= 1 ? 2 : 1;
  static constexpr int ST = MODE == 0 ? (BN == 128 ? 3 : 4) : MODE == 1 ? (BN == 128 ? 2 : 3) : (BN == 128 ? 3 : 6);
  static constexpr int CTAS = MODE == 0 ? 2 : 1;
  static constexpr int ISSUE_GROUP = ST >= 12 ? 4 : ST >= 6 ? 3 : ST >= 4 ? 2 : 1;   // ring stages a producer thread fills per barrier wait
  static constexpr int RING = ST * KPS * (A_STAGE + BN * BK * 2);
  // split-K only: fp32 receive buffer for the partial-tile rows this CTA owns, one slot per
  // cluster rank, behind the ring (peers write into it while this CTA may still be computing)
  static constexpr int RECV_ROWS = (MODE >= 2 ? 64 : 128) + 8;
  static constexpr int RECV = RECV_ROWS * (BN + 4) * 4;
};

// Decode (M <= 64) plan, settled by measurement on the Qwen2.5-1.5B shapes (a layer's four GEMMs, B = 1..64):
// split-K aims for one CTA per SM, keeps the partial sums below half the weight bytes and at least two
// k-blocks per CTA; the deep single-CTA ring (mode 3) gained 4 % and is used.
constexpr int SPLIT_TARGET_CTAS = 148, SPLIT_TRAFFIC_DIV = 2, SPLIT_MIN_KB = 2;

struct Tc5Params {
  const void* bias; const void* residual; const void* aux; void* out;
  int64_t M, N, K, ldo, ldr, ldaux;
  int bias_dtype, epilogue, splits, kb_per_split;
  const void* x;   // convolution input (implicit-GEMM mode only)
  Tc5Conv g;
  // persistent kernel: shared-memory plan chosen by the host (bytes from the aligned base)
  int pst, pstage;      // ring stages and bytes per stage
  int wr, w_off;        // weights resident: all k-blocks of the CTA's weight tile stay in shared memory at w_off
  int pncb, c_off;      // C buffers (bulk-copy epilogue) and where they start
  int npa;              // persistent kernel: activation producer threads (1 or 2), ring stages dealt round-robin
  int kps;              // persistent kernel: k-blocks per ring stage (1 or 2): one barrier hand-off covers that many
  int nfast;            // persistent kernel: column tiles fastest in the tile order
  // one-tile kernel, M <= 64: scale the output rows by the RMSNorm factor of the input rows / write
  // sum-of-squares partials of the output rows
  const float* sumsq_in; float* sumsq_out;
  float norm_eps;
  int sumsq_in_cols;
  // CTA-pair kernel with split-K (p.splits > 1): fp32 partial sums [split][M][N] instead of outputs
  float* partial;
  // one-tile kernel, M <= 64, 128-wide tiles: rotary embedding + q / KV-cache destinations in the final pass
  Tc5Args::Rope rope;
};

template <typename T> struct AbFormat;
template <> struct AbFormat<__half> { static constexpr int value = 0; };
template <> struct AbFormat<__nv_bfloat16> { static constexpr int value = 1; };


// The epilogue code runs once or a few times per CTA, so it is written as short rolled loops
// over 16-column units: straight-line code unrolled over a whole tile row costs more in
// instruction fetch (cold instruction cache on every SM) than in execution.

// v[i] += bias[n + i]
template <int CNT>
__device__ __forceinline__ void add_bias(const Tc5Params& p, float (&v)[CNT], int64_t n, int cnt) {
  if (!p.bias) return;
  if (p.bias_dtype == B200_F32) {
    const float* __restrict__ bp = static_cast<const float*>(p.bias) + n;
#pragma unroll
    for (int i = 0; i < CNT; ++i) if (i < cnt) v[i] += bp[i];
  } else if (p.bias_dtype == B200_BF16) {
    const __nv_bfloat16* __restrict__ bp = static_cast<const __nv_bfloat16*>(p.bias) + n;
#pragma unroll
    for (int i = 0; i < CNT; ++i) if (i < cnt) v[i] += __bfloat162float(bp[i]);
  } else if (p.bias_dtype == B200_F16) {
    const __half* __restrict__ bp = static_cast<const __half*>(p.bias) + n;
#pragma unroll
    for (int i = 0; i < CNT; ++i) if (i < cnt) v[i] += __half2float(bp[i]);
  } else {
#pragma unroll
    for (int i = 0; i < CNT; ++i) if (i < cnt) v[i] += load_as_f32(p.bias, n + i, p.bias_dtype);   // (static indices keep v in registers)
  }
}

// CNT (8 or 16) consecutive values of row `row` of a [*, ld] matrix of T starting at column n
template <typename T, int CNT>
__device__ __forceinline__ void load_cols(const T* __restrict__ base, int64_t ld, int64_t row, int64_t n, int cnt, float (&f)[CNT]) {
  const T* src = base + row * ld + n;
  if (cnt == CNT && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
    for (int j = 0; j < CNT / 8; ++j) {
      float t[8];
      unpack8<T>(reinterpret_cast<const uint4*>(src)[j], t);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[8 * j + i] = t[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < CNT; ++i) f[i] = i < cnt ? to_f32<T>(src[i]) : 0.f;
  }
}

template <typename T, int CNT>
__device__ __forceinline__ void store_cols(T* __restrict__ dst, const float (&v)[CNT], int cnt) {
  if (cnt == CNT && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
    for (int j = 0; j < CNT / 8; ++j) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = v[8 * j + i];
      reinterpret_cast<uint4*>(dst)[j] = pack8<T>(f);
    }
  } else {
#pragma unroll
    for (int i = 0; i < CNT; ++i) if (i < cnt) dst[i] = from_f32<T>(v[i]);
  }
}

// bias / residual / activation on CNT consecutive outputs of row m starting at column n, then store
template <typename T, int CNT>
__device__ __forceinline__ void finish_cols(const Tc5Params& p, float (&v)[CNT], int64_t m, int64_t n) {
  const int cnt = static_cast<int>(p.N - n < CNT ? p.N - n : CNT);
  add_bias<CNT>(p, v, n, cnt);
  if (p.residual) {
    float r[CNT];
    load_cols<T, CNT>(static_cast<const T*>(p.residual), p.ldr, m, n, cnt, r);
#pragma unroll
    for (int i = 0; i < CNT; i += 2) {
      round2<T>(v[i], v[i + 1]);
      v[i] += r[i]; v[i + 1] += r[i + 1];
    }
  }
  if (p.epilogue & B200_EPI_RELU) {
#pragma unroll
    for (int i = 0; i < CNT; ++i) v[i] = fmaxf(v[i], 0.f);
  }
  if (p.epilogue & B200_EPI_SILU_MUL) {
    float x[CNT];
    load_cols<T, CNT>(static_cast<const T*>(p.aux), p.ldaux, m, n, cnt, x);
#pragma unroll
    for (int i = 0; i < CNT; ++i) v[i] = round_as<T>(silu_f32(round_as<T>(v[i]))) * x[i];
  }
  store_cols<T, CNT>(static_cast<T*>(p.out) + m * p.ldo + n, v, cnt);
}

// finish_cols with the residual already in registers (16 values as two 16-byte words); no silu_mul term
template <typename T>
__device__ __forceinline__ void finish_cols_res(const Tc5Params& p, float (&v)[16], int64_t m, int64_t n, const uint4& r0, const uint4& r1) {
  const int cnt = static_cast<int>(p.N - n < 16 ? p.N - n : 16);
  add_bias<16>(p, v, n, cnt);
  float r[16], t[8];
  unpack8<T>(r0, t);
#pragma unroll
  for (int i = 0; i < 8; ++i) r[i] = t[i];
  unpack8<T>(r1, t);
#pragma unroll
  for (int i = 0; i < 8; ++i) r[8 + i] = t[i];
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    round2<T>(v[i], v[i + 1]);
    v[i] += r[i]; v[i + 1] += r[i + 1];
  }
  if (p.epilogue & B200_EPI_RELU) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
  }
  store_cols<T, 16>(static_cast<T*>(p.out) + m * p.ldo + n, v, cnt);
}

// gated-MLP epilogue: CNT gate accumulators (merged columns n_merged..) and the matching up
// accumulators (merged columns n_merged + 64 ..) of row m -> CNT outputs starting at column n_out
template <typename T, int CNT>
__device__ __forceinline__ void finish_glu_cols(const Tc5Params& p, float (&g)[CNT], float (&u)[CNT], int64_t m, int64_t n_merged, int64_t n_out) {
  add_bias<CNT>(p, g, n_merged, CNT);
  add_bias<CNT>(p, u, n_merged + 64, CNT);
#pragma unroll
  for (int i = 0; i < CNT; i += 2) {   // pairs: the three roundings to T go through packed conversions
    float g0 = g[i], g1 = g[i + 1], u0 = u[i], u1 = u[i + 1];
    round2<T>(g0, g1);
    g0 = silu_f32(g0); g1 = silu_f32(g1);
    round2<T>(g0, g1);
    round2<T>(u0, u1);
    g[i] = g0 * u0; g[i + 1] = g1 * u1;
  }
  store_cols<T, CNT>(static_cast<T*>(p.out) + m * p.ldo + n_out, g, CNT);
}

// Final pass of the merged q/k/v projection of a decode step: `lo` / `hi` are columns col..col+3 and
// col+64..col+67 of head `head` (a 128-wide tile) for sequence b.  Adds the bias, rounds to T as the linear
// layer's output is rounded, applies x*cos + rotate_half(x)*sin with the roundings of the unfused
// operators (both products, then the sum) to query and key heads, and stores to rope(q) / the cache rows.
template <typename T>
__device__ __forceinline__ void finish_rope4(const Tc5Params& p, const float4& lo4, const float4& hi4, int64_t b, int head, int col) {
  float lo[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hi[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
  const int64_t n = static_cast<int64_t>(head) * 128 + col;
  add_bias<4>(p, lo, n, 4);
  add_bias<4>(p, hi, n + 64, 4);
#pragma unroll
  for (int i = 0; i < 4; ++i) { lo[i] = round_as<T>(lo[i]); hi[i] = round_as<T>(hi[i]); }
  const Tc5Args::Rope& r = p.rope;
  const int which = head < r.Hq ? 0 : (head < r.Hq + r.Hkv ? 1 : 2);
  if (which != 2) {
    const T* cs = static_cast<const T*>(r.cos) + b * 128 + col;
    const T* sn = static_cast<const T*>(r.sin) + b * 128 + col;
    float c0, c1, c2, c3, s0, s1, s2, s3, d0, d1, d2, d3, t0, t1, t2, t3;
    const uint2 cl = *reinterpret_cast<const uint2*>(cs), ch = *reinterpret_cast<const uint2*>(cs + 64);
    const uint2 sl = *reinterpret_cast<const uint2*>(sn), sh = *reinterpret_cast<const uint2*>(sn + 64);
    unpack2<T>(cl.x, c0, c1); unpack2<T>(cl.y, c2, c3); unpack2<T>(sl.x, s0, s1); unpack2<T>(sl.y, s2, s3);
    unpack2<T>(ch.x, d0, d1); unpack2<T>(ch.y, d2, d3); unpack2<T>(sh.x, t0, t1); unpack2<T>(sh.y, t2, t3);
    const float cl4[4] = {c0, c1, c2, c3}, sl4[4] = {s0, s1, s2, s3}, ch4[4] = {d0, d1, d2, d3}, sh4[4] = {t0, t1, t2, t3};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = lo[i], h = hi[i];
      lo[i] = round_as<T>(a * cl4[i]) + round_as<T>(-h * sl4[i]);
      hi[i] = round_as<T>(h * ch4[i]) + round_as<T>(a * sh4[i]);
    }
  }
  T* dst;
  if (which == 0) {
    dst = static_cast<T*>(r.q_out) + (b * r.Hq + head) * 128;
  } else {
    int64_t pos = load_index(r.cache_pos, 0, r.pos_dtype);
    if (pos < 0) pos += r.cache_len;
    if (pos < 0 || pos >= r.cache_len) return;
    const int hk = head - r.Hq - (which == 2 ? r.Hkv : 0);
    dst = static_cast<T*>(which == 1 ? r.k_cache : r.v_cache) + ((b * r.Hkv + hk) * r.cache_len + pos) * 128;
  }
  *reinterpret_cast<uint2*>(dst + col) = make_uint2(pack2<T>(lo[0], lo[1]), pack2<T>(lo[2], lo[3]));
  *reinterpret_cast<uint2*>(dst + col + 64) = make_uint2(pack2<T>(hi[0], hi[1]), pack2<T>(hi[2], hi[3]));
}

// four consecutive outputs of row m starting at column n (split-K final pass)
template <typename T>
__device__ __forceinline__ void finish4(const Tc5Params& p, const float4& acc, int64_t m, int64_t n) {
  float v[4] = {acc.x, acc.y, acc.z, acc.w};
  const int cnt = static_cast<int>(p.N - n < 4 ? p.N - n : 4);
  add_bias<4>(p, v, n, cnt);
  const T* __restrict__ res = static_cast<const T*>(p.residual);
  const T* __restrict__ aux = static_cast<const T*>(p.aux);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < cnt) {
      if (res) v[i] = round_as<T>(v[i]) + to_f32<T>(res[m * p.ldr + n + i]);
      if (p.epilogue & B200_EPI_RELU) v[i] = fmaxf(v[i], 0.f);
      if (p.epilogue & B200_EPI_SILU_MUL) v[i] = round_as<T>(silu_f32(round_as<T>(v[i]))) * to_f32<T>(aux[m * p.ldaux + n + i]);
    }
  }
  T* o = static_cast<T*>(p.out) + m * p.ldo + n;
  if (cnt == 4 && (reinterpret_cast<uintptr_t>(o) & 7u) == 0) {
    *reinterpret_cast<uint2*>(o) = make_uint2(pack2<T>(v[0], v[1]), pack2<T>(v[2], v[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) if (i < cnt) o[i] = from_f32<T>(v[i]);
  }
}

// four gate accumulators and the matching up accumulators of row m (split-K final pass)
template <typename T>
__device__ __forceinline__ void finish_glu4(const Tc5Params& p, const float4& gate, const float4& up, int64_t m, int64_t n_merged, int64_t n_out) {
  float g[4] = {gate.x, gate.y, gate.z, gate.w}, u[4] = {up.x, up.y, up.z, up.w};
  add_bias<4>(p, g, n_merged, 4);
  add_bias<4>(p, u, n_merged + 64, 4);
#pragma unroll
  for (int i = 0; i < 4; i += 2) {
    float g0 = g[i], g1 = g[i + 1], u0 = u[i], u1 = u[i + 1];
    round2<T>(g0, g1);
    g0 = silu_f32(g0); g1 = silu_f32(g1);
    round2<T>(g0, g1);
    round2<T>(u0, u1);
    g[i] = g0 * u0; g[i + 1] = g1 * u1;
  }
  T* o = static_cast<T*>(p.out) + m * p.ldo + n_out;
  if ((reinterpret_cast<uintptr_t>(o) & 7u) == 0) {
    *reinterpret_cast<uint2*>(o) = make_uint2(pack2<T>(g[0], g[1]), pack2<T>(g[2], g[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = from_f32<T>(g[i]);
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
__global__ void __launch_bounds__(224, Cfg<BN, MODE>::CTAS) gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_w, const Tc5Params p) {
  constexpr int ST = Cfg<BN, MODE>::ST, A_STAGE = Cfg<BN, MODE>::A_STAGE, ISSUE_GROUP = Cfg<BN, MODE>::ISSUE_GROUP, KPS = Cfg<BN, MODE>::KPS;
  constexpr int B_STAGE = BN * BK * 2, STAGE = KPS * (A_STAGE + B_STAGE);   // a stage: KPS activation tiles, then KPS weight tiles
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ __align__(8) uint64_t full_bar[ST], empty_bar[ST], acc_bar;
  __shared__ uint32_t tmem_holder;
  __shared__ int failed;
  // Row scaling (decode shapes): the RMSNorm in front of this layer is applied after the GEMM - the
  // caller has folded the gain into W's columns and each output row m is multiplied by
  // r_m = 1 / sqrt(sum(x_m^2) / K + eps) before the bias, since (r x) W^T = r (x W^T).
  constexpr bool CAN_NORM = !CONV && MODE >= 2;
  __shared__ float s_rinv[CAN_NORM ? 64 : 1];
  const bool norm = CAN_NORM && p.sumsq_in != nullptr;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int KB = static_cast<int>((p.K + BK - 1) / BK);
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int nkb = min(KB, kb0 + p.kb_per_split) - kb0;   // >= 1 by construction of the grid
  const int nstg = (nkb + KPS - 1) / KPS;                // ring stages this CTA fills
  auto stage_cnt = [&](int i) { return nkb - i * KPS < KPS ? nkb - i * KPS : KPS; };   // k-blocks of stage i
  // single-row-tile shapes and split-K stage the accumulator through shared memory (see the end of the kernel)
  const bool gather = CONV && !p.g.im2col;   // convolution A tile copied by the epilogue warps instead of TMA
  const bool staged = !CONV && (MODE >= 1 || p.splits > 1);   // MODE >= 1: known at compile time, the direct epilogue is dropped
  const bool glu = (p.epilogue & B200_EPI_GLU) != 0;       // host guarantees BN == 128 and N % 128 == 0
  const bool rope = CAN_NORM && BN == 128 && p.rope.cos != nullptr;   // tile = one attention head (host: BN == 128, N % 128 == 0)
  const int rows_valid = static_cast<int>(p.M - m0 < BM ? p.M - m0 : BM);
  constexpr int PART_PITCH = BN + 4;                      // floats; rows 16 bytes apart in bank space
  // fp32 staging tile: the ring itself without split-K (it is free once the last MMA has completed);
  // with split-K the receive buffer behind the ring.  Rows are handed out to the cluster ranks in
  // blocks of `rpo`; slot s of a CTA's buffer holds rank s's partial sums for the rows it owns.
  const int nsp = p.splits;
  float* part = reinterpret_cast<float*>(nsp > 1 ? smem + Cfg<BN, MODE>::RING : smem);
  const int rpo = (rows_valid + nsp - 1) / nsp;
  const int rank = nsp > 1 ? static_cast<int>(tc5::cluster_ctarank()) : 0;

  if (threadIdx.x == 0) {
    failed = 0;
    // a stage is full when both producers' copies have landed (or the 128 gather threads have arrived)
    for (int s = 0; s < ST; ++s) { tc5::mbar_init(&full_bar[s], gather ? 129 : 2); tc5::mbar_init(&empty_bar[s], 1); }
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

  // Two producer threads - thread 0 of warp 0 the activation tiles, thread 0 of warp 6 the weight
  // tiles.  A barrier wait that follows a TMA instruction costs the thread ~0.3 us whatever it waits
  // for (measured: one wait-then-copy per iteration issues 3 boxes per us, copies alone 30), so a
  // producer waits once per ISSUE_GROUP stages and then issues that many copies back to back.
  // Weights that no kernel of this stream writes are fetched before the predecessor has finished:
  // the weight producer simply runs ahead until the ring is full.
  const bool w_static = (p.epilogue & B200_EPI_W_STATIC) != 0;
  const int pre = w_static ? (nstg < ST ? nstg : ST) : 0;   // weight stages issued before the cluster start-up barrier
  const uint32_t ring_addr = tc5::smem_addr(smem), full0 = tc5::smem_addr(&full_bar[0]), empty0 = tc5::smem_addr(&empty_bar[0]);
  auto load_w_stage = [&](int i, int st) {   // the weight tiles of stage i into ring slot st
    const int cnt = stage_cnt(i);
    tc5::mbar_arrive_expect_tx_a(full0 + 8u * st, cnt * B_STAGE);
#pragma unroll
    for (int j = 0; j < KPS; ++j)
      if (j < cnt) tc5::tma_load_2d_a(ring_addr + st * STAGE + KPS * A_STAGE + j * B_STAGE, &map_w, full0 + 8u * st, (kb0 + i * KPS + j) * BK, n0);
  };
  if (warp == 6 && lane == 0) {
    for (int i = 0; i < pre; ++i) load_w_stage(i, i);
  }
  // Every CTA of the cluster must be running before any of them writes into a peer's shared memory, which
  // happens in the epilogue only: arrive here, wait there (by then the peers have long arrived; a full
  // barrier at this point was ~1 us on the critical path of every split-K GEMM).
  if (nsp > 1) { __syncwarp(); tc5::cluster_arrive(); }

  // Both producers: the first pass over the ring finds every stage free and waits for nothing; after
  // that a group of stages is waited for (the first wait is the long one, the rest answer at once) and
  // filled back to back.  `load(i, s)` issues k-block i into stage s.
  auto produce = [&](int from, auto&& load) {
    const int first = nstg < ST ? nstg : ST;
    for (int i = from; i < first; ++i) load(i, i);
    int i = first, st = 0;
    uint32_t par = 0;   // stage ST reuses slot 0 once the first phase of its barrier has completed
    while (i < nstg) {
      const int g = nstg - i < ISSUE_GROUP ? nstg - i : ISSUE_GROUP;
      int ss = st;
      uint32_t pp = par;
      for (int j = 0; j < g; ++j) {
        if (!tc5::mbar_wait_a(empty0 + 8u * ss, pp)) { failed = 1; atomicExch(&g_tc5_error, 1); return i; }
        if (++ss == ST) { ss = 0; pp ^= 1u; }
      }
      if (*reinterpret_cast<volatile int*>(&failed)) return i;
      for (int j = 0; j < g; ++j, ++i) {
        load(i, st);
        if (++st == ST) { st = 0; par ^= 1u; }
      }
    }
    return i;
  };
  auto drain = [&](int issued) {   // after a failure: wait (bounded) for this thread's own copies still in flight
    if (*reinterpret_cast<volatile int*>(&failed))
      for (int i = issued > ST ? issued - ST : 0; i < issued; ++i) tc5::mbar_wait(&full_bar[i % ST], (i / ST) & 1, 1u << 16);
  };

  if (warp == 6) {
    if (lane == 0) {   // ---- weight producer ----
      if (!w_static) pdl_wait();   // the weights may come from the kernel before this one
      drain(produce(pre, load_w_stage));
    }
  } else if (warp == 0) {
    if (lane == 0 && !gather) {   // ---- activation producer (the gather variant fills the A tile with the epilogue warps) ----
      pdl_wait();
      if (!CONV) {
        drain(produce(0, [&](int i, int st) {
          const int cnt = stage_cnt(i);
          tc5::mbar_arrive_expect_tx_a(full0 + 8u * st, cnt * A_STAGE);
#pragma unroll
          for (int j = 0; j < KPS; ++j)
            if (j < cnt) tc5::tma_load_2d_a(ring_addr + st * STAGE + j * A_STAGE, &map_a, full0 + 8u * st, (kb0 + i * KPS + j) * BK, m0);
        }));
      } else {
        // implicit GEMM: k-block = 64 channels of one filter tap; tap row / column / channel block are stepped
        const int cpb = p.g.C / BK;
        const int img = m0 / (p.g.Ho * p.g.Wo), rem = m0 - img * (p.g.Ho * p.g.Wo), oh = rem / p.g.Wo, ow = rem - oh * p.g.Wo;
        const int base_w = ow * p.g.sw - p.g.pw, base_h = oh * p.g.sh - p.g.ph;
        int cb = 0, sx = 0, r = 0;
        drain(produce(0, [&](int, int st) {
          tc5::mbar_arrive_expect_tx_a(full0 + 8u * st, A_STAGE);
          tc5::tma_load_im2col_4d_a(ring_addr + st * STAGE, &map_a, full0 + 8u * st, cb * BK, base_w, base_h, img, sx, r);
          if (++cb == cpb) { cb = 0; if (++sx == p.g.KW) { sx = 0; ++r; } }
        }));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::umma_idesc(BM, BN, AbFormat<T>::value);
      // this thread's scalar instructions set the pace of a decode GEMM (8 KB of weights per k-block): barrier
      // addresses and descriptor words are stepped by single additions; a stage that no later k-block
      // reuses is not handed back (a commit costs the thread ~50 cycles)
      const uint32_t ring_lo = tc5::desc_sw128_lo(ring_addr);
      uint32_t a_lo = ring_lo, ph = 0;
      int s = 0;
      for (int i = 0; i < nstg; ++i) {
        if (!tc5::mbar_wait_a(full0 + 8u * s, ph)) { failed = 1; atomicExch(&g_tc5_error, 2); break; }
        const int cnt = stage_cnt(i);
#pragma unroll
        for (int j = 0; j < KPS; ++j)
          if (j < cnt) tc5::umma_f16_kblock(tmem_base, a_lo + j * (A_STAGE >> 4), a_lo + ((KPS * A_STAGE + j * B_STAGE) >> 4), idesc, i * KPS + j);
        if (i + ST < nstg) tc5::umma_commit_a(empty0 + 8u * s);
        a_lo += STAGE >> 4;
        if (++s == ST) { s = 0; ph ^= 1u; a_lo = ring_lo; }
      }
      tc5::umma_commit(&acc_bar);
    }
  } else {
    pdl_wait();   // residual, bias, split-K scratch and convolution inputs come from earlier kernels
    const int q = warp & 3;  // warps 2,3,4,5 -> TMEM lane quarters 2,3,0,1
    if (gather) {
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
    if (CAN_NORM && norm) {
      // r of the rows of this tile, from the sum-of-squares partials the producer of x left behind: all
      // partials of a row are requested at once, then added in index order.  Needed in the final pass only.
      const int row = static_cast<int>(threadIdx.x) - 64;
      if (row < 64) {
        float rinv = 0.f;
        if (row < rows_valid) {
          const float* sp = p.sumsq_in + static_cast<int64_t>(m0 + row) * p.sumsq_in_cols;
          float part[NORM_MAX_PARTS];
#pragma unroll
          for (int j = 0; j < NORM_MAX_PARTS; ++j) part[j] = j < p.sumsq_in_cols ? __ldcg(sp + j) : 0.f;
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < NORM_MAX_PARTS; ++j) ss += part[j];
          rinv = 1.0f / sqrtf(ss / static_cast<float>(p.K) + p.norm_eps);
        }
        s_rinv[row] = rinv;
      }
    }
    bool ok = true;
    if (lane == 0) ok = tc5::mbar_wait(&acc_bar, 0);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok && lane == 0) { failed = 1; atomicExch(&g_tc5_error, 3); }
    ok = ok && !*reinterpret_cast<volatile int*>(&failed);
    ok = __all_sync(0xffffffffu, ok);
    const int64_t m = m0 + q * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (nsp > 1) { __syncwarp(); tc5::cluster_wait(); }   // (every epilogue warp, whatever `ok`: pairs with the arrive at start-up)
    if (ok && staged) {
      // ---- accumulator row -> fp32 staging buffer of the CTA that owns the row ----
      tc5::tc_fence_after();
      if (q * 32 < rows_valid) {   // warp-uniform: this lane quarter holds rows that exist
        const int r = q * 32 + lane;
        const bool row_ok = r < rows_valid;
        const int owner = row_ok ? r / rpo : 0, lr = r - owner * rpo;
        uint32_t dst = tc5::smem_addr(part + (rank * rpo + lr) * PART_PITCH);
        if (nsp > 1) dst = tc5::map_to_rank(dst, owner);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          __syncwarp();
          tc5::tmem_ld_32x16(t_row + c, v);
          tc5::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 4; ++j) tc5::st_cluster_f4(dst + (c + 4 * j) * 4, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          }
        }
      }
      tc5::tc_fence_before();
    } else if (ok && glu) {
      tc5::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 64; c += 16) {   // gate columns c..c+15 pair with up columns 64+c..
        float vg[16], vu[16];
        __syncwarp();
        tc5::tmem_ld_32x16(t_row + c, vg);
        tc5::tmem_ld_32x16(t_row + 64 + c, vu);
        tc5::tmem_ld_wait();
        if (m < p.M) finish_glu_cols<T, 16>(p, vg, vu, m, n0 + c, n0 / 2 + c);
      }
      tc5::tc_fence_before();
    } else if (ok) {
      tc5::tc_fence_after();
      float va[16], vb[16];   // two 16-column units in flight: the next tcgen05.ld runs under the current unit's stores
      tc5::tmem_ld_32x16(t_row, va);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        tc5::tmem_ld_wait();
        tc5::tmem_ld_32x16(t_row + c + 16, vb);
        if (m < p.M && n0 + c < p.N) finish_cols<T, 16>(p, va, m, n0 + c);
        __syncwarp();   // tcgen05.ld is warp-collective; lanes that skipped the stores rejoin here
        tc5::tmem_ld_wait();
        if (c + 32 < BN) tc5::tmem_ld_32x16(t_row + c + 32, va);
        if (m < p.M && n0 + c + 16 < p.N) finish_cols<T, 16>(p, vb, m, n0 + c + 16);
        __syncwarp();
      }
      tc5::tc_fence_before();
    }
  }

  // ---- staged epilogue.  The split-K CTAs of one output tile form a thread-block cluster along
  // z.  Every accumulator row has been written, as fp32, into the staging buffer of the CTA that
  // owns the row (remote shared-memory stores for the other ranks' rows); after ONE cluster
  // barrier each CTA sums the slots of its rows in rank order (deterministic) from its own shared
  // memory and finishes those outputs with coalesced stores.  No global scratch, no atomics;
  // after the barrier nobody touches a peer's memory, so CTAs may exit independently.
  if (staged) {
    // All 224 threads walk the owned rows as float4 units in row-major order.  The loop body is
    // kept short: it runs a handful of times per thread, so its cost is instruction count.
    constexpr int LOG_UNITS = BN == 64 ? 4 : 5;              // float4 units per tile row (staged tiles are 64 or 128 wide)
    const bool paired = glu || rope;
    const int log_pr = paired ? 4 : LOG_UNITS;               // gated / rotary: the 16 units of columns 0..63, each paired with +64
    const int my_rows = max(0, min(rpo, rows_valid - rank * rpo));
    const int total = my_rows << log_pr;
    const int slot = rpo * PART_PITCH;                       // floats between the slots of two ranks
    T* const outp = static_cast<T*>(p.out);
    const T* const resp = static_cast<const T*>(p.residual);
    const bool relu = (p.epilogue & B200_EPI_RELU) != 0;
    const int bias_kind = !p.bias ? 0 : p.bias_dtype == B200_F32 ? 1 : p.bias_dtype == AbFormat<T>::value + 1 ? 2 : 3;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(outp) & 7u) == 0 && (p.ldo & 3) == 0 && bias_kind < 3 &&
                        (!resp || ((reinterpret_cast<uintptr_t>(resp) & 7u) == 0 && (p.ldr & 3) == 0)) && !(p.epilogue & B200_EPI_SILU_MUL);
    // A thread meets the same four columns in every iteration (224 is a multiple of the units per row), so
    // their bias - a constant of the stream - is fetched once, before the barrier that the thread waits at anyway.
    const int my_col = (static_cast<int>(threadIdx.x) & ((1 << log_pr) - 1)) << 2;
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!paired && vec_ok && static_cast<int64_t>(n0) + my_col + 4 <= p.N) {
      if (bias_kind == 1) {
        const float* bp = static_cast<const float*>(p.bias) + n0 + my_col;
        bias4 = make_float4(__ldg(bp), __ldg(bp + 1), __ldg(bp + 2), __ldg(bp + 3));
      } else if (bias_kind == 2) {
        const T* bp = static_cast<const T*>(p.bias) + n0 + my_col;
        bias4 = make_float4(to_f32<T>(bp[0]), to_f32<T>(bp[1]), to_f32<T>(bp[2]), to_f32<T>(bp[3]));
      }
    }
    __syncwarp();
    if (nsp > 1) {
      if (warp < 2 || warp > 5) tc5::cluster_wait();   // the producer and MMA warps complete the start-up barrier here
      tc5::cluster_sync();
    } else {
      __syncthreads();
    }
    if (!*reinterpret_cast<volatile int*>(&failed)) {
      // the residual of a unit is requested one iteration ahead of its use
      const bool res_ahead = resp && vec_ok && !paired;
      auto residual_of = [&](int idx) {
        const int lr = idx >> log_pr;
        const int64_t n = static_cast<int64_t>(n0) + my_col;
        if (idx >= total || n + 4 > p.N) return make_uint2(0u, 0u);
        return *reinterpret_cast<const uint2*>(resp + (static_cast<int64_t>(m0) + rank * rpo + lr) * p.ldr + n);
      };
      uint2 res_next = res_ahead ? residual_of(static_cast<int>(threadIdx.x)) : make_uint2(0u, 0u);
      // The plain case (bias / residual / ReLU on whole float4 units, no row scale, no sum of squares) as a loop of
      // its own: every decision is made outside, the pointers step by a constant number of rows, two units in flight.
      const bool plain = !paired && vec_ok && static_cast<int64_t>(n0) + my_col + 4 <= p.N && !p.sumsq_out && !(CAN_NORM && norm);
      if (plain) {
        constexpr int ROWS_PER_STEP = 224 >> LOG_UNITS;   // 224 threads cover this many whole rows per iteration
        const int lr0 = static_cast<int>(threadIdx.x) >> LOG_UNITS;
        const float* src0 = part + lr0 * PART_PITCH + my_col;
        const int64_t row0 = static_cast<int64_t>(m0) + rank * rpo + lr0;
        T* o = outp + row0 * p.ldo + n0 + my_col;
        const T* r = resp ? resp + row0 * p.ldr + n0 + my_col : nullptr;
        const int64_t o_step = static_cast<int64_t>(ROWS_PER_STEP) * p.ldo, r_step = static_cast<int64_t>(ROWS_PER_STEP) * p.ldr;
        const int iters = lr0 < my_rows ? (my_rows - lr0 + ROWS_PER_STEP - 1) / ROWS_PER_STEP : 0;
        uint2 rn = (r && iters > 0) ? *reinterpret_cast<const uint2*>(r) : make_uint2(0u, 0u);
#pragma unroll 2
        for (int it = 0; it < iters; ++it) {
          const uint2 rc = rn;
          if (r && it + 1 < iters) rn = *reinterpret_cast<const uint2*>(r + r_step);
          const float* sp = src0;
          float4 acc = *reinterpret_cast<const float4*>(sp);
          for (int sl = 1; sl < nsp; ++sl) {
            sp += slot;
            const float4 t = *reinterpret_cast<const float4*>(sp);
            acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
          }
          acc.x += bias4.x; acc.y += bias4.y; acc.z += bias4.z; acc.w += bias4.w;
          if (r) {
            float r0, r1, r2, r3;
            unpack2<T>(rc.x, r0, r1);
            unpack2<T>(rc.y, r2, r3);
            acc.x = round_as<T>(acc.x) + r0; acc.y = round_as<T>(acc.y) + r1; acc.z = round_as<T>(acc.z) + r2; acc.w = round_as<T>(acc.w) + r3;
            r += r_step;
          }
          if (relu) { acc.x = fmaxf(acc.x, 0.f); acc.y = fmaxf(acc.y, 0.f); acc.z = fmaxf(acc.z, 0.f); acc.w = fmaxf(acc.w, 0.f); }
          *reinterpret_cast<uint2*>(o) = make_uint2(pack2<T>(acc.x, acc.y), pack2<T>(acc.z, acc.w));
          o += o_step;
          src0 += ROWS_PER_STEP * PART_PITCH;
        }
      }
#pragma unroll 1
      for (int idx = plain ? total : static_cast<int>(threadIdx.x); idx < total; idx += 224) {
        const uint2 res_cur = res_next;
        if (res_ahead) res_next = residual_of(idx + 224);
        const int lr = idx >> log_pr, col = my_col;
        const float* src = part + lr * PART_PITCH + col;
        float4 acc = *reinterpret_cast<const float4*>(src), up = make_float4(0.f, 0.f, 0.f, 0.f);
        if (paired) up = *reinterpret_cast<const float4*>(src + 64);
#pragma unroll 1
        for (int s = 1; s < nsp; ++s) {
          src += slot;
          const float4 t = *reinterpret_cast<const float4*>(src);
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
          if (paired) {
            const float4 u = *reinterpret_cast<const float4*>(src + 64);
            up.x += u.x; up.y += u.y; up.z += u.z; up.w += u.w;
          }
        }
        const int64_t mm = static_cast<int64_t>(m0) + rank * rpo + lr;
        const int64_t n = static_cast<int64_t>(n0) + col;
        if (CAN_NORM && norm) {
          const float rs = s_rinv[rank * rpo + lr];
          acc.x *= rs; acc.y *= rs; acc.z *= rs; acc.w *= rs;
          up.x *= rs; up.y *= rs; up.z *= rs; up.w *= rs;
        }
        if (glu) {
          finish_glu4<T>(p, acc, up, mm, n, n0 / 2 + col);
        } else if (rope) {
          finish_rope4<T>(p, acc, up, mm, n0 >> 7, col);
        } else if (vec_ok && n + 4 <= p.N) {
          acc.x += bias4.x; acc.y += bias4.y; acc.z += bias4.z; acc.w += bias4.w;
          if (resp) {
            const uint2 raw = res_cur;
            float r0, r1, r2, r3;
            unpack2<T>(raw.x, r0, r1);
            unpack2<T>(raw.y, r2, r3);
            acc.x = round_as<T>(acc.x) + r0; acc.y = round_as<T>(acc.y) + r1; acc.z = round_as<T>(acc.z) + r2; acc.w = round_as<T>(acc.w) + r3;
          }
          if (relu) { acc.x = fmaxf(acc.x, 0.f); acc.y = fmaxf(acc.y, 0.f); acc.z = fmaxf(acc.z, 0.f); acc.w = fmaxf(acc.w, 0.f); }
          *reinterpret_cast<uint2*>(outp + mm * p.ldo + n) = make_uint2(pack2<T>(acc.x, acc.y), pack2<T>(acc.z, acc.w));
          if (p.sumsq_out) {
            // Sum of squares of the rounded outputs over this row's block of 64 columns: the 16 lanes
            // of a half warp hold exactly that block (4 columns each; N % 64 == 0 by contract).
            round2<T>(acc.x, acc.y);
            round2<T>(acc.z, acc.w);
            float sq = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
            const unsigned am = __activemask();
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) sq += __shfl_xor_sync(am, sq, off);
            if ((lane & 15) == 0) p.sumsq_out[mm * (p.N >> 6) + (n >> 6)] = sq;
          }
        } else if (n < p.N) {
          finish4<T>(p, acc, mm, n);
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
//
// TS = true adds the bulk-copy epilogue for 16-bit outputs: the residual tile of tile i is
// fetched by TMA into a shared-memory C buffer while tile i is still being multiplied; the
// epilogue warps combine accumulator, bias and residual in that buffer (128-byte-swizzled
// 64-column sub-tiles, conflict-free 16-byte accesses); a dedicated thread (warp 6) writes the
// buffer out with TMA stores.  Residual reads and output writes are then large asynchronous
// copies - what a memory-bound layer (1x1 convolution, K = 64..256) needs to keep enough
// bytes in flight - instead of one dependent 32-byte access per thread and 16 columns.
template <int BN, bool TS> struct PCfg {
  static constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2, STAGE = A_STAGE + B_STAGE;
  static constexpr int ST = TS ? (BN == 256 ? 3 : (BN == 128 ? 5 : 8)) : (BN == 256 ? 4 : (BN == 128 ? 6 : 8));   // ring + C buffers fill the 227 KB
  static constexpr int CB = BM * BN * 2;               // one C buffer: BN/64 sub-tiles of [128 rows][128 bytes]
  static constexpr int NCB = TS ? (BN == 256 ? 1 : 2) : 0;
  static constexpr int SMEM = ST * STAGE + NCB * CB + 1024;
  // Weights resident (short reductions whose whole weight tile fits): the ring holds activation
  // tiles only, the rest goes to the weight tile and up to MAX_NCB C buffers.
  static constexpr int MAX_ST = 12, MAX_NCB = 4;
  static constexpr int SMEM_LIMIT = 227 * 1024 - 1024;   // dynamic part; the barriers are static shared memory
  // warps: 0 activation producer, 1 MMA, 2-5 epilogue; TS adds 6 store, 7-10 second epilogue group
  // (half the columns each); the gather variant adds 6-9 gather; then the weight producer and,
  // last, the second activation producer
  static constexpr int W_WARP = TS ? 11 : 6;
  static constexpr int A2_WARP = TS ? 12 : 7;           // second activation producer
  static constexpr int THREADS = (A2_WARP + 1) * 32;
  static constexpr int W_WARP_GATHER = 10;
  static constexpr int EPI_WARPS = TS ? 8 : 4;
};

// Position in the shared-memory ring (stage index and phase bit), stepped without a division:
// the persistent kernel's ring depth is a run-time value.
struct RingPos {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next(int stages) { if (++s == stages) { s = 0; ph ^= 1u; } }
};

template <typename T, int BN, bool CONV, bool TS, int KPS>
__global__ void __launch_bounds__(PCfg<BN, TS>::THREADS, 1)
    gemm_tc5p_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                     const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_o, const Tc5Params p,
                     const int tiles_m, const int n_tiles) {
  constexpr int A_STAGE = PCfg<BN, TS>::A_STAGE, B_STAGE = PCfg<BN, TS>::B_STAGE, CB = PCfg<BN, TS>::CB;
  constexpr int MAX_ST = PCfg<BN, TS>::MAX_ST, MAX_NCB = PCfg<BN, TS>::MAX_NCB;
  const int ST = p.pst, STAGE = p.pstage, NCB = p.pncb;
  const bool WR = p.wr != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* cbuf = smem + p.c_off;
  uint8_t* wres = smem + p.w_off;
  __shared__ __align__(8) uint64_t full_bar[MAX_ST], empty_bar[MAX_ST], acc_full[2], acc_empty[2];
  // C buffers: c_full = residual tile landed, c_ready = epilogue result written, c_free = store has read it
  __shared__ __align__(8) uint64_t c_full[MAX_NCB], c_ready[MAX_NCB], c_free[MAX_NCB];
  // resident weights: w_full = the weight tile has landed, w_empty = every MMA that reads it has completed
  __shared__ __align__(8) uint64_t w_full, w_empty;
  __shared__ uint32_t tmem_holder;
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = static_cast<int>((p.K + BK - 1) / BK);
  // Tile index -> row tile / column tile.  Rows fastest by default (the CTAs running together share
  // weight tiles); columns fastest (p.nfast) for short reductions over large activations: the column
  // tiles of one row tile then run together and share the activation tile in L2, and with a grid that
  // is a multiple of the column-tile count every CTA keeps one column tile - its resident weights - for good.
  const int tiles_n = static_cast<int>((p.N + BN - 1) / BN);
  auto tile_m = [&](int tile) { return p.nfast ? tile / tiles_n : tile % tiles_m; };
  auto tile_n = [&](int tile) { return p.nfast ? tile % tiles_n : tile / tiles_m; };

  if (threadIdx.x == 0) {
    failed = 0;
    // a stage is full when both producers' copies have landed (or the 128 gather threads have arrived)
    for (int s = 0; s < ST; ++s) { tc5::mbar_init(&full_bar[s], (CONV && !p.g.im2col) ? 129 : (WR ? 1 : 2)); tc5::mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { tc5::mbar_init(&acc_full[b], 1); tc5::mbar_init(&acc_empty[b], PCfg<BN, TS>::EPI_WARPS); }
    for (int b = 0; b < MAX_NCB; ++b) { tc5::mbar_init(&c_full[b], 1); tc5::mbar_init(&c_ready[b], PCfg<BN, TS>::EPI_WARPS); tc5::mbar_init(&c_free[b], 1); }
    tc5::mbar_init(&w_full, 1);
    tc5::mbar_init(&w_empty, 1);
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&map_a);
    tc5::prefetch_tensormap(&map_w);
    if (TS) { tc5::prefetch_tensormap(&map_o); if (p.residual) tc5::prefetch_tensormap(&map_r); }
  }
  if (warp == 1) { tc5::tmem_alloc(&tmem_holder, 2 * BN); tc5::tmem_relinquish(); }
  tc5::tc_fence_before();
  __syncthreads();
  tc5::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_trigger();
  auto dead = [&]() { return *reinterpret_cast<volatile int*>(&failed) != 0; };

  const bool gather_variant = CONV && !TS && !p.g.im2col;   // launched with 352 threads
  const int a_id = warp == 0 ? 0 : warp == PCfg<BN, TS>::A2_WARP ? 1 : -1;   // producer number among the activation producers (-1: not one)
  if (a_id >= 0 && a_id < p.npa) {
    // ---- activation producers: with two, the k-blocks alternate between them (a 3x3 convolution is bound
    // by how fast one thread gets its im2col boxes through; more than two measured no better) ----
    if (lane == 0) {
      pdl_wait();
      const int mine = a_id, deal = p.npa - 1;
      constexpr int kps = KPS;
      const bool c8 = CONV && p.g.c8, gathered = CONV && !p.g.im2col;
      const uint32_t ring_addr = tc5::smem_addr(smem), full0 = tc5::smem_addr(&full_bar[0]), empty0 = tc5::smem_addr(&empty_bar[0]);
      const int cpb = CONV ? (c8 ? 1 : p.g.C / BK) : 1;
      int it = 0, ti = 0, s = 0;
      uint32_t ph = 0, dst = ring_addr;
      bool alive = true;
      for (int tile = blockIdx.x; tile < n_tiles && alive && !dead(); tile += gridDim.x, ++ti) {
        const int m0 = tile_m(tile) * BM;
        int img = 0, base_w = 0, base_h = 0;   // convolution: first output pixel of the tile as a base position
        if (CONV) {
          img = m0 / (p.g.Ho * p.g.Wo);
          const int rem = m0 - img * (p.g.Ho * p.g.Wo), oh = rem / p.g.Wo;
          base_w = (rem - oh * p.g.Wo) * p.g.sw - p.g.pw;
          base_h = oh * p.g.sh - p.g.ph;
        }
        int cb = 0, sx = 0, r = 0;   // convolution: channel block within the filter tap, tap column, tap row - stepped, not divided
        for (int kb0 = 0; kb0 < KB; kb0 += kps, ++it) {
          const int cnt = KB - kb0 < kps ? KB - kb0 : kps;   // k-blocks of this stage
          const bool own = (it & deal) == mine;
          if (own && !tc5::mbar_wait_a(empty0 + 8u * s, ph ^ 1u)) { failed = 1; atomicExch(&g_tc5_error, 11); alive = false; break; }
          const uint32_t fb = full0 + 8u * s;
          if (own && !gathered) tc5::mbar_arrive_expect_tx_a(fb, cnt * A_STAGE);   // (gather variant: warps 6-9 fill the A tile)
#pragma unroll
          for (int j = 0; j < kps; ++j) {
            if (j >= cnt) break;
            const int kb = kb0 + j;
            if (own && !gathered) {
              const uint32_t dj = dst + j * A_STAGE;
              if (c8) {
                // 8-channel input: k-block = 8 filter taps, each a [128 pixels][16 B] box.  Taps past the
                // filter meet zero weights (outside the weight map), so their box only has to be finite: tap 0 again.
                for (int tt = 0; tt < 8; ++tt) {
                  const int tap = kb * 8 + tt, ta = tap < p.g.KH * p.g.KW ? tap : 0, rr = ta / p.g.KW;
                  tc5::tma_load_im2col_4d_a(dj + tt * (BM * 16), &map_a, fb, 0, base_w, base_h, img, ta - rr * p.g.KW, rr);
                }
              } else if (!CONV) {
                tc5::tma_load_2d_a(dj, &map_a, fb, kb * BK, m0);
              } else {
                tc5::tma_load_im2col_4d_a(dj, &map_a, fb, cb * BK, base_w, base_h, img, sx, r);
              }
            }
            if (CONV && ++cb == cpb) { cb = 0; if (++sx == p.g.KW) { sx = 0; ++r; } }
          }
          dst += STAGE;
          if (++s == ST) { s = 0; ph ^= 1u; dst = ring_addr; }
        }
      }
      if (dead()) {  // wait (bounded) for our own copies still in flight
        for (int i = it > ST ? it - ST : 0; i < it; ++i) tc5::mbar_wait(&full_bar[i % ST], (i / ST) & 1, 1u << 16);
      }
    }
  } else if (warp == (gather_variant ? PCfg<BN, TS>::W_WARP_GATHER : PCfg<BN, TS>::W_WARP)) {
    // ---- weight producer ----
    if (lane == 0) {
      if (!(p.epilogue & B200_EPI_W_STATIC)) pdl_wait();
      auto load_w = [&](uint8_t* dst, uint64_t* bar, int kb, int n0) {
        if (CONV && p.g.c8) {
          for (int tt = 0; tt < 8; ++tt) tc5::tma_load_2d(dst + tt * (BN * 16), &map_w, bar, (kb * 8 + tt) * 8, n0);
        } else {
          tc5::tma_load_2d(dst, &map_w, bar, kb * BK, n0);
        }
      };
      if (WR) {
        // Resident weights: every CTA would otherwise fetch the same few lines of a small weight
        // matrix from L2 for every tile, all at the same time (measured: those loads, not the
        // activations, set the pace of a 3x3 convolution over 64 channels).  The tile is loaded
        // once and again only when the CTA moves to another column tile.
        int cur_n0 = -1, loads = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !dead(); tile += gridDim.x) {
          const int n0 = tile_n(tile) * BN;
          if (n0 == cur_n0) continue;
          if (loads > 0 && !tc5::mbar_wait(&w_empty, (loads - 1) & 1)) { failed = 1; atomicExch(&g_tc5_error, 19); break; }
          tc5::mbar_arrive_expect_tx(&w_full, KB * B_STAGE);
          for (int kb = 0; kb < KB; ++kb) load_w(wres + kb * B_STAGE, &w_full, kb, n0);
          cur_n0 = n0;
          ++loads;
        }
        if (dead() && loads > 0) tc5::mbar_wait(&w_full, (loads - 1) & 1, 1u << 16);
      } else {
        const bool c8 = CONV && p.g.c8;
        constexpr int kps = KPS;
        const uint32_t ring_addr = tc5::smem_addr(smem) + kps * A_STAGE, full0 = tc5::smem_addr(&full_bar[0]), empty0 = tc5::smem_addr(&empty_bar[0]);
        int it = 0, s = 0;
        uint32_t ph = 0, dst = ring_addr;
        bool alive = true;
        for (int tile = blockIdx.x; tile < n_tiles && alive && !dead(); tile += gridDim.x) {
          const int n0 = tile_n(tile) * BN;
          for (int kb0 = 0; kb0 < KB; kb0 += kps, ++it) {
            const int cnt = KB - kb0 < kps ? KB - kb0 : kps;
            if (!tc5::mbar_wait_a(empty0 + 8u * s, ph ^ 1u)) { failed = 1; atomicExch(&g_tc5_error, 19); alive = false; break; }
            tc5::mbar_arrive_expect_tx_a(full0 + 8u * s, cnt * B_STAGE);
#pragma unroll
            for (int j = 0; j < kps; ++j) {
              if (j >= cnt) break;
              if (c8) load_w(smem + s * STAGE + A_STAGE, &full_bar[s], kb0 + j, n0);   // (c8: one k-block per stage)
              else tc5::tma_load_2d_a(dst + j * B_STAGE, &map_w, full0 + 8u * s, (kb0 + j) * BK, n0);
            }
            dst += STAGE;
            if (++s == ST) { s = 0; ph ^= 1u; dst = ring_addr; }
          }
        }
        if (dead()) {
          for (int i = it > ST ? it - ST : 0; i < it; ++i) tc5::mbar_wait(&full_bar[i % ST], (i / ST) & 1, 1u << 16);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::umma_idesc(BM, BN, AbFormat<T>::value);
      // Everything the loop needs per k-block is kept as a 32-bit value stepped by one addition: barrier
      // addresses, the operand descriptors' low words, the phase bit.
      const bool c8 = CONV && p.g.c8;
      const uint32_t ring_addr = tc5::smem_addr(smem), full0 = tc5::smem_addr(&full_bar[0]), empty0 = tc5::smem_addr(&empty_bar[0]);
      const uint32_t ring_lo = tc5::desc_sw128_lo(ring_addr), wres_lo = tc5::desc_sw128_lo(tc5::smem_addr(wres));
      const uint32_t stage_lo = static_cast<uint32_t>(STAGE) >> 4;
      constexpr int kps = KPS;
      int ti = 0, cur_n0 = -1, w_loads = 0, s = 0;
      uint32_t ph = 0, a_lo = ring_lo;
      bool alive = true;
      for (int tile = blockIdx.x; tile < n_tiles && alive && !dead(); tile += gridDim.x, ++ti) {
        const int b = ti & 1;
        const int n0 = tile_n(tile) * BN;
        if (WR && n0 != cur_n0) {   // the resident weight tile of this column tile
          if (!tc5::mbar_wait(&w_full, w_loads & 1)) { failed = 1; atomicExch(&g_tc5_error, 20); break; }
          cur_n0 = n0;
          ++w_loads;
        }
        if (!tc5::mbar_wait(&acc_empty[b], ((ti >> 1) & 1) ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 12); break; }
        tc5::tc_fence_after();
        const uint32_t acc = tmem_base + b * BN;
        uint32_t w_lo = wres_lo;
        for (int kb = 0; kb < KB; kb += kps) {
          const int cnt = KB - kb < kps ? KB - kb : kps;
          if (!tc5::mbar_wait_a(full0 + 8u * s, ph)) { failed = 1; atomicExch(&g_tc5_error, 13); alive = false; break; }
          if (c8) {   // unswizzled operands: one MMA covers two taps (2 x 16 bytes of K); one k-block per stage
            const uint32_t a_addr = ring_addr + s * STAGE, b_addr = WR ? tc5::smem_addr(wres + kb * B_STAGE) : a_addr + A_STAGE;
            const uint32_t ak = BM * 16u, am = 128u, bk = BN * 16u, bm = 128u;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc5::umma_f16(acc, tc5::umma_desc_nosw(a_addr + k * 2 * (BM * 16), ak, am), tc5::umma_desc_nosw(b_addr + k * 2 * (BN * 16), bk, bm), idesc,
                            (kb | k) != 0);
          } else {
#pragma unroll
            for (int j = 0; j < kps; ++j)
              if (j < cnt)
                tc5::umma_f16_kblock(acc, a_lo + j * (A_STAGE >> 4), WR ? w_lo + j * (B_STAGE >> 4) : a_lo + ((kps * A_STAGE + j * B_STAGE) >> 4), idesc, kb + j);
          }
          tc5::umma_commit_a(empty0 + 8u * s);
          w_lo += cnt * (B_STAGE >> 4);
          a_lo += stage_lo;
          if (++s == ST) { s = 0; ph ^= 1u; a_lo = ring_lo; }
        }
        if (!alive) break;
        tc5::umma_commit(&acc_full[b]);
        if (WR) {   // last tile of this column tile: the weight producer may overwrite the tile once these MMAs are done
          const int next = tile + static_cast<int>(gridDim.x);
          if (next < n_tiles && tile_n(next) * BN != n0) tc5::umma_commit(&w_empty);
        }
      }
    }
  } else if (warp < 6 || (TS && warp >= 7 && warp < 11)) {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    // bulk-copy epilogue: two warps per lane quarter, each takes half of the tile's columns
    const int c_begin = (TS && warp >= 7) ? BN / 2 : 0, c_end = (TS && warp < 6) ? BN / 2 : BN;
    pdl_wait();
    const bool glu = (p.epilogue & B200_EPI_GLU) != 0;
    int ti = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
      const int b = ti & 1;
      const int m0 = tile_m(tile) * BM, n0 = tile_n(tile) * BN;
      bool ok = true;
      if (lane == 0) ok = tc5::mbar_wait(&acc_full[b], (ti >> 1) & 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) { failed = 1; atomicExch(&g_tc5_error, 14); }
      ok = __all_sync(0xffffffffu, ok && !dead());
      if (!ok) break;
      tc5::tc_fence_after();
      const int64_t m = static_cast<int64_t>(m0) + q * 32 + lane;
      const uint32_t t_row = tmem_base + b * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (TS) {
        const int cb = ti % NCB, u = ti / NCB;
        bool okc = true;   // residual landed / buffer free
        if (lane == 0) okc = p.residual ? tc5::mbar_wait(&c_full[cb], u & 1) : tc5::mbar_wait(&c_free[cb], (u & 1) ^ 1);
        okc = __shfl_sync(0xffffffffu, okc ? 1 : 0, 0) != 0;
        if (!okc) { if (lane == 0) { failed = 1; atomicExch(&g_tc5_error, 17); } break; }
        const int r = q * 32 + lane, swz = r & 7;
        const uint32_t crow = tc5::smem_addr(cbuf + cb * CB) + r * 128;
        const bool relu = (p.epilogue & B200_EPI_RELU) != 0, has_res = p.residual != nullptr;
        // one 16-column unit: bias in fp32, then packed 16-bit pairs (one conversion per pair; the
        // residual add and the ReLU are exact in packed arithmetic) - conversions are quarter-rate
        const bool bias_f32_vec = p.bias && p.bias_dtype == B200_F32 && (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0 && (n0 & 3) == 0;
        auto unit = [&](float (&v)[16], int c) {
          const int64_t n = static_cast<int64_t>(n0) + c;
          if (bias_f32_vec && n + 16 <= p.N) {
            const float4* bp = reinterpret_cast<const float4*>(static_cast<const float*>(p.bias) + n);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 bv = __ldg(bp + i);
              v[4 * i] += bv.x; v[4 * i + 1] += bv.y; v[4 * i + 2] += bv.z; v[4 * i + 3] += bv.w;
            }
          } else {
            const int cnt = static_cast<int>(p.N - n < 16 ? (p.N - n < 0 ? 0 : p.N - n) : 16);
            add_bias<16>(p, v, n, cnt);
          }
          const int k = (c & 63) >> 3;
          const uint32_t a0 = crow + (c >> 6) * (BM * 128) + ((k ^ swz) << 4), a1 = crow + (c >> 6) * (BM * 128) + (((k + 1) ^ swz) << 4);
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = pack2<T>(v[2 * i], v[2 * i + 1]);
          if (has_res) {
            uint32_t r[8];
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a0));
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(a1));
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = add2<T>(o[i], r[i]);
          }
          if (relu) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = relu2<T>(o[i]);
          }
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a1), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
        };
        float va[16], vb[16];   // two units in flight: the next tcgen05.ld runs under the current unit's math
        __syncwarp();
        tc5::tmem_ld_32x16(t_row + c_begin, va);
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 32) {
          tc5::tmem_ld_wait();
          tc5::tmem_ld_32x16(t_row + c + 16, vb);
          unit(va, c);
          tc5::tmem_ld_wait();
          if (c + 32 < c_end) tc5::tmem_ld_32x16(t_row + c + 32, va);
          unit(vb, c + 16);
        }
        tc5::fence_proxy_async();   // the TMA store reads these generic-proxy writes
        __syncwarp();
        if (lane == 0) mbar_arrive(&c_ready[cb]);
      } else if (glu) {
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 16) {   // c counts gate columns: block h = c / 64 of 128 merged columns
          float vg[16], vu[16];
          const int col = (c >> 6) * 128 + (c & 63);
          __syncwarp();
          tc5::tmem_ld_32x16(t_row + col, vg);
          tc5::tmem_ld_32x16(t_row + col + 64, vu);
          tc5::tmem_ld_wait();
          const int64_t nm = static_cast<int64_t>(n0) + col;
          if (m < p.M && nm < p.N) finish_glu_cols<T, 16>(p, vg, vu, m, nm, (static_cast<int64_t>(n0) + (c >> 6) * 128) / 2 + (c & 63));
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          __syncwarp();
          tc5::tmem_ld_32x16(t_row + c, v);
          tc5::tmem_ld_wait();
          const int64_t n = static_cast<int64_t>(n0) + c;
          if (m < p.M && n < p.N) finish_cols<T, 16>(p, v, m, n);
        }
      }
      tc5::tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);   // this warp has drained its quarter of the accumulator
    }
  } else if (TS) {
    // ---- C-buffer store and residual prefetch (one thread of warp 6) ----
    // The thread that learns first that a buffer is free again (its store has been read out) is
    // the one that refills it with the residual tile of the tile that will use it next.
    if (warp == 6 && lane == 0) {
      pdl_wait();   // the output buffer may still be read by the kernel before this one
      const bool has_res = p.residual != nullptr;
      const int my_tiles = static_cast<int>(blockIdx.x) < n_tiles ? (n_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x) : 0;
      auto load_residual = [&](int ti) {
        const int tile = blockIdx.x + ti * gridDim.x, cb = ti % NCB;
        const int m0 = tile_m(tile) * BM, n0 = tile_n(tile) * BN;
        tc5::mbar_arrive_expect_tx(&c_full[cb], CB);
        for (int j = 0; j < BN / 64; ++j) tc5::tma_load_2d(cbuf + cb * CB + j * (BM * 128), &map_r, &c_full[cb], n0 + 64 * j, m0);
      };
      int res_issued = 0;
      if (has_res)
        for (; res_issued < NCB && res_issued < my_tiles; ++res_issued) load_residual(res_issued);
      int ti = 0;
      for (int tile = blockIdx.x; tile < n_tiles && !dead(); tile += gridDim.x, ++ti) {
        const int m0 = tile_m(tile) * BM, n0 = tile_n(tile) * BN;
        const int cb = ti % NCB, u = ti / NCB;
        if (!tc5::mbar_wait(&c_ready[cb], u & 1)) { failed = 1; atomicExch(&g_tc5_error, 18); break; }
        for (int j = 0; j < BN / 64; ++j)
          if (n0 + 64 * j < p.N) tc5::tma_store_2d(&map_o, cbuf + cb * CB + j * (BM * 128), n0 + 64 * j, m0);
        tc5::tma_store_commit();
        tc5::tma_store_wait_read();
        if (!has_res) mbar_arrive(&c_free[cb]);
        else if (res_issued < my_tiles) load_residual(res_issued++);   // == ti + NCB
      }
      if (dead())   // wait (bounded) for residual copies still in flight
        for (int i = res_issued > NCB ? res_issued - NCB : 0; i < res_issued; ++i) tc5::mbar_wait(&c_full[i % NCB], (i / NCB) & 1, 1u << 16);
      tc5::tma_store_wait_all();
    }
  } else if (CONV && !p.g.im2col) {
    // ---- A-operand gather (warps 6-9): thread r owns tile row r, i.e. one output pixel per tile ----
    constexpr int LAG = 2;
    const int row = (warp - 6) * 32 + lane;
    const int cpb = p.g.C / BK;
    const uint32_t row_off = row * 128, swz = row & 7;
    pdl_wait();
    int it = 0;          // k-blocks issued
    RingPos rp;
    int arrived = 0;     // k-blocks signalled
    bool alive = true;
    for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const int64_t mrow = static_cast<int64_t>(tile_m(tile)) * BM + row;
      const bool row_ok = mrow < p.M;
      const int64_t mm = row_ok ? mrow : 0;
      const int ow = static_cast<int>(mm % p.g.Wo), oh = static_cast<int>((mm / p.g.Wo) % p.g.Ho);
      const int64_t img = mm / (static_cast<int64_t>(p.g.Wo) * p.g.Ho);
      const int ih0 = oh * p.g.sh - p.g.ph, iw0 = ow * p.g.sw - p.g.pw;
      const T* xb = static_cast<const T*>(p.x) + img * p.g.H * p.g.W * p.g.C;
      for (int kb = 0; kb < KB && alive; ++kb, ++it, rp.next(ST)) {
        const int s = rp.s;
        if (!tc5::mbar_wait(&empty_bar[s], rp.ph ^ 1u) || dead()) { failed = 1; atomicExch(&g_tc5_error, 15); alive = false; break; }
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

// ---- CTA-pair kernel: 256 x 256 tiles on two SMs (cta_group::2) ------------------------------------
// A 128 x 256 tile per CTA needs 48 KB of operands per 4.2 MFLOP; at the rate the L2 feeds the SMs
// (measured ~11 TB/s over all SMs) that bounds the persistent kernel at ~1 PFLOP/s.  Here the two CTAs
// of a cluster share one 256 x 256 tile: each loads its own 128 rows of A and its own 128 of the 256 B
// rows (32 KB per k-block and CTA for the same 4.2 MFLOP), rank 0 issues M = 256 MMAs that read both
// CTAs' shared memory and write both CTAs' tensor memory.  Linear layers only; the epilogue is the plain
// one (accumulator rows -> registers -> global), overlapped with the next tile through the two accumulators.
// warps: 0 / 7 activation producers, 6 / 8 weight producers, 1 MMA (rank 0) and TMEM, 2-5 epilogue of columns
// 0..127, 9-12 epilogue of columns 128..255 (a tile that nothing follows - the last of a CTA, every split-K unit -
// is drained in half the time).
constexpr int PAIR_BN = 256, PAIR_ST = 6, PAIR_THREADS = 416;
constexpr int PAIR_A_STAGE = BM * BK * 2, PAIR_B_STAGE = (PAIR_BN / 2) * BK * 2, PAIR_STAGE = PAIR_A_STAGE + PAIR_B_STAGE;
constexpr int PAIR_SMEM = PAIR_ST * PAIR_STAGE + 1024;

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Tc5Params p, const int tiles_m,
                     const int n_tiles) {
  constexpr int ST = PAIR_ST, BN = PAIR_BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // full_bar / acc_empty are used in rank 0 only (its MMA thread waits on them); empty_bar / acc_full in both
  __shared__ __align__(8) uint64_t full_bar[ST], empty_bar[ST], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc5::cluster_ctarank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int KB = static_cast<int>((p.K + BK - 1) / BK);
  // Work units: (tile, split).  With split-K (few tiles, long reduction) a unit covers p.kb_per_split
  // k-blocks of its tile and leaves fp32 partial sums in p.partial; a second kernel adds them up.
  const int n_units = n_tiles * p.splits;
  auto unit_kb0 = [&](int unit) { return (unit / n_tiles) * p.kb_per_split; };
  auto unit_nkb = [&](int unit) { const int k0 = unit_kb0(unit); return (KB - k0 < p.kb_per_split ? KB - k0 : p.kb_per_split); };
  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < ST; ++s) { tc5::mbar_init(&full_bar[s], 2); tc5::mbar_init(&empty_bar[s], 1); }   // full: rank 0's two producers of the k-block
    for (int b = 0; b < 2; ++b) { tc5::mbar_init(&acc_full[b], 1); tc5::mbar_init(&acc_empty[b], 16); }    // empty: eight epilogue warps of each CTA
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&map_a);
    tc5::prefetch_tensormap(&map_w);
  }
  if (warp == 1) { tc5::tmem_alloc_pair(&tmem_holder, 2 * BN); tc5::tmem_relinquish_pair(); }
  tc5::tc_fence_before();
  __syncthreads();
  tc5::cluster_sync();   // the peer's barriers exist before anything arrives on them
  tc5::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_trigger();
  auto dead = [&]() { return *reinterpret_cast<volatile int*>(&failed) != 0; };
  const uint32_t ring_addr = tc5::smem_addr(smem), full0 = tc5::smem_addr(&full_bar[0]), empty0 = tc5::smem_addr(&empty_bar[0]);

  const int a_id = warp == 0 ? 0 : warp == 7 ? 1 : -1, b_id = warp == 6 ? 0 : warp == 8 ? 1 : -1;
  if (a_id >= 0 || b_id >= 0) {
    // ---- producers: k-blocks alternate between the two threads of an operand (2 <= ring depth) ----
    if (lane == 0) {
      const bool is_a = a_id >= 0;
      const int mine = is_a ? a_id : b_id;
      if (is_a || !(p.epilogue & B200_EPI_W_STATIC)) pdl_wait();
      const CUtensorMap* map = is_a ? &map_a : &map_w;
      const uint32_t lead_full0 = tc5::map_to_rank(full0, 0);
      int it = 0, s = 0;
      uint32_t ph = 0, dst = ring_addr + (is_a ? 0 : PAIR_A_STAGE);
      const uint32_t dst0 = dst;
      bool alive = true;
      for (int unit = pair; unit < n_units && alive && !dead(); unit += n_pairs) {
        const int tile = unit % n_tiles;
        const int row0 = (is_a ? (tile % tiles_m) : (tile / tiles_m)) * 256 + static_cast<int>(rank) * 128;   // this CTA's half
        const int kb0 = unit_kb0(unit), kb1 = kb0 + unit_nkb(unit);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if ((it & 1) == mine) {
            if (!tc5::mbar_wait_a(empty0 + 8u * s, ph ^ 1u)) { failed = 1; atomicExch(&g_tc5_error, 40); alive = false; break; }
            if (rank == 0) tc5::mbar_arrive_expect_tx_a(full0 + 8u * s, 2 * PAIR_A_STAGE);   // both CTAs' halves of this operand
            tc5::tma_load_2d_pair(dst, map, lead_full0 + 8u * s, kb * BK, row0);
          }
          dst += PAIR_STAGE;
          if (++s == ST) { s = 0; ph ^= 1u; dst = dst0; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer (rank 0 only) ----
      constexpr uint32_t idesc = tc5::umma_idesc(256, BN, AbFormat<T>::value);
      const uint32_t ring_lo = tc5::desc_sw128_lo(ring_addr);
      const uint32_t acc_full0 = tc5::smem_addr(&acc_full[0]), acc_empty0 = tc5::smem_addr(&acc_empty[0]);
      int ti = 0, s = 0;
      uint32_t ph = 0, a_lo = ring_lo;
      bool alive = true;
      for (int unit = pair; unit < n_units && alive && !dead(); unit += n_pairs, ++ti) {
        const int b = ti & 1;
        if (!tc5::mbar_wait_a(acc_empty0 + 8u * b, ((ti >> 1) & 1) ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 41); break; }
        tc5::tc_fence_after();
        const uint32_t acc = tmem_base + b * BN;
        const int nkb = unit_nkb(unit);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!tc5::mbar_wait_a(full0 + 8u * s, ph)) { failed = 1; atomicExch(&g_tc5_error, 42); alive = false; break; }
          tc5::umma_f16_kblock_pair(acc, a_lo, a_lo + (PAIR_A_STAGE >> 4), idesc, kb);
          tc5::umma_commit_pair(empty0 + 8u * s);   // frees the stage in both CTAs
          a_lo += PAIR_STAGE >> 4;
          if (++s == ST) { s = 0; ph ^= 1u; a_lo = ring_lo; }
        }
        if (!alive) break;
        tc5::umma_commit_pair(acc_full0 + 8u * b);
      }
    }
  } else {
    // ---- epilogue (warps 2-5 and 9-12): this CTA's 128 accumulator rows, columns c_lo .. c_lo + 127 ----
    const int q = warp & 3;
    const int c_lo = warp >= 9 ? BN / 2 : 0, c_hi = c_lo + BN / 2;
    pdl_wait();
    const bool glu = (p.epilogue & B200_EPI_GLU) != 0;
    const bool res_fast = p.splits == 1 && !glu && p.residual && !(p.epilogue & B200_EPI_SILU_MUL) && p.ldr % 8 == 0 && p.N % 8 == 0 &&
                          (reinterpret_cast<uintptr_t>(p.residual) & 15u) == 0;
    const uint32_t lead_acc_empty0 = tc5::map_to_rank(tc5::smem_addr(&acc_empty[0]), 0);
    int ti = 0;
    for (int unit = pair; unit < n_units; unit += n_pairs, ++ti) {
      const int b = ti & 1;
      const int tile = unit % n_tiles;
      const int64_t m = static_cast<int64_t>(tile % tiles_m) * 256 + rank * 128 + q * 32 + lane;
      const int64_t n0 = static_cast<int64_t>(tile / tiles_m) * BN;
      // Residual rows are read 32 columns (four 16-byte words) at a time, one step ahead of their use and the
      // first step before the accumulator is waited for: a load per step issued and consumed in place would
      // put an L2 round trip between any two steps of this thread's row.
      uint4 rc[4], rn[4];
      const T* rrow = res_fast && m < p.M ? static_cast<const T*>(p.residual) + m * p.ldr + n0 : nullptr;
      auto fetch = [&](int c, uint4 (&r)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          r[j] = (rrow && n0 + c + 8 * j < p.N) ? __ldg(reinterpret_cast<const uint4*>(rrow + c) + j) : make_uint4(0u, 0u, 0u, 0u);
      };
      if (res_fast) fetch(c_lo, rc);
      bool ok = true;
      if (lane == 0) ok = tc5::mbar_wait(&acc_full[b], (ti >> 1) & 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) { failed = 1; atomicExch(&g_tc5_error, 43); }
      ok = __all_sync(0xffffffffu, ok && !dead());
      if (!ok) break;
      tc5::tc_fence_after();
      const uint32_t t_row = tmem_base + b * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (res_fast) {
        float va[16], vb[16];
#pragma unroll 1
        for (int c = c_lo; c < c_hi; c += 32) {
          __syncwarp();
          tc5::tmem_ld_32x16(t_row + c, va);
          tc5::tmem_ld_32x16(t_row + c + 16, vb);
          if (c + 32 < c_hi) fetch(c + 32, rn);
          tc5::tmem_ld_wait();
          if (m < p.M && n0 + c < p.N) finish_cols_res<T>(p, va, m, n0 + c, rc[0], rc[1]);
          if (m < p.M && n0 + c + 16 < p.N) finish_cols_res<T>(p, vb, m, n0 + c + 16, rc[2], rc[3]);
#pragma unroll
          for (int j = 0; j < 4; ++j) rc[j] = rn[j];
        }
      } else if (p.splits > 1) {
        // raw partial sums of this unit's k-range (N % 8 == 0: 32-byte units stay inside the row); two 16-column
        // units in flight, 256-bit stores (a lane's store is one whole sector)
        float* dst = p.partial + (static_cast<int64_t>(unit / n_tiles) * p.M + m) * p.N + n0;
        float va[16], vb[16];
        __syncwarp();
        tc5::tmem_ld_32x16(t_row + c_lo, va);
#pragma unroll 1
        for (int c = c_lo; c < c_hi; c += 32) {
          tc5::tmem_ld_wait();
          tc5::tmem_ld_32x16(t_row + c + 16, vb);
          if (m < p.M) {
            if (n0 + c < p.N) tc5::st_global_f8(dst + c, va);
            if (n0 + c + 8 < p.N) tc5::st_global_f8(dst + c + 8, va + 8);
          }
          __syncwarp();
          tc5::tmem_ld_wait();
          if (c + 32 < c_hi) tc5::tmem_ld_32x16(t_row + c + 32, va);
          if (m < p.M) {
            if (n0 + c + 16 < p.N) tc5::st_global_f8(dst + c + 16, vb);
            if (n0 + c + 24 < p.N) tc5::st_global_f8(dst + c + 24, vb + 8);
          }
          __syncwarp();
        }
      } else if (glu) {
#pragma unroll 1
        for (int c = c_lo / 2; c < c_hi / 2; c += 16) {   // c counts gate columns: block c / 64 of 128 merged columns
          float vg[16], vu[16];
          const int col = (c >> 6) * 128 + (c & 63);
          __syncwarp();
          tc5::tmem_ld_32x16(t_row + col, vg);
          tc5::tmem_ld_32x16(t_row + col + 64, vu);
          tc5::tmem_ld_wait();
          const int64_t nm = n0 + col;
          if (m < p.M && nm < p.N) finish_glu_cols<T, 16>(p, vg, vu, m, nm, (n0 + (c >> 6) * 128) / 2 + (c & 63));
        }
      } else {
        float va[16], vb[16];   // two units in flight: the next tcgen05.ld runs under the current unit's math
        __syncwarp();
        tc5::tmem_ld_32x16(t_row + c_lo, va);
#pragma unroll 1
        for (int c = c_lo; c < c_hi; c += 32) {
          tc5::tmem_ld_wait();
          tc5::tmem_ld_32x16(t_row + c + 16, vb);
          if (m < p.M && n0 + c < p.N) finish_cols<T, 16>(p, va, m, n0 + c);
          tc5::tmem_ld_wait();
          if (c + 32 < c_hi) tc5::tmem_ld_32x16(t_row + c + 32, va);
          if (m < p.M && n0 + c + 16 < p.N) finish_cols<T, 16>(p, vb, m, n0 + c + 16);
        }
      }
      tc5::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive_cluster(lead_acc_empty0 + 8u * b);   // this warp has drained its quarter of the accumulator
    }
  }
  tc5::tc_fence_before();
  __syncthreads();
  tc5::cluster_sync();   // neither CTA leaves while the other may still signal its barriers or read its shared memory
  if (warp == 1) { tc5::tc_fence_after(); tc5::tmem_dealloc_pair(tmem_base, 2 * BN); }
}

// Second half of the pair kernel's split-K: out = epilogue(sum over splits of the fp32 partial sums), eight
// consecutive columns per thread.  The partial sums of all splits (at most PAIR_MAX_SPLITS) are requested before
// the first is used - one memory round trip per output instead of one per split, which is what this kernel's
// time consists of - and added in index order (the result does not depend on timing); they are zeroed behind
// the read, as every user of the shared split-K workspace leaves it.
constexpr int PAIR_MAX_SPLITS = 8;
template <typename T>
__global__ void __launch_bounds__(256) pair_splitk_reduce_kernel(const Tc5Params p) {
  pdl_trigger();
  pdl_wait();
  const int64_t per_row = p.N / 8, total = p.M * per_row, plane = p.M * p.N;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = i / per_row, n = (i - m * per_row) * 8;
    float* const q = p.partial + m * p.N + n;
    float a[PAIR_MAX_SPLITS][8];
#pragma unroll
    for (int s = 0; s < PAIR_MAX_SPLITS; ++s)
      if (s < p.splits) tc5::ld_global_cg_f8(q + s * plane, a[s]);
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < PAIR_MAX_SPLITS; ++s) {
      if (s < p.splits) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += a[s][i];
        tc5::st_global_f8(q + s * plane, zero);   // the workspace is shared with kernels that expect it zeroed
      }
    }
    finish_cols<T, 8>(p, v, m, n);
  }
}

// The same with the RMSNorm of the finished row as a tail: one block per output row (N / 8 threads, N <= 2048), so
// that the row's sum of squares can be formed inside the block.  norm_out[m, :] = rmsnorm(out[m, :]) * gain with the
// roundings of the stand-alone kernel: the sum runs over the outputs as stored (rounded to T), x * r is rounded to T
// before the gain when round_mid is set.
struct NormTailParams { const void* gain; void* out; int64_t ld; float eps; int round_mid; };

template <typename T>
__global__ void __launch_bounds__(256) pair_splitk_reduce_norm_kernel(const Tc5Params p, const NormTailParams nt) {
  __shared__ float warp_ss[8];
  pdl_trigger();
  pdl_wait();
  const int64_t m = blockIdx.x, plane = p.M * p.N;
  const int64_t n = static_cast<int64_t>(threadIdx.x) * 8;
  const bool act = n < p.N;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  uint4 graw = make_uint4(0u, 0u, 0u, 0u);
  float ss = 0.f;
  if (act) {
    float* const q = p.partial + m * p.N + n;
    float a[PAIR_MAX_SPLITS][8];
#pragma unroll
    for (int s = 0; s < PAIR_MAX_SPLITS; ++s)
      if (s < p.splits) tc5::ld_global_cg_f8(q + s * plane, a[s]);
    graw = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(nt.gain) + n));
    const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < PAIR_MAX_SPLITS; ++s) {
      if (s < p.splits) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += a[s][i];
        tc5::st_global_f8(q + s * plane, zero);
      }
    }
    finish_cols<T, 8>(p, v, m, n);
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = round_as<T>(v[i]); ss += v[i] * v[i]; }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) warp_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) tot += warp_ss[w];
  if (!act) return;
  const float r = 1.0f / sqrtf(tot / static_cast<float>(p.N) + nt.eps);
  float g[8];
  unpack8<T>(graw, g);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float x = v[i] * r;
    if (nt.round_mid) x = round_as<T>(x);
    v[i] = x * g[i];
  }
  *reinterpret_cast<uint4*>(static_cast<T*>(nt.out) + m * nt.ld + n) = pack8<T>(v);
}

// ---- 7x7 / stride-2 stem convolution on the 8-channel padded input ------------------------------
// The im2col route moves one 16-byte row per (pixel, tap): 7168 TMA rows per 128-pixel tile.  Here a
// persistent CTA walks consecutive output rows of an image and keeps the input rows it needs in a
// shared-memory window (16 row slots): stepping to the next output row loads only sh new input rows
// (7 KB instead of 114 KB of boxes).  Each input row is stored de-interleaved - odd pixels in one
// plane, even pixels in the other, 16 bytes per pixel - so that for a fixed filter tap the pixels of
// consecutive output columns (stride 2 in the input) are consecutive 16-byte entries of one plane:
// exactly the unswizzled K-major core-matrix layout (8 rows x 16 bytes contiguous), and the MMA reads
// the A operand straight from the window.  One MMA (K = 16) covers taps (r, 2k) and (r, 2k+1): the
// second tap sits in the other plane at a constant distance, which is the descriptor's K step.
// Tile = one output row (Wo <= 128 pixels; accumulator rows beyond Wo are computed and never stored).
struct StemParams {
  const void* x; const void* bias; int bias_dtype, relu;
  int batch, H, W, Ho, Wo, KH, sh, ph, N;
  int tiles, tiles_per_cta;
};
constexpr int STEM_BN = 64, STEM_SLOTS = 16, STEM_ENTRIES = 132, STEM_PLANE = STEM_ENTRIES * 16, STEM_SLOT = 2 * STEM_PLANE;
constexpr int STEM_W_STAGE = STEM_BN * 128;                  // one filter row: 8 taps x [64 rows][16 B]
constexpr int STEM_CB = BM * STEM_BN * 2, STEM_NT = 4;       // C buffer; tiles the row loaders may run ahead
constexpr int STEM_THREADS = 352;                            // warps: 0 weights, 1 MMA, 2-5 epilogue, 6 store, 7-10 row loaders

template <typename T>
__global__ void __launch_bounds__(STEM_THREADS, 1)
    conv_stem_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_o, const StemParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* wres = smem;                                   // KH filter rows of weights, resident
  uint8_t* cbuf = smem + 8 * STEM_W_STAGE;                // 2 C buffers
  uint8_t* window = cbuf + 2 * STEM_CB;                   // 16 row slots
  __shared__ __align__(8) uint64_t w_full, tile_full[STEM_NT], tile_done[STEM_NT], acc_full[2], acc_empty[2], c_ready[2], c_free[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int failed;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = blockIdx.x * p.tiles_per_cta;
  const int my_tiles = first >= p.tiles ? 0 : (p.tiles - first < p.tiles_per_cta ? p.tiles - first : p.tiles_per_cta);

  if (threadIdx.x == 0) {
    failed = 0;
    tc5::mbar_init(&w_full, 1);
    for (int s = 0; s < STEM_NT; ++s) { tc5::mbar_init(&tile_full[s], 128); tc5::mbar_init(&tile_done[s], 1); }
    for (int b = 0; b < 2; ++b) {
      tc5::mbar_init(&acc_full[b], 1); tc5::mbar_init(&acc_empty[b], 4);
      tc5::mbar_init(&c_ready[b], 4); tc5::mbar_init(&c_free[b], 1);
    }
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&map_w);
    tc5::prefetch_tensormap(&map_o);
  }
  // the window starts as zeros: the margins of every plane (pixels left and right of the image) stay zero
  for (int i = threadIdx.x; i < STEM_SLOTS * STEM_SLOT / 16; i += STEM_THREADS) reinterpret_cast<uint4*>(window)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 1) { tc5::tmem_alloc(&tmem_holder, 2 * STEM_BN); tc5::tmem_relinquish(); }
  tc5::fence_proxy_async();
  tc5::tc_fence_before();
  __syncthreads();
  tc5::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_trigger();
  auto dead = [&]() { return *reinterpret_cast<volatile int*>(&failed) != 0; };
  auto fail = [&](int code) { failed = 1; atomicExch(&g_tc5_error, code); };

  if (warp == 0) {
    // ---- weights: filter row r = 8 boxes of [64 channels][16 B]; the 8th tap lies outside the weight matrix (zeros) ----
    if (lane == 0 && my_tiles > 0) {
      tc5::mbar_arrive_expect_tx(&w_full, p.KH * STEM_W_STAGE);
      for (int r = 0; r < p.KH; ++r)
        for (int tt = 0; tt < 8; ++tt)
          tc5::tma_load_2d(wres + r * STEM_W_STAGE + tt * (STEM_BN * 16), &map_w, &w_full, tt < 7 ? (r * 7 + tt) * 8 : p.KH * 7 * 8 + 8, 0);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0 && my_tiles > 0) {
      constexpr uint32_t idesc = tc5::umma_idesc(BM, STEM_BN, AbFormat<T>::value);
      if (!tc5::mbar_wait(&w_full, 0)) fail(31);
      for (int ti = 0; ti < my_tiles && !dead(); ++ti) {
        const int b = ti & 1, st = ti % STEM_NT;
        const int tile = first + ti, oh = tile % p.Ho, ih_lo = oh * p.sh - p.ph;
        if (!tc5::mbar_wait(&acc_empty[b], ((ti >> 1) & 1) ^ 1)) { fail(32); break; }
        if (!tc5::mbar_wait(&tile_full[st], (ti / STEM_NT) & 1)) { fail(33); break; }
        tc5::tc_fence_after();
        const uint32_t acc = tmem_base + b * STEM_BN;
        for (int r = 0; r < p.KH; ++r) {
          const uint32_t a_row = tc5::smem_addr(window + ((ih_lo + r + STEM_SLOTS) & (STEM_SLOTS - 1)) * STEM_SLOT);
          const uint32_t b_row = tc5::smem_addr(wres + r * STEM_W_STAGE);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc5::umma_f16(acc, tc5::umma_desc_nosw(a_row + k * 16, STEM_PLANE + 16, 128),
                          tc5::umma_desc_nosw(b_row + k * 2 * (STEM_BN * 16), STEM_BN * 16, 128), idesc, (r | k) != 0);
        }
        tc5::umma_commit(&acc_full[b]);
        tc5::umma_commit(&tile_done[st]);
      }
    }
  } else if (warp < 6) {
    // ---- epilogue warps 2-5: TMEM -> bias (+ReLU) -> packed 16-bit -> swizzled C buffer ----
    const int q = warp & 3;
    const int r = q * 32 + lane, swz = r & 7;
    const bool relu = p.relu != 0;
    Tc5Params bp{};   // add_bias reads bias, dtype and N from the GEMM parameter block
    bp.bias = p.bias; bp.bias_dtype = p.bias_dtype; bp.N = p.N;
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int b = ti & 1;
      bool ok = true;
      if (lane == 0) ok = tc5::mbar_wait(&acc_full[b], (ti >> 1) & 1) && tc5::mbar_wait(&c_free[b], ((ti >> 1) & 1) ^ 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) fail(34);
      ok = __all_sync(0xffffffffu, ok && !dead());
      if (!ok) break;
      tc5::tc_fence_after();
      const uint32_t t_row = tmem_base + b * STEM_BN + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t crow = tc5::smem_addr(cbuf + b * STEM_CB) + r * 128;
#pragma unroll 1
      for (int c = 0; c < STEM_BN; c += 16) {
        float v[16];
        __syncwarp();
        tc5::tmem_ld_32x16(t_row + c, v);
        tc5::tmem_ld_wait();
        const int cnt = p.N - c < 16 ? (p.N - c < 0 ? 0 : p.N - c) : 16;
        add_bias<16>(bp, v, c, cnt);
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = pack2<T>(v[2 * i], v[2 * i + 1]);
        if (relu) {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = relu2<T>(o[i]);
        }
        const int k = c >> 3;
        const uint32_t a0 = crow + ((k ^ swz) << 4), a1 = crow + (((k + 1) ^ swz) << 4);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a0), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a1), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
      }
      tc5::fence_proxy_async();
      tc5::tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&c_ready[b]); mbar_arrive(&acc_empty[b]); }
    }
  } else if (warp == 6) {
    // ---- store thread: one bulk tensor store of [Wo pixels][64 channels] per tile ----
    if (lane == 0) {
      pdl_wait();   // the output buffer may still be read by the kernel before this one
      for (int ti = 0; ti < my_tiles && !dead(); ++ti) {
        const int b = ti & 1;
        if (!tc5::mbar_wait(&c_ready[b], (ti >> 1) & 1)) { fail(35); break; }
        tc5::tma_store_2d(&map_o, cbuf + b * STEM_CB, 0, (first + ti) * p.Wo);
        tc5::tma_store_commit();
        tc5::tma_store_wait_read();
        mbar_arrive(&c_free[b]);
      }
      tc5::tma_store_wait_all();
    }
  } else {
    // ---- row loaders (warps 7-10): de-interleave the new input rows of each tile into the window ----
    const int t = threadIdx.x - 7 * 32;   // 0..127
    pdl_wait();
    int have_n = -1, have_hi = 0;          // image whose rows the window holds, highest row loaded
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int tile = first + ti, n = tile / p.Ho, oh = tile - n * p.Ho;
      const int ih_lo = oh * p.sh - p.ph, ih_hi = ih_lo + p.KH - 1;
      const bool fresh = n != have_n;
      // slots about to be overwritten were last read by tile ti-4 at the latest (16 slots, KH + 4 sh <= 16);
      // a new image overwrites rows the previous tile may still be reading
      bool ok = true;
      if (fresh && ti >= 1) ok = tc5::mbar_wait(&tile_done[(ti - 1) % STEM_NT], ((ti - 1) / STEM_NT) & 1);
      else if (ti >= STEM_NT) ok = tc5::mbar_wait(&tile_done[ti % STEM_NT], ((ti / STEM_NT) & 1) ^ 1);
      if (!ok || dead()) { fail(36); break; }
      const int from = fresh ? ih_lo : (have_hi + 1 > ih_lo ? have_hi + 1 : ih_lo);
      for (int ih = from; ih <= ih_hi; ++ih) {
        uint8_t* slot = window + ((ih + STEM_SLOTS) & (STEM_SLOTS - 1)) * STEM_SLOT;
        const bool in = ih >= 0 && ih < p.H;
        const T* src = static_cast<const T*>(p.x) + (static_cast<int64_t>(n) * p.H + (in ? ih : 0)) * p.W * 8;
        for (int px = t; px < p.W; px += 128) {
          const uint32_t dst = tc5::smem_addr(slot + ((px & 1) ? 0 : STEM_PLANE) + (((px - (px & 1)) >> 1) + 2) * 16);
          cp_async16_zfill(dst, src + px * 8, in ? 16 : 0);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      tc5::fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's async-proxy reads
      mbar_arrive(&tile_full[ti % STEM_NT]);
      have_n = n;
      have_hi = ih_hi;
    }
  }
  __syncthreads();
  if (warp == 1) { tc5::tc_fence_after(); tc5::tmem_dealloc(tmem_base, 2 * STEM_BN); }
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

}  // namespace

// Tiled tensor map of up to five dimensions with a 128-byte swizzle (dims / box innermost first,
// strides in bytes for dimensions 1..rank-1).  Used by kernels outside this file.
bool tma_encode_sw128(CUtensorMap* map, int dtype, int rank, const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || rank < 1 || rank > 5) return false;
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
  const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*,
                                   const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeIm2colFn encode_im2col_fn() {
  static EncodeIm2colFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeIm2col", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeIm2colFn>(p);
  }
  return fn;
}

// NHWC activations [N, H, W, C] as an im2col-mode map: 64 channels x 128 output positions per
// load, 128-byte swizzle, zero fill outside the image.  The bounding box of base positions runs
// from -pad to (size - 1) + pad - (filter - 1) in each spatial dimension and is walked with the
// convolution stride, so consecutive positions are consecutive output pixels.
bool make_im2col_map(CUtensorMap* map, const void* x, const Tc5Conv& g, int dtype) {
  EncodeIm2colFn fn = encode_im2col_fn();
  if (!fn || g.batch <= 0) return false;
  if (g.ph > 127 || g.pw > 127 || g.KH > 128 || g.KW > 128 || g.sh > 8 || g.sw > 8) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.C), static_cast<cuuint64_t>(g.W), static_cast<cuuint64_t>(g.H), static_cast<cuuint64_t>(g.batch)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.C) * 2, static_cast<cuuint64_t>(g.W) * g.C * 2, static_cast<cuuint64_t>(g.H) * g.W * g.C * 2};
  const int lower[2] = {-g.pw, -g.ph};
  const int upper[2] = {g.pw - (g.KW - 1), g.ph - (g.KH - 1)};
  const cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(g.sw), static_cast<cuuint32_t>(g.sh), 1};
  const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 4, const_cast<void*>(x), dims, strides, lower, upper, BK, BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 8-channel variants: no swizzle, 16-byte inner box (one filter tap of 8 channels)
bool make_map_c8(CUtensorMap* map, const void* w, int64_t rows, int64_t K, int64_t ld, int box_rows, int dtype) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {8, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 2, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_im2col_map_c8(CUtensorMap* map, const void* x, const Tc5Conv& g, int dtype) {
  EncodeIm2colFn fn = encode_im2col_fn();
  if (!fn || g.batch <= 0 || g.C != 8) return false;
  if (g.ph > 127 || g.pw > 127 || g.KH > 128 || g.KW > 128 || g.sh > 8 || g.sw > 8) return false;
  const cuuint64_t dims[4] = {8, static_cast<cuuint64_t>(g.W), static_cast<cuuint64_t>(g.H), static_cast<cuuint64_t>(g.batch)};
  const cuuint64_t strides[3] = {16, static_cast<cuuint64_t>(g.W) * 16, static_cast<cuuint64_t>(g.H) * g.W * 16};
  const int lower[2] = {-g.pw, -g.ph};
  const int upper[2] = {g.pw - (g.KW - 1), g.ph - (g.KH - 1)};
  const cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(g.sw), static_cast<cuuint32_t>(g.sh), 1};
  const CUtensorMapDataType dt = dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 4, const_cast<void*>(x), dims, strides, lower, upper, 8, BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Tc5Plan { int bn, splits, kb_per_split; int64_t tiles_n, tiles_m; };

constexpr int MAX_SPLITS = 8;   // portable cluster size

Tc5Plan plan_for_bn(int bn, int64_t M, int64_t N, int64_t K) {
  Tc5Plan pl;
  const int64_t tm = ceil_div(M, BM);
  pl.bn = bn;
  pl.tiles_n = ceil_div(N, pl.bn);
  pl.tiles_m = tm;
  const int64_t tiles = pl.tiles_n * tm, KB = ceil_div(K, BK);
  int64_t splits = 1;
  if (tiles < 100) {
    // a split-K CTA carries ring + receive buffer, so one fits per SM: never more CTAs than SMs
    splits = SPLIT_TARGET_CTAS / tiles;
    const int64_t by_traffic = K / (SPLIT_TRAFFIC_DIV * (M < BM ? M : BM));   // partial sums stay below the weight bytes
    if (splits > by_traffic) splits = by_traffic;
    if (splits > KB / SPLIT_MIN_KB) splits = KB / SPLIT_MIN_KB;             // at least this many k-blocks per CTA
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;   // the splits of a tile form one thread-block cluster
    if (splits < 1) splits = 1;
  }
  pl.kb_per_split = static_cast<int>(ceil_div(KB, splits));
  pl.splits = static_cast<int>(ceil_div(KB, pl.kb_per_split));
  return pl;
}

Tc5Plan plan_tc5(int64_t M, int64_t N, int64_t K, bool glu = false) {
  const int64_t tm = ceil_div(M, BM);
  if (glu) return plan_for_bn(128, M, N, K);   // the gated epilogue pairs columns c and c+64 of a 128-wide tile
  if (ceil_div(N, 128) * tm >= 148) return plan_for_bn(128, M, N, K);   // enough 128-wide tiles for every SM
  if (tm >= 2) {
    // Too few wide tiles: either 64-wide tiles or wide tiles with split-K.  Take the wide ones when
    // split-K can still put (nearly) as many CTAs to work - they re-read the activations half as often.
    const Tc5Plan wide = plan_for_bn(128, M, N, K), narrow = plan_for_bn(64, M, N, K);
    const int64_t cw = wide.tiles_n * wide.tiles_m * wide.splits, cn = narrow.tiles_n * narrow.tiles_m * narrow.splits;
    return cw * 10 >= cn * 8 ? wide : narrow;
  }
  // decode (one row tile): 128-wide tiles - half as many k-block hand-offs per weight byte as 64-wide ones
  // (per layer of the 1.5B model: level at 64 rows, 39 -> 35 us at 8 rows), and a tile is one attention head
  return plan_for_bn(128, M, N, K);
}

template <typename T, int BN, bool CONV, int MODE = 0>
int launch(const Tc5Args& a, const Tc5Plan& plan, cudaStream_t st, const Tc5Conv* g = nullptr) {
  Tc5Plan pl = plan;
  constexpr int SMEM_RING = Cfg<BN, MODE>::RING + 1024, SMEM_SPLIT = SMEM_RING + Cfg<BN, MODE>::RECV;
  static_assert(SMEM_SPLIT <= 227 * 1024, "ring + receive buffer exceed the shared memory of an SM");
  struct DeviceState { bool configured; int fit[MAX_SPLITS + 1]; };
  static PerDevice<DeviceState> state_on;
  DeviceState* ds = state_on.slot();
  if (!ds) return B200_ENOTSUP;
  if (!ds->configured) {
    if (cudaFuncSetAttribute(gemm_tc5_kernel<T, BN, CONV, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_SPLIT) != cudaSuccess) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    ds->configured = true;
  }
  // The clusters of one launch should all be resident at once (a second wave would double the
  // time of these short kernels).  How many clusters of a given size fit depends on how the SMs
  // are grouped, so ask the runtime, once per cluster size, and shrink the split until they fit.
  if (pl.splits > 1) {
    int* fit = ds->fit;
    const int64_t tiles = pl.tiles_n * pl.tiles_m;
    int splits = pl.splits;
    for (; splits > 1; --splits) {
      if (fit[splits] == 0) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(static_cast<unsigned>(pl.tiles_n), static_cast<unsigned>(pl.tiles_m), static_cast<unsigned>(splits));
        q.blockDim = dim3(224);
        q.dynamicSmemBytes = SMEM_SPLIT;
        cudaLaunchAttribute ca;
        ca.id = cudaLaunchAttributeClusterDimension;
        ca.val.clusterDim.x = 1; ca.val.clusterDim.y = 1; ca.val.clusterDim.z = static_cast<unsigned>(splits);
        q.attrs = &ca;
        q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc5_kernel<T, BN, CONV, MODE>, &q) != cudaSuccess) { cudaGetLastError(); n = -1; }
        fit[splits] = n > 0 ? n : -1;
      }
      if (fit[splits] >= tiles) break;
    }
    const int64_t KB = ceil_div(a.K, BK);
    pl.kb_per_split = static_cast<int>(ceil_div(KB, splits));
    pl.splits = static_cast<int>(ceil_div(KB, pl.kb_per_split));
  }
  const int SMEM = pl.splits > 1 ? SMEM_SPLIT : SMEM_RING;
  CUtensorMap ma, mw;
  if (!make_map(&mw, a.W, a.N, a.K, a.ldw, BN, a.dtype)) return B200_ENOTSUP;
  Tc5Params p;
  p.x = a.A;
  p.g = g ? *g : Tc5Conv{};
  if (CONV) {
    p.g.im2col = make_im2col_map(&ma, a.A, p.g, a.dtype) ? 1 : 0;
    if (!p.g.im2col) ma = mw;   // unused: the epilogue warps gather the A tile
  } else if (!make_map(&ma, a.A, a.M, a.K, a.lda, Cfg<BN, MODE>::AROWS, a.dtype)) {
    return B200_ENOTSUP;
  }
  p.bias = a.bias; p.residual = a.residual; p.aux = a.aux; p.out = a.out;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo; p.ldr = a.ldr; p.ldaux = a.ldaux;
  p.bias_dtype = a.bias_dtype; p.epilogue = a.epilogue; p.splits = pl.splits; p.kb_per_split = pl.kb_per_split;
  p.norm_eps = a.norm_eps; p.sumsq_in = a.sumsq_in; p.sumsq_in_cols = a.sumsq_in_cols; p.sumsq_out = a.sumsq_out;
  if ((a.sumsq_in || a.sumsq_out) && (CONV || MODE < 2)) return B200_ENOTSUP;
  p.rope = a.rope;
  if (a.rope.cos && (CONV || MODE < 2 || BN != 128 || a.N % 128)) return B200_ENOTSUP;
  if (CONV && pl.splits != 1) return B200_ENOTSUP;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pl.tiles_n), static_cast<unsigned>(pl.tiles_m), static_cast<unsigned>(pl.splits));
  cfg.blockDim = dim3(224);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  int n_attrs = 0;
  if (pdl_enabled()) {
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  if (pl.splits > 1) {   // the split-K CTAs of one tile exchange partial sums through distributed shared memory
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = 1;
    attrs[n_attrs].val.clusterDim.y = 1;
    attrs[n_attrs].val.clusterDim.z = static_cast<unsigned>(pl.splits);
    ++n_attrs;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  cudaLaunchKernelEx(&cfg, gemm_tc5_kernel<T, BN, CONV, MODE>, ma, mw, p);
  B200_CHECK_LAUNCH("gemm_tc5_kernel");
  return B200_OK;
}

// Persistent-kernel choices settled by measurement on ResNet-50 at batch 256 and Qwen prefill:
// column tiles fastest for reductions up to K = 256, a second activation producer thread for
// convolutions only, weight tiles resident whenever they fit.
constexpr int COLUMN_FASTEST_MAX_K = 256;

template <typename T, int BN, bool CONV, bool TS>
int launch_persistent(const Tc5Args& a, cudaStream_t st, const Tc5Conv* g = nullptr) {
  using PC = PCfg<BN, TS>;
  static_assert(PC::SMEM <= PC::SMEM_LIMIT, "ring + C buffers exceed the shared memory of an SM");
  static PerDevice<bool> configured_on;
  bool* configured = configured_on.slot();
  if (!configured) return B200_ENOTSUP;
  if (!*configured) {
    if (cudaFuncSetAttribute(gemm_tc5p_kernel<T, BN, CONV, TS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PC::SMEM_LIMIT) != cudaSuccess ||
        (BN <= 128 && cudaFuncSetAttribute(gemm_tc5p_kernel<T, BN, CONV, TS, BN <= 128 ? 2 : 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           PC::SMEM_LIMIT) != cudaSuccess)) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    *configured = true;
  }
  CUtensorMap ma, mw, mr, mo;
  Tc5Params p;
  p.g = g ? *g : Tc5Conv{};
  if (CONV && p.g.c8) {
    if (!make_map_c8(&mw, a.W, a.N, a.K, a.ldw, BN, a.dtype) || !make_im2col_map_c8(&ma, a.A, p.g, a.dtype)) return B200_ENOTSUP;
    p.g.im2col = 1;
  } else if (!make_map(&mw, a.W, a.N, a.K, a.ldw, BN, a.dtype)) {
    return B200_ENOTSUP;
  } else if (CONV) {
    p.g.im2col = make_im2col_map(&ma, a.A, p.g, a.dtype) ? 1 : 0;
    if (!p.g.im2col) {
      if (TS) return B200_ENOTSUP;   // warp 6 cannot both gather and store
      ma = mw;
    }
  } else if (!make_map(&ma, a.A, a.M, a.K, a.lda, BM, a.dtype)) {
    return B200_ENOTSUP;
  }
  mr = mw; mo = mw;
  if (TS) {   // output (and residual) as [M, N] maps with 64-column x 128-row boxes
    if (!make_map(&mo, a.out, a.M, a.N, a.ldo, BM, a.dtype)) return B200_ENOTSUP;
    if (a.residual && !make_map(&mr, a.residual, a.M, a.N, a.ldr, BM, a.dtype)) return B200_ENOTSUP;
  }
  p.bias = a.bias; p.residual = a.residual; p.aux = a.aux; p.out = a.out;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo; p.ldr = a.ldr; p.ldaux = a.ldaux;
  p.bias_dtype = a.bias_dtype; p.epilogue = a.epilogue; p.splits = 1; p.kb_per_split = static_cast<int>(ceil_div(a.K, BK));
  p.sumsq_in = nullptr; p.sumsq_out = nullptr; p.norm_eps = 0.f; p.sumsq_in_cols = 0;
  p.x = a.A;
  const int64_t tiles_m = ceil_div(a.M, BM), tiles = tiles_m * ceil_div(a.N, BN);
  if (tiles >= (1ll << 31)) return B200_ENOTSUP;
  int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  const int64_t tiles_n = ceil_div(a.N, BN);
  p.nfast = 0;
  if (a.K <= COLUMN_FASTEST_MAX_K && tiles_n > 1 && tiles_n <= grid / 4 && tiles >= 2 * grid) {
    p.nfast = 1;
    grid -= grid % static_cast<int>(tiles_n);   // every CTA stays on one column tile
  }

  // shared-memory plan
  p.pst = PC::ST; p.pstage = PC::STAGE; p.wr = 0; p.w_off = 0; p.pncb = TS ? PC::NCB : 1; p.c_off = PC::ST * PC::STAGE;
  int SMEM = PC::SMEM;
  const int64_t w_bytes = ceil_div(a.K, BK) * PC::B_STAGE;
  if ((!CONV || p.g.im2col) && w_bytes <= 96 * 1024 && tiles >= 2 * grid) {
    const int avail = PC::SMEM_LIMIT - 1024 - static_cast<int>(w_bytes);
    for (int stages = (a.K <= BK ? 4 : 6); stages >= 4; stages -= 2) {
      const int left = avail - stages * PC::A_STAGE;
      const int ncb = TS ? (left / PC::CB < PC::MAX_NCB ? left / PC::CB : PC::MAX_NCB) : 0;
      if (left < 0 || (TS && ncb < PC::NCB)) continue;
      p.wr = 1; p.pst = stages; p.pstage = PC::A_STAGE; p.w_off = stages * PC::A_STAGE;
      p.c_off = p.w_off + static_cast<int>(w_bytes); p.pncb = TS ? ncb : 1;
      SMEM = p.c_off + (TS ? ncb : 0) * PC::CB + 1024;
      break;
    }
  }
  // Two k-blocks per ring stage where a k-block of MMAs is short (tiles up to 128 wide: 0.05-0.13 us against
  // ~0.3 us for a barrier hand-off between the single-thread roles): half as many hand-offs per tile.  From
  // nine k-blocks per tile - the 3x3 convolutions and long reductions (ResNet-50 at batch 256: 3x3 over 64
  // channels 178 -> 146 us, over 512 channels 90 -> 68 us) - and from four where the ring has an even number
  // of stages; shorter, memory-bound reductions on an odd ring keep it (pairing would lose a k-block of
  // buffering: 1x1/2 512 -> 1024 went 88 -> 109 us).
  // A compile-time parameter of the kernel: with a run-time count the longer issue loops cost what the
  // halved hand-offs gained.  (Not for the unswizzled 8-channel operands and the gathered A tile.)
  p.kps = 1;
  if (BN <= 128 && (!CONV || (p.g.im2col && !p.g.c8)) && p.pst >= 4 && (ceil_div(a.K, BK) >= 9 || (ceil_div(a.K, BK) >= 4 && p.pst % 2 == 0))) {
    p.kps = 2;
    p.pst /= 2;
    p.pstage *= 2;
  }
  // Two activation producers for convolutions through im2col boxes.  (Dealing k-blocks to more threads than the
  // ring has stages would be wrong, not just useless: a producer learns how far the MMAs have got only from its
  // own waits, one ring pass back at a time, and a parity wait cannot tell a barrier two phases behind from the
  // phase it expects.  Two is below every ring depth used here.)
  p.npa = CONV && p.g.im2col && ceil_div(a.K, BK) >= 2 ? 2 : 1;
  const dim3 block((CONV && !TS && !p.g.im2col) ? 352 : PC::THREADS);
  if (p.kps == 2)
    launch_pdl(gemm_tc5p_kernel<T, BN, CONV, TS, BN <= 128 ? 2 : 1>, dim3(grid), block, SMEM, st, ma, mw, mr, mo, p, static_cast<int>(tiles_m),
               static_cast<int>(tiles));
  else
    launch_pdl(gemm_tc5p_kernel<T, BN, CONV, TS, 1>, dim3(grid), block, SMEM, st, ma, mw, mr, mo, p, static_cast<int>(tiles_m), static_cast<int>(tiles));
  B200_CHECK_LAUNCH("gemm_tc5p_kernel");
  return B200_OK;
}

// The CTA-pair kernel takes a linear layer when its 256 x 256 tiles give at least half of the 74 pairs a tile
// (even half empty it beats 128-wide tiles on every SM) and the reduction is long enough to hide the plain epilogue.
bool pair_shape(const Tc5Args& a) {
  // (N >= 1024: a tall activation matrix against one or two column tiles - the 1x1 convolutions 1024 -> 256 / 512
  // over 50176 pixels - measured slower here than with the bulk-copy epilogue of the persistent kernel)
  if (a.M <= 128 || a.N < 1024 || a.K < 1024) return false;
  return ceil_div(a.M, 256) * ceil_div(a.N, 256) >= 37;
}

// Few tiles but a long reduction (the down projection of a 512- or 1024-token prompt: 12 or 24 tiles, K = 8960): the
// pairs split K among themselves and leave fp32 partial sums in the caller's workspace; measured 21.8 us (512 rows)
// and 30.7 us (1024) against 33.9 and 70.5 us for 128 x 128 tiles with split-K inside a cluster.  Returns the split
// count (1: none).
int pair_splits(int64_t M, int64_t N, int64_t K) {
  if (M <= 128 || N < 256 || K < 4096 || N % 8) return 1;
  const int64_t tiles = ceil_div(M, 256) * ceil_div(N, 256), KB = ceil_div(K, BK);
  if (tiles >= 37 || tiles < 12) return 1;   // (fewer than 12 tiles: up to 256 rows, left to the one-tile kernel)
  int64_t s = 74 / tiles;
  if (s > KB / 16) s = KB / 16;   // at least 16 k-blocks per unit
  if (s > PAIR_MAX_SPLITS) s = PAIR_MAX_SPLITS;
  if (s < 2) return 1;
  const int64_t per = ceil_div(KB, s);
  return static_cast<int>(ceil_div(KB, per));
}

int64_t pair_splitk_bytes(int64_t M, int64_t N, int splits) { return splits > 1 ? splits * M * N * 4 : 0; }

template <typename T> int launch_pair(const Tc5Args& a, cudaStream_t st, int splits = 1) {
  static PerDevice<bool> configured_on;
  bool* configured = configured_on.slot();
  if (!configured) return B200_ENOTSUP;
  if (!*configured) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM) != cudaSuccess) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    *configured = true;
  }
  CUtensorMap ma, mw;
  if (!make_map(&ma, a.A, a.M, a.K, a.lda, BM, a.dtype) || !make_map(&mw, a.W, a.N, a.K, a.ldw, PAIR_BN / 2, a.dtype)) return B200_ENOTSUP;
  Tc5Params p = {};
  p.bias = a.bias; p.residual = a.residual; p.aux = a.aux; p.out = a.out;
  p.M = a.M; p.N = a.N; p.K = a.K; p.ldo = a.ldo; p.ldr = a.ldr; p.ldaux = a.ldaux;
  p.bias_dtype = a.bias_dtype; p.epilogue = a.epilogue;
  p.splits = splits; p.kb_per_split = static_cast<int>(ceil_div(ceil_div(a.K, BK), splits));
  p.partial = static_cast<float*>(a.workspace);
  p.x = a.A;
  const int64_t tiles_m = ceil_div(a.M, 256), tiles = tiles_m * ceil_div(a.N, PAIR_BN), units = tiles * splits;
  if (units >= (1ll << 30) || splits > PAIR_MAX_SPLITS) return B200_ENOTSUP;
  if (splits > 1 && (!a.workspace || a.workspace_bytes < pair_splitk_bytes(a.M, a.N, splits) || (reinterpret_cast<uintptr_t>(a.workspace) & 31u)))   // 256-bit accesses
    return B200_ENOTSUP;
  const int pairs = static_cast<int>(units < sm_count() / 2 ? units : sm_count() / 2);
  launch_pdl(gemm_pair_kernel<T>, dim3(2 * pairs), dim3(PAIR_THREADS), PAIR_SMEM, st, ma, mw, p, static_cast<int>(tiles_m), static_cast<int>(tiles));
  B200_CHECK_LAUNCH("gemm_pair_kernel");
  if (splits > 1) {
    const Tc5Args::NormTail& t = a.norm_tail;
    const bool tail = t.out && t.gain && t.done && a.N <= 2048 && a.M < (1ll << 31) && t.ld % 8 == 0 && aligned16(t.out) && aligned16(t.gain) &&
                      !(a.epilogue & B200_EPI_SILU_MUL);
    if (tail) {
      const NormTailParams nt{t.gain, t.out, t.ld, t.eps, t.round_mid};
      const int threads = static_cast<int>(ceil_div(a.N / 8, 32) * 32);
      launch_pdl(pair_splitk_reduce_norm_kernel<T>, dim3(static_cast<unsigned>(a.M)), dim3(threads), 0, st, p, nt);
      B200_CHECK_LAUNCH("pair_splitk_reduce_norm_kernel");
      *t.done = 1;
    } else {
      const int64_t work = a.M * (a.N / 8);
      const int blocks = static_cast<int>(ceil_div(work, 256) < 4 * sm_count() ? ceil_div(work, 256) : 4 * sm_count());
      launch_pdl(pair_splitk_reduce_kernel<T>, dim3(blocks), dim3(256), 0, st, p);
      B200_CHECK_LAUNCH("pair_splitk_reduce_kernel");
    }
  }
  return B200_OK;
}

// Tile width of the persistent kernel for a shape, or 0 when the shape should stay on the
// one-tile-per-CTA kernel (too few tiles to fill the SMs with wide tiles).
int persistent_bn(int64_t M, int64_t N, int64_t K, bool glu, bool residual) {
  const int64_t tm = ceil_div(M, BM);
  // One row tile: the one-tile kernel, except for a very wide N (the vocabulary projection of a decode step:
  // 1187 one-tile CTAs run in eight waves and pay their start-up eight times; measured 123 us for 467 MB).
  if (tm < 2) return (K > 512 && ceil_div(N, 256) >= 2 * 148) ? 256 : 0;
  // short reductions are memory-bound: 128-wide tiles leave room for two C buffers (see PCfg)
  // (a tile wider than N only multiplies and copies padding: 64 output channels take 64-wide tiles)
  if (K > 512 && N > 128 && ceil_div(N, 256) * tm >= 2 * 148) return 256;
  // Short reductions are memory-bound and the column tiles of a row tile run far apart in time, so every
  // column tile reads its activation tile from DRAM again: a 256-wide tile halves those reads.  It pays
  // where two C buffers still fit beside the resident weights (K <= 64: 1x1 expansions 64 -> 256 went from
  // 0.78 to 0.91 of their HBM time) or where no residual tile has to be prefetched into the one buffer.
  if (N >= 256 && (K <= 64 || (K <= 256 && !residual)) && ceil_div(N, 256) * tm >= 2 * 148) return 256;
  if ((N > 64 || glu) && ceil_div(N, 128) * tm >= 148) return 128;
  if (!glu && ceil_div(N, 64) * tm >= 148) return 64;
  return 0;
}

// The bulk-copy epilogue handles 16-bit outputs with bias, residual and ReLU.
bool tma_store_ok(const Tc5Args& a) {
  if (a.epilogue & (B200_EPI_GLU | B200_EPI_SILU_MUL)) return false;
  if (a.K > 2048) return false;   // long reductions hide the plain epilogue and prefer the deeper ring
  if (!aligned16(a.out) || a.ldo % 8 || a.N % 8) return false;
  if (a.residual && (!aligned16(a.residual) || a.ldr % 8)) return false;
  return true;
}

template <typename T, bool CONV> int dispatch_persistent_t(int bn, bool ts, const Tc5Args& a, cudaStream_t st, const Tc5Conv* g) {
  if (ts) {
    int rc = bn == 256 ? launch_persistent<T, 256, CONV, true>(a, st, g) : bn == 128 ? launch_persistent<T, 128, CONV, true>(a, st, g)
                                                                                     : launch_persistent<T, 64, CONV, true>(a, st, g);
    if (rc != B200_ENOTSUP) return rc;
  }
  return bn == 256 ? launch_persistent<T, 256, CONV, false>(a, st, g) : bn == 128 ? launch_persistent<T, 128, CONV, false>(a, st, g)
                                                                                  : launch_persistent<T, 64, CONV, false>(a, st, g);
}

template <bool CONV> int dispatch_persistent(int bn, const Tc5Args& a, cudaStream_t st, const Tc5Conv* g) {
  const bool ts = tma_store_ok(a);
  if (a.dtype == B200_BF16) return dispatch_persistent_t<__nv_bfloat16, CONV>(bn, ts, a, st, g);
  return dispatch_persistent_t<__half, CONV>(bn, ts, a, st, g);
}

// The stem kernel takes 7-wide filters with stride 2 and padding 3 along W on an 8-channel input whose
// output rows fit one tile (Wo <= 128); other stems go through the im2col path.
template <typename T>
int launch_stem_rows(const Tc5Args& a, const Tc5Conv& g, cudaStream_t st) {
  if (g.C != 8 || g.KW != 7 || g.sw != 2 || g.pw != 3 || g.sh != 2 || g.KH < 1 || g.KH > 8 || g.Wo > BM || g.W > 256 ||
      g.Wo != (g.W + 2 * g.pw - g.KW) / g.sw + 1 || g.batch <= 0 || a.residual || a.N > STEM_BN || a.N % 8 ||
      a.K != static_cast<int64_t>(g.KH) * g.KW * 8 || a.ldw % 8 || !aligned16(a.A) || !aligned16(a.W) || !tma_store_ok(a))
    return B200_ENOTSUP;
  constexpr int SMEM = 8 * STEM_W_STAGE + 2 * STEM_CB + STEM_SLOTS * STEM_SLOT + 1024;
  static PerDevice<bool> configured_on;
  bool* configured = configured_on.slot();
  if (!configured) return B200_ENOTSUP;
  if (!*configured) {
    if (cudaFuncSetAttribute(conv_stem_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    *configured = true;
  }
  CUtensorMap mw, mo;
  if (!make_map_c8(&mw, a.W, a.N, a.K, a.ldw, STEM_BN, a.dtype) || !make_map(&mo, a.out, a.M, a.N, a.ldo, g.Wo, a.dtype)) return B200_ENOTSUP;
  const int64_t tiles = static_cast<int64_t>(g.batch) * g.Ho;
  if (tiles >= (1ll << 31) || a.M != tiles * g.Wo) return B200_ENOTSUP;
  StemParams p;
  p.x = a.A; p.bias = a.bias; p.bias_dtype = a.bias_dtype; p.relu = (a.epilogue & B200_EPI_RELU) ? 1 : 0;
  p.batch = g.batch; p.H = g.H; p.W = g.W; p.Ho = g.Ho; p.Wo = g.Wo; p.KH = g.KH; p.sh = g.sh; p.ph = g.ph; p.N = static_cast<int>(a.N);
  p.tiles = static_cast<int>(tiles);
  const int sms = sm_count();
  p.tiles_per_cta = static_cast<int>(ceil_div(tiles, tiles < sms ? tiles : sms));
  const int grid = static_cast<int>(ceil_div(tiles, p.tiles_per_cta));
  launch_pdl(conv_stem_rows_kernel<T>, dim3(grid), dim3(STEM_THREADS), SMEM, st, mw, mo, p);
  B200_CHECK_LAUNCH("conv_stem_rows_kernel");
  return B200_OK;
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

// Scratch of the tcgen05 path: none for the cluster split-K of the one-tile kernel (partial sums meet in
// distributed shared memory); fp32 partial sums for the split-K of the CTA-pair kernel.
int64_t linear_tc5_workspace_bytes(int64_t M, int64_t N, int64_t K) { return pair_splitk_bytes(M, N, pair_splits(M, N, K)); }

int linear_tc5(const Tc5Args& a, cudaStream_t st) {
  if (!tc5_enabled()) return B200_ENOTSUP;
  if (a.dtype != B200_BF16 && a.dtype != B200_F16) return B200_ENOTSUP;
  if (a.K % 8 || a.lda % 8 || a.ldw % 8 || !aligned16(a.A) || !aligned16(a.W)) return B200_ENOTSUP;
  if (a.M >= (1ll << 31) || a.N >= (1ll << 31) || a.K >= (1ll << 31)) return B200_ENOTSUP;
  const bool glu = (a.epilogue & B200_EPI_GLU) != 0;
  if (glu && (a.N % 128 || (a.epilogue & ~(B200_EPI_GLU | B200_EPI_W_STATIC)) || a.residual)) return B200_ENOTSUP;
  if (a.sumsq_in || a.sumsq_out) {   // carried by the staged epilogue of the decode kernel
    if (a.M > 64) return B200_ENOTSUP;
    if (a.sumsq_in && (a.sumsq_in_cols <= 0 || a.sumsq_in_cols > NORM_MAX_PARTS || (a.epilogue & B200_EPI_SILU_MUL))) return B200_ENOTSUP;
    const int tb = a.dtype == B200_BF16 ? B200_BF16 : B200_F16;
    if (a.sumsq_out && (a.N % 64 || glu || (a.epilogue & B200_EPI_SILU_MUL) || (reinterpret_cast<uintptr_t>(a.out) & 7u) || a.ldo % 4 ||
                        (a.bias && a.bias_dtype != B200_F32 && a.bias_dtype != tb) ||
                        (a.residual && ((reinterpret_cast<uintptr_t>(a.residual) & 7u) || a.ldr % 4))))
      return B200_ENOTSUP;
  }
  if (a.rope.cos) {   // merged q/k/v projection with rotary embedding and cache write: decode shapes, one head per 128-wide tile
    const Tc5Args::Rope& r = a.rope;
    const bool aligned = aligned16(r.cos) && aligned16(r.sin) && aligned16(r.q_out) && aligned16(r.k_cache) && aligned16(r.v_cache);
    if (a.M > 64 || !r.sin || !r.q_out || !r.k_cache || !r.v_cache || !r.cache_pos || !aligned || r.Hq <= 0 || r.Hkv <= 0 ||
        a.N != static_cast<int64_t>(r.Hq + 2 * r.Hkv) * 128 || a.residual || a.sumsq_out || glu || (a.epilogue & ~B200_EPI_W_STATIC) ||
        (r.pos_dtype != B200_I64 && r.pos_dtype != B200_I32) || r.cache_len <= 0)
      return B200_ENOTSUP;
    const Tc5Plan pl = plan_tc5(a.M, a.N, a.K, false);
    if (pl.bn != 128 || pl.tiles_m != 1) return B200_ENOTSUP;
    return a.dtype == B200_BF16 ? launch<__nv_bfloat16, 128, false, 2>(a, pl, st) : launch<__half, 128, false, 2>(a, pl, st);
  }
  if (pair_shape(a)) {
    const int rc = a.dtype == B200_BF16 ? launch_pair<__nv_bfloat16>(a, st) : launch_pair<__half>(a, st);
    if (rc != B200_ENOTSUP) return rc;
  }
  if (const int ps = pair_splits(a.M, a.N, a.K); ps > 1 && !glu) {   // (falls through when the caller gave no workspace)
    const int rc = a.dtype == B200_BF16 ? launch_pair<__nv_bfloat16>(a, st, ps) : launch_pair<__half>(a, st, ps);
    if (rc != B200_ENOTSUP) return rc;
  }
  if (const int bn = (a.sumsq_in || a.sumsq_out) ? 0 : persistent_bn(a.M, a.N, a.K, glu, a.residual != nullptr))
    return dispatch_persistent<false>(bn, a, st, nullptr);
  const Tc5Plan pl = plan_tc5(a.M, a.N, a.K, glu);
  if (pl.tiles_m > 65535 || pl.splits > 65535) return B200_ENOTSUP;
  if (pl.tiles_m == 1 && a.M <= 64) {
    if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false, 2>(a, pl, st) : launch<__nv_bfloat16, 128, false, 2>(a, pl, st);
    return pl.bn == 64 ? launch<__half, 64, false, 2>(a, pl, st) : launch<__half, 128, false, 2>(a, pl, st);
  }
  if (pl.tiles_m == 1) {
    if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false, 1>(a, pl, st) : launch<__nv_bfloat16, 128, false, 1>(a, pl, st);
    return pl.bn == 64 ? launch<__half, 64, false, 1>(a, pl, st) : launch<__half, 128, false, 1>(a, pl, st);
  }
  if (pl.splits > 1) {   // split-K CTAs sit alone on their SM (ring + receive buffer): give them the deeper ring of mode 1
    if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false, 1>(a, pl, st) : launch<__nv_bfloat16, 128, false, 1>(a, pl, st);
    return pl.bn == 64 ? launch<__half, 64, false, 1>(a, pl, st) : launch<__half, 128, false, 1>(a, pl, st);
  }
  if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, false>(a, pl, st) : launch<__nv_bfloat16, 128, false>(a, pl, st);
  return pl.bn == 64 ? launch<__half, 64, false>(a, pl, st) : launch<__half, 128, false>(a, pl, st);
}

int conv_tc5(const Tc5Args& a, const Tc5Conv& g, cudaStream_t st) {
  if (!tc5_enabled()) return B200_ENOTSUP;
  if (a.dtype != B200_BF16 && a.dtype != B200_F16) return B200_ENOTSUP;
  if (a.M >= (1ll << 31) || a.N >= (1ll << 31) || (a.epilogue & ~(B200_EPI_RELU | B200_EPI_W_STATIC))) return B200_ENOTSUP;
  if (g.C == 8 && !(a.epilogue & ~(B200_EPI_RELU | B200_EPI_W_STATIC))) {   // 7x7 stem: rows kept in a shared-memory window
    const int rc = a.dtype == B200_BF16 ? launch_stem_rows<__nv_bfloat16>(a, g, st) : launch_stem_rows<__half>(a, g, st);
    if (rc != B200_ENOTSUP) return rc;
  }
  if (g.C == 8) {   // stem convolution on the padded RGB input: persistent kernel, 64-wide tiles, bulk-copy epilogue
    if (a.K != static_cast<int64_t>(g.KH) * g.KW * 8 || a.ldw % 8 || !aligned16(a.A) || !aligned16(a.W) || a.N > 64 || a.N % 8 ||
        a.M < 2 * BM || !tma_store_ok(a))
      return B200_ENOTSUP;
    Tc5Conv g8 = g;
    g8.c8 = 1;
    return a.dtype == B200_BF16 ? launch_persistent<__nv_bfloat16, 64, true, true>(a, st, &g8) : launch_persistent<__half, 64, true, true>(a, st, &g8);
  }
  if (g.C % BK || a.K != static_cast<int64_t>(g.KH) * g.KW * g.C || a.ldw % 8 || !aligned16(a.A) || !aligned16(a.W)) return B200_ENOTSUP;
  if (const int bn = persistent_bn(a.M, a.N, a.K, false, a.residual != nullptr)) return dispatch_persistent<true>(bn, a, st, &g);
  Tc5Plan pl;
  pl.bn = a.N >= 128 ? 128 : 64;
  pl.tiles_n = ceil_div(a.N, pl.bn);
  pl.tiles_m = ceil_div(a.M, BM);
  pl.splits = 1;
  pl.kb_per_split = static_cast<int>(a.K / BK);
  if (pl.tiles_m > 65535) return B200_ENOTSUP;
  if (a.dtype == B200_BF16) return pl.bn == 64 ? launch<__nv_bfloat16, 64, true, 0>(a, pl, st, &g) : launch<__nv_bfloat16, 128, true, 0>(a, pl, st, &g);
  return pl.bn == 64 ? launch<__half, 64, true, 0>(a, pl, st, &g) : launch<__half, 128, true, 0>(a, pl, st, &g);
}

}  // namespace b200

namespace b200 {
__global__ void wait_timeout_selftest_kernel(uint32_t probes) {
  __shared__ __align__(8) uint64_t bar;
  tc5::mbar_init(&bar, 1);
  tc5::fence_barrier_init();
  if (!tc5::mbar_wait(&bar, 0, probes)) atomicExch(&g_tc5_error, 99);   // nobody arrives: the bounded wait must give up
}
}  // namespace b200

extern "C" int b200_debug_wait_timeout(int probes, void* stream) {
  B200_CHECK_ARG(probes > 0 && probes <= (1 << 20), "b200_debug_wait_timeout: probes must be in 1..2^20");
  b200::wait_timeout_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t>(probes));
  B200_CHECK_LAUNCH("wait_timeout_selftest_kernel");
  return B200_OK;
}

extern "C" int b200_debug_device_error(int* code, int clear) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, b200::g_tc5_error, sizeof(int));
  if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "b200_debug_device_error: %s", cudaGetErrorString(e));
  const int att = b200::attn_prefill_tc5_error(clear != 0);
  if (code) *code = v ? v : (att > 0 ? att : 0);
  if (clear && v) {
    v = 0;
    cudaMemcpyToSymbol(b200::g_tc5_error, &v, sizeof(int));
  }
  return B200_OK;
}
