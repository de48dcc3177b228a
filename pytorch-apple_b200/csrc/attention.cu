// Fused attention for head_dim 128 on the warp-level tensor-core path.
//
// One warp owns a 16-row score tile: 16 query positions of one head (prefill) or
// the group of query heads that share one KV head, padded to 16 (decode).  K and V
// rows go from global memory straight into MMA fragments with 16-byte loads:
//   * S = Q K^T: inside every 32-wide slice of the head dim, thread t of a quad owns
//     dims 8t..8t+7 for both Q and K - a consistent permutation of the contraction
//     index, so the dot products are unchanged;
//   * O = P V: thread (g, t) loads dims 8g..8g+7 (+64) of keys {2t, 2t+1, 2t+8, 2t+9}
//     and assembles the B fragments with byte permutes; output column "g" of MMA
//     tile j therefore is head dim 8g + j, which the store undoes.
// Softmax is the usual online form in fp32; P is rounded to the activation dtype
// for the second MMA, as the unfused graph rounds the probabilities.
#include "mma.cuh"

#include <stdlib.h>

namespace b200 {

constexpr int HD = 128;          // head dim
constexpr float LOG2E = 1.4426950408889634f;
constexpr float MASKED = -1e30f; // additive mask values at or below this are "masked out"

template <typename T> struct AttnWarp {
  uint32_t q[4][2][4];  // [32-dim slice][row half g / g+8][4 x 32-bit]
  float o[2][8][4];     // [64-dim half][tile j][c0..c3]
  float m[2], l[2];     // running max / sum for rows g and g+8

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[a][j][e] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }

  // q_lo / q_hi: rows g and g+8 (nullptr -> zero row)
  __device__ __forceinline__ void load_q(const T* q_lo, const T* q_hi, int t) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 lo = q_lo ? *reinterpret_cast<const uint4*>(q_lo + 32 * c + 8 * t) : make_uint4(0, 0, 0, 0);
      const uint4 hi = q_hi ? *reinterpret_cast<const uint4*>(q_hi + 32 * c + 8 * t) : make_uint4(0, 0, 0, 0);
      q[c][0][0] = lo.x; q[c][0][1] = lo.y; q[c][0][2] = lo.z; q[c][0][3] = lo.w;
      q[c][1][0] = hi.x; q[c][1][1] = hi.y; q[c][1][2] = hi.z; q[c][1][3] = hi.w;
    }
  }

  // One block of 16 keys starting at row `kb`.  k_base/v_base point at key 0 of this
  // (batch, kv head); key stride in elements.  add[j][e]: additive mask (already in
  // the score domain) for rows (g, g+8) x keys (8j+2t, 8j+2t+1): index [j][2*half+e].
  __device__ __forceinline__ void step(const T* k_base, const T* v_base, int64_t k_stride, int64_t v_stride, int64_t kb,
                                       int64_t n_keys, float scale, const float (&add)[2][4], int g, int t) {
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    // ---- issue all loads for this block -----------------------------------------
    uint4 kf[2][4];  // [key tile][32-dim slice]
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t key = kb + 8 * j + g;
      const T* kr = k_base + key * k_stride + 8 * t;
#pragma unroll
      for (int c = 0; c < 4; ++c) kf[j][c] = key < n_keys ? ld_global_nc_v4(kr + 32 * c) : zero4;
    }
    uint4 vf[2][4];  // [64-dim half][key slot 2t, 2t+1, 2t+8, 2t+9]
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int64_t key = kb + 2 * t + (s & 1) + 8 * (s >> 1);
      const T* vr = v_base + key * v_stride + 8 * g;
#pragma unroll
      for (int a = 0; a < 2; ++a) vf[a][s] = key < n_keys ? ld_global_nc_v4(vr + 64 * a) : zero4;
    }
    compute(kf, vf, kb, n_keys, scale, add, t);
  }

  // Same block, fragments already in registers (from global memory or from a shared-memory stage).
  __device__ __forceinline__ void compute(const uint4 (&kf)[2][4], const uint4 (&vf)[2][4], int64_t kb, int64_t n_keys, float scale,
                                          const float (&add)[2][4], int t) {
    // ---- S = Q K^T ---------------------------------------------------------------
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t a1[4] = {q[c][0][0], q[c][1][0], q[c][0][1], q[c][1][1]};
        const uint32_t a2[4] = {q[c][0][2], q[c][1][2], q[c][0][3], q[c][1][3]};
        const uint32_t b1[2] = {kf[j][c].x, kf[j][c].y};
        const uint32_t b2[2] = {kf[j][c].z, kf[j][c].w};
        MmaType<T>::mma(s[j], a1, b1);
        MmaType<T>::mma(s[j], a2, b2);
      }
    }
    // ---- online softmax ------------------------------------------------------------
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t key = kb + 8 * j + 2 * t + (e & 1);
        const float v = key < n_keys ? s[j][e] * scale + add[j][e] : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m[h], mx[h]);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      corr[h] = exp2f((m[h] - m_use) * LOG2E);  // m = -inf -> 0
      m[h] = m_new;
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float p = exp2f((s[j][2 * h + e] - m_use) * LOG2E);
          s[j][2 * h + e] = p;
          rs += p;
        }
      rs += __shfl_xor_sync(0xffffffffu, rs, 1);
      rs += __shfl_xor_sync(0xffffffffu, rs, 2);
      l[h] = l[h] * corr[h] + rs;
    }
    // ---- O = O * corr + P V -----------------------------------------------------------
    const uint32_t pa[4] = {pack2<T>(s[0][0], s[0][1]), pack2<T>(s[0][2], s[0][3]), pack2<T>(s[1][0], s[1][1]),
                            pack2<T>(s[1][2], s[1][3])};
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&vf[a][0]);
      const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&vf[a][1]);
      const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&vf[a][2]);
      const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&vf[a][3]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
        const uint32_t b[2] = {__byte_perm(r0[j >> 1], r1[j >> 1], sel), __byte_perm(r2[j >> 1], r3[j >> 1], sel)};
        o[a][j][0] *= corr[0]; o[a][j][1] *= corr[0];
        o[a][j][2] *= corr[1]; o[a][j][3] *= corr[1];
        MmaType<T>::mma(o[a][j], pa, b);
      }
    }
  }
};

// head dim held in o[a][j][2*h + e]  (h: row half) for thread (g, t)
__device__ __forceinline__ int out_dim(int a, int j, int e, int t) { return 64 * a + 8 * (2 * t + e) + j; }

// ===========================================================================
// Decode: one query token, G = Hq / Hkv query heads share each KV head.
// grid = (splits, Hkv, B), 128 threads.  Partials: acc [B][Hkv][splits][G][HD] fp32,
// then ml [B][Hkv][splits][G][2] fp32 (running max in the log2 domain, sum).
// ===========================================================================
struct DecodeParams {
  const void* q; const void* k; const void* v; const void* mask;
  float* part_acc; float* part_ml;
  int64_t B, S;
  int Hq, Hkv, G;
  int64_t q_bs, kv_bs, kv_hs, mask_bs;
  int split_len, splits;
  float scale;
  int mask_dtype;
  int l2_ahead;   // blocks per warp requested into L2 ahead of the shared-memory ring
};

constexpr int DEC_MAX_BLOCKS = 128;  // 16-key blocks per split (split_len <= 2048)

// Phase time stamps for tuning, compiled in only with -DB200NN_TC5_TRACE (never in the shipped library).
#ifdef B200NN_TC5_TRACE
constexpr int ATR_CTAS = 1280, ATR_N = 8;
__device__ unsigned long long g_attn_trace[ATR_CTAS][ATR_N];
#define ATTN_STAMP(i)                                                                                   \
  do {                                                                                                  \
    const int cta_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);                    \
    if (threadIdx.x == 0 && cta_ < ATR_CTAS) {                                                          \
      unsigned long long t_;                                                                            \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                            \
      g_attn_trace[cta_][i] = t_;                                                                       \
    }                                                                                                   \
  } while (0)
#else
#define ATTN_STAMP(i)
#endif

constexpr int DEC_STAGE_BYTES = 2 * 16 * HD * 2;  // 16 keys of K and of V
constexpr int DEC_MAX_SPLIT = 512;             // keys per split (mask values of a split are staged in shared memory)
constexpr int DEC_ACC_PITCH = HD + 4;          // row pitch of the cross-warp accumulator (spreads the heads over banks)

// The decode kernel works on the transposed problem, so that the (at most 8) query heads of a
// KV group sit on the 8-wide N side of the m16n8k16 MMA and no tensor-core row is wasted:
//   S^T[16 keys x 8 heads] = K[16 x 128] Q^T        A = K rows from shared memory (ldmatrix),
//                                                   B = Q^T, 16 registers loaded once;
//   O^T[128 dims x 8 heads] += V^T[128 x 16] P^T    A = V^T via ldmatrix.trans,
//                                                   B = P^T, the S^T accumulators transposed
//                                                       in registers with movmatrix.
// Thread (g = lane / 4, t = lane % 4) owns heads 2t, 2t+1: scores of keys g and g+8, and
// output dims 16j+g, 16j+g+8.  Running max and sum are kept in the log2 domain; the sum is
// a per-thread partial (its keys only) until the end; the output accumulators are rescaled
// only when some head's running max moved.
//
// Each warp streams its own 16-key blocks (blocks warp, warp+4, ...) through a private ring of
// STAGES shared-memory stages filled with cp.async.  16-byte chunk c of row r is stored at chunk
// c ^ (r & 7), which makes every ldmatrix (8 rows x 16 bytes, rows 256 bytes apart)
// bank-conflict free.  STAGES = 3: two blocks in flight while a third is consumed, two CTAs per
// SM; STAGES = 2: one in flight, three CTAs per SM (more CTAs to cover each other's start-up
// and wind-down).
//
// Nothing on the way into the main loop waits for the whole CTA: each warp looks only at the
// mask entries of its own blocks (ballots into a register bit set: which blocks have an
// unmasked key and need to be fetched at all), and reads the two mask values a lane needs per
// block straight from global memory (L1 hits after the scan).  The four warps meet once, at
// the end, to merge their partial results through the shared memory their rings occupied.
template <typename T, int STAGES>
__global__ void __launch_bounds__(128, STAGES == 2 ? 3 : 2) attn_decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t dsm[];
  __shared__ float s_m[4][8], s_l[4][8];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hk = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t s_begin = static_cast<int64_t>(split) * p.split_len;
  const int64_t s_end = min(p.S, s_begin + p.split_len);
  const int n_keys = static_cast<int>(s_end - s_begin);
  const int nblk = (n_keys + 15) / 16;

  ATTN_STAMP(0);
  pdl_trigger();
  pdl_wait();   // q, the new cache rows and the mask come from the kernels before this one
  ATTN_STAMP(1);

  // ---- per-lane addressing -------------------------------------------------------------
  // cp.async: lane copies chunk (lane & 15) of rows 2i + (lane >> 4), i = 0..7
  const int hi = lane >> 4, ch = lane & 15;
  const uint32_t cp_off = hi * 256 + ((ch ^ hi) << 4);   // chunk ^ (row & 7) = (ch ^ hi) ^ (2i & 7)
  const T* k_lane = static_cast<const T*>(p.k) + b * p.kv_bs + hk * p.kv_hs + (s_begin + hi) * HD + ch * 8;
  const T* v_lane = static_cast<const T*>(p.v) + b * p.kv_bs + hk * p.kv_hs + (s_begin + hi) * HD + ch * 8;
  // ldmatrix: lane supplies one row address of 8x8 matrix (lane >> 3)
  const int mi = lane >> 3, mr = lane & 7;
  const uint32_t k_off = (8 * (mi & 1) + mr) * 256 + (((mi >> 1) ^ mr) << 4);   // ^ (ks << 5) selects dims 16ks..16ks+15
  const uint32_t v_off = (8 * (mi >> 1) + mr) * 256 + (((mi & 1) ^ mr) << 4);   // ^ (j << 5) selects dims 16j..16j+15
  const uint32_t ring = smem_u32(dsm) + warp * (STAGES * DEC_STAGE_BYTES);

  // copy block `blk` (16 keys x 256 B of K and of V) into ring stage `st`
  auto issue = [&](int blk, int st) {
    const uint32_t sk = ring + st * DEC_STAGE_BYTES + cp_off;
    const T* ks = k_lane + static_cast<int64_t>(blk) * 16 * HD;
    const T* vs = v_lane + static_cast<int64_t>(blk) * 16 * HD;
    const int rows_left = n_keys - blk * 16;
    if (rows_left >= 16) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t d = (sk ^ (((2 * i) & 7) << 4)) + i * 512;
        cp_async16(d, ks + i * 2 * HD, 16);
        cp_async16(d + 16 * HD * 2, vs + i * 2 * HD, 16);
      }
    } else {   // rows past the end are zero-filled (their probabilities are zero, but 0 * garbage must stay 0)
#pragma unroll 1
      for (int i = 0; i < 8; ++i) {
        const uint32_t d = (sk ^ (((2 * i) & 7) << 4)) + i * 512;
        const bool ok = 2 * i + hi < rows_left;
        cp_async16(d, ok ? ks + i * 2 * HD : k_lane, ok ? 16 : 0);
        cp_async16(d + 16 * HD * 2, ok ? vs + i * 2 * HD : v_lane, ok ? 16 : 0);
      }
    }
  };

  // Ask for a block's K and V rows (two contiguous 4 KB runs) to be brought into L2.  The ring
  // keeps at most one or two blocks per warp in flight (shared memory is the limit); requests
  // into L2 cost no shared memory, so the DRAM latency is paid there and the ring copies that
  // follow find their lines in L2.
  const T* k_blk0 = static_cast<const T*>(p.k) + b * p.kv_bs + hk * p.kv_hs + s_begin * HD;
  const T* v_blk0 = static_cast<const T*>(p.v) + b * p.kv_bs + hk * p.kv_hs + s_begin * HD;
  auto l2_prefetch = [&](int blk) {
    if (lane == 0 && blk < nblk) {
      const int rows = min(16, n_keys - blk * 16);
      const uint32_t bytes = static_cast<uint32_t>(rows) * HD * 2;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(k_blk0 + static_cast<int64_t>(blk) * 16 * HD), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(v_blk0 + static_cast<int64_t>(blk) * 16 * HD), "r"(bytes) : "memory");
    }
  };

  // The first blocks of every warp are fetched before the mask has been looked at (they are
  // almost always needed): the mask scan and the query loads hide behind these copies.
  int cur = warp < nblk ? warp : -1, nxt = -1;
  if (cur >= 0) issue(cur, 0);
  cp_async_commit();
  if (STAGES > 2) {
    nxt = warp + 4 < nblk ? warp + 4 : -1;
    if (nxt >= 0) issue(nxt, 1);
    cp_async_commit();
  }
  for (int dd = 0; dd < p.l2_ahead; ++dd) l2_prefetch(warp + 4 * (STAGES - 1 + dd));

  // ---- which of this warp's blocks have an unmasked key: bit j <-> block warp + 4j ----
  const char* mask_row = p.mask ? static_cast<const char*>(p.mask) : nullptr;
  const int64_t mask_base = b * p.mask_bs + s_begin;
  uint32_t vbits = 0;
#pragma unroll
  for (int i = 0; i < DEC_MAX_SPLIT / 128; ++i) {
    const int idx = i * 32 + lane, blk = warp + 4 * (idx >> 4), key = blk * 16 + (idx & 15);
    float mv = -INFINITY;
    if (key < n_keys) mv = mask_row ? load_as_f32(mask_row, mask_base + key, p.mask_dtype) : 0.f;
    const uint32_t bal = __ballot_sync(0xffffffffu, mv > MASKED);
    vbits |= ((bal & 0xffffu) ? 1u : 0u) << (2 * i) | ((bal >> 16) ? 1u : 0u) << (2 * i + 1);
  }
  auto is_valid = [&](int blk) { return ((vbits >> ((blk - warp) >> 2)) & 1u) != 0u; };
  auto next_valid = [&](int blk) {  // first valid block of this warp at or after blk (stride 4)
    while (blk < nblk && !is_valid(blk)) blk += 4;
    return blk;
  };

  // Q^T fragments: head g, dims 16ks + 2t, +1 and 16ks + 2t + 8, +9
  uint32_t qf[8][2];
  {
    const T* qr = static_cast<const T*>(p.q) + b * p.q_bs + (static_cast<int64_t>(hk) * p.G + g) * HD + 2 * t;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qf[ks][0] = g < p.G ? *reinterpret_cast<const uint32_t*>(qr + 16 * ks) : 0u;
      qf[ks][1] = g < p.G ? *reinterpret_cast<const uint32_t*>(qr + 16 * ks + 8) : 0u;
    }
  }
  ATTN_STAMP(2);

  float o[8][4];   // [dim tile j][dims 16j+g (0,1) / 16j+g+8 (2,3)  x  heads 2t (0,2) / 2t+1 (1,3)]
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float sl = p.scale * LOG2E;

  // additive mask (log2 domain) of key `key` of this split for this lane's two score rows
  auto mask_of = [&](int key) {
    if (key >= n_keys) return -INFINITY;
    return mask_row ? load_as_f32(mask_row, mask_base + key, p.mask_dtype) * LOG2E : 0.f;
  };

  int fetch = next_valid(warp + (STAGES > 2 ? 8 : 4));   // next block to copy
  int st_fetch = STAGES > 2 ? 2 : 1, st_use = 0;
  while (cur >= 0) {
    int fetched = -1;
    if (STAGES > 2) {
      cp_async_wait<1>();
      __syncwarp();   // every lane's copies for this stage have landed; the stage consumed last time is free
      if (fetch < nblk) {
        issue(fetch, st_fetch);
        fetched = fetch;
        const int pb = fetch + 4 * p.l2_ahead;
        if (p.l2_ahead && pb < nblk && is_valid(pb)) l2_prefetch(pb);
        fetch = next_valid(fetch + 4);
      }
      cp_async_commit();
      st_fetch = (st_fetch + 1) % STAGES;
    } else {
      __syncwarp();   // every lane has finished with the stage consumed last time
      if (fetch < nblk) {
        issue(fetch, st_fetch);
        fetched = fetch;
        const int pb = fetch + 4 * p.l2_ahead;
        if (p.l2_ahead && pb < nblk && is_valid(pb)) l2_prefetch(pb);
        fetch = next_valid(fetch + 4);
      }
      cp_async_commit();
      st_fetch ^= 1;
      cp_async_wait<1>();
      __syncwarp();
    }

    if (is_valid(cur)) {
      const uint32_t sk = ring + st_use * DEC_STAGE_BYTES, sv = sk + 16 * HD * 2;
      const float mk0 = mask_of(cur * 16 + g), mk1 = mask_of(cur * 16 + g + 8);
      // ---- S^T = K Q^T (two accumulators halve the dependent chain) ----
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ks += 2) {
        uint32_t a0[4], a1[4];
        ldmatrix_x4(a0, sk + (k_off ^ (ks << 5)));
        ldmatrix_x4(a1, sk + (k_off ^ ((ks + 1) << 5)));
        MmaType<T>::mma(sa, a0, qf[ks]);
        MmaType<T>::mma(sb, a1, qf[ks + 1]);
      }
      const float v0 = fmaf(sa[0] + sb[0], sl, mk0), v1 = fmaf(sa[1] + sb[1], sl, mk0);   // key g:   heads 2t, 2t+1
      const float v2 = fmaf(sa[2] + sb[2], sl, mk1), v3 = fmaf(sa[3] + sb[3], sl, mk1);   // key g+8: heads 2t, 2t+1
      // ---- online softmax over the 16 keys (lanes that differ in g) ----
      float mx0 = fmaxf(v0, v2), mx1 = fmaxf(v1, v3);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      if (__any_sync(0xffffffffu, mn0 > m0 || mn1 > m1)) {
        const float c0 = ex2_approx(m0 - (mn0 == -INFINITY ? 0.f : mn0)), c1 = ex2_approx(m1 - (mn1 == -INFINITY ? 0.f : mn1));
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j][0] *= c0; o[j][1] *= c1; o[j][2] *= c0; o[j][3] *= c1; }
        l0 *= c0; l1 *= c1;
        m0 = mn0; m1 = mn1;
      }
      const float u0 = m0 == -INFINITY ? 0.f : m0, u1 = m1 == -INFINITY ? 0.f : m1;
      const float p0 = ex2_approx(v0 - u0), p1 = ex2_approx(v1 - u1), p2 = ex2_approx(v2 - u0), p3 = ex2_approx(v3 - u1);
      l0 += p0 + p2;
      l1 += p1 + p3;
      // ---- O^T += V^T P^T ----
      const uint32_t pb[2] = {movmatrix_trans(pack2<T>(p0, p1)), movmatrix_trans(pack2<T>(p2, p3))};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, sv + (v_off ^ (j << 5)));
        MmaType<T>::mma(o[j], a, pb);
      }
    }
    st_use = (st_use + 1) % STAGES;
    if (STAGES > 2) { cur = nxt; nxt = fetched; }
    else cur = fetched;
  }
  cp_async_wait<0>();
  ATTN_STAMP(3);

  // ---- merge the four warps: every warp parks its accumulators (and running max / sum) in the
  // shared memory its own ring occupied; after one barrier thread d adds up dim d of every head ----
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, off);
    l1 += __shfl_xor_sync(0xffffffffu, l1, off);
  }
  __syncwarp();   // all lanes are done reading the ring
  float* slab = reinterpret_cast<float*>(dsm + warp * (STAGES * DEC_STAGE_BYTES));   // [8 heads][DEC_ACC_PITCH]
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    slab[(2 * t) * DEC_ACC_PITCH + 16 * j + g] = o[j][0];
    slab[(2 * t + 1) * DEC_ACC_PITCH + 16 * j + g] = o[j][1];
    slab[(2 * t) * DEC_ACC_PITCH + 16 * j + g + 8] = o[j][2];
    slab[(2 * t + 1) * DEC_ACC_PITCH + 16 * j + g + 8] = o[j][3];
  }
  if (g == 0) { s_m[warp][2 * t] = m0; s_m[warp][2 * t + 1] = m1; s_l[warp][2 * t] = l0; s_l[warp][2 * t + 1] = l1; }
  __syncthreads();
  const int64_t pidx = ((b * p.Hkv + hk) * p.splits + split) * p.G;
  const int d = threadIdx.x;
#pragma unroll 1
  for (int h = 0; h < p.G; ++h) {
    const float ma = fmaxf(fmaxf(s_m[0][h], s_m[1][h]), fmaxf(s_m[2][h], s_m[3][h]));
    const float mu = ma == -INFINITY ? 0.f : ma;
    float acc = 0.f, lr = 0.f;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      const float f = ex2_approx(s_m[wi][h] - mu);
      acc += reinterpret_cast<const float*>(dsm + wi * (STAGES * DEC_STAGE_BYTES))[h * DEC_ACC_PITCH + d] * f;
      lr += s_l[wi][h] * f;
    }
    p.part_acc[(pidx + h) * HD + d] = acc;
    if (d == 0) {
      p.part_ml[(pidx + h) * 2] = ma;      // log2 domain
      p.part_ml[(pidx + h) * 2 + 1] = lr;
    }
  }
  ATTN_STAMP(4);
}

#ifdef B200NN_TC5_TRACE
}  // namespace b200
extern "C" int b200_debug_attn_trace(unsigned long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, b200::g_attn_trace, sizeof(unsigned long long) * b200::ATR_CTAS * b200::ATR_N) == cudaSuccess ? 0 : -3;
}
namespace b200 {
#endif

// grid = B*Hq blocks of 128 threads (one per head dim)
template <typename T>
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                                T* __restrict__ out, int Hq, int Hkv, int G, int splits) {
  const int64_t bh = blockIdx.x, b = bh / Hq;
  const int h = static_cast<int>(bh % Hq), hk = h / G, r = h % G;
  pdl_wait();
  pdl_trigger();
  const int64_t base = (b * Hkv + hk) * splits;
  float m_all = -INFINITY;
  for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, part_ml[((base + s) * G + r) * 2]);
  const float m_use = m_all == -INFINITY ? 0.f : m_all;
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const int64_t i = (base + s) * G + r;
    const float f = ex2_approx(part_ml[i * 2] - m_use);   // maxima are stored in the log2 domain
    l += part_ml[i * 2 + 1] * f;
    acc += part_acc[i * HD + threadIdx.x] * f;
  }
  out[bh * HD + threadIdx.x] = from_f32<T>(l > 0.f ? acc / l : 0.f);
}

// ===========================================================================
// Prefill: grid = (ceil(T/64), Hq, B), 4 warps x 16 query rows, all keys streamed.
// ===========================================================================
struct PrefillParams {
  const void* q; const void* k; const void* v; const void* mask; void* out;
  int64_t B, T, S;
  int Hq, Hkv;
  int64_t qs[3], ks[3], vs[3];
  int64_t mask_b, mask_t;
  float scale;
  int mask_dtype;
};

template <typename T>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const __grid_constant__ PrefillParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int h = blockIdx.y, hk = h / (p.Hq / p.Hkv);
  const int64_t b = blockIdx.z;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * 64 + warp * 16;
  if (row0 >= p.T) return;
  const int64_t r_lo = row0 + g, r_hi = row0 + g + 8;
  const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  AttnWarp<T> w;
  w.init();
  w.load_q(r_lo < p.T ? qb + r_lo * p.qs[2] : nullptr, r_hi < p.T ? qb + r_hi * p.qs[2] : nullptr, t);
  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
  const int64_t mrow[2] = {b * p.mask_b + min(r_lo, p.T - 1) * p.mask_t, b * p.mask_b + min(r_hi, p.T - 1) * p.mask_t};

  for (int64_t kb = 0; kb < p.S; kb += 16) {
    float add[2][4];
    bool any = !p.mask;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t key = kb + 8 * j + 2 * t + (e & 1);
        float mv = 0.f;
        if (p.mask && key < p.S) {
          mv = load_as_f32(p.mask, mrow[e >> 1] + key, p.mask_dtype);
          any = any || mv > MASKED;
        }
        add[j][e] = mv;
      }
    if (!__any_sync(0xffffffffu, any)) continue;  // whole 16x16 tile masked out
    w.step(kbase, vbase, p.ks[2], p.vs[2], kb, p.S, p.scale, add, g, t);
  }

  // out[b][row][h][:]
  T* ob = static_cast<T*>(p.out) + (b * p.T * p.Hq + h) * HD;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int64_t row = hh ? r_hi : r_lo;
    if (row >= p.T) continue;
    const float inv = w.l[hh] > 0.f ? 1.f / w.l[hh] : 0.f;
    T* orow = ob + row * p.Hq * HD;
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float vals[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[j] = w.o[a][j][2 * hh + e] * inv;
        *reinterpret_cast<uint4*>(orow + 64 * a + 8 * (2 * t + e)) = pack8<T>(vals);
      }
  }
}

struct DecodePlan { int split_len; int splits; };

static DecodePlan plan_decode(int64_t B, int Hkv, int64_t S) {
  const int64_t want = 2 * 148;  // fixed so that the workspace size does not depend on the device
  if (B * Hkv * ceil_div(S, 512) >= 4 * 148) {  // plenty of work: longer splits amortise the per-split prologue
    DecodePlan big;
    big.split_len = 512;
    big.splits = static_cast<int>(ceil_div(S, 512));
    return big;
  }
  int len = 256;
  while (len > 64 && B * Hkv * ceil_div(S, len) < want) len >>= 1;
  DecodePlan d;
  d.split_len = len;
  d.splits = static_cast<int>(ceil_div(S, len));
  return d;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_attn_decode_workspace_bytes(int64_t B, int Hq, int Hkv, int64_t S, int D) {
  if (B <= 0 || Hkv <= 0 || Hq <= 0 || S <= 0) return 0;
  const DecodePlan d = plan_decode(B, Hkv, S);
  const int G = Hq / Hkv;
  return B * Hkv * d.splits * G * (static_cast<int64_t>(D) + 2) * 4;
}

extern "C" int b200_attn_decode(const void* q, const void* k, const void* v, const void* mask, void* out, int64_t B, int Hq,
                                int Hkv, int64_t S, int D, int64_t q_batch_stride, int64_t kv_batch_stride,
                                int64_t kv_head_stride, int64_t mask_batch_stride, float scale, int dtype, void* workspace,
                                int64_t workspace_bytes, void* stream) {
  B200_CHECK_ARG(q && k && v && out && B >= 0 && Hq > 0 && Hkv > 0 && S > 0, "b200_attn_decode: bad arguments");
  B200_CHECK_ARG(D == HD, "b200_attn_decode: head_dim %d not supported (128 only)", D);
  B200_CHECK_ARG(Hq % Hkv == 0 && Hq / Hkv <= 8, "b200_attn_decode: query heads per KV head must divide and be <= 8");
  B200_CHECK_ARG(B <= 65535 && Hkv <= 65535, "b200_attn_decode: batch or head count too large");
  if (B == 0) return B200_OK;
  if (!(aligned16(q) && aligned16(k) && aligned16(v) && q_batch_stride % 8 == 0 && kv_batch_stride % 8 == 0 && kv_head_stride % 8 == 0))
    B200_FAIL(B200_EALIGN, "b200_attn_decode: operands must be 16-byte aligned with strides multiple of 8");
  const DecodePlan d = plan_decode(B, Hkv, S);
  const int64_t need = b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D);
  if (!workspace || workspace_bytes < need)
    B200_FAIL(B200_EINVAL, "b200_attn_decode: workspace of %lld bytes required (got %lld)", (long long)need, (long long)workspace_bytes);
  DecodeParams p;
  p.q = q; p.k = k; p.v = v; p.mask = mask;
  p.G = Hq / Hkv;
  p.part_acc = static_cast<float*>(workspace);
  p.part_ml = p.part_acc + B * Hkv * d.splits * p.G * HD;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.q_bs = q_batch_stride; p.kv_bs = kv_batch_stride; p.kv_hs = kv_head_stride; p.mask_bs = mask_batch_stride;
  p.split_len = d.split_len; p.splits = d.splits; p.scale = scale; p.mask_dtype = dtype;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>(d.splits), static_cast<unsigned>(Hkv), static_cast<unsigned>(B));
  static int stages = 0, l2_ahead = 0;   // ring depth per warp: 2 (three CTAs per SM) or 3 (two CTAs per SM)
  if (stages == 0) {
    const char* e = getenv("B200NN_ATTN_STAGES");
    stages = (e && e[0] == '3') ? 3 : 2;
    const char* a = getenv("B200NN_ATTN_L2_AHEAD");
    l2_ahead = a && a[0] ? atoi(a) : 0;   // measured: requests into L2 ahead of the ring only slow the kernel down
    if (l2_ahead < 0 || l2_ahead > 8) l2_ahead = 0;
  }
  p.l2_ahead = l2_ahead;
  B200_DISPATCH_HALF(dtype, T, {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<T, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 3 * DEC_STAGE_BYTES);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * DEC_STAGE_BYTES);
      if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "attn_decode_kernel attribute: %s", cudaGetErrorString(e));
      configured = true;
    }
    if (stages == 2) launch_pdl(attn_decode_kernel<T, 2>, grid, dim3(128), 4 * 2 * DEC_STAGE_BYTES, st, p);
    else launch_pdl(attn_decode_kernel<T, 3>, grid, dim3(128), 4 * 3 * DEC_STAGE_BYTES, st, p);
    launch_pdl(attn_decode_merge_kernel<T>, dim3(static_cast<unsigned>(B * Hq)), dim3(128), 0, st, static_cast<const float*>(p.part_acc),
               static_cast<const float*>(p.part_ml), static_cast<T*>(out), Hq, Hkv, p.G, d.splits);
  });
  B200_CHECK_LAUNCH("attn_decode_kernel");
  return B200_OK;
}

extern "C" int b200_attn_prefill(const void* q, const void* k, const void* v, const void* mask, void* out, int64_t B, int Hq,
                                 int Hkv, int64_t T, int64_t S, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                                 const int64_t v_strides[3], int64_t mask_b, int64_t mask_t, float scale, int dtype,
                                 void* stream) {
  B200_CHECK_ARG(q && k && v && out && B >= 0 && Hq > 0 && Hkv > 0 && T >= 0 && S > 0 && q_strides && k_strides && v_strides,
                 "b200_attn_prefill: bad arguments");
  B200_CHECK_ARG(D == HD, "b200_attn_prefill: head_dim %d not supported (128 only)", D);
  B200_CHECK_ARG(Hq % Hkv == 0, "b200_attn_prefill: Hq must be a multiple of Hkv");
  B200_CHECK_ARG(B <= 65535 && Hq <= 65535, "b200_attn_prefill: batch or head count too large");
  if (B == 0 || T == 0) return B200_OK;
  bool ok = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out);
  for (int i = 0; i < 3; ++i) ok = ok && q_strides[i] % 8 == 0 && k_strides[i] % 8 == 0 && v_strides[i] % 8 == 0;
  if (!ok) B200_FAIL(B200_EALIGN, "b200_attn_prefill: operands must be 16-byte aligned with strides multiple of 8");
  PrefillParams p;
  p.q = q; p.k = k; p.v = v; p.mask = mask; p.out = out; p.B = B; p.T = T; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  for (int i = 0; i < 3; ++i) { p.qs[i] = q_strides[i]; p.ks[i] = k_strides[i]; p.vs[i] = v_strides[i]; }
  p.mask_b = mask_b; p.mask_t = mask_t; p.scale = scale; p.mask_dtype = dtype;
  dim3 grid(static_cast<unsigned>(ceil_div(T, 64)), static_cast<unsigned>(Hq), static_cast<unsigned>(B));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_HALF(dtype, T_, { attn_prefill_kernel<T_><<<grid, 128, 0, st>>>(p); });
  B200_CHECK_LAUNCH("attn_prefill_kernel");
  return B200_OK;
}
