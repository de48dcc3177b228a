// Fused attention for head_dim 128 on the warp-level tensor-core path (mma.sync m16n8k16,
// fp32 accumulation, online softmax in the log2 domain).  K and V rows are staged in shared
// memory with cp.async under an XOR swizzle and read with ldmatrix / ldmatrix.trans; the
// probabilities are rounded to the activation dtype for the second MMA, as the unfused graph
// rounds them.  Two kernels: prefill (64 query rows per CTA) and split-KV decode (one query
// token, the query heads of a KV group on the N side of the MMA).
#include "attention.cuh"
#include "gemm_tc5.cuh"
#include "mma.cuh"
#include "tc5.cuh"

#include <stdlib.h>

namespace b200 {

constexpr int HD = 128;          // head dim
constexpr float LOG2E = 1.4426950408889634f;
constexpr float MASKED = -1e30f; // additive mask values at or below this are "masked out"

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
  void* out;      // cluster-merge mode: final output [B][Hq][HD] in the activation dtype
};


constexpr int DEC_STAGE_BYTES = 2 * 16 * HD * 2;  // 16 keys of K and of V
constexpr int DEC_MAX_SPLIT = 2048;            // keys per split (mask values of a split are staged in shared memory)
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
//
// CM = true ("cluster merge"): the splits of one (sequence, KV head) form a thread-block cluster
// along x.  Instead of writing its partial result to global memory for a second kernel, every
// CTA stores head h's partial (accumulator, max, sum) into the receive buffer of cluster rank h
// (distributed shared memory); after one cluster barrier every rank combines the splits of the
// heads it owns (head h belongs to rank h % splits) and writes the final output.  2 <= splits <= 16.
template <typename T, int STAGES, bool CM>
__global__ void __launch_bounds__(128, STAGES == 2 ? 3 : 2) attn_decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t dsm[];
  __shared__ float s_m[4][8], s_l[4][8];
  // partials of the heads this CTA owns (head h belongs to cluster rank h % splits), by [owned head * splits + source rank]
  __shared__ __align__(16) float recv_acc[CM ? 16 : 1][HD];
  __shared__ float recv_ml[CM ? 16 : 1][2];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hk = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int64_t s_begin = static_cast<int64_t>(split) * p.split_len;
  const int64_t s_end = min(p.S, s_begin + p.split_len);
  const int n_keys = static_cast<int>(s_end - s_begin);
  const int nblk = (n_keys + 15) / 16;

  pdl_trigger();
  if (CM) tc5::cluster_sync();   // every CTA of the cluster runs before anyone writes into a peer (overlaps the predecessor)
  pdl_wait();   // q, the new cache rows and the mask come from the kernels before this one

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

  // ---- which of this warp's blocks have an unmasked key: bit j <-> block warp + 4j ----
  const char* mask_row = p.mask ? static_cast<const char*>(p.mask) : nullptr;
  const int64_t mask_base = b * p.mask_bs + s_begin;
  uint32_t vbits = 0;
#pragma unroll
  for (int i = 0; i < DEC_MAX_SPLIT / 128; ++i) {
    if (i * 128 >= n_keys) break;   // (uniform) every pass covers 128 keys of the split
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
        fetch = next_valid(fetch + 4);
      }
      cp_async_commit();
      st_fetch = (st_fetch + 1) % STAGES;
    } else {
      __syncwarp();   // every lane has finished with the stage consumed last time
      if (fetch < nblk) {
        issue(fetch, st_fetch);
        fetched = fetch;
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
    if (CM) {   // partial of head h -> the receive buffer of the cluster rank that owns the head
      const int owner = h % p.splits, slot = (h / p.splits) * p.splits + split;
      const uint32_t dst = tc5::map_to_rank(smem_u32(&recv_acc[slot][d]), owner);
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(acc) : "memory");
      if (d == 0) {
        const uint32_t dml = tc5::map_to_rank(smem_u32(&recv_ml[slot][0]), owner);
        asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(dml), "f"(ma), "f"(lr) : "memory");
      }
    } else {
      p.part_acc[(pidx + h) * HD + d] = acc;
      if (d == 0) {
        p.part_ml[(pidx + h) * 2] = ma;      // log2 domain
        p.part_ml[(pidx + h) * 2 + 1] = lr;
      }
    }
  }
  if (CM) {
    tc5::cluster_sync();   // all partials have landed; nobody touches a peer's memory afterwards
    for (int h = split; h < p.G; h += p.splits) {   // the heads this CTA owns
      const int base = (h / p.splits) * p.splits;
      float m_all = -INFINITY;
      for (int r = 0; r < p.splits; ++r) m_all = fmaxf(m_all, recv_ml[base + r][0]);
      const float m_use = m_all == -INFINITY ? 0.f : m_all;
      float acc = 0.f, l = 0.f;
      for (int r = 0; r < p.splits; ++r) {
        const float f = ex2_approx(recv_ml[base + r][0] - m_use);
        l += recv_ml[base + r][1] * f;
        acc += recv_acc[base + r][d] * f;
      }
      static_cast<T*>(p.out)[((b * p.Hq) + static_cast<int64_t>(hk) * p.G + h) * HD + d] = from_f32<T>(l > 0.f ? acc / l : 0.f);
    }
  }
}

// grid = B*Hq blocks of 128 threads (one per head dim)
template <typename T>
__global__ void __launch_bounds__(128) attn_decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                                T* __restrict__ out, int Hq, int Hkv, int G, int splits) {
  const int64_t bh = blockIdx.x, b = bh / Hq;
  const int h = static_cast<int>(bh % Hq), hk = h / G, r = h % G;
  pdl_wait();
  pdl_trigger();
  const int64_t base = (b * Hkv + hk) * splits;
  // (the loads of different splits are independent: unrolled, they overlap instead of queueing up one
  // L2 round trip each - 256 splits of a 32768-row cache took 20 us that way)
  float m_all = -INFINITY;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, __ldg(&part_ml[((base + s) * G + r) * 2]));
  const float m_use = m_all == -INFINITY ? 0.f : m_all;
  float acc = 0.f, l = 0.f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) {
    const int64_t i = (base + s) * G + r;
    const float f = ex2_approx(__ldg(&part_ml[i * 2]) - m_use);   // maxima are stored in the log2 domain
    l += __ldg(&part_ml[i * 2 + 1]) * f;
    acc += __ldg(&part_acc[i * HD + threadIdx.x]) * f;
  }
  out[bh * HD + threadIdx.x] = from_f32<T>(l > 0.f ? acc / l : 0.f);
}

// ===========================================================================
// Prefill: grid = (ceil(T/64), Hq, B), 4 warps x 16 query rows, all keys streamed.
// ===========================================================================

constexpr int PF_BK = 64;                              // keys per shared-memory tile
constexpr int PF_KV_BYTES = 2 * PF_BK * HD * 2;        // K tile + V tile
constexpr int PF_STAGE_BYTES = PF_KV_BYTES + 64 * PF_BK * 2;   // + the 64 x 64 tile of a 16-bit mask
constexpr int PF_SMEM = 2 * PF_STAGE_BYTES;            // double buffer

// One CTA = 64 query rows of one head (16 per warp).  K and V tiles of 64 keys are copied into
// shared memory once per CTA with cp.async (double-buffered; chunk c of row r at c ^ (r & 7)) and
// read by all four warps with ldmatrix: K rows as the B operand of S = Q K^T, V rows through
// ldmatrix.trans as the B operand of O += P V; P goes from the score accumulators straight
// into A fragments.  Online softmax in the log2 domain, lazy rescale, 64-key tiles whose mask
// entries are all <= -1e30 for a warp's 16 rows are skipped by that warp.
template <typename T>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const __grid_constant__ PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t psm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int h = blockIdx.y, hk = h / (p.Hq / p.Hkv);
  const int64_t b = blockIdx.z;
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * 64 + warp * 16;
  const int64_t r_lo = row0 + g, r_hi = row0 + g + 8;
  const bool warp_live = row0 < p.T;   // a warp past the end still copies tiles and meets the barriers

  // Q as A fragments: slice ks covers dims 16ks..16ks+15
  uint32_t qf[8][4];
  {
    const T* qb = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + 2 * t;
    const T* q0 = qb + r_lo * p.qs[2];
    const T* q1 = qb + r_hi * p.qs[2];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qf[ks][0] = r_lo < p.T ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks) : 0u;
      qf[ks][1] = r_hi < p.T ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks) : 0u;
      qf[ks][2] = r_lo < p.T ? *reinterpret_cast<const uint32_t*>(q0 + 16 * ks + 8) : 0u;
      qf[ks][3] = r_hi < p.T ? *reinterpret_cast<const uint32_t*>(q1 + 16 * ks + 8) : 0u;
    }
  }
  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
  const uint32_t sm0 = smem_u32(psm);
  // A mask in the activation dtype with 16-byte-aligned rows travels with the K/V tiles: its
  // 64 x 64 tile is copied with cp.async (chunk c of row r at c ^ (r & 7)).  Reading the mask
  // straight from global memory, two bytes at a time, cost three times the rest of the kernel.
  const bool mask_staged = p.mask != nullptr && p.mask_staged;
  const T* mask_t = static_cast<const T*>(p.mask);

  auto issue = [&](int64_t kb, int st) {   // tile of keys kb..kb+63 -> stage st
    const uint32_t sk = sm0 + st * PF_STAGE_BYTES, sv = sk + PF_BK * HD * 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = i * 128 + threadIdx.x, row = idx >> 4, ch = idx & 15;
      const bool ok = kb + row < p.S;
      const uint32_t off = row * 256 + ((ch ^ (row & 7)) << 4);
      cp_async16(sk + off, ok ? static_cast<const void*>(kbase + (kb + row) * p.ks[2] + ch * 8) : static_cast<const void*>(kbase), ok ? 16 : 0);
      cp_async16(sv + off, ok ? static_cast<const void*>(vbase + (kb + row) * p.vs[2] + ch * 8) : static_cast<const void*>(vbase), ok ? 16 : 0);
    }
    if (mask_staged) {
      const uint32_t smk = sk + PF_KV_BYTES;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = i * 128 + threadIdx.x, row = idx >> 3, ch = idx & 7;   // 64 rows x 8 chunks of 8 keys
        const int64_t qrow = min(static_cast<int64_t>(blockIdx.x) * 64 + row, p.T - 1);
        const bool ok = kb + ch * 8 < p.S;   // S is a multiple of 8 here; chunks past the end are never read as valid keys
        cp_async16(smk + row * 128 + ((ch ^ (row & 7)) << 4),
                   ok ? static_cast<const void*>(mask_t + b * p.mask_b + qrow * p.mask_t + kb + ch * 8) : static_cast<const void*>(mask_t), ok ? 16 : 0);
      }
    }
  };

  // ldmatrix lane addressing inside a tile
  const int mi = lane >> 3, mr = lane & 7;
  const uint32_t k_off = ((mi >> 1) * 8 + mr) * 256 + (((mi & 1) ^ mr) << 4);   // + 16-key group * 4096, ^ (dim slice << 5)
  const uint32_t v_off = ((mi & 1) * 8 + mr) * 256 + (((mi >> 1) ^ mr) << 4);   // + 16-key group * 4096, ^ (dim pair << 5)

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl = p.scale * LOG2E;
  const int64_t mrow[2] = {b * p.mask_b + min(r_lo, p.T - 1) * p.mask_t, b * p.mask_b + min(r_hi, p.T - 1) * p.mask_t};

  const int n_tiles = static_cast<int>((p.S + PF_BK - 1) / PF_BK);
  issue(0, 0);
  cp_async_commit();
  for (int j = 0; j < n_tiles; ++j) {
    const int64_t kb = static_cast<int64_t>(j) * PF_BK;
    if (j + 1 < n_tiles) issue(kb + PF_BK, (j + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();   // tile j has landed for every thread

    // ---- additive mask (log2 domain) for rows g, g+8 x keys 8nt + 2t, +1 ----
    float mk[8][4];
    bool any = false;
    if (mask_staged) {
      const uint32_t smk = sm0 + (j & 1) * PF_STAGE_BYTES + PF_KV_BYTES;
      const int rl = warp * 16 + g;   // tile rows rl and rl + 8 ((rl + 8) & 7 == rl & 7)
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        uint32_t w0, w1;
        const uint32_t off = ((nt ^ (rl & 7)) << 4) + 4 * t;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w0) : "r"(smk + rl * 128 + off));
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w1) : "r"(smk + (rl + 8) * 128 + off));
        unpack2<T>(w0, mk[nt][0], mk[nt][1]);
        unpack2<T>(w1, mk[nt][2], mk[nt][3]);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (kb + 8 * nt + 2 * t + (e & 1) >= p.S) mk[nt][e] = -INFINITY;
          any = any || mk[nt][e] > MASKED;
          mk[nt][e] *= LOG2E;
        }
    } else {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int64_t key = kb + 8 * nt + 2 * t + (e & 1);
          float mv = 0.f;
          if (key >= p.S) mv = -INFINITY;
          else if (p.mask) mv = load_as_f32(p.mask, mrow[e >> 1] + key, p.mask_dtype);
          any = any || mv > MASKED;
          mk[nt][e] = mv * LOG2E;
        }
    }
    if (warp_live && __any_sync(0xffffffffu, any)) {
      const uint32_t sk = sm0 + (j & 1) * PF_STAGE_BYTES, sv = sk + PF_BK * HD * 2;
      // ---- S = Q K^T ----
      float sc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t kf[4];
          ldmatrix_x4(kf, sk + np * 4096 + (k_off ^ (ks << 5)));
          const uint32_t b0[2] = {kf[0], kf[1]}, b1[2] = {kf[2], kf[3]};
          MmaType<T>::mma(sc[2 * np], qf[ks], b0);
          MmaType<T>::mma(sc[2 * np + 1], qf[ks], b1);
        }
      // ---- online softmax ----
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sc[nt][e] = fmaf(sc[nt][e], sl, mk[nt][e]);
          mx[e >> 1] = fmaxf(mx[e >> 1], sc[nt][e]);
        }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
        mx[hh] = fmaxf(mx[hh], m_run[hh]);
      }
      if (__any_sync(0xffffffffu, mx[0] > m_run[0] || mx[1] > m_run[1])) {
        const float c0 = ex2_approx(m_run[0] - (mx[0] == -INFINITY ? 0.f : mx[0])), c1 = ex2_approx(m_run[1] - (mx[1] == -INFINITY ? 0.f : mx[1]));
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) { o[jj][0] *= c0; o[jj][1] *= c0; o[jj][2] *= c1; o[jj][3] *= c1; }
        l_run[0] *= c0; l_run[1] *= c1;
        m_run[0] = mx[0]; m_run[1] = mx[1];
      }
      const float u0 = m_run[0] == -INFINITY ? 0.f : m_run[0], u1 = m_run[1] == -INFINITY ? 0.f : m_run[1];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        sc[nt][0] = ex2_approx(sc[nt][0] - u0); sc[nt][1] = ex2_approx(sc[nt][1] - u0);
        sc[nt][2] = ex2_approx(sc[nt][2] - u1); sc[nt][3] = ex2_approx(sc[nt][3] - u1);
        l_run[0] += sc[nt][0] + sc[nt][1];
        l_run[1] += sc[nt][2] + sc[nt][3];
      }
      // ---- O += P V ----
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t pa[4] = {pack2<T>(sc[2 * kk][0], sc[2 * kk][1]), pack2<T>(sc[2 * kk][2], sc[2 * kk][3]),
                                pack2<T>(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), pack2<T>(sc[2 * kk + 1][2], sc[2 * kk + 1][3])};
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, sv + kk * 4096 + (v_off ^ (dp << 5)));
          const uint32_t b0[2] = {vf[0], vf[1]}, b1[2] = {vf[2], vf[3]};
          MmaType<T>::mma(o[2 * dp], pa, b0);
          MmaType<T>::mma(o[2 * dp + 1], pa, b1);
        }
      }
    }
    __syncthreads();   // every warp is done with stage j & 1 before tile j + 2 is copied into it
  }
  cp_async_wait<0>();

  if (!warp_live) return;
  // row sums live as per-thread partials over the thread's key columns: finish them across the quad
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
  // out[b][row][h][:]
  T* ob = static_cast<T*>(p.out) + (b * p.T * p.Hq + h) * HD + 2 * t;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int64_t row = hh ? r_hi : r_lo;
    if (row >= p.T) continue;
    const float inv = l_run[hh] > 0.f ? 1.f / l_run[hh] : 0.f;
    T* orow = ob + row * p.Hq * HD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
      *reinterpret_cast<uint32_t*>(orow + 8 * nt) = pack2<T>(o[nt][2 * hh] * inv, o[nt][2 * hh + 1] * inv);
  }
}

struct DecodePlan { int split_len; int splits; bool cluster; };

static DecodePlan plan_decode(int64_t B, int Hkv, int64_t S, int G = 8, int resident16 = 0) {
  const int64_t want = 2 * 148;  // fixed so that the workspace size does not depend on the device
  // Caches of 512 .. 16384 rows: up to eight splits per (sequence, KV head), merged inside the kernel by a cluster
  // (measured faster than the two-kernel form at every batch size: B=8 14.7 vs 19.6 us, B=1 12.2 vs 13.4 us).
  if (S >= 8 * 64 && S <= 8 * DEC_MAX_SPLIT && G <= 8) {
    // Among the split counts min(G, 6)..8 take the one with the shortest estimated time: waves of
    // CTAs (three CTAs per SM are resident at a time) x keys per split.  Measured at B=64, S=4352:
    // 8 splits (2.3 waves of 544 keys) 55.2 us, 7 splits 59.1, 6 splits (1.7 waves of 736 keys) 52.2;
    // at B=32: 8 splits 34.2 us, 6 splits 28.6.  Fewer, longer splits lose again even when they fit
    // one wave (3 splits of 1456 keys: 54.7 us; 4 splits: 64.0): SMs left with two CTAs stream slower.
    DecodePlan c;
    c.cluster = false;
    int64_t best = 0;
    // Small batches, where eight splits per KV head leave SMs idle, use clusters of 16 (a non-portable size) as long
    // as all of them are resident at once (`resident16`, asked of the device): B=1 12.2 -> 8.0 us, B=8 13.1 -> 10.8,
    // B=10 12.0; with a second wave of clusters they lose (B=12: 20.4 us).
    const int n_hi = (resident16 > 0 && B * Hkv <= resident16) ? 16 : 8;
    for (int n = n_hi; n >= (G < 6 ? (G < 2 ? 2 : G) : 6); --n) {
      const int len = static_cast<int>(ceil_div(ceil_div(S, n), 16) * 16);
      if (len > DEC_MAX_SPLIT || ceil_div(S, len) != n) continue;
      const int64_t waves = ceil_div(B * Hkv * n, 3 * 148);
      const int64_t cost = waves * (len + 96);   // + 96 keys' worth of start-up and merge per wave
      if (!c.cluster || cost < best) {
        best = cost;
        c.split_len = len;
        c.splits = n;
        c.cluster = true;
      }
    }
    if (c.cluster) return c;
  }
  if (B * Hkv * ceil_div(S, 512) >= 4 * 148) {  // plenty of work: longer splits amortise the per-split prologue
    DecodePlan big;
    big.split_len = 512;
    big.splits = static_cast<int>(ceil_div(S, 512));
    big.cluster = false;
    return big;
  }
  int len = 256;
  while (len > 64 && B * Hkv * ceil_div(S, len) < want) len >>= 1;
  DecodePlan d;
  d.split_len = len;
  d.splits = static_cast<int>(ceil_div(S, len));
  d.cluster = false;
  return d;
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_attn_decode_workspace_bytes(int64_t B, int Hq, int Hkv, int64_t S, int D) {
  if (B <= 0 || Hkv <= 0 || Hq <= 0 || S <= 0) return 0;
  const int G = Hq / Hkv;
  const DecodePlan d = plan_decode(B, Hkv, S, G);
  if (d.cluster) return 0;   // the splits are merged inside the kernel through distributed shared memory
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
  // clusters of 16 CTAs are a non-portable size: how many the device keeps resident at once is asked once per device
  // (0 = not asked yet, -1 = not available)
  static PerDevice<int> resident16_on;
  int* resident16 = resident16_on.slot();
  if (!resident16) B200_FAIL(B200_ELAUNCH, "attn_decode_kernel: no current device");
  if (*resident16 == 0) {
    *resident16 = -1;
    int n16 = 0;
    bool ok16 = true;
    // (the attribute is per kernel instantiation: both activation types get it, whichever asks first)
    ok16 = cudaFuncSetAttribute(attn_decode_kernel<__nv_bfloat16, 2, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
           cudaFuncSetAttribute(attn_decode_kernel<__half, 2, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    B200_DISPATCH_HALF(dtype, T, {
      ok16 = ok16 && cudaFuncSetAttribute(attn_decode_kernel<T, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * DEC_STAGE_BYTES) == cudaSuccess;
      if (ok16) {
        cudaLaunchConfig_t qc = {};
        qc.gridDim = dim3(16, 1, 1);
        qc.blockDim = dim3(128);
        qc.dynamicSmemBytes = 4 * 2 * DEC_STAGE_BYTES;
        cudaLaunchAttribute ca;
        ca.id = cudaLaunchAttributeClusterDimension;
        ca.val.clusterDim.x = 16; ca.val.clusterDim.y = 1; ca.val.clusterDim.z = 1;
        qc.attrs = &ca;
        qc.numAttrs = 1;
        ok16 = cudaOccupancyMaxActiveClusters(&n16, attn_decode_kernel<T, 2, true>, &qc) == cudaSuccess && n16 >= 1;
      }
    });
    cudaGetLastError();
    if (ok16) *resident16 = n16;
  }
  const DecodePlan d = plan_decode(B, Hkv, S, Hq / Hkv, *resident16);
  const int64_t need = b200_attn_decode_workspace_bytes(B, Hq, Hkv, S, D);
  if (need > 0 && (!workspace || workspace_bytes < need))
    B200_FAIL(B200_EINVAL, "b200_attn_decode: workspace of %lld bytes required (got %lld)", (long long)need, (long long)workspace_bytes);
  DecodeParams p;
  p.q = q; p.k = k; p.v = v; p.mask = mask;
  p.G = Hq / Hkv;
  p.part_acc = static_cast<float*>(workspace);
  p.part_ml = p.part_acc + B * Hkv * d.splits * p.G * HD;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.q_bs = q_batch_stride; p.kv_bs = kv_batch_stride; p.kv_hs = kv_head_stride; p.mask_bs = mask_batch_stride;
  p.split_len = d.split_len; p.splits = d.splits; p.scale = scale; p.mask_dtype = dtype;
  p.out = out;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>(d.splits), static_cast<unsigned>(Hkv), static_cast<unsigned>(B));
  B200_DISPATCH_HALF(dtype, T, {
    static PerDevice<bool> configured_on;
    bool* configured = configured_on.slot();
    if (!configured) B200_FAIL(B200_ELAUNCH, "attn_decode_kernel: no current device");
    if (!*configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<T, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * DEC_STAGE_BYTES);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel<T, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * DEC_STAGE_BYTES);
      if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "attn_decode_kernel attribute: %s", cudaGetErrorString(e));
      *configured = true;
    }
    if (d.cluster) {   // one kernel: the splits of a (sequence, KV head) are a cluster along x and merge in shared memory
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(128);
      cfg.dynamicSmemBytes = 4 * 2 * DEC_STAGE_BYTES;
      cfg.stream = st;
      cudaLaunchAttribute attrs[2];
      int n_attrs = 0;
      attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
      attrs[n_attrs].val.clusterDim.x = static_cast<unsigned>(d.splits);
      attrs[n_attrs].val.clusterDim.y = 1;
      attrs[n_attrs].val.clusterDim.z = 1;
      ++n_attrs;
      if (pdl_enabled()) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
      }
      cfg.attrs = attrs;
      cfg.numAttrs = n_attrs;
      cudaLaunchKernelEx(&cfg, attn_decode_kernel<T, 2, true>, p);
    } else {
      launch_pdl(attn_decode_kernel<T, 2, false>, grid, dim3(128), 4 * 2 * DEC_STAGE_BYTES, st, p);
      launch_pdl(attn_decode_merge_kernel<T>, dim3(static_cast<unsigned>(B * Hq)), dim3(128), 0, st, static_cast<const float*>(p.part_acc),
                 static_cast<const float*>(p.part_ml), static_cast<T*>(out), Hq, Hkv, p.G, d.splits);
    }
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
  p.mask_staged = (mask && aligned16(mask) && mask_b % 8 == 0 && mask_t % 8 == 0 && S % 8 == 0) ? 1 : 0;   // mask dtype == activation dtype by contract
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (tc5_enabled()) {   // tcgen05 kernel first; the mma.sync kernel below takes what it cannot (odd strides, other mask types)
    const int rc = attn_prefill_tc5(p, dtype, st);
    if (rc == B200_ELAUNCH) B200_FAIL(B200_ELAUNCH, "attn_prefill_tc5_kernel: launch failed");
    if (rc != B200_ENOTSUP) return rc;
  }
  dim3 grid(static_cast<unsigned>(ceil_div(T, 64)), static_cast<unsigned>(Hq), static_cast<unsigned>(B));
  B200_DISPATCH_HALF(dtype, T_, {
    static PerDevice<bool> configured_on;
    bool* configured = configured_on.slot();
    if (!configured) B200_FAIL(B200_ELAUNCH, "attn_prefill_kernel: no current device");
    if (!*configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
      if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "attn_prefill_kernel attribute: %s", cudaGetErrorString(e));
      *configured = true;
    }
    attn_prefill_kernel<T_><<<grid, 128, PF_SMEM, st>>>(p);
  });
  B200_CHECK_LAUNCH("attn_prefill_kernel");
  return B200_OK;
}
