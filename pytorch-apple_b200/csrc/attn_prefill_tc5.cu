// Prefill attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory, operands staged by TMA), head_dim 128.
//
// One CTA = 128 query rows of one head.  Q sits in shared memory for the CTA's life; K, V and the
// matching 128 x 64 tile of the additive mask arrive by TMA in 64-key tiles through a two-stage
// ring (all with the 128-byte swizzle).  Per key tile:
//   S[128 x 64]  = Q K^T        tcgen05.mma, K tile as the K-major B operand, S in tensor memory
//   softmax      one thread per query row reads its S row with tcgen05.ld, adds the mask, keeps
//                the running max / sum (log2 domain) and writes the probabilities, rounded to the
//                activation type as the unfused graph rounds them, into shared memory in the
//                K-major swizzled layout of an A operand
//   O[128x128]  += P V          tcgen05.mma, V tile as the MN-major B operand (V rows are keys, the
//                head dimension is the contiguous one); O stays in tensor memory for the whole CTA
//   correction   only when the running max of some row of a warp moved does that warp read its 32 rows
//                of O, rescale them and write them back (tcgen05.ld / tcgen05.st) before the product.
// S is double-buffered in tensor memory: the tensor core computes S of the next key tile while the
// softmax warps work on the current one.
// Key tiles whose mask tile holds no unmasked entry for these 128 rows are neither fetched nor
// multiplied: four scanner warps read the mask rows of the CTA tile by tile (the mask is the only
// statement of what is attended; nothing assumes it is causal) and leave a verdict per key tile in
// shared memory, which the other roles follow as the scan runs ahead of them.
// Warp roles: warps 11-14 mask scanners (tile j by warp 11 + j % 4), warps 0 and 10 TMA producers, warp 1 MMA issuer (and owner of the tensor-memory allocation),
// warps 2-9 softmax: warp w works on the 32 tensor-memory lanes (query rows) of quarter w % 4, warps 2-5 on
// the first 32 keys of a tile, warps 6-9 on the other 32 - two threads per row, so that every scheduler
// has two softmax warps to interleave (one warp per scheduler ran its dependent instruction stream at a
// quarter of the issue rate); the two halves of a row exchange their maxima through shared memory.  Every
// barrier wait is bounded; on a time-out the CTA records a code in the library's device error
// word, stops issuing, frees its tensor memory and returns.
#include "attention.cuh"
#include "tc5.cuh"

namespace b200 {

// time-out code of the last failed wait in this file's kernel (reported through b200_debug_device_error)
__device__ int g_attn5_error = 0;
#define g_tc5_error g_attn5_error

namespace {

constexpr int PD = 128;                        // head dim
constexpr int BQ = 128, BKV = 64;
constexpr int Q_BYTES = 2 * BQ * 128;          // two 64-column panels of [128 rows][128 bytes]
constexpr int K_BYTES = 2 * BKV * 128;         // two panels of [64 keys][128 bytes]
constexpr int V_BYTES = 2 * BKV * 128;
constexpr int M_BYTES = BQ * 128;              // [128 rows][64 keys] of a 16-bit mask
constexpr int STAGE = K_BYTES + V_BYTES + M_BYTES;
constexpr int NST = 3;
constexpr int P_BYTES = BQ * 128;              // [128 rows][64 keys]
constexpr int PF5_SMEM = Q_BYTES + NST * STAGE + 2 * P_BYTES + 1024;   // probabilities double-buffered
constexpr int MAX_TILES = 512;                 // key tiles per launch (S <= 32768)
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float MASKED_F = -1e30f;
constexpr int TMEM_COLS = 256;                 // S: columns 0..63 and 64..127 (double buffer), O: columns 128..255

template <typename T> struct Fmt;
template <> struct Fmt<__half> { static constexpr int value = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr int value = 1; };

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive1(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc5::smem_addr(bar)) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(480, 1)
    attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_m, const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem;
  uint8_t* st_s = smem + Q_BYTES;
  uint8_t* p_s = st_s + NST * STAGE;
  __shared__ __align__(8) uint64_t q_full, kv_full[NST], kv_empty[NST], s_full[2], p_ready, o_full;
  __shared__ uint32_t tmem_holder;
  __shared__ uint8_t s_flag[MAX_TILES];   // per key tile: 0 not scanned yet, 1 to be processed, 2 fully masked for these rows
  __shared__ float s_max[2][2][BQ];   // [tile parity][half][row]: the halves' maxima of a tile
  __shared__ float s_sum[2][BQ];      // [half][row]: the halves' sums, exchanged once at the end
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads fastest (the CTAs that share a mask tile run together and find it in L2), late row blocks -
  // the ones with the most key tiles under a causal mask - first
  const int h = blockIdx.x, b = blockIdx.z;
  const int q0 = static_cast<int>(gridDim.y - 1 - blockIdx.y) * BQ;
  const int hk = h / (p.Hq / p.Hkv);
  const int b_m = p.mask_b == 0 ? 0 : b;   // a mask without a batch stride is shared by all sequences
  const int n_tiles = static_cast<int>((p.S + BKV - 1) / BKV);
  const int rows_valid = static_cast<int>(p.T - q0 < BQ ? p.T - q0 : BQ);
  const bool has_mask = p.mask != nullptr;

  if (threadIdx.x == 0) {
    failed = 0;
    tc5::mbar_init(&q_full, 1);
    for (int s = 0; s < NST; ++s) { tc5::mbar_init(&kv_full[s], 2); tc5::mbar_init(&kv_empty[s], 1); }
    tc5::mbar_init(&s_full[0], 1);
    tc5::mbar_init(&s_full[1], 1);
    tc5::mbar_init(&p_ready, 256);
    tc5::mbar_init(&o_full, 1);
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&map_q);
    tc5::prefetch_tensormap(&map_k);
    tc5::prefetch_tensormap(&map_v);
    if (has_mask) tc5::prefetch_tensormap(&map_m);
  }
  for (int j = threadIdx.x; j < MAX_TILES; j += blockDim.x) s_flag[j] = has_mask ? 0 : 1;
  if (warp == 1) { tc5::tmem_alloc(&tmem_holder, TMEM_COLS); tc5::tmem_relinquish(); }
  tc5::tc_fence_before();
  __syncthreads();
  tc5::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_trigger();
  pdl_wait();   // q, k, v and the mask come from earlier kernels

  // row of the query tile a softmax thread works on (the tensor-memory lane its warp may read) and its half of the keys
  const int r = 32 * (warp & 3) + lane;
  const int half = (warp - 2) >> 2;

  // First key tile at or after j that must be processed, -1 when there is none, -2 when the scanners stopped answering.
  auto next_tile = [&](int j) -> int {
    const volatile uint8_t* flag = s_flag;
    for (; j < n_tiles; ++j) {
      uint32_t spin = 0;
      uint8_t f = flag[j];
      while (f == 0) {
        if (++spin > (1u << 22)) return -2;
        f = flag[j];
      }
      if (f == 1) return j;
    }
    return -1;
  };

  if (warp >= 11) {
    // ---- scanners: does key tile j hold an unmasked entry for these 128 rows (lane l: rows l, l+32, l+64, l+96) ----
    if (has_mask) {
      const T* m0 = static_cast<const T*>(p.mask) + static_cast<int64_t>(b) * p.mask_b + static_cast<int64_t>(q0) * p.mask_t;
      for (int j = warp - 11; j < n_tiles; j += 4) {
        const int64_t key0 = static_cast<int64_t>(j) * BKV;
        bool any = false;
        if (key0 + BKV <= p.S) {
          uint4 v[4][8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const bool row_ok = lane + 32 * q < rows_valid;
            const uint4* src = reinterpret_cast<const uint4*>(m0 + static_cast<int64_t>(lane + 32 * q) * p.mask_t + key0);
#pragma unroll
            for (int c = 0; c < 8; ++c) v[q][c] = row_ok ? __ldg(src + c) : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float f[8];
              unpack8<T>(v[q][c], f);
#pragma unroll
              for (int e = 0; e < 8; ++e) any = any || f[e] > MASKED_F;
            }
        } else {
          for (int q = 0; q < 4; ++q)
            if (lane + 32 * q < rows_valid)
              for (int e = 0; e < BKV; ++e)
                if (key0 + e < p.S && to_f32<T>(m0[static_cast<int64_t>(lane + 32 * q) * p.mask_t + key0 + e]) > MASKED_F) any = true;
        }
        const bool valid = __ballot_sync(0xffffffffu, any) != 0u;
        if (lane == 0) *reinterpret_cast<volatile uint8_t*>(&s_flag[j]) = valid ? 1 : 2;
      }
    }
  } else if (warp == 0 || warp == 10) {
    // ---- two TMA producers (one issuing thread sustains ~60 GB/s): warp 0 brings Q, the K tiles and the
    // mask tiles, warp 10 the V tiles.  One instruction per tile: the maps split the head dimension into
    // (64, 2), so a box lands as two [rows][128-byte] panels.
    if (lane == 0) {
      const bool kside = warp == 0;
      if (kside) {
        tc5::mbar_arrive_expect_tx(&q_full, Q_BYTES);
        tc5::tma_load_5d(q_s, &map_q, &q_full, 0, q0, 0, h, b);
      }
      int n = 0;
      for (int jc = 0;; ++n) {
        const int j = next_tile(jc), st = n % NST;
        jc = j + 1;
        if (j < 0) {
          if (j == -2) { failed = 1; atomicExch(&g_tc5_error, 30); }
          break;
        }
        if (!tc5::mbar_wait(&kv_empty[st], ((n / NST) & 1) ^ 1)) { failed = 1; atomicExch(&g_tc5_error, 31); break; }
        if (*reinterpret_cast<volatile int*>(&failed)) break;
        uint8_t* dst = st_s + st * STAGE;
        if (kside) {
          tc5::mbar_arrive_expect_tx(&kv_full[st], K_BYTES + (has_mask ? M_BYTES : 0));
          tc5::tma_load_5d(dst, &map_k, &kv_full[st], 0, j * BKV, 0, hk, b);
          if (has_mask) tc5::tma_load_3d(dst + K_BYTES + V_BYTES, &map_m, &kv_full[st], j * BKV, q0, b_m);
        } else {
          tc5::mbar_arrive_expect_tx(&kv_full[st], V_BYTES);
          tc5::tma_load_5d(dst + K_BYTES, &map_v, &kv_full[st], 0, j * BKV, 0, hk, b);
        }
      }
      // on a failure elsewhere the copies in flight must land before the CTA leaves
      if (*reinterpret_cast<volatile int*>(&failed))
        for (int i = n > NST ? n - NST : 0; i < n; ++i) tc5::mbar_wait(&kv_full[i % NST], (i / NST) & 1, 1u << 16);
    }
  } else if (warp == 1) {
    if (lane == 0) {   // ---- MMA issuer ----
      constexpr uint32_t idesc_s = tc5::umma_idesc(BQ, BKV, Fmt<T>::value);
      constexpr uint32_t idesc_o = tc5::umma_idesc(BQ, PD, Fmt<T>::value) | (1u << 16);   // B operand MN-major
      const uint32_t tm_o = tmem_base + 128, q_addr = tc5::smem_addr(q_s), p_addr = tc5::smem_addr(p_s);
      auto issue_s = [&](int n) {   // S[n & 1] = Q K(n)^T; false when the tile did not arrive
        const int st = n % NST;
        if (!tc5::mbar_wait(&kv_full[st], (n / NST) & 1)) return false;
        tc5::tc_fence_after();
        const uint32_t k_addr = tc5::smem_addr(st_s + st * STAGE);
#pragma unroll
        for (int kk = 0; kk < PD / 16; ++kk) {   // 16 head dims per instruction; panel kk / 4, 32-byte step inside it
          const uint64_t da = tc5::umma_desc_sw128(q_addr + (kk >> 2) * (BQ * 128)) + 2 * (kk & 3);
          const uint64_t db = tc5::umma_desc_sw128(k_addr + (kk >> 2) * (BKV * 128)) + 2 * (kk & 3);
          tc5::umma_f16(tmem_base + 64 * (n & 1), da, db, idesc_s, kk != 0);
        }
        tc5::umma_commit(&s_full[n & 1]);
        return true;
      };
      int cur = next_tile(0);
      bool ok = cur >= 0 && tc5::mbar_wait(&q_full, 0);
      if (cur >= 0 && !ok) { failed = 1; atomicExch(&g_tc5_error, 32); }
      if (ok && !issue_s(0)) { ok = false; failed = 1; atomicExch(&g_tc5_error, 33); }
      for (int n = 0; ok && cur >= 0; ++n) {
        // the next tile's scores are computed while the softmax warps work on this one
        const int nxt = next_tile(cur + 1);
        if (nxt == -2 || (nxt >= 0 && !issue_s(n + 1))) { failed = 1; atomicExch(&g_tc5_error, 33); break; }
        if (!tc5::mbar_wait(&p_ready, n & 1)) { failed = 1; atomicExch(&g_tc5_error, 34); break; }
        tc5::tc_fence_after();
        const int st = n % NST;
        const uint32_t v_addr = tc5::smem_addr(st_s + st * STAGE) + K_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {     // 16 keys per instruction = two 8-key groups of the V panels
          const uint64_t da = tc5::umma_desc_sw128(p_addr + (n & 1) * P_BYTES) + 2 * k;
          const uint64_t db = tc5::umma_desc_sw128_mn(v_addr + k * 2048, BKV * 128, 1024);
          tc5::umma_f16(tm_o, da, db, idesc_o, (n | k) != 0);
        }
        tc5::umma_commit(&o_full);
        tc5::umma_commit(&kv_empty[st]);
        cur = nxt;
      }
    }
  } else if (warp < 10) {
    // ---- softmax: two threads per query row, 32 keys of the tile each ----
    constexpr int HK = BKV / 2;   // keys per thread
    const int quarter = warp & 3;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(32 * quarter) << 16);
    const float scale = p.scale;
    float m_run = -INFINITY, l_run = 0.f;   // running max of the row (log2 domain, both halves agree), sum of this half
    bool alive = true;
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {   // every lane polls; the warp leaves together
      const bool got = __all_sync(0xffffffffu, tc5::mbar_wait(bar, parity));
      if (!got && lane == 0) { failed = 1; atomicExch(&g_tc5_error, code); }
      return got;
    };
    int n = 0;
    for (int jc = 0;; ++n) {
      int j = 0;
      if (lane == 0) j = next_tile(jc);
      j = __shfl_sync(0xffffffffu, j, 0);
      jc = j + 1;
      if (j < 0) {
        if (j == -2) { alive = false; if (lane == 0) { failed = 1; atomicExch(&g_tc5_error, 38); } }
        break;
      }
      const int st = n % NST;
      if (!wait_all(&s_full[n & 1], (n >> 1) & 1, 35)) { alive = false; break; }
      tc5::tc_fence_after();
      const uint8_t* m_row = st_s + st * STAGE + K_BYTES + V_BYTES + r * 128;
      const int key0 = j * BKV + half * HK;
      // u = score * scale + mask for this thread's 32 keys (natural-log domain; ex2 takes u * log2 e)
      float u[HK];
      tc5::tmem_ld_32x16(t_row + 64 * (n & 1) + half * HK, *reinterpret_cast<float(*)[16]>(&u[0]));
      tc5::tmem_ld_32x16(t_row + 64 * (n & 1) + half * HK + 16, *reinterpret_cast<float(*)[16]>(&u[16]));
      tc5::tmem_ld_wait();
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < HK / 8; ++c) {
        float mk[8];
        if (has_mask) unpack8<T>(*reinterpret_cast<const uint4*>(m_row + (((half * 4 + c) ^ (r & 7)) << 4)), mk);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float v = has_mask ? fmaf(u[8 * c + e], scale, mk[e]) : u[8 * c + e] * scale;
          u[8 * c + e] = v;
          mx[e & 3] = fmaxf(mx[e & 3], v);
        }
      }
      if (key0 + HK > p.S) {   // the last tile of a cache whose length is not a multiple of 64: keys past the end
#pragma unroll
        for (int e = 0; e < HK; ++e)
          if (key0 + e >= p.S) u[e] = -INFINITY;
        mx[0] = mx[1] = mx[2] = mx[3] = -INFINITY;
#pragma unroll
        for (int e = 0; e < HK; ++e) mx[e & 3] = fmaxf(mx[e & 3], u[e]);
      }
      const float mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * LOG2E_F;
      // the row's maximum over both halves: exchange through shared memory (one barrier of the 64 threads of the quarter)
      s_max[n & 1][half][r] = mine;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      const float m_new = fmaxf(m_run, fmaxf(mine, s_max[n & 1][half ^ 1][r]));
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ex2(m_run - m_use);   // exactly 1 while the max stands; 0 for the first tile
      // Some row's max moved: rescale this warp's half of the 32 rows of O, once the previous product
      // has finished.  (That wait is skipped otherwise: the probabilities are double-buffered, and
      // S of this tile being complete means the product before the previous one is, so the barrier
      // is never more than one phase behind when it is looked at again.)
      if (n > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!wait_all(&o_full, (n - 1) & 1, 36)) { alive = false; break; }
        tc5::tc_fence_after();
        {
#pragma unroll
          for (int c = 0; c < PD / 32; ++c) {
            float t[16];
            tc5::tmem_ld_32x16(t_row + 128 + half * 64 + 16 * c, t);
            tc5::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) t[e] *= alpha;
            tc5::tmem_st_32x16(t_row + 128 + half * 64 + 16 * c, t);
          }
          tc5::tmem_st_wait();
        }
      }
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* p_row = p_s + (n & 1) * P_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < HK / 8; ++c) {
        float pr[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pr[e] = ex2(fmaf(u[8 * c + e], LOG2E_F, -m_use));
          sum[e & 3] += pr[e];
        }
        *reinterpret_cast<uint4*>(p_row + (((half * 4 + c) ^ (r & 7)) << 4)) = pack8<T>(pr);
      }
      tc5::fence_proxy_async();   // the probabilities are read by the tensor core (async proxy)
      tc5::tc_fence_before();     // this thread's tcgen05.ld / st are complete before S and O are touched again
      mbar_arrive1(&p_ready);
      l_run = l_run * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      m_run = m_new;
    }
    const int N = n;   // tiles processed
    // the row's sum over both halves
    s_sum[half][r] = l_run;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    const float l_all = l_run + s_sum[half ^ 1][r];
    if (alive && N > 0) alive = wait_all(&o_full, (N - 1) & 1, 37);
    if (alive) {
      tc5::tc_fence_after();
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;   // a row whose mask admits no key gives zeros
      T* orow = static_cast<T*>(p.out) + ((static_cast<int64_t>(b) * p.T + q0 + r) * p.Hq + h) * PD + half * 64;
#pragma unroll
      for (int c = 0; c < PD / 32; ++c) {   // this thread's 64 of the row's 128 output columns
        float t[16];
        if (N > 0) {
          tc5::tmem_ld_32x16(t_row + 128 + half * 64 + 16 * c, t);
          tc5::tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) t[e] = 0.f;
        }
        if (r < rows_valid) {
          float f0[8], f1[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) { f0[e] = t[e] * inv; f1[e] = t[8 + e] * inv; }
          reinterpret_cast<uint4*>(orow)[2 * c] = pack8<T>(f0);
          reinterpret_cast<uint4*>(orow)[2 * c + 1] = pack8<T>(f1);
        }
      }
    }
  }
  tc5::tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc5::tc_fence_after(); tc5::tmem_dealloc(tmem_base, TMEM_COLS); }
}

template <typename T>
int launch_prefill_tc5(const PrefillParams& p, int dtype, cudaStream_t st) {
  static PerDevice<bool> configured_on;
  bool* configured = configured_on.slot();
  if (!configured) return B200_ENOTSUP;
  if (!*configured) {
    if (cudaFuncSetAttribute(attn_prefill_tc5_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF5_SMEM) != cudaSuccess) {
      cudaGetLastError();
      return B200_ENOTSUP;
    }
    *configured = true;
  }
  CUtensorMap mq, mk, mv, mm;
  auto st_of = [](int64_t elems, uint64_t fallback) { return elems > 0 ? static_cast<uint64_t>(elems) * 2 : fallback; };
  // [batch, head, row, 128] as (64, rows, 2, heads, batch): a box of (64, rows, 2) lands as two panels of [rows][128 bytes]
  auto map5 = [&](CUtensorMap* m, const void* base, int64_t rows, int heads, const int64_t* strides, uint32_t box_rows) {
    const uint64_t dims[5] = {64, static_cast<uint64_t>(rows), 2, static_cast<uint64_t>(heads), static_cast<uint64_t>(p.B)};
    const uint64_t str[4] = {st_of(strides[2], PD * 2), 128, st_of(strides[1], PD * 2), st_of(strides[0], PD * 2)};
    const uint32_t box[5] = {64, box_rows, 2, 1, 1};
    return tma_encode_sw128(m, dtype, 5, base, dims, str, box);
  };
  if (!map5(&mq, p.q, p.T, p.Hq, p.qs, BQ) || !map5(&mk, p.k, p.S, p.Hkv, p.ks, BKV) || !map5(&mv, p.v, p.S, p.Hkv, p.vs, BKV)) return B200_ENOTSUP;
  mm = mq;
  if (p.mask) {
    const uint64_t dims[3] = {static_cast<uint64_t>(p.S), static_cast<uint64_t>(p.T), static_cast<uint64_t>(p.mask_b == 0 ? 1 : p.B)};
    const uint64_t str[2] = {st_of(p.mask_t, static_cast<uint64_t>(p.S) * 2), st_of(p.mask_b, static_cast<uint64_t>(p.S) * 2)};
    const uint32_t box[3] = {64, BQ, 1};
    if (!tma_encode_sw128(&mm, dtype, 3, p.mask, dims, str, box)) return B200_ENOTSUP;
  }
  dim3 grid(static_cast<unsigned>(p.Hq), static_cast<unsigned>((p.T + BQ - 1) / BQ), static_cast<unsigned>(p.B));
  launch_pdl(attn_prefill_tc5_kernel<T>, grid, dim3(480), PF5_SMEM, st, mq, mk, mv, mm, p);
  return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ELAUNCH;
}

}  // namespace

#undef g_tc5_error
int attn_prefill_tc5_error(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn5_error, sizeof(int)) != cudaSuccess) return -1;
  if (clear && v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn5_error, &zero, sizeof(int));
  }
  return v;
}

int attn_prefill_tc5(const PrefillParams& p, int dtype, cudaStream_t stream) {
  if (dtype != B200_BF16 && dtype != B200_F16) return B200_ENOTSUP;
  if (p.S > static_cast<int64_t>(BKV) * MAX_TILES || p.T >= (1ll << 31) || p.Hq % p.Hkv) return B200_ENOTSUP;
  if (p.mask && (!p.mask_staged || p.mask_dtype != dtype)) return B200_ENOTSUP;   // the mask tile travels by TMA in the activation type
  // TMA: 16-byte aligned bases (checked by the caller) and strides that are multiples of 16 bytes
  for (int i = 0; i < 3; ++i)
    if (p.qs[i] % 8 || p.ks[i] % 8 || p.vs[i] % 8 || p.qs[i] < 0 || p.ks[i] < 0 || p.vs[i] < 0) return B200_ENOTSUP;
  if (p.mask && (p.mask_b < 0 || p.mask_t < p.S || p.mask_t % 8)) return B200_ENOTSUP;
  return dtype == B200_BF16 ? launch_prefill_tc5<__nv_bfloat16>(p, dtype, stream) : launch_prefill_tc5<__half>(p, dtype, stream);
}

}  // namespace b200
