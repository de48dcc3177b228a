// Gather / scatter kernels (embedding, KV-cache index_copy) and rotary embedding.
// Gathers and scatters move raw bytes, so their results are bit-exact.
#include "common.cuh"

namespace b200 {

// out[s, :] = table[ids[s], :], rows as raw bytes.  blockDim.x threads walk one row.
template <bool VEC16>
__global__ void __launch_bounds__(256) embedding_kernel(const uint8_t* __restrict__ table, const void* __restrict__ ids,
                                                        uint8_t* __restrict__ out, int64_t vocab, int64_t row_bytes,
                                                        int ids_dtype) {
  const int64_t s = blockIdx.x;
  const int64_t id = load_index(ids, s, ids_dtype);
  const bool ok = id >= 0 && id < vocab;
  const uint8_t* src = table + (ok ? id : 0) * row_bytes;
  uint8_t* dst = out + s * row_bytes;
  if (VEC16) {
    const int64_t n = row_bytes >> 4;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = ok ? ld_global_nc_v4(reinterpret_cast<const uint4*>(src) + i) : make_uint4(0, 0, 0, 0);
  } else {
    for (int64_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = ok ? src[i] : uint8_t(0);
  }
}

// dst[o, index[l], :] = src[o, l, :]; one block per (o, l) row.
template <bool VEC16>
__global__ void __launch_bounds__(128) index_copy_rows_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                                              const void* __restrict__ index, int64_t dim_size,
                                                              int64_t inner_bytes, int64_t n_index, int64_t src_outer_bytes,
                                                              int64_t src_index_bytes, int index_dtype) {
  const int64_t o = blockIdx.x / n_index, l = blockIdx.x % n_index;
  int64_t pos = load_index(index, l, index_dtype);
  if (pos < 0) pos += dim_size;
  if (pos < 0 || pos >= dim_size) return;  // out-of-range index: leave the destination untouched
  const uint8_t* s = src + o * src_outer_bytes + l * src_index_bytes;
  uint8_t* d = dst + (o * dim_size + pos) * inner_bytes;
  if (VEC16) {
    const int64_t n = inner_bytes >> 4;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
  } else {
    for (int64_t i = threadIdx.x; i < inner_bytes; i += blockDim.x) d[i] = s[i];
  }
}

// cos/sin tables: angle = fp32(position) * inv_freq[d mod half] as one fp32 product.
template <typename TO>
__global__ void __launch_bounds__(128) rope_table_kernel(const float* __restrict__ inv_freq, const void* __restrict__ positions,
                                                         TO* __restrict__ cos_out, TO* __restrict__ sin_out, int64_t n_pos,
                                                         int head_dim, int pos_dtype) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_pos * head_dim) return;
  const int64_t p = i / head_dim;
  const int d = static_cast<int>(i % head_dim);
  const float pos = pos_dtype == B200_F32 ? static_cast<const float*>(positions)[p]
                                          : static_cast<float>(load_index(positions, p, pos_dtype));
  const float ang = __fmul_rn(pos, inv_freq[d % (head_dim >> 1)]);
  cos_out[i] = from_f32<TO>(cosf(ang));
  sin_out[i] = from_f32<TO>(sinf(ang));
}

struct RopeParams {
  const void* x;
  const void* cos_t;
  const void* sin_t;
  void* y;
  void* cache;
  const void* cache_pos;
  int64_t B, H, T;
  int D;
  int64_t xs[3];  // element strides of x over (b, h, t); D is contiguous
  int64_t cache_len;
  int pos_dtype;
};

// One thread per pair of 16-byte packs (dims d..d+7 and d+D/2..d+D/2+7): both halves of a
// rotation are read once.  Products are rounded in pairs (one packed conversion per two
// values; the conversion unit is the scarce one), index arithmetic in IDX (32-bit when the
// tensor allows it).
template <typename T, typename IDX>
__device__ __forceinline__ void rope_rotate_block(const RopeParams& p, unsigned block) {
  const IDX half_packs = static_cast<IDX>(p.D >> 4);
  const IDX gid = static_cast<IDX>(block) * 128 + threadIdx.x;
  const IDX total = static_cast<IDX>(p.B * p.H * p.T) * half_packs;
  if (gid >= total) return;
  const IDX row = gid / half_packs;
  const int pk = static_cast<int>(gid - row * half_packs);
  const IDX bh = row / static_cast<IDX>(p.T);
  const int64_t t = static_cast<int64_t>(row - bh * static_cast<IDX>(p.T));
  const IDX b = bh / static_cast<IDX>(p.H);
  const int64_t h = static_cast<int64_t>(bh - b * static_cast<IDX>(p.H));
  const uint4* xr = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + static_cast<int64_t>(b) * p.xs[0] + h * p.xs[1] + t * p.xs[2]);
  const int64_t tab = (static_cast<int64_t>(b) * p.T + t) * p.D;
  const uint4* ct = reinterpret_cast<const uint4*>(static_cast<const T*>(p.cos_t) + tab);
  const uint4* st = reinterpret_cast<const uint4*>(static_cast<const T*>(p.sin_t) + tab);
  const int hp = static_cast<int>(half_packs);
  const uint4 rlo = ld_global_nc_v4(xr + pk), rhi = ld_global_nc_v4(xr + pk + hp);
  const uint4 rclo = __ldg(ct + pk), rchi = __ldg(ct + pk + hp), rslo = __ldg(st + pk), rshi = __ldg(st + pk + hp);
  float lo[8], hi[8], c[8], s[8], olo[8], ohi[8];
  unpack8<T>(rlo, lo);
  unpack8<T>(rhi, hi);
  unpack8<T>(rclo, c);
  unpack8<T>(rslo, s);
#pragma unroll
  for (int k = 0; k < 8; k += 2) {   // first half: x1*cos + (-x2)*sin
    float a0 = lo[k] * c[k], a1 = lo[k + 1] * c[k + 1], b0 = -hi[k] * s[k], b1 = -hi[k + 1] * s[k + 1];
    round2<T>(a0, a1);
    round2<T>(b0, b1);
    olo[k] = a0 + b0; olo[k + 1] = a1 + b1;
  }
  unpack8<T>(rchi, c);
  unpack8<T>(rshi, s);
#pragma unroll
  for (int k = 0; k < 8; k += 2) {   // second half: x2*cos + x1*sin
    float a0 = hi[k] * c[k], a1 = hi[k + 1] * c[k + 1], b0 = lo[k] * s[k], b1 = lo[k + 1] * s[k + 1];
    round2<T>(a0, a1);
    round2<T>(b0, b1);
    ohi[k] = a0 + b0; ohi[k + 1] = a1 + b1;
  }
  T* dst;
  if (p.cache) {
    int64_t pos = load_index(p.cache_pos, t, p.pos_dtype);
    if (pos < 0) pos += p.cache_len;
    if (pos < 0 || pos >= p.cache_len) return;
    dst = static_cast<T*>(p.cache) + (static_cast<int64_t>(bh) * p.cache_len + pos) * p.D;
  } else {
    dst = static_cast<T*>(p.y) + static_cast<int64_t>(row) * p.D;
  }
  reinterpret_cast<uint4*>(dst)[pk] = pack8<T>(olo);
  reinterpret_cast<uint4*>(dst)[pk + hp] = pack8<T>(ohi);
}

template <typename T, typename IDX>
__global__ void __launch_bounds__(128) rope_rotate_kernel(const __grid_constant__ RopeParams p) {
  rope_rotate_block<T, IDX>(p, blockIdx.x);
}

// q and k of one attention layer in one launch: the first `q_blocks` blocks rotate q, the rest k.
template <typename T>
__global__ void __launch_bounds__(128) rope_rotate_pair_kernel(const __grid_constant__ RopeParams pq, const __grid_constant__ RopeParams pk,
                                                               const unsigned q_blocks) {
  pdl_wait();
  pdl_trigger();
  if (blockIdx.x < q_blocks) rope_rotate_block<T, uint32_t>(pq, blockIdx.x);
  else rope_rotate_block<T, uint32_t>(pk, blockIdx.x - q_blocks);
}

// Many positions (prefill): one thread per (sequence, position, pack pair) walks ALL heads.  The
// cos / sin values of a position are the same for every head, so they are loaded once per thread
// instead of once per head, and the loads of four heads are in flight together.
template <typename T>
__global__ void __launch_bounds__(128) rope_rotate_heads_kernel(const __grid_constant__ RopeParams p) {
  const int hp = p.D >> 4;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * 128 + threadIdx.x;
  if (gid >= p.B * p.T * hp) return;
  const int pk = static_cast<int>(gid % hp);
  const int64_t bt = gid / hp, b = bt / p.T, t = bt - b * p.T;
  const int64_t tab = (b * p.T + t) * p.D;
  const uint4* ct = reinterpret_cast<const uint4*>(static_cast<const T*>(p.cos_t) + tab);
  const uint4* st = reinterpret_cast<const uint4*>(static_cast<const T*>(p.sin_t) + tab);
  float clo[8], chi[8], slo[8], shi[8];
  unpack8<T>(__ldg(ct + pk), clo);
  unpack8<T>(__ldg(ct + pk + hp), chi);
  unpack8<T>(__ldg(st + pk), slo);
  unpack8<T>(__ldg(st + pk + hp), shi);
  const T* xb = static_cast<const T*>(p.x) + b * p.xs[0] + t * p.xs[2];
  constexpr int U = 4;
  for (int64_t h0 = 0; h0 < p.H; h0 += U) {
    uint4 rlo[U], rhi[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (h0 + u < p.H) {
        const uint4* xr = reinterpret_cast<const uint4*>(xb + (h0 + u) * p.xs[1]);
        rlo[u] = ld_global_nc_v4(xr + pk);
        rhi[u] = ld_global_nc_v4(xr + pk + hp);
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (h0 + u >= p.H) break;
      float lo[8], hi[8], olo[8], ohi[8];
      unpack8<T>(rlo[u], lo);
      unpack8<T>(rhi[u], hi);
#pragma unroll
      for (int k = 0; k < 8; k += 2) {
        float a0 = lo[k] * clo[k], a1 = lo[k + 1] * clo[k + 1], b0 = -hi[k] * slo[k], b1 = -hi[k + 1] * slo[k + 1];
        round2<T>(a0, a1);
        round2<T>(b0, b1);
        olo[k] = a0 + b0; olo[k + 1] = a1 + b1;
        float c0 = hi[k] * chi[k], c1 = hi[k + 1] * chi[k + 1], d0 = lo[k] * shi[k], d1 = lo[k + 1] * shi[k + 1];
        round2<T>(c0, c1);
        round2<T>(d0, d1);
        ohi[k] = c0 + d0; ohi[k + 1] = c1 + d1;
      }
      T* dst = static_cast<T*>(p.y) + ((b * p.H + h0 + u) * p.T + t) * p.D;
      reinterpret_cast<uint4*>(dst)[pk] = pack8<T>(olo);
      reinterpret_cast<uint4*>(dst)[pk + hp] = pack8<T>(ohi);
    }
  }
}

struct QkvPostParams {
  const void* x[3];     // q, k, v: [B, H, T, D] views, D contiguous
  int64_t xs[3][3];     // element strides over (b, h, t)
  const void* cos_t; const void* sin_t;
  void* q_out; void* k_cache; void* v_cache;
  const void* cache_pos;
  int64_t B, T, cache_len;
  int Hq, Hkv, D, pos_dtype;
};

// One launch for the three per-token steps between the QKV projection and attention:
// RoPE on q (to a dense [B,Hq,T,D] buffer), RoPE on k written straight into the key cache
// at row cache_pos[t], and v copied into the value cache at the same row.
template <typename T>
__global__ void __launch_bounds__(128) qkv_rope_cache_kernel(const __grid_constant__ QkvPostParams p) {
  const int packs = p.D >> 3, half_packs = packs >> 1, H = p.Hq + 2 * p.Hkv;
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_trigger();
  if (gid >= p.B * H * p.T * packs) return;
  const int pk = static_cast<int>(gid % packs);
  int64_t r = gid / packs;
  const int64_t t = r % p.T; r /= p.T;
  int h = static_cast<int>(r % H);
  const int64_t b = r / H;
  const int which = h < p.Hq ? 0 : (h < p.Hq + p.Hkv ? 1 : 2);
  if (which == 1) h -= p.Hq;
  if (which == 2) h -= p.Hq + p.Hkv;
  const T* xr = static_cast<const T*>(p.x[which]) + b * p.xs[which][0] + h * p.xs[which][1] + t * p.xs[which][2];
  uint4 result;
  if (which == 2) {
    result = *(reinterpret_cast<const uint4*>(xr) + pk);
  } else {
    const int64_t tab = (b * p.T + t) * p.D;
    float xv[8], ov[8], c[8], s[8], out[8];
    unpack8<T>(*(reinterpret_cast<const uint4*>(xr) + pk), xv);
    unpack8<T>(*(reinterpret_cast<const uint4*>(xr) + (pk < half_packs ? pk + half_packs : pk - half_packs)), ov);
    unpack8<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.cos_t) + tab) + pk), c);
    unpack8<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.sin_t) + tab) + pk), s);
    const float sign = pk < half_packs ? -1.f : 1.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = round_as<T>(xv[k] * c[k]) + round_as<T>(sign * ov[k] * s[k]);
    result = pack8<T>(out);
  }
  T* dst;
  if (which == 0) {
    dst = static_cast<T*>(p.q_out) + ((b * p.Hq + h) * p.T + t) * p.D;
  } else {
    int64_t pos = load_index(p.cache_pos, t, p.pos_dtype);
    if (pos < 0) pos += p.cache_len;
    if (pos < 0 || pos >= p.cache_len) return;
    dst = static_cast<T*>(which == 1 ? p.k_cache : p.v_cache) + ((b * p.Hkv + h) * p.cache_len + pos) * p.D;
  }
  reinterpret_cast<uint4*>(dst)[pk] = result;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_qkv_rope_cache(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v, const void* cos_t,
                                   const void* sin_t, void* q_out, void* k_cache, void* v_cache, const void* cache_pos,
                                   int64_t cache_len, int pos_dtype, void* stream) {
  B200_CHECK_ARG(q && k && v && q->data && k->data && v->data && cos_t && sin_t && q_out && k_cache && v_cache && cache_pos,
                 "b200_qkv_rope_cache: bad arguments");
  B200_CHECK_ARG(q->ndim == 4 && k->ndim == 4 && v->ndim == 4 && q->dtype == k->dtype && k->dtype == v->dtype,
                 "b200_qkv_rope_cache: q, k, v must be 4-D tensors of one dtype");
  QkvPostParams p;
  const b200_tensor* ts[3] = {q, k, v};
  bool ok = aligned16(cos_t) && aligned16(sin_t) && aligned16(q_out) && aligned16(k_cache) && aligned16(v_cache);
  for (int i = 0; i < 3; ++i) {
    p.x[i] = ts[i]->data;
    ok = ok && aligned16(ts[i]->data) && ts[i]->stride[3] == 1;
    for (int d = 0; d < 3; ++d) { p.xs[i][d] = ts[i]->stride[d]; ok = ok && ts[i]->stride[d] % 8 == 0; }
  }
  B200_CHECK_ARG(k->shape[1] == v->shape[1] && q->shape[0] == k->shape[0] && q->shape[2] == k->shape[2] && q->shape[3] == k->shape[3] &&
                 v->shape[0] == k->shape[0] && v->shape[2] == k->shape[2] && v->shape[3] == k->shape[3] && q->shape[3] % 16 == 0,
                 "b200_qkv_rope_cache: shape mismatch");
  if (!ok) B200_FAIL(B200_EALIGN, "b200_qkv_rope_cache: operands must be 16-byte aligned with strides multiple of 8");
  p.cos_t = cos_t; p.sin_t = sin_t; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache; p.cache_pos = cache_pos;
  p.B = q->shape[0]; p.T = q->shape[2]; p.cache_len = cache_len;
  p.Hq = static_cast<int>(q->shape[1]); p.Hkv = static_cast<int>(k->shape[1]); p.D = static_cast<int>(q->shape[3]); p.pos_dtype = pos_dtype;
  const int64_t total = p.B * (p.Hq + 2 * p.Hkv) * p.T * (p.D >> 3);
  if (total == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_HALF(q->dtype, T, { launch_pdl(qkv_rope_cache_kernel<T>, dim3(static_cast<unsigned>(ceil_div(total, 128))), dim3(128), 0, st, p); });
  B200_CHECK_LAUNCH("qkv_rope_cache_kernel");
  return B200_OK;
}

extern "C" int b200_embedding(const void* table, const void* ids, void* out, int64_t n_ids, int64_t vocab,
                              int64_t row_bytes, int ids_dtype, void* stream) {
  B200_CHECK_ARG(table && ids && out && n_ids >= 0 && vocab > 0 && row_bytes > 0, "b200_embedding: bad arguments");
  B200_CHECK_ARG(ids_dtype == B200_I64 || ids_dtype == B200_I32, "b200_embedding: ids must be int32/int64");
  if (n_ids == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = row_bytes % 16 == 0 && aligned16(table) && aligned16(out);
  const int threads = row_bytes >= 16 * 256 ? 256 : (row_bytes >= 16 * 64 ? 64 : 32);
  if (vec) embedding_kernel<true><<<static_cast<unsigned>(n_ids), threads, 0, st>>>(
        static_cast<const uint8_t*>(table), ids, static_cast<uint8_t*>(out), vocab, row_bytes, ids_dtype);
  else embedding_kernel<false><<<static_cast<unsigned>(n_ids), threads, 0, st>>>(
        static_cast<const uint8_t*>(table), ids, static_cast<uint8_t*>(out), vocab, row_bytes, ids_dtype);
  B200_CHECK_LAUNCH("embedding_kernel");
  return B200_OK;
}

extern "C" int b200_index_copy(const void* base, void* dst, const void* src, const void* index, int64_t outer,
                               int64_t dim_size, int64_t inner, int64_t n_index, int64_t src_outer_stride,
                               int64_t src_index_stride, int elem_bytes, int index_dtype, void* stream) {
  B200_CHECK_ARG(base && dst && src && index && outer >= 0 && dim_size > 0 && inner > 0 && n_index >= 0 && elem_bytes > 0,
                 "b200_index_copy: bad arguments");
  B200_CHECK_ARG(index_dtype == B200_I64 || index_dtype == B200_I32, "b200_index_copy: index must be int32/int64");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (base != dst) {
    cudaError_t e = cudaMemcpyAsync(dst, base, static_cast<size_t>(outer * dim_size * inner) * elem_bytes,
                                    cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "b200_index_copy: %s", cudaGetErrorString(e));
  }
  if (outer == 0 || n_index == 0) return B200_OK;
  const int64_t inner_bytes = inner * elem_bytes, so = src_outer_stride * elem_bytes, si = src_index_stride * elem_bytes;
  const bool vec = inner_bytes % 16 == 0 && so % 16 == 0 && si % 16 == 0 && aligned16(dst) && aligned16(src);
  const unsigned grid = static_cast<unsigned>(outer * n_index);
  const int threads = inner_bytes >= 16 * 128 ? 128 : 32;
  if (vec) index_copy_rows_kernel<true><<<grid, threads, 0, st>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src),
                                                                  index, dim_size, inner_bytes, n_index, so, si, index_dtype);
  else index_copy_rows_kernel<false><<<grid, threads, 0, st>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src),
                                                               index, dim_size, inner_bytes, n_index, so, si, index_dtype);
  B200_CHECK_LAUNCH("index_copy_rows_kernel");
  return B200_OK;
}

extern "C" int b200_rope_table(const float* inv_freq, const void* positions, void* cos_out, void* sin_out, int64_t n_pos,
                               int head_dim, int pos_dtype, int out_dtype, void* stream) {
  B200_CHECK_ARG(inv_freq && positions && cos_out && sin_out && n_pos >= 0 && head_dim > 0 && head_dim % 2 == 0,
                 "b200_rope_table: bad arguments");
  if (n_pos == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(ceil_div(n_pos * head_dim, 128));
  B200_DISPATCH_FLOAT(out_dtype, T, {
    rope_table_kernel<T><<<grid, 128, 0, st>>>(inv_freq, positions, static_cast<T*>(cos_out), static_cast<T*>(sin_out), n_pos,
                                               head_dim, pos_dtype);
  });
  B200_CHECK_LAUNCH("rope_table_kernel");
  return B200_OK;
}

namespace {
// Fills `p` from the operands of one rotation; B200_OK or the error code (message set).
int rope_params(RopeParams& p, const char* who, const b200_tensor* x, const void* cos_t, const void* sin_t, void* y, void* kv_cache,
                const void* cache_pos, int64_t cache_len, int pos_dtype) {
  B200_CHECK_ARG(x && x->data && x->ndim == 4 && cos_t && sin_t && (y || kv_cache), "%s: bad arguments", who);
  B200_CHECK_ARG(x->stride[3] == 1 && x->shape[3] % 16 == 0, "%s: head_dim must be contiguous and a multiple of 16", who);
  B200_CHECK_ARG(!kv_cache || cache_pos, "%s: cache write needs cache_pos", who);
  p.x = x->data; p.cos_t = cos_t; p.sin_t = sin_t; p.y = y; p.cache = kv_cache; p.cache_pos = cache_pos;
  p.B = x->shape[0]; p.H = x->shape[1]; p.T = x->shape[2]; p.D = static_cast<int>(x->shape[3]);
  for (int i = 0; i < 3; ++i) p.xs[i] = x->stride[i];
  p.cache_len = cache_len; p.pos_dtype = pos_dtype;
  const bool ok = aligned16(x->data) && aligned16(cos_t) && aligned16(sin_t) && aligned16(kv_cache ? kv_cache : y) &&
                  p.xs[0] % 8 == 0 && p.xs[1] % 8 == 0 && p.xs[2] % 8 == 0;
  if (!ok) B200_FAIL(B200_EALIGN, "%s: operands must be 16-byte aligned with strides multiple of 8", who);
  return B200_OK;
}

int rope_launch(const RopeParams& p, int dtype, bool to_cache, cudaStream_t st) {
  const int64_t total = p.B * p.H * p.T * (p.D >> 4);
  if (total == 0) return B200_OK;
  const int64_t grid = ceil_div(total, 128);
  B200_CHECK_ARG(grid < (1ll << 31), "b200_rope_rotate: tensor too large");
  const bool small = total + 128 < (1ll << 32);
  const int64_t per_head = p.B * p.T * (p.D >> 4);
  B200_DISPATCH_HALF(dtype, T, {
    if (!to_cache && p.H >= 2 && per_head >= 4 * 64 * 148)   // enough positions to fill the GPU with one thread per (position, pack pair): below that (2048 tokens: 6.2 against 5.2 us) one thread per head wins
      rope_rotate_heads_kernel<T><<<static_cast<unsigned>(ceil_div(per_head, 128)), 128, 0, st>>>(p);
    else if (small) rope_rotate_kernel<T, uint32_t><<<static_cast<unsigned>(grid), 128, 0, st>>>(p);
    else rope_rotate_kernel<T, int64_t><<<static_cast<unsigned>(grid), 128, 0, st>>>(p);
  });
  B200_CHECK_LAUNCH("rope_rotate_kernel");
  return B200_OK;
}
}  // namespace

extern "C" int b200_rope_rotate(const b200_tensor* x, const void* cos_t, const void* sin_t, void* y, void* kv_cache,
                                const void* cache_pos, int64_t cache_len, int pos_dtype, void* stream) {
  RopeParams p;
  if (const int rc = rope_params(p, "b200_rope_rotate", x, cos_t, sin_t, y, kv_cache, cache_pos, cache_len, pos_dtype)) return rc;
  return rope_launch(p, x->dtype, kv_cache != nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_rope_rotate_pair(const b200_tensor* q, const b200_tensor* k, const void* cos_t, const void* sin_t, void* q_out,
                                     void* k_out, void* stream) {
  RopeParams pq, pk;
  if (const int rc = rope_params(pq, "b200_rope_rotate_pair", q, cos_t, sin_t, q_out, nullptr, nullptr, 0, 0)) return rc;
  if (const int rc = rope_params(pk, "b200_rope_rotate_pair", k, cos_t, sin_t, k_out, nullptr, nullptr, 0, 0)) return rc;
  B200_CHECK_ARG(q->dtype == k->dtype && pq.B == pk.B && pq.T == pk.T && pq.D == pk.D, "b200_rope_rotate_pair: q and k differ in dtype, batch, positions or head_dim");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t tq = pq.B * pq.H * pq.T * (pq.D >> 4), tk = pk.B * pk.H * pk.T * (pk.D >> 4);
  const int64_t per_head = pq.B * pq.T * (pq.D >> 4);
  // long prompts take the kernel that walks the heads of a position (two launches); an empty side needs none
  if (tq == 0 || tk == 0 || per_head >= 4 * 64 * 148 || tq + tk + 256 >= (1ll << 32)) {
    if (const int rc = rope_launch(pq, q->dtype, false, st)) return rc;
    return rope_launch(pk, k->dtype, false, st);
  }
  const unsigned qb = static_cast<unsigned>(ceil_div(tq, 128)), kb = static_cast<unsigned>(ceil_div(tk, 128));
  B200_DISPATCH_HALF(q->dtype, T, { launch_pdl(rope_rotate_pair_kernel<T>, dim3(qb + kb), dim3(128), 0, st, pq, pk, qb); });
  B200_CHECK_LAUNCH("rope_rotate_pair_kernel");
  return B200_OK;
}
