// Fused elementwise chains, strided copies and fills.
//
// A chain is a short program (b200_ew_op[]) evaluated per output element in fp32
// with the result of every op rounded to the dtype the IR assigns to it.  Chains
// that the two model families actually contain (relu, add, add+relu, silu*mul,
// scalar scale) are recognised on the host and run as 128-bit vectorised kernels
// over flat memory; everything else goes through a strided interpreter.
#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// Dimension coalescing shared by ew_chain and strided_copy.
// ---------------------------------------------------------------------------
struct IterDims {
  int ndim;
  int64_t shape[B200_MAX_DIMS];
  int64_t stride[1 + B200_EW_MAX_INPUTS][B200_MAX_DIMS];  // [0] = output
};

// Merge adjacent dims that are contiguous for every operand; drop size-1 dims.
static int64_t coalesce(const b200_tensor* out, const b200_tensor* const* ins, int n_in, IterDims* it) {
  int nd = 0;
  int64_t total = 1;
  for (int d = 0; d < out->ndim; ++d) {
    int64_t ext = out->shape[d];
    total *= ext;
    if (ext == 1) continue;
    bool merged = false;
    if (nd > 0) {
      bool ok = it->stride[0][nd - 1] == out->stride[d] * ext;
      for (int k = 0; ok && k < n_in; ++k) ok = it->stride[1 + k][nd - 1] == ins[k]->stride[d] * ext;
      if (ok) {
        it->shape[nd - 1] *= ext;
        it->stride[0][nd - 1] = out->stride[d];
        for (int k = 0; k < n_in; ++k) it->stride[1 + k][nd - 1] = ins[k]->stride[d];
        merged = true;
      }
    }
    if (!merged) {
      it->shape[nd] = ext;
      it->stride[0][nd] = out->stride[d];
      for (int k = 0; k < n_in; ++k) it->stride[1 + k][nd] = ins[k]->stride[d];
      ++nd;
    }
  }
  if (nd == 0) {
    nd = 1;
    it->shape[0] = 1;
    for (int k = 0; k <= n_in; ++k) it->stride[k][0] = 1;
  }
  it->ndim = nd;
  return total;
}

// ---------------------------------------------------------------------------
// Generic interpreter.
// ---------------------------------------------------------------------------
struct ChainParams {
  IterDims it;
  void* out;
  const void* in[B200_EW_MAX_INPUTS];
  int out_dtype;
  int in_dtype[B200_EW_MAX_INPUTS];
  int n_in, n_ops;
  int64_t total;
  b200_ew_op ops[B200_EW_MAX_OPS];
};

__device__ __forceinline__ float apply_op(int opcode, float a, float b, float imm) {
  switch (opcode) {
    case B200_EW_RELU: return a != a ? a : fmaxf(a, 0.f);
    case B200_EW_SILU: return a / (1.f + expf(-a));
    case B200_EW_NEG: return -a;
    case B200_EW_RSQRT: return rsqrtf(a);
    case B200_EW_COS: return cosf(a);
    case B200_EW_SIN: return sinf(a);
    case B200_EW_ADD: return a + b;
    case B200_EW_MUL: return a * b;
    case B200_EW_DIV: return a / b;
    case B200_EW_SUB: return a - b;
    case B200_EW_ADD_S: return a + imm;
    case B200_EW_MUL_S: return a * imm;
    case B200_EW_DIV_S: return a / imm;
    case B200_EW_POW_S: return imm == 2.f ? a * a : powf(a, imm);
    case B200_EW_SUB_S: return a - imm;
    case B200_EW_RSUB_S: return imm - a;
    case B200_EW_CAST: return a;
    case B200_EW_SIGMOID: return 1.f / (1.f + expf(-a));
    case B200_EW_EXP: return expf(a);
    case B200_EW_SQRT: return sqrtf(a);
    case B200_EW_TANH: return tanhf(a);
    case B200_EW_GELU: return 0.5f * a * (1.f + erff(a * 0.70710678118654752f));
    case B200_EW_MAX: return fmaxf(a, b);
    case B200_EW_MIN: return fminf(a, b);
  }
  return a;
}

__global__ void __launch_bounds__(256) ew_chain_generic_kernel(const __grid_constant__ ChainParams p) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t off[1 + B200_EW_MAX_INPUTS] = {0, 0, 0, 0, 0};
    int64_t rem = i;
    for (int d = p.it.ndim - 1; d >= 0; --d) {
      const int64_t ext = p.it.shape[d];
      const int64_t c = rem % ext;
      rem /= ext;
      off[0] += c * p.it.stride[0][d];
#pragma unroll
      for (int k = 0; k < B200_EW_MAX_INPUTS; ++k)
        if (k < p.n_in) off[1 + k] += c * p.it.stride[1 + k][d];
    }
    float slot[B200_EW_MAX_INPUTS + B200_EW_MAX_OPS];
#pragma unroll
    for (int k = 0; k < B200_EW_MAX_INPUTS; ++k)
      slot[k] = k < p.n_in ? load_as_f32(p.in[k], off[1 + k], p.in_dtype[k]) : 0.f;
    float r = slot[0];
    for (int j = 0; j < p.n_ops; ++j) {
      const b200_ew_op op = p.ops[j];
      const float a = slot[op.a];
      const float b = op.b >= 0 ? slot[op.b] : 0.f;
      r = round_to(apply_op(op.opcode, a, b, op.imm), op.round_dtype);
      slot[B200_EW_MAX_INPUTS + j] = r;
    }
    store_from_f32(p.out, off[0], p.out_dtype, r);
  }
}

// ---------------------------------------------------------------------------
// Vectorised flat kernels for the recognised chains.
// ---------------------------------------------------------------------------
enum FlatKind { FLAT_NONE = 0, FLAT_RELU, FLAT_ADD, FLAT_ADD_RELU, FLAT_SILU_MUL, FLAT_MUL, FLAT_MUL_S, FLAT_ADD_S };

template <typename T, int KIND> __device__ __forceinline__ float flat_eval(float a, float b, float imm) {
  if (KIND == FLAT_RELU) return a != a ? a : fmaxf(a, 0.f);
  if (KIND == FLAT_ADD) return a + b;
  if (KIND == FLAT_ADD_RELU) { float s = round_as<T>(a + b); return s != s ? s : fmaxf(s, 0.f); }
  if (KIND == FLAT_SILU_MUL) { float s = round_as<T>(silu_f32(a)); return s * b; }
  if (KIND == FLAT_MUL) return a * b;
  if (KIND == FLAT_MUL_S) return a * imm;
  if (KIND == FLAT_ADD_S) return a + imm;
  return a;
}

// 8 elements (16 bytes) per thread per step; n8 = number of full 8-packs.
template <typename T, int KIND, bool BINARY>
__global__ void __launch_bounds__(256) ew_flat_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                      int64_t n, float imm) {
  const int64_t n8 = n >> 3;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const uint4* a4 = reinterpret_cast<const uint4*>(a);
  const uint4* b4 = reinterpret_cast<const uint4*>(b);
  uint4* o4 = reinterpret_cast<uint4*>(out);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    float fa[8], fb[8], fo[8];
    unpack8<T>(ld_global_nc_v4(a4 + i), fa);
    if (BINARY) unpack8<T>(ld_global_nc_v4(b4 + i), fb);
#pragma unroll
    for (int k = 0; k < 8; ++k) fo[k] = flat_eval<T, KIND>(fa[k], BINARY ? fb[k] : 0.f, imm);
    o4[i] = pack8<T>(fo);
  }
  // tail (< 8 elements) by the first threads of block 0
  if (blockIdx.x == 0) {
    const int64_t i = (n8 << 3) + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(flat_eval<T, KIND>(to_f32<T>(a[i]), BINARY ? to_f32<T>(b[i]) : 0.f, imm));
  }
}

static FlatKind classify_flat(const b200_ew_op* ops, int n_ops, int n_in, int dt) {
  auto same = [&](int j) { return ops[j].round_dtype == dt; };
  if (n_ops == 1 && same(0)) {
    const b200_ew_op& o = ops[0];
    if (n_in == 1 && o.a == 0) {
      if (o.opcode == B200_EW_RELU) return FLAT_RELU;
      if (o.opcode == B200_EW_MUL_S) return FLAT_MUL_S;
      if (o.opcode == B200_EW_ADD_S) return FLAT_ADD_S;
    }
    if (n_in == 2 && ((o.a == 0 && o.b == 1) || (o.a == 1 && o.b == 0))) {
      if (o.opcode == B200_EW_ADD) return FLAT_ADD;
      if (o.opcode == B200_EW_MUL) return FLAT_MUL;
    }
  }
  if (n_ops == 2 && n_in == 2 && same(0) && same(1)) {
    const b200_ew_op &o0 = ops[0], &o1 = ops[1];
    const int r0 = B200_EW_MAX_INPUTS;  // slot of op 0's result
    if (o0.opcode == B200_EW_ADD && ((o0.a == 0 && o0.b == 1) || (o0.a == 1 && o0.b == 0)) &&
        o1.opcode == B200_EW_RELU && o1.a == r0)
      return FLAT_ADD_RELU;
    // silu(in0) * in1, in either operand order of the mul
    if (o0.opcode == B200_EW_SILU && o0.a == 0 && o1.opcode == B200_EW_MUL &&
        ((o1.a == r0 && o1.b == 1) || (o1.a == 1 && o1.b == r0)))
      return FLAT_SILU_MUL;
  }
  return FLAT_NONE;
}

template <typename T>
static void launch_flat(FlatKind kind, const void* a, const void* b, void* out, int64_t n, float imm, cudaStream_t st) {
  const int64_t n8 = n >> 3;
  int64_t blocks = ceil_div(n8 > 0 ? n8 : 1, 256);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  const T* pa = static_cast<const T*>(a);
  const T* pb = static_cast<const T*>(b);
  T* po = static_cast<T*>(out);
  switch (kind) {
    case FLAT_RELU: ew_flat_kernel<T, FLAT_RELU, false><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    case FLAT_MUL_S: ew_flat_kernel<T, FLAT_MUL_S, false><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    case FLAT_ADD_S: ew_flat_kernel<T, FLAT_ADD_S, false><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    case FLAT_ADD: ew_flat_kernel<T, FLAT_ADD, true><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    case FLAT_MUL: ew_flat_kernel<T, FLAT_MUL, true><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    case FLAT_ADD_RELU: ew_flat_kernel<T, FLAT_ADD_RELU, true><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    case FLAT_SILU_MUL: ew_flat_kernel<T, FLAT_SILU_MUL, true><<<blocks, 256, 0, st>>>(pa, pb, po, n, imm); break;
    default: break;
  }
}

// ---------------------------------------------------------------------------
// Strided copy.
// ---------------------------------------------------------------------------
struct CopyParams {
  IterDims it;
  void* out;
  const void* in;
  int out_dtype, in_dtype;
  int64_t total;
};

// Planar -> interleaved for up to 8 channels of a 16-bit type: in [N, C, H, W] contiguous,
// out [N, C, H, W] viewed with strides (S0, 1, 8 W, 8) - channels-last with room for 8.  One
// thread per pixel: C coalesced 2-byte reads (one per plane), then the pixel's 16-byte slot is
// read, the C channels replaced and written back whole (channels C..7 keep their contents), so
// DRAM sees full sectors instead of masked 2-byte writes.
__global__ void __launch_bounds__(256) interleave8_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int64_t pixels,
                                                          int64_t hw, int C, int64_t out_s0) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= pixels) return;
  const int64_t n = gid / hw, r = gid - n * hw;
  const uint16_t* src = in + n * C * hw + r;
  uint4* slot = reinterpret_cast<uint4*>(out + n * out_s0 + r * 8);
  uint16_t v[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) v[c] = c < C ? src[c * hw] : uint16_t(0);
  uint4 cur = *slot;
  uint32_t w[4] = {cur.x, cur.y, cur.z, cur.w};
#pragma unroll
  for (int c = 0; c < 8; ++c)
    if (c < C) w[c >> 1] = (c & 1) ? ((w[c >> 1] & 0x0000ffffu) | (static_cast<uint32_t>(v[c]) << 16)) : ((w[c >> 1] & 0xffff0000u) | v[c]);
  *slot = make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename U>
__global__ void __launch_bounds__(256) strided_copy_raw_kernel(const __grid_constant__ CopyParams p) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t oo = 0, io = 0, rem = i;
    for (int d = p.it.ndim - 1; d >= 0; --d) {
      const int64_t ext = p.it.shape[d];
      const int64_t c = rem % ext;
      rem /= ext;
      oo += c * p.it.stride[0][d];
      io += c * p.it.stride[1][d];
    }
    static_cast<U*>(p.out)[oo] = static_cast<const U*>(p.in)[io];
  }
}

__global__ void __launch_bounds__(256) strided_copy_convert_kernel(const __grid_constant__ CopyParams p) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += stride) {
    int64_t oo = 0, io = 0, rem = i;
    for (int d = p.it.ndim - 1; d >= 0; --d) {
      const int64_t ext = p.it.shape[d];
      const int64_t c = rem % ext;
      rem /= ext;
      oo += c * p.it.stride[0][d];
      io += c * p.it.stride[1][d];
    }
    if (p.in_dtype == B200_I64 && p.out_dtype == B200_I32)
      static_cast<int32_t*>(p.out)[oo] = static_cast<int32_t>(static_cast<const int64_t*>(p.in)[io]);
    else if (p.in_dtype == B200_I32 && p.out_dtype == B200_I64)
      static_cast<int64_t*>(p.out)[oo] = static_cast<const int32_t*>(p.in)[io];
    else
      store_from_f32(p.out, oo, p.out_dtype, load_as_f32(p.in, io, p.in_dtype));
  }
}

template <typename T> __global__ void __launch_bounds__(256) fill_kernel(T* out, int64_t n, T value) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}

static int grid_for(int64_t total) {
  int64_t blocks = ceil_div(total > 0 ? total : 1, 256);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(blocks > cap ? cap : blocks);
}

static bool check_tensor(const b200_tensor* t) {
  return t && t->data && t->ndim >= 0 && t->ndim <= B200_MAX_DIMS && dtype_size(t->dtype) > 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_ew_chain(const b200_tensor* out, const b200_tensor* ins, int n_in, const b200_ew_op* ops,
                             int n_ops, void* stream) {
  B200_CHECK_ARG(check_tensor(out), "b200_ew_chain: bad output tensor");
  B200_CHECK_ARG(n_in >= 1 && n_in <= B200_EW_MAX_INPUTS, "b200_ew_chain: n_in=%d out of range", n_in);
  B200_CHECK_ARG(n_ops >= 1 && n_ops <= B200_EW_MAX_OPS, "b200_ew_chain: n_ops=%d out of range", n_ops);
  const b200_tensor* inp[B200_EW_MAX_INPUTS];
  for (int k = 0; k < n_in; ++k) {
    B200_CHECK_ARG(check_tensor(&ins[k]) && ins[k].ndim == out->ndim, "b200_ew_chain: bad input %d", k);
    for (int d = 0; d < out->ndim; ++d)
      B200_CHECK_ARG(ins[k].shape[d] == out->shape[d], "b200_ew_chain: input %d shape differs at dim %d", k, d);
    inp[k] = &ins[k];
  }
  for (int j = 0; j < n_ops; ++j) {
    const int lim = B200_EW_MAX_INPUTS + j;
    B200_CHECK_ARG(ops[j].a >= 0 && ops[j].a < lim && (ops[j].a >= B200_EW_MAX_INPUTS || ops[j].a < n_in),
                   "b200_ew_chain: op %d operand a=%d invalid", j, ops[j].a);
    B200_CHECK_ARG(ops[j].b < lim && (ops[j].b < 0 || ops[j].b >= B200_EW_MAX_INPUTS || ops[j].b < n_in),
                   "b200_ew_chain: op %d operand b=%d invalid", j, ops[j].b);
  }
  ChainParams p;
  p.total = coalesce(out, inp, n_in, &p.it);
  if (p.total == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // flat, same 16-bit dtype, aligned -> vector kernels
  const int dt = out->dtype;
  bool flat = p.it.ndim == 1 && p.it.stride[0][0] == 1 && (dt == B200_BF16 || dt == B200_F16) && aligned16(out->data);
  for (int k = 0; flat && k < n_in; ++k)
    flat = p.it.stride[1 + k][0] == 1 && ins[k].dtype == dt && aligned16(ins[k].data);
  if (flat) {
    const FlatKind kind = classify_flat(ops, n_ops, n_in, dt);
    if (kind != FLAT_NONE) {
      const void* a = ins[0].data;
      const void* b = n_in > 1 ? ins[1].data : ins[0].data;
      if ((kind == FLAT_ADD || kind == FLAT_MUL) && ops[0].a == 1) { a = ins[1].data; b = ins[0].data; }
      if (dt == B200_BF16) launch_flat<__nv_bfloat16>(kind, a, b, out->data, p.total, ops[0].imm, st);
      else launch_flat<__half>(kind, a, b, out->data, p.total, ops[0].imm, st);
      B200_CHECK_LAUNCH("ew_flat_kernel");
      return B200_OK;
    }
  }
  p.out = out->data;
  p.out_dtype = out->dtype;
  p.n_in = n_in;
  p.n_ops = n_ops;
  for (int k = 0; k < B200_EW_MAX_INPUTS; ++k) {
    p.in[k] = k < n_in ? ins[k].data : nullptr;
    p.in_dtype[k] = k < n_in ? ins[k].dtype : 0;
  }
  for (int j = 0; j < n_ops; ++j) p.ops[j] = ops[j];
  ew_chain_generic_kernel<<<grid_for(p.total), 256, 0, st>>>(p);
  B200_CHECK_LAUNCH("ew_chain_generic_kernel");
  return B200_OK;
}

extern "C" int b200_strided_copy(const b200_tensor* out, const b200_tensor* in, void* stream) {
  B200_CHECK_ARG(check_tensor(out) && check_tensor(in) && in->ndim == out->ndim, "b200_strided_copy: bad tensors");
  for (int d = 0; d < out->ndim; ++d)
    B200_CHECK_ARG(in->shape[d] == out->shape[d], "b200_strided_copy: shape differs at dim %d", d);
  if (out->ndim == 4 && out->dtype == in->dtype && dtype_size(out->dtype) == 2 && out->shape[1] >= 2 && out->shape[1] <= 8) {
    // planar -> channels-last with 8-channel slots (the input repack of a convolution network)
    const int64_t N = out->shape[0], C = out->shape[1], H = out->shape[2], W = out->shape[3], hw = H * W;
    const bool planar = in->stride[3] == 1 && in->stride[2] == W && in->stride[1] == hw && (N == 1 || in->stride[0] == C * hw);
    const bool slots = out->stride[1] == 1 && out->stride[3] == 8 && out->stride[2] == 8 * W && (N == 1 || out->stride[0] % 8 == 0) &&
                       aligned16(out->data);
    if (planar && slots && N * hw > 0) {
      const int64_t pixels = N * hw;
      interleave8_kernel<<<static_cast<unsigned>(ceil_div(pixels, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const uint16_t*>(in->data), static_cast<uint16_t*>(out->data), pixels, hw, static_cast<int>(C), N == 1 ? 0 : out->stride[0]);
      B200_CHECK_LAUNCH("interleave8_kernel");
      return B200_OK;
    }
  }
  CopyParams p;
  const b200_tensor* inp[1] = {in};
  p.total = coalesce(out, inp, 1, &p.it);
  if (p.total == 0) return B200_OK;
  p.out = out->data;
  p.in = in->data;
  p.out_dtype = out->dtype;
  p.in_dtype = in->dtype;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int esz = dtype_size(out->dtype);
  if (out->dtype == in->dtype) {
    const int last = p.it.ndim - 1;
    if (p.it.ndim == 1 && p.it.stride[0][0] == 1 && p.it.stride[1][0] == 1) {
      cudaError_t e = cudaMemcpyAsync(p.out, p.in, static_cast<size_t>(p.total) * esz, cudaMemcpyDeviceToDevice, st);
      if (e != cudaSuccess) B200_FAIL(B200_ELAUNCH, "b200_strided_copy: %s", cudaGetErrorString(e));
      return B200_OK;
    }
    // 16-byte units when the innermost run is contiguous on both sides and everything is aligned
    const int per16 = 16 / esz;
    bool v16 = p.it.stride[0][last] == 1 && p.it.stride[1][last] == 1 && p.it.shape[last] % per16 == 0 &&
               aligned16(p.out) && aligned16(p.in);
    for (int d = 0; v16 && d < last; ++d) v16 = p.it.stride[0][d] % per16 == 0 && p.it.stride[1][d] % per16 == 0;
    if (v16) {
      p.it.shape[last] /= per16;
      for (int d = 0; d < last; ++d) { p.it.stride[0][d] /= per16; p.it.stride[1][d] /= per16; }
      p.total /= per16;
      strided_copy_raw_kernel<uint4><<<grid_for(p.total), 256, 0, st>>>(p);
    } else if (esz == 2) strided_copy_raw_kernel<uint16_t><<<grid_for(p.total), 256, 0, st>>>(p);
    else if (esz == 4) strided_copy_raw_kernel<uint32_t><<<grid_for(p.total), 256, 0, st>>>(p);
    else if (esz == 8) strided_copy_raw_kernel<uint64_t><<<grid_for(p.total), 256, 0, st>>>(p);
    else strided_copy_raw_kernel<uint8_t><<<grid_for(p.total), 256, 0, st>>>(p);
  } else {
    strided_copy_convert_kernel<<<grid_for(p.total), 256, 0, st>>>(p);
  }
  B200_CHECK_LAUNCH("strided_copy_kernel");
  return B200_OK;
}

extern "C" int b200_fill(void* out, int64_t n, double value, int dtype, void* stream) {
  B200_CHECK_ARG(out != nullptr && n >= 0, "b200_fill: bad arguments");
  if (n == 0) return B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = grid_for(n);
  switch (dtype) {
    case B200_F32: fill_kernel<float><<<g, 256, 0, st>>>(static_cast<float*>(out), n, static_cast<float>(value)); break;
    case B200_F16: fill_kernel<__half><<<g, 256, 0, st>>>(static_cast<__half*>(out), n, __float2half_rn(static_cast<float>(value))); break;
    case B200_BF16: fill_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<__nv_bfloat16*>(out), n, __float2bfloat16_rn(static_cast<float>(value))); break;
    case B200_I32: fill_kernel<int32_t><<<g, 256, 0, st>>>(static_cast<int32_t*>(out), n, static_cast<int32_t>(value)); break;
    case B200_I64: fill_kernel<int64_t><<<g, 256, 0, st>>>(static_cast<int64_t*>(out), n, static_cast<int64_t>(value)); break;
    case B200_U8: fill_kernel<uint8_t><<<g, 256, 0, st>>>(static_cast<uint8_t*>(out), n, static_cast<uint8_t>(value)); break;
    default: B200_FAIL(B200_ENOTSUP, "b200_fill: dtype %d", dtype);
  }
  B200_CHECK_LAUNCH("fill_kernel");
  return B200_OK;
}
