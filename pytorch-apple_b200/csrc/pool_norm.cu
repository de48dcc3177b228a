// CNN-side bandwidth kernels: pooling, inference batch-norm, and the one-off
// weight preparation that folds batch-norm into convolution weights.
// Activations are NCHW in shape with arbitrary strides; threads are laid out so
// that the memory-contiguous axis (W for NCHW, C for channels-last) varies fastest.
#include "common.cuh"

namespace b200 {

struct Pool4D {
  const void* x;
  void* y;
  int64_t N, C, H, W, OH, OW;
  int64_t xs[4], ys[4];
  int x_dtype, y_dtype;
  int kh, kw, sh, sw, ph, pw;
  int channels_last;  // thread order: (n, oh, ow, c) instead of (n, c, oh, ow)
};

__device__ __forceinline__ void decode_nchw(const Pool4D& p, int64_t i, int64_t& n, int64_t& c, int64_t& oh, int64_t& ow) {
  if (p.channels_last) {
    c = i % p.C; i /= p.C;
    ow = i % p.OW; i /= p.OW;
    oh = i % p.OH; n = i / p.OH;
  } else {
    ow = i % p.OW; i /= p.OW;
    oh = i % p.OH; i /= p.OH;
    c = i % p.C; n = i / p.C;
  }
}

__global__ void __launch_bounds__(256) max_pool2d_kernel(const __grid_constant__ Pool4D p) {
  const int64_t total = p.N * p.C * p.OH * p.OW;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int64_t n, c, oh, ow;
  decode_nchw(p, i, n, c, oh, ow);
  float best = -INFINITY;
  for (int r = 0; r < p.kh; ++r) {
    const int64_t ih = oh * p.sh - p.ph + r;
    if (ih < 0 || ih >= p.H) continue;
    for (int s = 0; s < p.kw; ++s) {
      const int64_t iw = ow * p.sw - p.pw + s;
      if (iw < 0 || iw >= p.W) continue;
      const float v = load_as_f32(p.x, n * p.xs[0] + c * p.xs[1] + ih * p.xs[2] + iw * p.xs[3], p.x_dtype);
      best = (v > best || v != v) ? v : best;
    }
  }
  store_from_f32(p.y, n * p.ys[0] + c * p.ys[1] + oh * p.ys[2] + ow * p.ys[3], p.y_dtype, best);
}

// Channels-last fast path: one thread owns 8 consecutive channels (16 bytes) of one output
// pixel; every tap is one 128-bit load.  NaN propagates as in the generic kernel.
template <typename T>
__global__ void __launch_bounds__(256) max_pool2d_cl8_kernel(const __grid_constant__ Pool4D p) {
  const int c8 = static_cast<int>(p.C / 8);
  const int64_t total = p.N * p.OH * p.OW * c8;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % c8) * 8; i /= c8;
  const int ow = static_cast<int>(i % p.OW); i /= p.OW;
  const int oh = static_cast<int>(i % p.OH);
  const int64_t n = i / p.OH;
  const T* xb = static_cast<const T*>(p.x) + n * p.xs[0] + c;
  float best[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) best[k] = -INFINITY;
  if (p.kh == 3 && p.kw == 3) {
    // The ResNet stem pool: all nine taps are requested before the first comparison (nine loads in
    // flight per thread instead of one after the other: 0.44 -> of the copy peak before).
    uint4 tap[9];
    bool in[9];
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const int ih = oh * p.sh - p.ph + r, iw = ow * p.sw - p.pw + s;
        in[3 * r + s] = ih >= 0 && ih < p.H && iw >= 0 && iw < p.W;
        if (in[3 * r + s]) tap[3 * r + s] = ld_global_nc_v4(xb + ih * p.xs[2] + iw * p.xs[3]);
      }
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      if (!in[j]) continue;
      float v[8];
      unpack8<T>(tap[j], v);
#pragma unroll
      for (int k = 0; k < 8; ++k) best[k] = (v[k] > best[k] || v[k] != v[k]) ? v[k] : best[k];
    }
    *reinterpret_cast<uint4*>(static_cast<T*>(p.y) + n * p.ys[0] + oh * p.ys[2] + ow * p.ys[3] + c) = pack8<T>(best);
    return;
  }
  for (int r = 0; r < p.kh; ++r) {
    const int ih = oh * p.sh - p.ph + r;
    if (ih < 0 || ih >= p.H) continue;
    for (int s = 0; s < p.kw; ++s) {
      const int iw = ow * p.sw - p.pw + s;
      if (iw < 0 || iw >= p.W) continue;
      float v[8];
      unpack8<T>(ld_global_nc_v4(xb + ih * p.xs[2] + iw * p.xs[3]), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) best[k] = (v[k] > best[k] || v[k] != v[k]) ? v[k] : best[k];
    }
  }
  *reinterpret_cast<uint4*>(static_cast<T*>(p.y) + n * p.ys[0] + oh * p.ys[2] + ow * p.ys[3] + c) = pack8<T>(best);
}

__global__ void __launch_bounds__(256) adaptive_avg_pool2d_kernel(const __grid_constant__ Pool4D p) {
  const int64_t total = p.N * p.C * p.OH * p.OW;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int64_t n, c, oh, ow;
  decode_nchw(p, i, n, c, oh, ow);
  const int64_t h0 = (oh * p.H) / p.OH, h1 = ((oh + 1) * p.H + p.OH - 1) / p.OH;
  const int64_t w0 = (ow * p.W) / p.OW, w1 = ((ow + 1) * p.W + p.OW - 1) / p.OW;
  float sum = 0.f;
  for (int64_t ih = h0; ih < h1; ++ih)
    for (int64_t iw = w0; iw < w1; ++iw)
      sum += load_as_f32(p.x, n * p.xs[0] + c * p.xs[1] + ih * p.xs[2] + iw * p.xs[3], p.x_dtype);
  store_from_f32(p.y, n * p.ys[0] + c * p.ys[1] + oh * p.ys[2] + ow * p.ys[3], p.y_dtype,
                 sum / static_cast<float>((h1 - h0) * (w1 - w0)));
}

__global__ void __launch_bounds__(256) batch_norm_kernel(const __grid_constant__ Pool4D p, const void* gamma, const void* beta,
                                                         const void* mean, const void* var, float eps, int param_dtype,
                                                         int relu) {
  const int64_t total = p.N * p.C * p.OH * p.OW;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int64_t n, c, h, w;
  decode_nchw(p, i, n, c, h, w);
  const float g = gamma ? load_as_f32(gamma, c, param_dtype) : 1.f;
  const float b = beta ? load_as_f32(beta, c, param_dtype) : 0.f;
  const float m = load_as_f32(mean, c, param_dtype);
  const float inv = 1.0f / sqrtf(load_as_f32(var, c, param_dtype) + eps);
  float v = load_as_f32(p.x, n * p.xs[0] + c * p.xs[1] + h * p.xs[2] + w * p.xs[3], p.x_dtype);
  v = (v - m) * inv * g + b;
  if (relu) v = fmaxf(v, 0.f);
  store_from_f32(p.y, n * p.ys[0] + c * p.ys[1] + h * p.ys[2] + w * p.ys[3], p.y_dtype, v);
}

// w OIHW -> [O][KH][KW][I_pad] scaled by gamma/sqrt(var+eps); bias = beta + (conv_bias - mean)*scale.
__global__ void __launch_bounds__(256) conv_weight_prep_kernel(const void* w, const void* conv_bias, const void* gamma,
                                                               const void* beta, const void* mean, const void* var, void* w_out,
                                                               float* bias_out, int O, int I, int KH, int KW, int I_pad, float eps,
                                                               int w_dtype, int param_dtype, int out_dtype) {
  const int64_t per_o = static_cast<int64_t>(KH) * KW * I_pad;
  const int64_t total = per_o * O;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int o = static_cast<int>(i / per_o);
  int64_t r = i % per_o;
  const int ci = static_cast<int>(r % I_pad); r /= I_pad;
  const int s = static_cast<int>(r % KW);
  const int kr = static_cast<int>(r / KW);
  float scale = 1.f;
  if (var) scale = (gamma ? load_as_f32(gamma, o, param_dtype) : 1.f) / sqrtf(load_as_f32(var, o, param_dtype) + eps);
  float v = 0.f;
  if (ci < I) v = load_as_f32(w, ((static_cast<int64_t>(o) * I + ci) * KH + kr) * KW + s, w_dtype) * scale;
  store_from_f32(w_out, i, out_dtype, v);
  if (r == 0 && ci == 0 && s == 0 && kr == 0) {
    float b = conv_bias ? load_as_f32(conv_bias, o, param_dtype) : 0.f;
    if (var) b = (beta ? load_as_f32(beta, o, param_dtype) : 0.f) + (b - load_as_f32(mean, o, param_dtype)) * scale;
    bias_out[o] = b;
  }
}

static int fill_pool(Pool4D* p, const b200_tensor* x, const b200_tensor* y) {
  if (!x || !y || !x->data || !y->data || x->ndim != 4 || y->ndim != 4) return -1;
  p->x = x->data; p->y = y->data;
  p->N = x->shape[0]; p->C = x->shape[1]; p->H = x->shape[2]; p->W = x->shape[3];
  p->OH = y->shape[2]; p->OW = y->shape[3];
  if (y->shape[0] != p->N || y->shape[1] != p->C) return -1;
  for (int i = 0; i < 4; ++i) { p->xs[i] = x->stride[i]; p->ys[i] = y->stride[i]; }
  p->x_dtype = x->dtype; p->y_dtype = y->dtype;
  p->channels_last = (y->stride[1] == 1 && p->C > 1) ? 1 : 0;
  p->kh = p->kw = p->sh = p->sw = 1; p->ph = p->pw = 0;
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_max_pool2d(const b200_tensor* x, const b200_tensor* y, int kh, int kw, int sh, int sw, int ph, int pw,
                               void* stream) {
  Pool4D p;
  B200_CHECK_ARG(fill_pool(&p, x, y) == 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0, "b200_max_pool2d: bad arguments");
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw;
  const int64_t total = p.N * p.C * p.OH * p.OW;
  if (total == 0) return B200_OK;
  const bool half_types = p.x_dtype == p.y_dtype && (p.x_dtype == B200_F16 || p.x_dtype == B200_BF16);
  if (half_types && p.channels_last && p.C % 8 == 0 && p.xs[1] == 1 && p.ys[1] == 1 && aligned16(p.x) && aligned16(p.y) &&
      p.xs[0] % 8 == 0 && p.xs[2] % 8 == 0 && p.xs[3] % 8 == 0 && p.ys[0] % 8 == 0 && p.ys[2] % 8 == 0 && p.ys[3] % 8 == 0) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(total / 8, 256));
    if (p.x_dtype == B200_F16) max_pool2d_cl8_kernel<__half><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    else max_pool2d_cl8_kernel<__nv_bfloat16><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    B200_CHECK_LAUNCH("max_pool2d_cl8_kernel");
    return B200_OK;
  }
  max_pool2d_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  B200_CHECK_LAUNCH("max_pool2d_kernel");
  return B200_OK;
}

extern "C" int b200_adaptive_avg_pool2d(const b200_tensor* x, const b200_tensor* y, void* stream) {
  Pool4D p;
  B200_CHECK_ARG(fill_pool(&p, x, y) == 0 && p.OH > 0 && p.OW > 0, "b200_adaptive_avg_pool2d: bad arguments");
  const int64_t total = p.N * p.C * p.OH * p.OW;
  if (total == 0) return B200_OK;
  adaptive_avg_pool2d_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  B200_CHECK_LAUNCH("adaptive_avg_pool2d_kernel");
  return B200_OK;
}

extern "C" int b200_batch_norm(const b200_tensor* x, const b200_tensor* y, const void* gamma, const void* beta,
                               const void* mean, const void* var, float eps, int param_dtype, int relu, void* stream) {
  Pool4D p;
  B200_CHECK_ARG(fill_pool(&p, x, y) == 0 && mean && var, "b200_batch_norm: bad arguments");
  B200_CHECK_ARG(p.OH == p.H && p.OW == p.W, "b200_batch_norm: shape mismatch");
  const int64_t total = p.N * p.C * p.H * p.W;
  if (total == 0) return B200_OK;
  batch_norm_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      p, gamma, beta, mean, var, eps, param_dtype, relu);
  B200_CHECK_LAUNCH("batch_norm_kernel");
  return B200_OK;
}

extern "C" int b200_conv_weight_prep(const void* w, const void* conv_bias, const void* gamma, const void* beta,
                                     const void* mean, const void* var, void* w_out, float* bias_out, int O, int I, int KH,
                                     int KW, int I_pad, float eps, int w_dtype, int param_dtype, int out_dtype, void* stream) {
  B200_CHECK_ARG(w && w_out && bias_out && O > 0 && I > 0 && KH > 0 && KW > 0 && I_pad >= I, "b200_conv_weight_prep: bad arguments");
  B200_CHECK_ARG((var == nullptr) == (mean == nullptr), "b200_conv_weight_prep: mean and var go together");
  const int64_t total = static_cast<int64_t>(O) * KH * KW * I_pad;
  conv_weight_prep_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, conv_bias, gamma, beta, mean, var, w_out, bias_out, O, I, KH, KW, I_pad, eps, w_dtype, param_dtype, out_dtype);
  B200_CHECK_LAUNCH("conv_weight_prep_kernel");
  return B200_OK;
}
