// Interface between the GEMM dispatcher (gemm.cu) and the tcgen05 kernel (gemm_tc5.cu).
#pragma once
#include "common.cuh"

namespace b200 {

struct Tc5Args {
  const void* A; const void* W; const void* bias; const void* residual; const void* aux; void* out;
  int64_t M, N, K, lda, ldw, ldo, ldr, ldaux;
  int dtype, bias_dtype, epilogue;
  void* workspace;          // unused by the tcgen05 path (split-K needs no global scratch); kept for the dispatcher's fallbacks
  int64_t workspace_bytes;
  // Decode shapes (M <= 64) only.  sumsq_in != nullptr: every output row m is multiplied, before the
  // bias, by r_m = 1 / sqrt(s_m / K + norm_eps), s_m = sum of sumsq_in[m * sumsq_in_cols + 0..sumsq_in_cols)
  // - the RMSNorm of the input rows, applied after the GEMM (the caller folds the gain into W's columns).
  // sumsq_out != nullptr: the kernel also writes, for every output row m and every block of 64 output
  // columns j, the sum of squares of the (rounded) outputs: sumsq_out[m * (N / 64) + j].
  float norm_eps = 0.f;
  const float* sumsq_in = nullptr;
  int sumsq_in_cols = 0;
  float* sumsq_out = nullptr;
  // Decode shapes only, out == nullptr: the GEMM is the merged q/k/v projection of one token per row
  // (N = (Hq + 2 Hkv) * 128, head h = columns [128 h, 128 h + 128)) and its final pass applies the rotary
  // embedding and writes the destinations of the three groups itself: rope(q) to q_out [M, Hq, 128],
  // rope(k) and v into row cache_pos[0] of the caches [M, Hkv, cache_len, 128].
  struct Rope {
    const void* cos = nullptr; const void* sin = nullptr;   // [M, 128] tables of the rows' positions
    void* q_out = nullptr; void* k_cache = nullptr; void* v_cache = nullptr;
    const void* cache_pos = nullptr;
    int64_t cache_len = 0;
    int Hq = 0, Hkv = 0, pos_dtype = 0;
  } rope;
  // RMSNorm of the output rows as a tail of the GEMM (b200_linear_rmsnorm): norm_out[m, :] =
  // rmsnorm(out[m, :]) * gain, same roundings as b200_rmsnorm.  Only the split-K reduce kernel of the
  // CTA-pair path can take it (one block per output row); it sets *done, otherwise the caller runs the
  // RMSNorm kernel after the GEMM.
  struct NormTail {
    const void* gain = nullptr; void* out = nullptr;
    int64_t ld = 0;
    float eps = 0.f;
    int round_mid = 0;
    int* done = nullptr;
  } norm_tail;
};

// Geometry of an NHWC convolution run as an implicit GEMM (A rows are output pixels,
// k runs over (filter row, filter column, channel)).
struct Tc5Conv {
  int H, W, C, KH, KW, sh, sw, ph, pw, Ho, Wo;
  int batch = 0;    // images
  int im2col = 0;   // set by conv_tc5: the A tile comes from an im2col-mode tensor map (else gathered by threads)
  int c8 = 0;       // 8-channel input (the padded RGB stem): one filter tap per 16-byte K chunk, unswizzled operands
};

// y = epi(conv(x, w) + bias + residual) on the tcgen05 path; needs C % 64 == 0, or C == 8
// (stem convolution after channel padding) with O <= 64.
// Args: A = x [N,H,W,C], W = packed weights [O, KH*KW*C], M = N*Ho*Wo, N = O, K = KH*KW*C.
int conv_tc5(const Tc5Args& a, const Tc5Conv& g, cudaStream_t stream);

// out = epi(A W^T + bias + residual) on the tcgen05 path.  Returns B200_ENOTSUP when the
// operands do not meet the TMA alignment rules (the caller then uses the mma.sync tiles).
int linear_tc5(const Tc5Args& a, cudaStream_t stream);
bool tc5_enabled();
// Scratch bytes linear_tc5 needs for (M, N, K): always 0.
int64_t linear_tc5_workspace_bytes(int64_t M, int64_t N, int64_t K);

}  // namespace b200
