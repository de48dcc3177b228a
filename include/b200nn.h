/*
 * b200nn - fixed library of hand-written sm_100a kernels behind a C ABI.
 *
 * This is the device side of the CUDA backend for the PyTorch-IR compiler: the
 * Python host (cuda_compiler / cuda_runtime) lowers an IR subgraph to a list of
 * calls into this library and issues them through ctypes.  The reference
 * backend has no native boundary of its own - it JIT-compiles CUDA C strings with
 * NVRTC through CuPy and calls cuBLAS via cupy.matmul - so every entry point
 * below cites the reference kernel template or executor dispatch it replaces.
 *
 * Conventions
 *   - every call returns 0 on success or a negative B200_E* code; the message is
 *     available from b200_last_error() (thread local);
 *   - calls only enqueue work on `stream` (a cudaStream_t passed as void*); they
 *     never synchronise, never allocate device memory and never free it, so a
 *     sequence of calls can be captured into a CUDA graph;
 *   - device pointers are plain pointers; sizes are element counts unless a name
 *     says bytes; `dtype` arguments take the B200_* codes below;
 *   - strided operands are described by b200_tensor (element strides).
 */
#ifndef B200NN_H
#define B200NN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200NN_VERSION 1

/* status codes */
#define B200_OK 0
#define B200_EINVAL (-1)   /* bad argument (shape, dtype, null pointer)        */
#define B200_EALIGN (-2)   /* pointer or stride not aligned as the kernel needs */
#define B200_ELAUNCH (-3)  /* the CUDA runtime refused the launch               */
#define B200_ENOTSUP (-4)  /* combination not implemented                       */
#define B200_ELIMIT (-5)   /* size beyond a documented maximum                  */

/* element types */
#define B200_F32 0
#define B200_F16 1
#define B200_BF16 2
#define B200_I32 3
#define B200_I64 4
#define B200_U8 5

#define B200_MAX_DIMS 6

typedef struct b200_tensor {
  void* data;
  int32_t dtype;
  int32_t ndim;
  int64_t shape[B200_MAX_DIMS];
  int64_t stride[B200_MAX_DIMS]; /* in elements; 0 = broadcast */
} b200_tensor;

int b200_version(void);
const char* b200_last_error(void);
/* Diagnostic: the kernels' bounded waits (mbarrier waits of the tcgen05 GEMM) record a
 * non-zero code in a device variable when they give up instead of hanging.  Reads (and
 * optionally clears) it; this call synchronises the device. */
int b200_debug_device_error(int* code, int clear);
/* Self-test of the time-out path, for hosts that want to see it work: launches a one-thread
 * kernel that waits on a barrier nobody will ever arrive at, with the library's bounded wait
 * limited to `probes` polls.  The wait gives up, the kernel records code 99 and returns
 * normally; b200_debug_device_error then reports 99 and the context stays usable.
 * No counterpart in the reference (its kernels never wait on one another). */
int b200_debug_wait_timeout(int probes, void* stream);
/* sm count, compute capability and opt-in shared memory of device `dev`. */
int b200_device_info(int dev, int* sm_count, int* cc_major, int* cc_minor, int64_t* smem_optin_bytes);

/* ------------------------------------------------------------------------- *
 * Fused elementwise chains.
 * Replaces the NVRTC-generated `fused_ew_<i>` kernels
 * (cuda_compiler/cuda_codegen.py:47-142, launched at
 * cuda_runtime/cuda_executor.py:358-376).  The reference emits one __half
 * kernel per chain and indexes every operand with the flat output index; here a
 * chain is a short program interpreted per element in fp32, operands may be
 * broadcast/strided, and every intermediate is rounded to the dtype the IR gives
 * it, which is what ATen does op by op.
 * ------------------------------------------------------------------------- */
enum b200_ew_opcode {
  B200_EW_RELU = 1, B200_EW_SILU, B200_EW_NEG, B200_EW_RSQRT, B200_EW_COS, B200_EW_SIN,
  B200_EW_ADD, B200_EW_MUL, B200_EW_DIV, B200_EW_SUB,
  B200_EW_ADD_S, B200_EW_MUL_S, B200_EW_DIV_S, B200_EW_POW_S, B200_EW_SUB_S, B200_EW_CAST,
  B200_EW_SIGMOID, B200_EW_EXP, B200_EW_SQRT, B200_EW_TANH, B200_EW_GELU, B200_EW_RSUB_S, B200_EW_MAX, B200_EW_MIN
};

#define B200_EW_MAX_INPUTS 4
#define B200_EW_MAX_OPS 12

typedef struct b200_ew_op {
  int32_t opcode;      /* b200_ew_opcode */
  int32_t a;           /* operand slot: 0..3 = inputs, 4+i = result of op i */
  int32_t b;           /* second operand slot (binary ops), else -1 */
  int32_t round_dtype; /* B200_F32/F16/BF16: dtype the result is rounded to */
  float imm;           /* scalar for the *_S opcodes */
} b200_ew_op;

/* out[i] = chain(in0[i], in1[i], ...).  Inputs must already be expressed in the
 * output's index space (same ndim and shape, stride 0 where broadcast). */
int b200_ew_chain(const b200_tensor* out, const b200_tensor* ins, int n_in,
                  const b200_ew_op* ops, int n_ops, void* stream);

/* Strided gather copy with dtype conversion: out[idx] = (out dtype) in[idx].
 * Replaces transpose_kernel / slice_kernel / expand_kernel / cat_2_kernel
 * (cuda_compiler/cuda_templates.py:164-302), which the reference executor
 * substitutes with CuPy views and implicit copies
 * (cuda_runtime/cuda_executor.py:596-649).
 * A 16-bit [N, C<=8, H, W] output whose strides are (s0, 1, 8W, 8) is treated as a window
 * of a channels-last buffer with 8-channel slots: each pixel's 16-byte slot is read,
 * the C channels replaced and the slot written back, so all 8 channels of every slot
 * must be addressable (they keep their contents). */
int b200_strided_copy(const b200_tensor* out, const b200_tensor* in, void* stream);

/* full_kernel (cuda_templates.py:304-313): fill `n` elements with `value`. */
int b200_fill(void* out, int64_t n, double value, int dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Row reductions.
 * ------------------------------------------------------------------------- */
/* rmsnorm_kernel (cuda_templates.py:458-506; matcher
 * cuda_compiler/subgraph_analyzer.py:667-756): y = x * rsqrt(mean(x^2)+eps) * w.
 * fp32 math.  With round_mid != 0 the normalised value is rounded to the
 * activation dtype before the multiply by w, as the unfused ATen chain does.
 * x, y: [rows, cols] with row strides in elements; w: [cols]. */
int b200_rmsnorm(const void* x, const void* w, void* y, int64_t rows, int64_t cols,
                 int64_t x_row_stride, int64_t y_row_stride, float eps, int dtype,
                 int round_mid, void* stream);

/* softmax_kernel / masked_softmax_kernel (cuda_templates.py:9-80, 525-594;
 * dispatch cuda_executor.py:378-427): y = softmax(x*scale + mask) over the last
 * axis.  x and y are contiguous [d0, d1, d2, cols]; the additive mask (may be
 * NULL) is addressed as mask[i0*ms0 + i1*ms1 + i2*ms2 + c], so [B,1,T,S],
 * [B,1,1,S] and full-shape masks all work (the reference indexes the mask with
 * the flat score index and cannot broadcast).  fp32 math; with round_steps != 0
 * the product x*scale and the sum with the mask are each rounded to `in_dtype`,
 * as the unfused ATen ops would. */
int b200_softmax(const void* x, const void* mask, void* y, int64_t d0, int64_t d1, int64_t d2,
                 int64_t cols, int64_t ms0, int64_t ms1, int64_t ms2, float scale, int in_dtype,
                 int mask_dtype, int out_dtype, int round_steps, void* stream);

/* mean_last_dim_kernel (cuda_templates.py:82-97): y[r] = mean(x[r, :]). */
int b200_mean_last_dim(const void* x, void* y, int64_t rows, int64_t cols, int in_dtype,
                       int out_dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Indexing (bit-exact).
 * ------------------------------------------------------------------------- */
/* embedding_kernel (cuda_templates.py:99-112; step subgraph_analyzer.py:381-393):
 * out[s, :] = table[ids[s], :].  ids are int64 or int32 as given (the reference
 * casts to int32 on device each call, cuda_executor.py:535).  Rows are copied
 * as raw bytes; an id outside [0, vocab) yields a zero row. */
int b200_embedding(const void* table, const void* ids, void* out, int64_t n_ids, int64_t vocab,
                   int64_t row_bytes, int ids_dtype, void* stream);

/* index_copy_kernel (cuda_templates.py:134-162; step subgraph_analyzer.py:411-428):
 * dst viewed as [outer, dim_size, inner]; dst[o, index[l], :] = src[o, l, :].
 * When base != dst the whole of base is copied to dst first (the reference's
 * out-of-place semantics); when base == dst only the indexed rows are written.
 * src may be strided: src element (o, l, i) is at o*src_outer_stride +
 * l*src_index_stride + i (inner is contiguous). */
int b200_index_copy(const void* base, void* dst, const void* src, const void* index,
                    int64_t outer, int64_t dim_size, int64_t inner, int64_t n_index,
                    int64_t src_outer_stride, int64_t src_index_stride, int elem_bytes,
                    int index_dtype, void* stream);

/* Greedy token choice: out[r] = argmax(x[r, :]) as int64 (lowest index wins ties).
 * Not a reference kernel: the reference downloads logits and uses numpy on the
 * host (benchmarks/benchmark_qwen.py). */
int b200_argmax_rows(const void* x, int64_t* out, int64_t rows, int64_t cols, int64_t row_stride,
                     int dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Rotary embedding.
 * ------------------------------------------------------------------------- */
/* rope_kernel (cuda_templates.py:114-132; correct math metal_kernels/rope.metal:34-44):
 * cos/sin tables [n_pos, head_dim] with angle = fp32(pos) * inv_freq[d mod head_dim/2]. */
int b200_rope_table(const float* inv_freq, const void* positions, void* cos_out, void* sin_out,
                    int64_t n_pos, int head_dim, int pos_dtype, int out_dtype, void* stream);

/* Fused rotate, replacing the mul/slice/neg/cat/mul/add chain the reference runs
 * as 7 elementwise and copy steps per tensor (math: metal_kernels/rope_rotate.metal:41-61):
 * y = x*cos + rotate_half(x)*sin for x [batch, heads, seq, head_dim] (arbitrary
 * strides, head_dim contiguous), cos/sin [batch, seq, head_dim].  Each product
 * and the sum are rounded to `dtype`, as the unfused chain does.
 * If kv_cache != NULL the result is written there instead of y, at row
 * cache_pos[s] of a [batch, heads, cache_len, head_dim] cache (the index_copy the
 * graph applies next). */
int b200_rope_rotate(const b200_tensor* x, const void* cos_t, const void* sin_t, void* y,
                     void* kv_cache, const void* cache_pos, int64_t cache_len, int pos_dtype,
                     void* stream);

/* b200_rope_rotate on q and k of one attention layer (same batch, positions, head_dim and
 * tables; their own head counts and strides) to dense q_out / k_out, in one launch where
 * one thread per (head, position) is the faster form (up to ~4700 positions; longer prompts
 * run the two rotations one after the other).  Same roundings as two b200_rope_rotate calls.
 * Replaces the two rotate chains of a prefill layer (metal_kernels/rope_rotate.metal:41-61;
 * steps subgraph_analyzer.py:395-428). */
int b200_rope_rotate_pair(const b200_tensor* q, const b200_tensor* k, const void* cos_t,
                          const void* sin_t, void* q_out, void* k_out, void* stream);

/* The three per-token steps between the QKV projection and decode attention in one
 * launch: RoPE on q -> q_out [B,Hq,T,D] dense; RoPE on k -> key cache row cache_pos[t];
 * v -> value cache row cache_pos[t] (caches [B,Hkv,cache_len,D], updated in place).
 * Replaces two rotate chains and two index_copy_kernel launches
 * (cuda_templates.py:114-162; steps subgraph_analyzer.py:395-428).  q, k, v are
 * [B,H,T,D] views with arbitrary strides over (b,h,t); cos/sin are [B,T,D]. */
int b200_qkv_rope_cache(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                        const void* cos_t, const void* sin_t, void* q_out, void* k_cache,
                        void* v_cache, const void* cache_pos, int64_t cache_len, int pos_dtype,
                        void* stream);

/* ------------------------------------------------------------------------- *
 * Pooling / normalisation for the CNN path (NCHW logical shape, any strides, so
 * channels-last storage is simply a stride pattern).
 * ------------------------------------------------------------------------- */
/* max_pool2d_kernel (cuda_templates.py:315-352). */
int b200_max_pool2d(const b200_tensor* x, const b200_tensor* y, int kh, int kw, int sh, int sw,
                    int ph, int pw, void* stream);
/* adaptive_avg_pool2d_kernel (cuda_templates.py:354-383); fp32 sum / count. */
int b200_adaptive_avg_pool2d(const b200_tensor* x, const b200_tensor* y, void* stream);
/* batch_norm_kernel (cuda_templates.py:432-456), inference statistics. */
int b200_batch_norm(const b200_tensor* x, const b200_tensor* y, const void* gamma, const void* beta,
                    const void* mean, const void* var, float eps, int param_dtype, int relu,
                    void* stream);
/* Weight preparation, run once per weight set: folds inference batch-norm into
 * the preceding convolution (math of npu_runtime/weight_loader.py:74-99) and
 * repacks OIHW weights to [O, KH, KW, I_pad] in the compute dtype.
 * w_out: [O, KH*KW*I_pad]; bias_out: fp32 [O].  gamma..var and conv_bias may be NULL. */
int b200_conv_weight_prep(const void* w, const void* conv_bias, const void* gamma, const void* beta,
                          const void* mean, const void* var, void* w_out, float* bias_out,
                          int O, int I, int KH, int KW, int I_pad, float eps, int w_dtype,
                          int param_dtype, int out_dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Dense contractions.
 * ------------------------------------------------------------------------- */
/* epilogue flags */
#define B200_EPI_RELU 1
#define B200_EPI_SILU_MUL 2 /* out = silu(acc) * aux (aux shaped like out) */
/* Gated MLP in one GEMM: W holds the gate and up projections interleaved in blocks of 64
 * rows ([128j, 128j+64) gate rows 64j.., [128j+64, 128j+128) up rows 64j..); N counts
 * the merged rows (a multiple of 128) and out has N/2 columns:
 * out[:, 64j+c] = silu(acc[:, 128j+c]) * acc[:, 128j+64+c]. */
#define B200_EPI_GLU 4
/* Hint: W is a constant of the stream (a model weight), so the kernel may begin fetching it
 * before the previous kernel in the stream has finished (programmatic dependent launch). */
#define B200_EPI_W_STATIC 8

/* CUBLASStep("gemm") (subgraph_analyzer.py:168-224, dispatch cuda_executor.py:182-208,
 * which calls cupy.matmul and a separate bias-add kernel):
 *   out[M,N] = epi( A[M,K] * W[N,K]^T + bias[N] + residual[M,N] )
 * A, W, out, residual share `dtype` (f16/bf16), fp32 accumulation; bias dtype is
 * `bias_dtype`.  lda/ldw/ldo/ldr are row strides in elements.  Any M.  Operands that
 * meet the TMA rules (16-byte aligned, strides multiples of 8 elements) run on the
 * tcgen05 path: one tile per CTA with split-K inside a thread-block cluster (partial sums
 * meet in distributed shared memory, no scratch) for M <= 128 and for shapes with few
 * tiles, a persistent kernel with 128 x 64..256 tiles, or 256 x 256 tiles on pairs of CTAs
 * (cta_group::2) for M > 128, N >= 1024, K >= 1024.  `workspace` (zero-initialised by the
 * caller once, left zeroed by every call; b200_linear_workspace_bytes gives the size, 0
 * when none is needed) serves two cases: the pair kernel's split-K for 12..36 tiles with
 * K >= 4096 (fp32 partial sums in a 32-byte aligned workspace, added in index order by a second kernel; without a
 * workspace the shape takes the cluster split-K instead), and the weight-streaming
 * fallback for operands with M <= 64 that miss the TMA rules. */
int b200_linear(const void* A, const void* W, const void* bias, const void* residual, void* out,
                int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldo, int64_t ldr,
                int dtype, int bias_dtype, int epilogue, const void* aux, int64_t ldaux,
                void* workspace, int64_t workspace_bytes, void* stream);
int64_t b200_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* b200_linear followed by b200_rmsnorm of its output rows: out as b200_linear (bias,
 * residual, B200_EPI_RELU / _W_STATIC; no aux, no gated epilogue), norm_out[m, :] =
 * rmsnorm(out[m, :]) * norm_weight with the roundings of b200_rmsnorm (round_mid as there),
 * row stride ldn.  Replaces a CUBLASStep("gemm") (cuda_executor.py:182-208) and the
 * `rmsnorm_kernel` launch that reads its result (cuda_templates.py:458-506).  Where the GEMM
 * takes the CTA-pair split-K path (see b200_linear) and N <= 2048 the kernel that adds up the
 * partial sums also normalises the finished row - one launch less; every other shape runs
 * the two kernels one after the other inside this call. */
int b200_linear_rmsnorm(const void* A, const void* W, const void* bias, const void* residual,
                        void* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw,
                        int64_t ldo, int64_t ldr, int dtype, int bias_dtype, int epilogue,
                        void* workspace, int64_t workspace_bytes, const void* norm_weight,
                        void* norm_out, int64_t ldn, float norm_eps, int round_mid, void* stream);

/* Decode-shape (M <= 64) linear layer with the neighbouring RMSNorm folded in, replacing a
 * `rmsnorm_kernel` launch (cuda_templates.py:458-506, matcher subgraph_analyzer.py:667-756)
 * plus the CUBLASStep("gemm") that consumes it (cuda_executor.py:182-208).
 *   sumsq_in != NULL: A holds the UN-normalised rows x and W holds the weights with the
 *     RMSNorm gain folded into their columns (W'[n,k] = W[n,k] * gain[k], prepared once by
 *     the caller).  Since (r x) W^T = r (x W^T), the kernel multiplies output row m by
 *     r_m = 1 / sqrt(s_m / K + norm_eps) before the bias, where s_m is the sum of
 *     sumsq_in[m * sumsq_in_cols + 0 .. sumsq_in_cols) (fp32, added in index order; at most
 *     32 partials).  The normalised activations are never rounded to the 16-bit type, so
 *     results differ from b200_rmsnorm + b200_linear by rounding only.
 *   sumsq_out != NULL: besides `out` the kernel writes sumsq_out[m * (N / 64) + j] = sum of
 *     squares of the rounded outputs out[m, 64 j .. 64 j + 63] - the partials the next
 *     normalising layer consumes.  Needs N % 64 == 0.
 * Everything else as b200_linear (bias, residual, B200_EPI_RELU / _GLU / _W_STATIC); no
 * aux operand, no workspace.  B200_ENOTSUP when the operands do not fit the fused kernel. */
int b200_linear_norm(const void* A, const void* W, const void* bias, const void* residual, void* out,
                     int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldo, int64_t ldr,
                     int dtype, int bias_dtype, int epilogue, float norm_eps,
                     const float* sumsq_in, int sumsq_in_cols, float* sumsq_out, void* stream);

/* The merged q/k/v projection of a decode step (one token per sequence, M = sequences <= 64)
 * with everything that follows it before attention: replaces the three CUBLASStep("gemm")
 * projections (cuda_executor.py:182-208), the `rope_kernel` launches on q and k
 * (cuda_templates.py:114-132) and the two `index_copy_kernel` KV-cache writes
 * (cuda_templates.py:134-162).  W holds the q, k and v weight rows one after the other,
 * N = (Hq + 2 Hkv) * 128 (head dimension 128); columns [128 h, 128 h + 128) are head h.
 * The kernel's final pass adds the bias, rounds to the 16-bit type as the linear layer's
 * output is rounded, applies x * cos + rotate_half(x) * sin to query and key heads with the
 * roundings of the unfused operators (both products, then the sum) and stores
 *   rope(q) to q_out [M, Hq, 128],
 *   rope(k) and v to row cache_pos[0] of k_cache / v_cache [M, Hkv, cache_len, 128] (in place;
 *   a negative position counts from the end, a position outside the cache writes nothing).
 * cos_t / sin_t: [M, 128] tables of the rows' positions in the activation type.  sumsq_in /
 * sumsq_in_cols / norm_eps as in b200_linear_norm (NULL: no row scaling).  epilogue: 0 or
 * B200_EPI_W_STATIC.  Results are bit-identical to b200_linear_norm followed by
 * b200_qkv_rope_cache.  B200_ENOTSUP when the operands do not fit the fused kernel. */
int b200_linear_qkv_rope(const void* A, const void* W, const void* bias, int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldw, int dtype, int bias_dtype, int epilogue, float norm_eps,
                         const float* sumsq_in, int sumsq_in_cols, const void* cos_t, const void* sin_t,
                         void* q_out, void* k_cache, void* v_cache, const void* cache_pos, int64_t cache_len,
                         int pos_dtype, int Hq, int Hkv, void* stream);

/* CUBLASStep("gemm_batched") and plain 2-D matmul (subgraph_analyzer.py:206-224,
 * dispatch cuda_executor.py:210-218): out[b1,b2,M,N] = A[b1,b2,M,K] @ B[b1,b2,K,N] with
 * independent element strides for every axis of every operand (0 = broadcast), so
 * transposed and expanded operands need no materialised copy.  fp32 accumulate. */
int b200_matmul_strided(const void* A, const void* B, void* out, int64_t b1, int64_t b2, int64_t M,
                        int64_t N, int64_t K, const int64_t a_strides[4], const int64_t b_strides[4],
                        const int64_t o_strides[4], int dtype, void* stream);

/* CUBLASStep("conv2d") (subgraph_analyzer.py:226-254; dispatch
 * cuda_executor.py:275-356, a host-side im2col loop + cupy.matmul): implicit-GEMM
 * convolution over channels-last activations.
 *   x: [N, H, W, C] (C contiguous), w: [O, KH, KW, C_pad] from b200_conv_weight_prep,
 *   y / residual: [N, Ho, Wo, O];  y = epi(conv(x, w) + bias + residual).
 * groups must be 1. */
int b200_conv2d_nhwc(const void* x, const void* w, const float* bias, const void* residual, void* y,
                     int N, int H, int W, int C, int C_pad, int O, int KH, int KW, int sh, int sw,
                     int ph, int pw, int Ho, int Wo, int dtype, int epilogue, void* stream);

/* ------------------------------------------------------------------------- *
 * Attention.
 * ------------------------------------------------------------------------- */
/* Decode attention over a static KV cache, replacing CUBLASStep("gemm_gqa") x2 plus
 * the scale / mask-add / softmax steps between them (subgraph_analyzer.py:819-861,
 * dispatch cuda_executor.py:226-273).
 *   q:   [B, Hq, D]   (one query token per sequence, D = 128)
 *   k,v: [B, Hkv, S, D] caches, row stride D, head stride S*D
 *   mask:[B, S] additive (the graph's attention_mask [B,1,1,S]); NULL = none
 *   out: [B, Hq, D]
 * Split-KV: for caches of 512..16384 rows (and at most 8 query heads per KV head) the up to eight splits
 * (sixteen for batches whose clusters are all resident at once) of a (sequence, KV head) form a thread-block cluster and merge in distributed shared memory
 * (no workspace: b200_attn_decode_workspace_bytes returns 0); otherwise partial
 * (max, sum, acc) per split go to `workspace` and are merged by a second kernel.  Key blocks whose mask entries are all <= -1e30 are skipped, which
 * leaves the result unchanged because their softmax weight underflows to 0. */
int b200_attn_decode(const void* q, const void* k, const void* v, const void* mask, void* out,
                     int64_t B, int Hq, int Hkv, int64_t S, int D, int64_t q_batch_stride,
                     int64_t kv_batch_stride, int64_t kv_head_stride, int64_t mask_batch_stride,
                     float scale, int dtype, void* workspace, int64_t workspace_bytes, void* stream);
int64_t b200_attn_decode_workspace_bytes(int64_t B, int Hq, int Hkv, int64_t S, int D);

/* Same computation as b200_attn_decode for callers that cannot allocate device memory
 * (a host runtime that owns every byte of the GPU, FFI glue that may only forward pointers
 * it was handed, code running where cudaMalloc is off limits).  This entry point has no
 * counterpart in the reference.  The split-KV partials go to an 8 MiB array that is part
 * of the library image (each GPU that loads the library holds it until exit); shapes whose
 * partials need more return B200_ELIMIT (caches of 512..16384 rows need none: their splits
 * merge inside the kernel; Hq=12, Hkv=2, S=32768 is refused for B > 21).  No
 * cudaMalloc, cudaFree or allocating library call is made.  The first call on a device
 * looks up the array's device address; make that call before any stream capture.  All
 * calls share the array: two calls whose kernels overlap on the GPU (different streams)
 * race.  Nothing in it needs clearing between calls - every partial is rewritten. */
int b200_attn_decode_noalloc(const void* q, const void* k, const void* v, const void* mask, void* out,
                             int64_t B, int Hq, int Hkv, int64_t S, int D, int64_t q_batch_stride,
                             int64_t kv_batch_stride, int64_t kv_head_stride, int64_t mask_batch_stride,
                             float scale, int dtype, void* stream);

/* Prefill attention, replacing CUBLASStep("gemm_batched") x2 with the softmax
 * between them and the materialised expand/transpose copies
 * (subgraph_analyzer.py:206-215; cuda_executor.py:210-218):
 *   q: [B, Hq, T, D] with strides (q_b, q_h, q_t, 1); k,v: [B, Hkv, S, D] likewise;
 *   mask: additive, addressed mask[b*mask_b + t*mask_t + s]; out: [B, T, Hq, D]
 *   contiguous (the layout the following o_proj consumes). */
int b200_attn_prefill(const void* q, const void* k, const void* v, const void* mask, void* out,
                      int64_t B, int Hq, int Hkv, int64_t T, int64_t S, int D,
                      const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                      int64_t mask_b, int64_t mask_t, float scale, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200NN_H */
