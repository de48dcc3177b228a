// Interface between the GEMM dispatcher (gemm.cu) and the tcgen05 kernel (gemm_tc5.cu).
#pragma once
#include "common.cuh"

namespace b200 {

struct Tc5Args {
  const void* A; const void* W; const void* bias; const void* residual; const void* aux; void* out;
  int64_t M, N, K, lda, ldw, ldo, ldr, ldaux;
  int dtype, bias_dtype, epilogue;
};

// out = epi(A W^T + bias + residual) on the tcgen05 path.  Returns B200_ENOTSUP when the
// operands do not meet the TMA alignment rules (the caller then uses the mma.sync tiles).
int linear_tc5(const Tc5Args& a, cudaStream_t stream);
bool tc5_enabled();

}  // namespace b200
