// Block-scaled fp8 GEMM launcher (see fp8_gemm_sm100.cu).  Counterpart of the stand-alone
// fp8 template in the reference tree (all2all/hip.py:17-59), which serves neither task.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

struct Fp8GemmArgs {
  const void* a;         // [M, K] e4m3, row-major (K contiguous)
  const void* b;         // [N, K] e4m3, row-major
  const float* a_scale;  // one scale per row of A and 128-wide K block
  const float* b_scale;  // one scale per 128 x 128 block of B
  void* c;               // [M, N] bf16 row-major
  int M, N, K;
  long long as_stride_m, as_stride_k, bs_stride_n, bs_stride_k;  // element strides of the scale tensors
  uint64_t timeout_ns;
  int* error_flag;       // device int, set to 1 if a pipeline wait expired (may be nullptr)
};

cudaError_t launch_fp8_gemm(const Fp8GemmArgs& args, cudaStream_t stream);

}  // namespace b200
