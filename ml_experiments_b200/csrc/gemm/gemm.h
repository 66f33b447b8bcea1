// C++ interface of the tcgen05/TMEM GEMM (torch-free; the binding layer fills this struct).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {

enum GemmEpilogue : int {
  EPI_NONE = 0,       // C = alpha * acc
  EPI_RELU2 = 1,      // C = relu(alpha * acc)^2
  EPI_AXPBY = 2,      // C = alpha * acc + beta * aux
  EPI_RELU2_BWD = 3,  // C = alpha * acc * 2 * sqrt(aux)      (aux = relu(pre)^2 saved by the forward)
};

enum GemmDtype : int { GEMM_BF16 = 0, GEMM_E4M3 = 1, GEMM_E5M2 = 2, GEMM_F32 = 3 };

// C[b] (M x N, row-major)  =  epilogue( A[b] (M x K)  *  B[b] (N x K)^T )
//   a_mn == 0 : A stored [M][K] (K contiguous, "K-major");  a_mn == 1 : A stored [K][M] ("MN-major")
//   b_mn == 0 : B stored [N][K];                             b_mn == 1 : B stored [K][N]
// Leading dimensions and batch strides are in elements. All row pitches must be multiples of 16 bytes.
struct GemmArgs {
  const void* A = nullptr;
  const void* B = nullptr;
  void* C = nullptr;
  const void* aux = nullptr;  // bf16 [batch][M][N], used by EPI_AXPBY / EPI_RELU2_BWD
  int batch = 1, M = 0, N = 0, K = 0;
  long long lda = 0, ldb = 0, ldc = 0, ldaux = 0;
  long long stride_a = 0, stride_b = 0, stride_c = 0, stride_aux = 0;
  int a_mn = 0, b_mn = 0;
  int a_dtype = GEMM_BF16, b_dtype = GEMM_BF16;  // both 2-byte or both 1-byte
  int c_dtype = GEMM_BF16;                       // GEMM_BF16 or GEMM_F32
  int epilogue = EPI_NONE;
  float alpha = 1.f, beta = 0.f;
  int split_k = 1;     // > 1 requires c_dtype == GEMM_F32 and accumulate-by-reduction (C is zeroed first unless accumulate)
  int accumulate = 0;  // 1: C += result (fp32 C only; performed with TMA reduce-add)
  int max_ctas = 0;    // 0 = one CTA per SM
  int* status = nullptr;  // device int; stays 0 unless a bounded wait expired
  cudaStream_t stream = nullptr;
};

// Throws std::runtime_error on invalid arguments / launch failure.
void gemm_sm100(const GemmArgs& args);

}  // namespace b200
