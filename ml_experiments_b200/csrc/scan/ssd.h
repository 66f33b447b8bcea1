// Chunked scalar-decay state-space scan on tcgen05 (see ssd_sm100.cu for the algorithm), torch-free interface.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

struct SsdArgs {
  const void* x = nullptr;        // bf16 [batch, L, H, P]
  const void* B = nullptr;        // bf16 [batch, L, Hb, N]
  const void* C = nullptr;        // bf16 [batch, L, Hb, N]
  const float* log_a = nullptr;   // fp32 [batch, L, H]  log of the per-step decay
  const float* g_off = nullptr;   // fp32 [batch, L, H]  weight of step j's outer product for outputs i > j and for the state
  const float* g_diag = nullptr;  // fp32 [batch, L, H]  weight of step i's own outer product in y_i
  void* y = nullptr;              // bf16 [batch, L, H, P]
  const float* init_state = nullptr;  // fp32 [batch, H, N, P] or null
  float* final_state = nullptr;       // fp32 [batch, H, N, P] or null
  int batch = 0, L = 0, H = 0, Hb = 0, N = 0, P = 0;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
};

bool ssd_fwd_supported(int L, int H, int Hb, int N, int P);
void ssd_fwd_sm100(const SsdArgs& a);

}  // namespace b200
