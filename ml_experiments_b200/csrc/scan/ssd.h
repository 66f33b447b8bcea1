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
  float* chunk_states = nullptr;      // fp32 [batch, H, L / 128, N, P] or null: the state after every 128-step chunk
  int batch = 0, L = 0, H = 0, Hb = 0, N = 0, P = 0;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
};

// Inputs and outputs of the backward's combining pass (ssd_aux.cu); every [.., P] / [.., N] tensor is bf16 and contiguous.
struct SsdPostArgs {
  const void *x = nullptr, *dy = nullptr, *y = nullptr;   // [batch, L, H, P]
  const void* dx_rev = nullptr;                            // [batch, L, H, P]  scan backwards in time, still time-reversed
  const void* dB_rev = nullptr;                            // [batch, L, H, N]  likewise
  const void* dC_heads = nullptr;                          // [batch, L, H, N]  per head, before the sum over a group
  const void *B = nullptr, *C = nullptr;                   // [batch, L, Hb, N]
  const float *g_off = nullptr, *g_diag = nullptr;         // [batch, L, H]
  void *dx = nullptr, *dB = nullptr, *dC = nullptr;        // [batch, L, H, P], [batch, L, Hb, N] x 2
  float *d_goff = nullptr, *d_gdiag = nullptr, *inner = nullptr;  // [batch, L, H]
  int batch = 0, L = 0, H = 0, Hb = 0, N = 0, P = 0;
  cudaStream_t stream = nullptr;
};

void ssd_flip_time(const void* src, void* dst, int batch, int L, long long row_bytes, cudaStream_t s);
void ssd_bwd_post(const SsdPostArgs& a);

bool ssd_fwd_supported(int L, int H, int Hb, int N, int P);
void ssd_fwd_sm100(const SsdArgs& a);

}  // namespace b200
