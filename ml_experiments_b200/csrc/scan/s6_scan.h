// S6 selective scan (torch-free interface). Tensors are channel-last:
//   u, z, y_pre, out, dy, du : bf16 [B][L][Din]      delta, ddelta : fp32 [B][L][Din]
//   Bm, Cm : fp32 [B][L][N]    A, dA : fp32 [Din][N]    Dv, dD : fp32 [Din]     N must be 16
//   chunk_state : fp32 [B][ceil(L/64)][Din][N], state at the start of every 64-step chunk (forward writes it)
//   dB_part, dC_part : fp32 [B][ceil(Din/64)][L][N] partial sums over 64-channel blocks (the caller sums dim 1)
#pragma once
#include <cuda_runtime.h>

namespace b200 {

int s6_channel_blocks(int Din);
int s6_num_chunks(int L);

void s6_scan_fwd(const void* u, const float* delta, const float* A, const float* Bm, const float* Cm, const float* Dv,
                 const void* z, void* y_pre, void* out, float* chunk_state, int batch, int L, int Din, int N,
                 cudaStream_t s);

// dy: gradient with respect to y_pre (before the silu(z) gate). dA and dD are accumulated into (zero them first).
void s6_scan_bwd(const void* u, const float* delta, const float* A, const float* Bm, const float* Cm, const float* Dv,
                 const void* dy, const float* chunk_state, void* du, float* ddelta, float* dA, float* dB_part,
                 float* dC_part, float* dD, int batch, int L, int Din, int N, cudaStream_t s);

}  // namespace b200
