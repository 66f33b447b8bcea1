// S6 selective scan (torch-free interface). Tensors are channel-last:
//   u, z, y_pre, out, dy, du : bf16 [B][L][Din]      delta, ddelta : fp32 [B][L][Din]
//   Bm, Cm : fp32 [B][L][N]    A, dA : fp32 [Din][N]    Dv, dD : fp32 [Din]     N must be 16
//   chunk_state : fp32 [B][ceil(L/64)][Din][N], state at the start of every 64-step chunk (forward writes it)
//   dB_part, dC_part : fp32 [B][ceil(Din/16)][L][N] partial sums over 16-channel blocks (the caller sums dim 1)
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

namespace b200 {
// Causal depthwise conv (width 4) + bias + SiLU. x: bf16 [B][L][*] with row pitch ldx (a channel slice of a wider
// tensor is fine), w: fp32 [C][4], bias: fp32 [C] or null, y / dy: bf16 [B][L][C] dense, dx: bf16 with pitch lddx.
// The backward accumulates into dw / dbias (zero them first).
void causal_conv1d_silu_fwd(const void* x, long long ldx, const float* w, const float* bias, void* y, int batch, int L,
                            int C, cudaStream_t s);
void causal_conv1d_silu_bwd(const void* x, long long ldx, const float* w, const float* bias, const void* dy, void* dx,
                            long long lddx, float* dw, float* dbias, int batch, int L, int C, cudaStream_t s);
}  // namespace b200
