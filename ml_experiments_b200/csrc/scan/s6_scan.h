// S6 selective scan (torch-free interface). Tensors are channel-last:
//   u, z, y_pre, out, dout, du, dz : bf16 [B][L][Din]      delta, ddelta : fp32 or bf16 [B][L][Din] (delta_bf16)
//   Bm, Cm : fp32 [B][L][N]    A, dA : fp32 [Din][N]    Dv, dD, delta_bias, ddelta_bias : fp32 [Din]     N must be 16
//   With `softplus` the step is softplus(delta + delta_bias) and ddelta / ddelta_bias are gradients of the raw values.
//   state : fp32 [B][ceil(L/16)][4][Din][4], the state at the start of every 16-step tile, states grouped in fours
//           (the forward writes it, the backward reads it)
//   dB_part, dC_part : fp32 [B][ceil(Din/32)][L][N] partial sums over 32-channel blocks (the caller sums dim 1)
#pragma once
#include <cuda_runtime.h>

namespace b200 {

int s6_channel_blocks(int Din);  // ceil(Din / 32)
int s6_num_chunks(int L);        // ceil(L / 16)
// States held per thread (2 or 4) by the forward and by the backward kernel: 4 = four warps per 32-channel block,
// 2 = eight warps per block (more warps per SM to hide latency, more shared-memory traffic). Default 2 / 4.
void s6_set_states_per_thread(int fwd_qs, int bwd_qs);

void s6_scan_fwd(const void* u, const void* delta, bool delta_bf16, const float* delta_bias, bool softplus, const float* A,
                 const float* Bm, const float* Cm, const float* Dv, const void* z, void* y_pre, void* out,
                 float* state, int batch, int L, int Din, int N, cudaStream_t s);

// dout: gradient of `out`. With z the gate's backward runs inside (needs y_pre; dz is written when non-null).
// dA, dD and ddelta_bias are accumulated into (zero them first).
void s6_scan_bwd(const void* u, const void* delta, bool delta_bf16, const float* delta_bias, bool softplus, const float* A,
                 const float* Bm, const float* Cm, const float* Dv, const void* z, const void* y_pre, const void* dout,
                 const float* state, void* du, void* ddelta, float* dA, float* dB_part, float* dC_part, float* dD,
                 void* dz, float* ddelta_bias, int batch, int L, int Din, int N, cudaStream_t s);

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
