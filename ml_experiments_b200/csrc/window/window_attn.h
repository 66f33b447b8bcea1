// Local window attention with a per-tap additive bias (1-D), torch-free interface.
//
//   s[b,l,h,w] = scale * q[b,l,h,:] . k[b, l + w - (K-1)/2, h, :] + bias[b,l,h,w]
//   P = softmax_w(s) ;  out[b,l,h,:] = sum_w P[b,l,h,w] * v[b, l + w - (K-1)/2, h, :]
//
// Keys / values beyond the sequence ends are zero vectors that still take part in the softmax (zero-padded windows).
// q, k, v, out, dout, dq, dk, dv : bf16 [B][L][H][D] (dense);  bias, P, dbias : fp32 [B][L][H][K].
// D in {16, 32, 64}, K <= 64. The forward writes P (the backward needs it).
#pragma once
#include <cuda_runtime.h>

namespace b200 {

void window_attn_fwd(const void* q, const void* k, const void* v, const float* bias, void* out, float* P, float scale,
                     int B, int L, int H, int D, int K, cudaStream_t s);
void window_attn_bwd(const void* q, const void* k, const void* v, const float* P, const void* dout, void* dq, void* dk,
                     void* dv, float* dbias, float scale, int B, int L, int H, int D, int K, cudaStream_t s);

}  // namespace b200
