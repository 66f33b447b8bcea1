// Telephone attention and adaptive local convolution with the tap formulas evaluated inside the gather kernel: no
// [B, L, H, S] position / weight tensors exist in memory, forward or backward.
//
// x : bf16 [B][L][H*D] (D in {8,16,32,64,128});  out : bf16 [B][L][H*D];  per (b, l, h) row, K <= 64 kernel taps.
//
// telephone (src/heuristic_secrets/models/telephone_attention.py:124-180, triton_telephone.py:149-357 of the reference):
//   s in [-half, half]:  rel = s*freq,  p = l + rel + phase,  valid = 0 <= p < L,
//   w = lerp(kern, |rel| / max_rec) * (1 + |rel|/L)^(-expo) * valid,   out += w * bilinear(x, clamp(p, 0, L - 1.001))
//   freq, phase : fp32 [B][L][H];  kern : fp32 [B][L][H][K];  expo : fp32 [B][L]
//   backward: dx (fp32, atomics, zero it first), dfreq, dphase [B][L][H], dkern [B][L][H][K], dexpo_h [B][L][H]
//   (the caller sums dexpo_h over heads).
//
// adaptive local conv (adaptive_local_conv.py:75-169, triton_adaptive_conv.py:81-318):
//   s in [-half, half]:  r = |s| / half_w,  p = l + center + s,  valid = 0 <= p < L,
//   base = (relu(lerp(kern, min(r, 1))) + 1) * exp(-r*r) * valid,   w = base / max(sum_s base, 1)
//   half_w, center : fp32 [B][L][H];  backward: dx, dhalf_w, dcenter, dkern.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
void tele_fused_fwd(const void* x, const float* freq, const float* phase, const float* kern, const float* expo, void* out,
                    int B, int L, int H, int D, int K, int half, float max_rec, cudaStream_t s);
void tele_fused_bwd(const void* x, const float* freq, const float* phase, const float* kern, const float* expo,
                    const void* dout, float* dx, float* dfreq, float* dphase, float* dkern, float* dexpo_h, int B, int L,
                    int H, int D, int K, int half, float max_rec, cudaStream_t s);
void alc_fused_fwd(const void* x, const float* half_w, const float* center, const float* kern, void* out, int B, int L,
                   int H, int D, int K, int half, cudaStream_t s);
void alc_fused_bwd(const void* x, const float* half_w, const float* center, const float* kern, const void* dout, float* dx,
                   float* dhalf_w, float* dcenter, float* dkern, int B, int L, int H, int D, int K, int half, cudaStream_t s);
}  // namespace b200
