// Weighted RMSNorm with a fused activation, forward and backward, for rows of any length C <= 4096:
//   y = act(w * x * rsqrt(mean(x^2) + eps)),   act in {identity, silu, sigmoid, tanh}
// One warp per row; x and y may each be bf16 or fp32. The forward saves rstd [R] (fp32). The backward writes dx (x's
// dtype) and accumulates dw [C] (fp32, zero it first) through per-block shared-memory partial sums; bf16 rows of 256,
// 512, 768 or 1024 columns take a variant with 16-byte accesses and the dw sums of all columns in registers.
// Counterpart of rmsnorm_silu_fwd_kernel / rmsnorm_fwd_kernel of the reference (src/heuristic_secrets/models/
// triton_telephone.py:109-146, triton_adaptive_conv.py:57-79), which have no fused backward.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
enum NormAct { NORM_ACT_NONE = 0, NORM_ACT_SILU = 1, NORM_ACT_SIGMOID = 2, NORM_ACT_TANH = 3 };
void rms_act_fwd(const void* x, bool x_bf16, const float* w, void* y, bool y_bf16, float* rstd, long long R, int C, float eps,
                 int act, cudaStream_t s);
// dres: optional second gradient of x's shape and dtype (a skip connection around the norm), added to dx.
// dlead: optional [R, lead] gradient (dy's dtype) of the first `lead` columns of y, added to dy's on the fly.
void rms_act_bwd(const void* x, bool x_bf16, const float* w, const float* rstd, const void* dy, bool dy_bf16,
                 const void* dres, const void* dlead, int lead, void* dx, float* dw, long long R, int C, int act,
                 cudaStream_t s);
}  // namespace b200
