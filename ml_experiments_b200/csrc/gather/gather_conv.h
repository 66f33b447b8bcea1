// Gather-convolution core shared by the telephone / adaptive-local-conv / scatter attention family:
//   out[b,l,h,:] = sum_s wgt[b,l,h,s] * lerp(x[b, floor(p), h, :], x[b, floor(p)+1, h, :], frac(p)),  p = pos[b,l,h,s]
// x : bf16 [B][L][H*D] (source)   out : bf16 [B][Lq][H*D]   pos, wgt : fp32 [B][Lq][H][S]   (Lq query rows gather from
// the L source rows; Lq = L for a whole-sequence call, smaller for a chunk)   D in {8,16,32,64,128}
// Backward: dwgt, dpos (fp32, same shape as wgt) and dx accumulated with vector atomics into fp32 [B][L][H*D]
// (zero it first). Positions are clamped to [0, pos_max] with pos_max <= L - 1 (the floor row is capped at L - 2, so with
// pos_max = L - 1 integer positions, the last row included, are read exactly); a clamped tap gets no position gradient.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
void gather_conv_fwd(const void* x, const float* pos, const float* wgt, void* out, int B, int L, int Lq, int H, int D,
                     int S, float pos_max, cudaStream_t s);
void gather_conv_bwd(const void* x, const float* pos, const float* wgt, const void* dout, float* dx, float* dpos,
                     float* dwgt, int B, int L, int Lq, int H, int D, int S, float pos_max, cudaStream_t s);
}  // namespace b200
