// MIMO-Jacobi state iteration (all iterations of the diffusion / injection loop in one launch), torch-free interface.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

struct JacobiArgs {
  // forward inputs, all fp32
  const float* Bm = nullptr;   // input map, logical [batch, R, L, N] with element strides b_s*
  const float* Cm = nullptr;   // output map, same logical shape, strides c_s*
  long long b_sb = 0, b_sr = 0, b_sl = 0, b_sn = 0;
  long long c_sb = 0, c_sr = 0, c_sl = 0, c_sn = 0;
  const float* theta = nullptr;  // [batch, L, N/2] contiguous
  const float* xr = nullptr;     // logical [batch, R, L], strides x_s*
  long long x_sb = 0, x_sr = 0, x_sl = 0;
  const float* alpha = nullptr;  // [batch, L, N] contiguous (decay, already through the sigmoid)
  const float* gamma = nullptr;  // [batch, L] contiguous (trapezoid weight, already through the sigmoid)
  const float* conv_w = nullptr; // [N, 3] depthwise diffusion taps
  const float* conv_b = nullptr; // [N]
  const float* inj_lambda = nullptr;  // device scalar or null (no sum / difference injection)
  const float* ro_lambda = nullptr;   // device scalar or null (no sum / difference readout)
  // forward outputs
  float* gated = nullptr;  // [batch, L, R * N]: rotated C times the final state, ready for the output projection
  float* Hs = nullptr;     // [n_iters, batch, R, L, N] states after every iteration (kept for the backward) or null
  // backward input and outputs (contiguous, zero-initialised where marked)
  const float* dgated = nullptr;  // [batch, L, R * N]
  float* dBm = nullptr;     // [batch, R, L, N]
  float* dCm = nullptr;     // [batch, R, L, N]
  float* dtheta = nullptr;  // [batch, L, N/2]
  float* dxr = nullptr;     // [batch, R, L]
  float* dalpha = nullptr;  // [batch, L, N]
  float* dgamma = nullptr;  // [batch, L]
  float* dconv_w = nullptr; // [N, 3]  zero-initialised (atomic sums)
  float* dconv_b = nullptr; // [N]     zero-initialised
  float* dlam = nullptr;    // [2]     zero-initialised: d inj_lambda, d ro_lambda
  int batch = 0, R = 0, L = 0, N = 0, n_iters = 0;
  cudaStream_t stream = nullptr;
};

bool jacobi_supported(int N, int n_iters);
void jacobi_fwd(const JacobiArgs& a);
void jacobi_bwd(const JacobiArgs& a);

}  // namespace b200
