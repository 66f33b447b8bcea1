// See norm_act.h.
#include "norm_act.h"

#include <cuda_bf16.h>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {
using bf16 = __nv_bfloat16;

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

template <int ACT>
__device__ __forceinline__ float act_fwd(float u) {
  if (ACT == NORM_ACT_SILU) return u / (1.f + __expf(-u));
  if (ACT == NORM_ACT_SIGMOID) return 1.f / (1.f + __expf(-u));
  if (ACT == NORM_ACT_TANH) return tanhf(u);
  return u;
}
template <int ACT>
__device__ __forceinline__ float act_grad(float u) {
  if (ACT == NORM_ACT_SILU) {
    const float s = 1.f / (1.f + __expf(-u));
    return s * (1.f + u * (1.f - s));
  }
  if (ACT == NORM_ACT_SIGMOID) {
    const float s = 1.f / (1.f + __expf(-u));
    return s * (1.f - s);
  }
  if (ACT == NORM_ACT_TANH) {
    const float t = tanhf(u);
    return 1.f - t * t;
  }
  return 1.f;
}

template <typename TI, typename TO, int ACT>
__global__ void __launch_bounds__(256)
rms_act_fwd_kernel(const TI* __restrict__ x, const float* __restrict__ w, TO* __restrict__ y, float* __restrict__ rstd,
                   long long R, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * 8;
  for (long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += warps) {
    const long long base = row * C;
    float ss = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float v = ldf(x, base + c);
      ss += v * v;
    }
    const float rs = rsqrtf(warp_sum(ss) / (float)C + eps);
    if (lane == 0) rstd[row] = rs;
    for (int c = lane; c < C; c += 32) stf(y, base + c, act_fwd<ACT>(w[c] * ldf(x, base + c) * rs));
  }
}

template <typename TI, typename TO, int ACT>
__global__ void __launch_bounds__(256)
rms_act_bwd_kernel(const TI* __restrict__ x, const float* __restrict__ w, const float* __restrict__ rstd,
                   const TO* __restrict__ dy, TI* __restrict__ dx, float* __restrict__ dw, long long R, int C) {
  extern __shared__ float s_dw[];  // [C]
  for (int c = threadIdx.x; c < C; c += 256) s_dw[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * 8;
  const float invC = 1.f / (float)C;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += warps) {
    const long long base = row * C;
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // the first 256 columns accumulate dw in registers
      const int c = lane + 32 * i;
      if (c < C) {
        const float xh = ldf(x, base + c) * rs, wc = w[c];
        const float g = ldf(dy, base + c) * act_grad<ACT>(wc * xh);
        dot += g * wc * xh;
        acc[i] += g * xh;
      }
    }
    for (int c = lane + 256; c < C; c += 32) {
      const float xh = ldf(x, base + c) * rs, wc = w[c];
      const float g = ldf(dy, base + c) * act_grad<ACT>(wc * xh);
      dot += g * wc * xh;
      atomicAdd(&s_dw[c], g * xh);
    }
    dot = warp_sum(dot) * invC;
    for (int c = lane; c < C; c += 32) {
      const float xh = ldf(x, base + c) * rs, wc = w[c];
      const float g = ldf(dy, base + c) * act_grad<ACT>(wc * xh);
      stf(dx, base + c, rs * (g * wc - xh * dot));
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < C && acc[i] != 0.f) atomicAdd(&s_dw[c], acc[i]);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += 256) {
    const float v = s_dw[c];
    if (v != 0.f) atomicAdd(&dw[c], v);
  }
}

void chk(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
int grid_for(long long R) {
  const long long need = (R + 7) / 8;
  return (int)(need < 148LL * 16 ? (need > 0 ? need : 1) : 148LL * 16);
}

#define DISPATCH_ACT(act, ...)                                                       \
  switch (act) {                                                                     \
    case NORM_ACT_NONE: { constexpr int ACT_ = NORM_ACT_NONE; __VA_ARGS__; break; }       \
    case NORM_ACT_SILU: { constexpr int ACT_ = NORM_ACT_SILU; __VA_ARGS__; break; }       \
    case NORM_ACT_SIGMOID: { constexpr int ACT_ = NORM_ACT_SIGMOID; __VA_ARGS__; break; } \
    case NORM_ACT_TANH: { constexpr int ACT_ = NORM_ACT_TANH; __VA_ARGS__; break; }       \
    default: throw std::runtime_error("rms_act: unknown activation");                \
  }
#define DISPATCH_IO(xb, yb, ...)                                                   \
  if (xb && yb) { using TI_ = bf16; using TO_ = bf16; __VA_ARGS__; }               \
  else if (xb && !yb) { using TI_ = bf16; using TO_ = float; __VA_ARGS__; }        \
  else if (!xb && yb) { using TI_ = float; using TO_ = bf16; __VA_ARGS__; }        \
  else { using TI_ = float; using TO_ = float; __VA_ARGS__; }
}  // namespace

void rms_act_fwd(const void* x, bool x_bf16, const float* w, void* y, bool y_bf16, float* rstd, long long R, int C, float eps,
                 int act, cudaStream_t s) {
  if (C < 1 || C > 4096) throw std::runtime_error("rms_act: row length must be in [1, 4096]");
  if (R == 0) return;
  DISPATCH_ACT(act, DISPATCH_IO(x_bf16, y_bf16, {
    rms_act_fwd_kernel<TI_, TO_, ACT_><<<grid_for(R), 256, 0, s>>>((const TI_*)x, w, (TO_*)y, rstd, R, C, eps);
  }));
  chk("rms_act_fwd");
}

void rms_act_bwd(const void* x, bool x_bf16, const float* w, const float* rstd, const void* dy, bool dy_bf16, void* dx,
                 float* dw, long long R, int C, int act, cudaStream_t s) {
  if (C < 1 || C > 4096) throw std::runtime_error("rms_act: row length must be in [1, 4096]");
  if (R == 0) return;
  DISPATCH_ACT(act, DISPATCH_IO(x_bf16, dy_bf16, {
    rms_act_bwd_kernel<TI_, TO_, ACT_><<<grid_for(R), 256, (size_t)C * sizeof(float), s>>>((const TI_*)x, w, rstd, (const TO_*)dy, (TI_*)dx, dw, R, C);
  }));
  chk("rms_act_bwd");
}

}  // namespace b200
