// See norm_act.h.
#include "norm_act.h"

#include <cuda_bf16.h>

#include <algorithm>
#include <cstdint>
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
                   const TO* __restrict__ dy, const TI* __restrict__ dres, const TO* __restrict__ dlead, int lead,
                   TI* __restrict__ dx, float* __restrict__ dw, long long R, int C) {
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
    // gradient of the normed row: dy plus, in the first `lead` columns, the gradient that came in through the slice
    auto gin = [&](int c) { return ldf(dy, base + c) + (c < lead ? ldf(dlead, row * lead + c) : 0.f); };
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // the first 256 columns accumulate dw in registers
      const int c = lane + 32 * i;
      if (c < C) {
        const float xh = ldf(x, base + c) * rs, wc = w[c];
        const float g = gin(c) * act_grad<ACT>(wc * xh);
        dot += g * wc * xh;
        acc[i] += g * xh;
      }
    }
    for (int c = lane + 256; c < C; c += 32) {
      const float xh = ldf(x, base + c) * rs, wc = w[c];
      const float g = gin(c) * act_grad<ACT>(wc * xh);
      dot += g * wc * xh;
      atomicAdd(&s_dw[c], g * xh);
    }
    dot = warp_sum(dot) * invC;
    for (int c = lane; c < C; c += 32) {
      const float xh = ldf(x, base + c) * rs, wc = w[c];
      const float g = gin(c) * act_grad<ACT>(wc * xh);
      stf(dx, base + c, rs * (g * wc - xh * dot) + (dres ? ldf(dres, base + c) : 0.f));
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

// two bf16 packed in a 32-bit word <-> fp32 (element 0 in the low half)
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t bf_pack(float lo, float hi) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&p);
}

// 16 bytes from shared memory, re-read at every use (a plain load of loop-invariant data would be hoisted into
// registers for the whole row loop, which the kernel below cannot spare)
__device__ __forceinline__ float4 lds128_volatile(const float* p) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"((uint32_t)__cvta_generic_to_shared(p)));
  return v;
}

// 16 bytes from global memory that the compiler may not merge with an earlier load of the same address
__device__ __forceinline__ uint4 ldg128_again(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Backward for bf16 rows of C = 256 * VPL columns: a lane owns VPL groups of 8 adjacent columns, moves everything with
// 16-byte accesses, keeps the weight-gradient sums of all its columns in registers over the rows it walks, and can add
// a second incoming gradient (`dres`: that of a skip connection around the norm) to dx in the same pass. x and dy are
// read twice (the second time from L1): holding a row between the passes costs the registers of the second resident block.
template <int VPL, int ACT>
__global__ void __launch_bounds__(256, 2)
rms_act_bwd_vec_kernel(const bf16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ rstd,
                       const bf16* __restrict__ dy, const bf16* __restrict__ dres, const bf16* __restrict__ dlead, int lead,
                       bf16* __restrict__ dx, float* __restrict__ dw, long long R) {
  constexpr int C = VPL * 256;
  __shared__ float s_dw[C];
  __shared__ __align__(16) float s_w[C];
  for (int c = threadIdx.x; c < C; c += 256) {
    s_dw[c] = 0.f;
    s_w[c] = w[c];
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * 8;
  const float invC = 1.f / (float)C;
  float acc[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
#pragma unroll 1
  for (long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); row < R; row += warps) {
    const long long base = row * C;
    const float rs = rstd[row];
    float dot = 0.f;
    {  // pass 1: the row's dot product and the weight-gradient terms
      uint4 xr[VPL], gr[VPL];
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const long long o = base + (j * 32 + lane) * 8;
        xr[j] = *reinterpret_cast<const uint4*>(x + o);
        gr[j] = *reinterpret_cast<const uint4*>(dy + o);
      }
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        const int c0 = (j * 32 + lane) * 8;
        const float4 w0 = lds128_volatile(s_w + c0), w1 = lds128_volatile(s_w + c0 + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const uint32_t xp[4] = {xr[j].x, xr[j].y, xr[j].z, xr[j].w};
        const uint32_t gp[4] = {gr[j].x, gr[j].y, gr[j].z, gr[j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float h0 = bf_lo(xp[q]) * rs, h1 = bf_hi(xp[q]) * rs;
          float g0 = bf_lo(gp[q]), g1 = bf_hi(gp[q]);
          if (j == 0 && c0 + 2 * q < lead) g0 += __bfloat162float(dlead[row * lead + c0 + 2 * q]);
          if (j == 0 && c0 + 2 * q + 1 < lead) g1 += __bfloat162float(dlead[row * lead + c0 + 2 * q + 1]);
          g0 *= act_grad<ACT>(wv[2 * q] * h0);
          g1 *= act_grad<ACT>(wv[2 * q + 1] * h1);
          dot = fmaf(g0 * wv[2 * q], h0, dot);
          dot = fmaf(g1 * wv[2 * q + 1], h1, dot);
          acc[j][2 * q] = fmaf(g0, h0, acc[j][2 * q]);
          acc[j][2 * q + 1] = fmaf(g1, h1, acc[j][2 * q + 1]);
        }
      }
    }
    dot = warp_sum(dot) * invC;
    // pass 2: x and dy again (the warp's own lines, still in L1), the skip's gradient, dx out
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c0 = (j * 32 + lane) * 8;
      const uint4 rr = dres ? *reinterpret_cast<const uint4*>(dres + base + c0) : make_uint4(0u, 0u, 0u, 0u);
      const uint4 xv = ldg128_again(x + base + c0), gv = ldg128_again(dy + base + c0);
      const float4 w0 = lds128_volatile(s_w + c0), w1 = lds128_volatile(s_w + c0 + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      const uint32_t xp[4] = {xv.x, xv.y, xv.z, xv.w};
      const uint32_t gp[4] = {gv.x, gv.y, gv.z, gv.w};
      const uint32_t rp[4] = {rr.x, rr.y, rr.z, rr.w};
      uint32_t op[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float h0 = bf_lo(xp[q]) * rs, h1 = bf_hi(xp[q]) * rs;
        float g0 = bf_lo(gp[q]), g1 = bf_hi(gp[q]);
        if (j == 0 && c0 + 2 * q < lead) g0 += __bfloat162float(dlead[row * lead + c0 + 2 * q]);
        if (j == 0 && c0 + 2 * q + 1 < lead) g1 += __bfloat162float(dlead[row * lead + c0 + 2 * q + 1]);
        g0 *= act_grad<ACT>(wv[2 * q] * h0);
        g1 *= act_grad<ACT>(wv[2 * q + 1] * h1);
        op[q] = bf_pack(fmaf(rs, g0 * wv[2 * q] - h0 * dot, bf_lo(rp[q])), fmaf(rs, g1 * wv[2 * q + 1] - h1 * dot, bf_hi(rp[q])));
      }
      *reinterpret_cast<uint4*>(dx + base + c0) = make_uint4(op[0], op[1], op[2], op[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (acc[j][e] != 0.f) atomicAdd(&s_dw[(j * 32 + lane) * 8 + e], acc[j][e]);
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

void rms_act_bwd(const void* x, bool x_bf16, const float* w, const float* rstd, const void* dy, bool dy_bf16,
                 const void* dres, const void* dlead, int lead, void* dx, float* dw, long long R, int C, int act,
                 cudaStream_t s) {
  if (dlead == nullptr) lead = 0;
  if (lead < 0 || lead > C) throw std::runtime_error("rms_act: lead columns out of range");
  if (C < 1 || C > 4096) throw std::runtime_error("rms_act: row length must be in [1, 4096]");
  if (R == 0) return;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx) |
                         reinterpret_cast<uintptr_t>(dres) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (x_bf16 && dy_bf16 && aligned && C % 256 == 0 && C <= 1024) {
    const int grid = (int)std::min<long long>((R + 7) / 8, 148LL * 4);
#define RMS_VEC(VPL_)                                                                                                  \
  DISPATCH_ACT(act, rms_act_bwd_vec_kernel<VPL_, ACT_><<<grid, 256, 0, s>>>((const bf16*)x, w, rstd, (const bf16*)dy,  \
                                                                             (const bf16*)dres, (const bf16*)dlead, lead,    \
                                                                             (bf16*)dx, dw, R))
    switch (C / 256) {
      case 1: RMS_VEC(1); break;
      case 2: RMS_VEC(2); break;
      case 3: RMS_VEC(3); break;
      default: RMS_VEC(4); break;
    }
#undef RMS_VEC
    chk("rms_act_bwd");
    return;
  }
  DISPATCH_ACT(act, DISPATCH_IO(x_bf16, dy_bf16, {
    rms_act_bwd_kernel<TI_, TO_, ACT_><<<grid_for(R), 256, (size_t)C * sizeof(float), s>>>((const TI_*)x, w, rstd, (const TO_*)dy, (const TI_*)dres, (const TO_*)dlead, lead, (TI_*)dx, dw, R, C);
  }));
  chk("rms_act_bwd");
}

}  // namespace b200
