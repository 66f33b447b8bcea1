// Gather-convolution kernels (see gather_conv.h). One group of D/4 adjacent lanes owns one (batch, position, head)
// row; each lane keeps 4 channels. Tap positions / weights are read 4 at a time; value rows are 8-byte bf16 loads
// that the group covers contiguously (coalesced 2*D bytes per row). The backward scatters with float4 atomics.
// Counterpart of the Triton kernels telephone_attn_fwd/bwd_kernel, adaptive_conv_fwd/bwd_kernel and
// _scatter_attn_fwd/bwd_kernel of the reference (src/heuristic_secrets/models/triton_telephone.py:149-357,
// triton_adaptive_conv.py:81-318, triton_scatter.py:26-238), which fuse the same gather with their tap formulas.
#include "gather_conv.h"

#include <cuda_bf16.h>

#include <cstdint>
#include <stdexcept>
#include <string>

namespace b200 {
namespace {
using bf16 = __nv_bfloat16;

__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
  const unsigned lane = threadIdx.x & 31u;
  const unsigned mask = (LPR == 32 ? 0xffffffffu : ((1u << LPR) - 1u)) << (lane & ~unsigned(LPR - 1));
#pragma unroll
  for (int s = LPR / 2; s > 0; s >>= 1) v += __shfl_xor_sync(mask, v, s);
  return v;
}

template <int LPR>
__global__ void __launch_bounds__(256)
gather_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ pos, const float* __restrict__ wgt,
                  bf16* __restrict__ out, int B, int L, int Lq, int H, int S, float pos_max) {
  constexpr int D = LPR * 4;
  const long long row = ((long long)blockIdx.x * 256 + threadIdx.x) / LPR;
  const int sub = threadIdx.x % LPR;
  if (row >= (long long)B * Lq * H) return;
  const int h = (int)(row % H);
  const long long bl = row / H;
  const int b = (int)(bl / Lq);
  const bf16* xb = x + (long long)b * L * H * D + h * D + sub * 4;
  const float* pr = pos + row * S;
  const float* wr = wgt + row * S;
  const float hi = pos_max;  // positions clamp into [0, pos_max]; the floor row is capped at L-2 so that p = L-1 reads row L-1 exactly
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < S; ++s) {
    const float w = wr[s];
    if (w == 0.f) continue;
    const float pc = fminf(fmaxf(pr[s], 0.f), hi);
    const int fl = min((int)pc, max(L - 2, 0));
    const int ce = min(fl + 1, L - 1);
    const float fr = pc - (float)fl;
    const float4 a = ld4(xb + (long long)fl * H * D), c = ld4(xb + (long long)ce * H * D);
    const float wa = w * (1.f - fr), wc = w * fr;
    acc.x += wa * a.x + wc * c.x; acc.y += wa * a.y + wc * c.y;
    acc.z += wa * a.z + wc * c.z; acc.w += wa * a.w + wc * c.w;
  }
  __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi2 = __floats2bfloat162_rn(acc.z, acc.w);
  *reinterpret_cast<uint2*>(out + row * D + sub * 4) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi2));
}

template <int LPR>
__global__ void __launch_bounds__(256)
gather_bwd_kernel(const bf16* __restrict__ x, const float* __restrict__ pos, const float* __restrict__ wgt,
                  const bf16* __restrict__ dout, float* __restrict__ dx, float* __restrict__ dpos,
                  float* __restrict__ dwgt, int B, int L, int Lq, int H, int S, float pos_max) {
  constexpr int D = LPR * 4;
  const long long row = ((long long)blockIdx.x * 256 + threadIdx.x) / LPR;
  const int sub = threadIdx.x % LPR;
  const bool active = row < (long long)B * Lq * H;
  const long long rr = active ? row : 0;
  const int h = (int)(rr % H);
  const long long bl = rr / H;
  const int b = (int)(bl / Lq);
  const bf16* xb = x + (long long)b * L * H * D + h * D + sub * 4;
  float* dxb = dx + (long long)b * L * H * D + h * D + sub * 4;
  const float* pr = pos + rr * S;
  const float* wr = wgt + rr * S;
  const float hi = pos_max;  // positions clamp into [0, pos_max]; the floor row is capped at L-2 so that p = L-1 reads row L-1 exactly
  const float4 g = ld4(dout + rr * D + sub * 4);
  for (int s = 0; s < S; ++s) {
    const float w = wr[s];
    const float p = pr[s];
    const float pc = fminf(fmaxf(p, 0.f), hi);
    const int fl = min((int)pc, max(L - 2, 0));
    const int ce = min(fl + 1, L - 1);
    const float fr = pc - (float)fl;
    const float4 a = ld4(xb + (long long)fl * H * D), c = ld4(xb + (long long)ce * H * D);
    const float da = g.x * a.x + g.y * a.y + g.z * a.z + g.w * a.w;
    const float dc = g.x * c.x + g.y * c.y + g.z * c.z + g.w * c.w;
    const float sa = group_sum<LPR>(da), sc = group_sum<LPR>(dc);
    if (active && sub == 0) {
      dwgt[rr * S + s] = sa * (1.f - fr) + sc * fr;
      dpos[rr * S + s] = (p >= 0.f && p <= hi) ? w * (sc - sa) : 0.f;
    }
    if (active && w != 0.f) {
      const float wa = w * (1.f - fr), wc = w * fr;
      atomicAdd(reinterpret_cast<float4*>(dxb + (long long)fl * H * D), make_float4(wa * g.x, wa * g.y, wa * g.z, wa * g.w));
      if (wc != 0.f)
        atomicAdd(reinterpret_cast<float4*>(dxb + (long long)ce * H * D), make_float4(wc * g.x, wc * g.y, wc * g.z, wc * g.w));
    }
  }
}

void chk(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

#define DISPATCH_LPR(D, ...)                                    \
  switch ((D) / 4) {                                            \
    case 2: { constexpr int LPR_ = 2; __VA_ARGS__; break; }            \
    case 4: { constexpr int LPR_ = 4; __VA_ARGS__; break; }            \
    case 8: { constexpr int LPR_ = 8; __VA_ARGS__; break; }            \
    case 16: { constexpr int LPR_ = 16; __VA_ARGS__; break; }          \
    case 32: { constexpr int LPR_ = 32; __VA_ARGS__; break; }          \
    default: throw std::runtime_error("gather_conv: head_dim must be 8, 16, 32, 64 or 128"); \
  }
}  // namespace

void gather_conv_fwd(const void* x, const float* pos, const float* wgt, void* out, int B, int L, int Lq, int H, int D,
                     int S, float pos_max, cudaStream_t s) {
  const long long rows = (long long)B * Lq * H;
  DISPATCH_LPR(D, {
    const int rpb = 256 / LPR_;
    gather_fwd_kernel<LPR_><<<(unsigned)((rows + rpb - 1) / rpb), 256, 0, s>>>((const bf16*)x, pos, wgt, (bf16*)out, B, L, Lq, H, S, pos_max);
  });
  chk("gather_conv_fwd");
}

void gather_conv_bwd(const void* x, const float* pos, const float* wgt, const void* dout, float* dx, float* dpos,
                     float* dwgt, int B, int L, int Lq, int H, int D, int S, float pos_max, cudaStream_t s) {
  const long long rows = (long long)B * Lq * H;
  DISPATCH_LPR(D, {
    const int rpb = 256 / LPR_;
    gather_bwd_kernel<LPR_><<<(unsigned)((rows + rpb - 1) / rpb), 256, 0, s>>>((const bf16*)x, pos, wgt, (const bf16*)dout, dx,
                                                                              dpos, dwgt, B, L, Lq, H, S, pos_max);
  });
  chk("gather_conv_bwd");
}

}  // namespace b200
