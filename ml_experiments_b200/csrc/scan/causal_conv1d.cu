// Causal depthwise conv1d (kernel width 4) fused with bias and SiLU, channel-last, forward and backward.
//   y[b,t,c] = silu(bias[c] + sum_k w[c][k] * x[b, t-3+k, c])
// A warp covers 256 adjacent channels (8 per lane, 16-byte accesses) and walks 64 time steps with the 4-tap window
// kept in registers. The backward recomputes the pre-activation, walks 3 steps past its tile for the taps that reach
// forward in time, and accumulates dw / dbias in registers before one atomic add per thread.
// Replaces causal_conv1d_cuda / nn.Conv1d of the reference Mamba mixer (zoology/mixers/mamba.py:155-169).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "s6_scan.h"

namespace b200 {
namespace {
using bf16 = __nv_bfloat16;
constexpr int TT = 64;

__device__ __forceinline__ void ld8(const bf16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
struct Raw4 { uint2 u; };
struct Raw8 { uint4 u; };
__device__ __forceinline__ void ldraw(const bf16* p, Raw8& r) { r.u = *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void ldraw(const bf16* p, Raw4& r) { r.u = *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ void cvt(const Raw8& r, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
__device__ __forceinline__ void cvt(const Raw4& r, float (&f)[4]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.u);
#pragma unroll
  for (int i = 0; i < 2; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
__device__ __forceinline__ void stn(bf16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void stn(bf16* p, const float (&f)[4]) {
  uint2 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
  h[0] = __floats2bfloat162_rn(f[0], f[1]);
  h[1] = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = u;
}
template <int N> struct RawOf;
template <> struct RawOf<8> { using type = Raw8; };
template <> struct RawOf<4> { using type = Raw4; };

// Each thread walks its time tile serially, so one row's DRAM latency per step would bound the kernel: the rows PF
// steps ahead are requested into L1 (no registers held), the demand loads then hit L1.
constexpr int PF = 8;
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ void cvt8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
}
__device__ __forceinline__ void st8(bf16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// grid (ceil(C/8/128), ceil(L/TT), B), 128 threads: thread = 8 channels
__global__ void __launch_bounds__(128)
conv_fwd_kernel(const bf16* __restrict__ x, long long ldx, const float* __restrict__ w, const float* __restrict__ bias,
                bf16* __restrict__ y, int L, int C) {
  const int c0 = (blockIdx.x * 128 + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * TT, b = blockIdx.z;
  float wk[4][8], bs[8], win[3][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int k = 0; k < 4; ++k) wk[k][i] = w[(c0 + i) * 4 + k];
    bs[i] = bias ? bias[c0 + i] : 0.f;
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int t = t0 - 3 + j;
    if (t >= 0) ld8(x + ((long long)b * L + t) * ldx + c0, win[j]);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j][i] = 0.f;
    }
  }
  const int tstop = min(t0 + TT, L);
#pragma unroll
  for (int j = 0; j < PF; ++j)
    if (t0 + j < tstop) prefetch_l1(x + ((long long)b * L + t0 + j) * ldx + c0);
  for (int t = t0; t < tstop; ++t) {
    float cur[8], o[8];
    if (t + PF < tstop) prefetch_l1(x + ((long long)b * L + t + PF) * ldx + c0);
    ld8(x + ((long long)b * L + t) * ldx + c0, cur);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float pre = bs[i] + wk[0][i] * win[0][i] + wk[1][i] * win[1][i] + wk[2][i] * win[2][i] + wk[3][i] * cur[i];
      o[i] = pre / (1.f + __expf(-pre));
      win[0][i] = win[1][i]; win[1][i] = win[2][i]; win[2][i] = cur[i];
    }
    st8(y + ((long long)b * L + t) * C + c0, o);
  }
}

// CPT channels per thread: 4 keeps the kernel at 96 registers (5 blocks per SM); once the rows are prefetched the kernel
// is bound by instruction issue at low occupancy, not by memory (8 channels: 168 registers, 243 us; 4 channels: 190 us;
// unrolling the time loop by 3 to rename the window rotation away costs a block per SM and runs at 235 us).
template <int CPT>
__global__ void __launch_bounds__(128)
conv_bwd_kernel(const bf16* __restrict__ x, long long ldx, const float* __restrict__ w, const float* __restrict__ bias,
                const bf16* __restrict__ dy, bf16* __restrict__ dx, long long lddx, float* __restrict__ dw,
                float* __restrict__ dbias, int L, int C) {
  const int c0 = (blockIdx.x * 128 + threadIdx.x) * CPT;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * TT, b = blockIdx.z;
  using Raw = typename RawOf<CPT>::type;
  float wk[4][CPT], bs[CPT], win[3][CPT], dp[3][CPT], dwa[4][CPT], dba[CPT];
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
#pragma unroll
    for (int k = 0; k < 4; ++k) { wk[k][i] = w[(c0 + i) * 4 + k]; dwa[k][i] = 0.f; }
    bs[i] = bias ? bias[c0 + i] : 0.f;
    dba[i] = 0.f;
#pragma unroll
    for (int j = 0; j < 3; ++j) dp[j][i] = 0.f;
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int t = t0 - 3 + j;
    if (t >= 0) {
      Raw r;
      ldraw(x + ((long long)b * L + t) * ldx + c0, r);
      cvt(r, win[j]);
    }
    else {
#pragma unroll
      for (int i = 0; i < CPT; ++i) win[j][i] = 0.f;
    }
  }
  const int tend = min(t0 + TT, L);
  // the rows of step t + 1 are requested before step t is computed (raw 16-byte registers), so two steps' loads are in flight
  Raw nx{}, ng{};
  if (t0 < L) {
    ldraw(x + ((long long)b * L + t0) * ldx + c0, nx);
    ldraw(dy + ((long long)b * L + t0) * C + c0, ng);
  }
  const int tlast = min(tend + 3, L);
#pragma unroll
  for (int j = 1; j < PF; ++j)
    if (t0 + j < tlast) {
      prefetch_l1(x + ((long long)b * L + t0 + j) * ldx + c0);
      prefetch_l1(dy + ((long long)b * L + t0 + j) * C + c0);
    }
  for (int t = t0; t < tend + 3; ++t) {
    float cur[CPT], g[CPT], dpre[CPT];
    const bool in = t < L;
    if (t + PF < tlast) {
      prefetch_l1(x + ((long long)b * L + t + PF) * ldx + c0);
      prefetch_l1(dy + ((long long)b * L + t + PF) * C + c0);
    }
    const Raw ux = nx, ug = ng;
    if (t + 1 < tend + 3 && t + 1 < L) {
      ldraw(x + ((long long)b * L + t + 1) * ldx + c0, nx);
      ldraw(dy + ((long long)b * L + t + 1) * C + c0, ng);
    }
    if (in) {
      cvt(ux, cur);
      cvt(ug, g);
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      if (in) {
        const float pre = bs[i] + wk[0][i] * win[0][i] + wk[1][i] * win[1][i] + wk[2][i] * win[2][i] + wk[3][i] * cur[i];
        const float sg = 1.f / (1.f + __expf(-pre));
        dpre[i] = g[i] * sg * (1.f + pre * (1.f - sg));
        if (t < tend) {  // parameters: every time step is counted by exactly one tile
          dwa[0][i] += dpre[i] * win[0][i]; dwa[1][i] += dpre[i] * win[1][i];
          dwa[2][i] += dpre[i] * win[2][i]; dwa[3][i] += dpre[i] * cur[i];
          dba[i] += dpre[i];
        }
      } else {
        dpre[i] = 0.f;
        cur[i] = 0.f;
      }
    }
    if (t - 3 >= t0) {  // dx[s] = w3 dpre[s] + w2 dpre[s+1] + w1 dpre[s+2] + w0 dpre[s+3], s = t - 3
      float o[CPT];
#pragma unroll
      for (int i = 0; i < CPT; ++i)
        o[i] = wk[3][i] * dp[0][i] + wk[2][i] * dp[1][i] + wk[1][i] * dp[2][i] + wk[0][i] * dpre[i];
      stn(dx + ((long long)b * L + t - 3) * lddx + c0, o);
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      dp[0][i] = dp[1][i]; dp[1][i] = dp[2][i]; dp[2][i] = dpre[i];
      win[0][i] = win[1][i]; win[1][i] = win[2][i]; win[2][i] = cur[i];
    }
  }
#pragma unroll
  for (int i = 0; i < CPT; ++i) {
#pragma unroll
    for (int k = 0; k < 4; ++k) atomicAdd(&dw[(c0 + i) * 4 + k], dwa[k][i]);
    if (dbias) atomicAdd(&dbias[c0 + i], dba[i]);
  }
}

void chk(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
}  // namespace

void causal_conv1d_silu_fwd(const void* x, long long ldx, const float* w, const float* bias, void* y, int batch, int L,
                            int C, cudaStream_t s) {
  if (C % 8 != 0 || ldx % 8 != 0) throw std::runtime_error("causal_conv1d: channels and row pitch must be multiples of 8");
  dim3 grid((C / 8 + 127) / 128, (L + TT - 1) / TT, batch);
  conv_fwd_kernel<<<grid, 128, 0, s>>>((const bf16*)x, ldx, w, bias, (bf16*)y, L, C);
  chk("causal_conv1d_silu_fwd");
}

void causal_conv1d_silu_bwd(const void* x, long long ldx, const float* w, const float* bias, const void* dy, void* dx,
                            long long lddx, float* dw, float* dbias, int batch, int L, int C, cudaStream_t s) {
  if (C % 8 != 0 || ldx % 8 != 0 || lddx % 8 != 0) throw std::runtime_error("causal_conv1d: channels and row pitch must be multiples of 8");
  dim3 grid((C / 4 + 127) / 128, (L + TT - 1) / TT, batch);
  conv_bwd_kernel<4><<<grid, 128, 0, s>>>((const bf16*)x, ldx, w, bias, (const bf16*)dy, (bf16*)dx, lddx, dw, dbias, L, C);
  chk("causal_conv1d_silu_bwd");
}

}  // namespace b200
