// RMS norm over the head dimension followed by the rotary map of the current speedrun GPT, forward and backward:
//   n = x * rsqrt(mean(x^2) + eps);   y[2i] = f1[2i] n[2i] + f2[2i] n[2i+1];   y[2i+1] = f1[2i+1] n[2i+1] + f2[2i+1] n[2i]
// with tables f1 = cos, f2 = sign-alternated sin per position (modded-nanogpt/train_gpt.py: `norm` + `Yarn.rotary`,
// i.e. F.rms_norm, a pair flip, two broadcast multiplies and an add: five elementwise kernels forward, about twelve in
// the backward graph). One warp per (token, head) row; a lane holds D / 32 consecutive elements, so a pair never
// leaves its lane. x may be a strided view (the q or k third of a fused projection); y and dx are contiguous.
// Paired-head layout: the table row is 2 D wide and head h reads columns (h % 2) * D onwards.
#include "fused.h"

#include <cuda_bf16.h>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// E (2 or 4) consecutive bf16 as one 4- or 8-byte access; every row and table offset is a multiple of E elements
template <int E>
__device__ __forceinline__ void ldE(const bf16* p, float (&o)[E]) {
  if constexpr (E == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    o[0] = a.x; o[1] = a.y;
  }
}
template <int E>
__device__ __forceinline__ void stE(bf16* p, const float (&o)[E]) {
  if constexpr (E == 4) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  } else {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(o[0], o[1]);
  }
}

template <int E>  // elements per lane: D = 32 * E
__global__ void __launch_bounds__(256) norm_rope_fwd_kernel(const bf16* __restrict__ x, long long st, long long sh,
                                                            const bf16* __restrict__ f1, const bf16* __restrict__ f2, int tab_w,
                                                            bf16* __restrict__ y, float* __restrict__ rstd, long long rows, int H,
                                                            int T, float eps) {
  constexpr int D = 32 * E;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int h = (int)(row % H);
  const long long bt = row / H;            // batch * T + t (batch entries share the tables)
  const int t = (int)(bt % T);
  const bf16* xp = x + bt * st + (long long)h * sh + lane * E;
  const long long tab = (long long)t * tab_w + (h % (tab_w / D)) * D + lane * E;
  float v[E], a[E], b[E];
  ldE<E>(xp, v);
  ldE<E>(f1 + tab, a);
  ldE<E>(f2 + tab, b);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) ss += v[e] * v[e];
  ss = wsum(ss);
  const float r = rsqrtf(ss / D + eps);
  if (lane == 0) rstd[row] = r;
  float o[E];
#pragma unroll
  for (int e = 0; e < E; e += 2) {
    const float n0 = v[e] * r, n1 = v[e + 1] * r;
    o[e] = a[e] * n0 + b[e] * n1;
    o[e + 1] = a[e + 1] * n1 + b[e + 1] * n0;
  }
  stE<E>(y + row * D + lane * E, o);
}

template <int E>
__global__ void __launch_bounds__(256) norm_rope_bwd_kernel(const bf16* __restrict__ x, long long st, long long sh,
                                                            const bf16* __restrict__ f1, const bf16* __restrict__ f2, int tab_w,
                                                            const float* __restrict__ rstd, const bf16* __restrict__ dy,
                                                            bf16* __restrict__ dx, long long rows, int H, int T) {
  constexpr int D = 32 * E;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int h = (int)(row % H);
  const long long bt = row / H;
  const int t = (int)(bt % T);
  const bf16* xp = x + bt * st + (long long)h * sh + lane * E;
  const bf16* gp = dy + row * D + lane * E;
  const long long tab = (long long)t * tab_w + (h % (tab_w / D)) * D + lane * E;
  const float r = rstd[row];
  float n[E], dn[E], g[E], a[E], b[E];
  ldE<E>(xp, n);
  ldE<E>(gp, g);
  ldE<E>(f1 + tab, a);
  ldE<E>(f2 + tab, b);
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < E; e += 2) {
    dn[e] = a[e] * g[e] + b[e + 1] * g[e + 1];        // n[e] enters y[e] through f1[e] and y[e+1] through f2[e+1]
    dn[e + 1] = a[e + 1] * g[e + 1] + b[e] * g[e];
    n[e] *= r;
    n[e + 1] *= r;
    dot += dn[e] * n[e] + dn[e + 1] * n[e + 1];
  }
  dot = wsum(dot) / D;
  float o[E];
#pragma unroll
  for (int e = 0; e < E; ++e) o[e] = r * (dn[e] - n[e] * dot);
  stE<E>(dx + row * D + lane * E, o);
}

void chk(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

void norm_rope_fwd(const void* x, long long st, long long sh, const void* f1, const void* f2, int tab_w, void* y, float* rstd,
                   long long rows, int H, int T, int D, float eps, cudaStream_t s) {
  const int blocks = (int)((rows * 32 + 255) / 256);
  if (D == 128) norm_rope_fwd_kernel<4><<<blocks, 256, 0, s>>>((const bf16*)x, st, sh, (const bf16*)f1, (const bf16*)f2, tab_w, (bf16*)y, rstd, rows, H, T, eps);
  else if (D == 64) norm_rope_fwd_kernel<2><<<blocks, 256, 0, s>>>((const bf16*)x, st, sh, (const bf16*)f1, (const bf16*)f2, tab_w, (bf16*)y, rstd, rows, H, T, eps);
  else throw std::runtime_error("norm_rope: head_dim must be 64 or 128");
  chk("norm_rope_fwd");
}

void norm_rope_bwd(const void* x, long long st, long long sh, const void* f1, const void* f2, int tab_w, const float* rstd,
                   const void* dy, void* dx, long long rows, int H, int T, int D, cudaStream_t s) {
  const int blocks = (int)((rows * 32 + 255) / 256);
  if (D == 128) norm_rope_bwd_kernel<4><<<blocks, 256, 0, s>>>((const bf16*)x, st, sh, (const bf16*)f1, (const bf16*)f2, tab_w, rstd, (const bf16*)dy, (bf16*)dx, rows, H, T);
  else if (D == 64) norm_rope_bwd_kernel<2><<<blocks, 256, 0, s>>>((const bf16*)x, st, sh, (const bf16*)f1, (const bf16*)f2, tab_w, rstd, (const bf16*)dy, (bf16*)dx, rows, H, T);
  else throw std::runtime_error("norm_rope: head_dim must be 64 or 128");
  chk("norm_rope_bwd");
}

}  // namespace b200
