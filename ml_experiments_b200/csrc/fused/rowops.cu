// Two small fused maps that the current speedrun GPT applies to every layer's activations (eager PyTorch issues one
// broadcast kernel per operator, and about twice as many again in the backward graph):
//   rowscale_add   out[r, :] = a[r, :] + g[r] * b[r, :]      rows r = (token, head), D = 64 or 128 columns; `a` optional
//                  (attention-output gate y * sigmoid(.), value-embedding mix v + 2 sigmoid(.) * ve)
//                  backward: db = g * dout, dg[r] = dout[r, :] . b[r, :]  (da = dout needs no kernel)
//   lincomb3       out = c0 x + c1 y + c2 z  over flat bf16 tensors, c on the device (residual / x0 / bigram mix)
//                  backward: dx = c0 dout, dy = c1 dout, dz = c2 dout, dc = (dout . x, dout . y, dout . z)
// Reference expressions: modded-nanogpt/train_gpt.py (`CausalSelfAttention.forward`, the layer loop of `GPT.forward`).
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

// a: optional, element strides st (between tokens) and sh (between heads); b, out contiguous [rows, D]; g [rows] bf16
template <int E>
__global__ void __launch_bounds__(256) rowscale_add_fwd_kernel(const bf16* __restrict__ a, long long st, long long sh,
                                                               const bf16* __restrict__ g, const bf16* __restrict__ b,
                                                               bf16* __restrict__ out, long long rows, int H) {
  constexpr int D = 32 * E;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float gv = __bfloat162float(g[row]);
  float bv[E], av[E], o[E];
  ldE<E>(b + row * D + lane * E, bv);
  if (a) ldE<E>(a + (row / H) * st + (row % H) * sh + lane * E, av);
#pragma unroll
  for (int e = 0; e < E; ++e) o[e] = (a ? av[e] : 0.f) + gv * bv[e];
  stE<E>(out + row * D + lane * E, o);
}

template <int E>
__global__ void __launch_bounds__(256) rowscale_add_bwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ b,
                                                               const bf16* __restrict__ dout, bf16* __restrict__ db,
                                                               bf16* __restrict__ dg, long long rows) {
  constexpr int D = 32 * E;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float gv = __bfloat162float(g[row]);
  float bv[E], dv[E], o[E];
  ldE<E>(b + row * D + lane * E, bv);
  ldE<E>(dout + row * D + lane * E, dv);
  float dot = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    o[e] = gv * dv[e];
    dot += dv[e] * bv[e];
  }
  stE<E>(db + row * D + lane * E, o);
  dot = wsum(dot);
  if (lane == 0) dg[row] = __float2bfloat16_rn(dot);
}

__global__ void __launch_bounds__(256) lincomb3_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                                           const bf16* __restrict__ z, const float* __restrict__ c,
                                                           bf16* __restrict__ out, long long n) {
  const float c0 = c[0], c1 = c[1], c2 = z ? c[2] : 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float a[4], b[4], d[4], o[4];
    ldE<4>(x + i, a);
    ldE<4>(y + i, b);
    if (z) ldE<4>(z + i, d);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = c0 * a[e] + c1 * b[e] + (z ? c2 * d[e] : 0.f);
    stE<4>(out + i, o);
  }
}

// dx, dy, dz written; dc accumulated by one atomic per block and coefficient (zero it first)
__global__ void __launch_bounds__(256) lincomb3_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                                           const bf16* __restrict__ z, const float* __restrict__ c,
                                                           const bf16* __restrict__ dout, bf16* __restrict__ dx,
                                                           bf16* __restrict__ dy, bf16* __restrict__ dz, float* __restrict__ dc,
                                                           long long n) {
  __shared__ float red[3][8];
  const float c0 = c[0], c1 = c[1], c2 = z ? c[2] : 0.f;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float a[4], b[4], d[4], g[4], o[4];
    ldE<4>(x + i, a);
    ldE<4>(y + i, b);
    ldE<4>(dout + i, g);
    if (z) ldE<4>(z + i, d);
#pragma unroll
    for (int e = 0; e < 4; ++e) { s0 += g[e] * a[e]; s1 += g[e] * b[e]; if (z) s2 += g[e] * d[e]; }
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = c0 * g[e];
    stE<4>(dx + i, o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = c1 * g[e];
    stE<4>(dy + i, o);
    if (z) {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = c2 * g[e];
      stE<4>(dz + i, o);
    }
  }
  s0 = wsum(s0); s1 = wsum(s1); s2 = wsum(s2);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { red[0][w] = s0; red[1][w] = s1; red[2][w] = s2; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[threadIdx.x][i];
    if (threadIdx.x < 2 || z) atomicAdd(dc + threadIdx.x, t);
  }
}

void chk(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
int flat_blocks(long long n) {
  long long b = (n / 4 + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  return b < 1 ? 1 : (int)b;
}

}  // namespace

void rowscale_add_fwd(const void* a, long long st, long long sh, const void* g, const void* b, void* out, long long rows, int H,
                      int D, cudaStream_t s) {
  const int blocks = (int)((rows * 32 + 255) / 256);
  if (D == 128) rowscale_add_fwd_kernel<4><<<blocks, 256, 0, s>>>((const bf16*)a, st, sh, (const bf16*)g, (const bf16*)b, (bf16*)out, rows, H);
  else if (D == 64) rowscale_add_fwd_kernel<2><<<blocks, 256, 0, s>>>((const bf16*)a, st, sh, (const bf16*)g, (const bf16*)b, (bf16*)out, rows, H);
  else throw std::runtime_error("rowscale_add: 64 or 128 columns");
  chk("rowscale_add_fwd");
}

void rowscale_add_bwd(const void* g, const void* b, const void* dout, void* db, void* dg, long long rows, int D, cudaStream_t s) {
  const int blocks = (int)((rows * 32 + 255) / 256);
  if (D == 128) rowscale_add_bwd_kernel<4><<<blocks, 256, 0, s>>>((const bf16*)g, (const bf16*)b, (const bf16*)dout, (bf16*)db, (bf16*)dg, rows);
  else if (D == 64) rowscale_add_bwd_kernel<2><<<blocks, 256, 0, s>>>((const bf16*)g, (const bf16*)b, (const bf16*)dout, (bf16*)db, (bf16*)dg, rows);
  else throw std::runtime_error("rowscale_add: 64 or 128 columns");
  chk("rowscale_add_bwd");
}

void lincomb3_fwd(const void* x, const void* y, const void* z, const float* c, void* out, long long n, cudaStream_t s) {
  if (n % 4 != 0) throw std::runtime_error("lincomb3: element count must be a multiple of 4");
  lincomb3_fwd_kernel<<<flat_blocks(n), 256, 0, s>>>((const bf16*)x, (const bf16*)y, (const bf16*)z, c, (bf16*)out, n);
  chk("lincomb3_fwd");
}

void lincomb3_bwd(const void* x, const void* y, const void* z, const float* c, const void* dout, void* dx, void* dy, void* dz,
                  float* dc, long long n, cudaStream_t s) {
  if (n % 4 != 0) throw std::runtime_error("lincomb3: element count must be a multiple of 4");
  lincomb3_bwd_kernel<<<flat_blocks(n), 256, 0, s>>>((const bf16*)x, (const bf16*)y, (const bf16*)z, c, (const bf16*)dout, (bf16*)dx, (bf16*)dy,
                                                     (bf16*)dz, dc, n);
  chk("lincomb3_bwd");
}

}  // namespace b200
