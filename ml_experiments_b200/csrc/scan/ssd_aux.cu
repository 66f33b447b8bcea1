// Elementwise companions of the SSD scan's backward (ops/ssd_scan.py::_SsdKernelGradFn). The backward runs the scan
// kernel three more times, two of them backwards in time; these two kernels do everything around those launches in one
// pass each, so no fp32 copy of a [batch, L, H, P] tensor is ever made:
//   flip_time      dst[b][L-1-l][:] = src[b][l][:]                     (bf16 rows, 16-byte vectors)
//   ssd_bwd_post   combines the three scan outputs with x, dy, y, B, C and the weights into dx, dB, dC and the three
//                  per-step scalars (d g_off, d g_diag, row sum minus column sum for the decay gradient); reads the two
//                  time-reversed scan outputs at their mirrored position, sums dB / dC over the heads of a B / C group.
#include "ssd.h"

#include <cuda_bf16.h>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;

__global__ void flip_time_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int L, int vec_per_row, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vec_per_row;
    const int v = (int)(i - row * vec_per_row);
    const long long b = row / L;
    const int l = (int)(row - b * L);
    dst[(b * L + (L - 1 - l)) * vec_per_row + v] = src[i];
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per (batch, step, B/C group); it walks the `rep` heads of the group. EP / EN = elements of P / N per lane.
template <int EP, int EN>
__global__ void __launch_bounds__(256) ssd_bwd_post_kernel(const SsdPostArgs a) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long nwarps = (long long)a.batch * a.L * a.Hb;
  if (warp >= nwarps) return;
  const int hb = (int)(warp % a.Hb);
  const long long bl = warp / a.Hb;
  const int l = (int)(bl % a.L);
  const long long b = bl / a.L;
  const long long bl_rev = b * a.L + (a.L - 1 - l);
  const int rep = a.H / a.Hb, P = EP * 32, N = EN * 32;
  float Bv[EN], Cv[EN], dBacc[EN], dCacc[EN];
  const bf16* Bp = reinterpret_cast<const bf16*>(a.B) + (bl * a.Hb + hb) * N;
  const bf16* Cp = reinterpret_cast<const bf16*>(a.C) + (bl * a.Hb + hb) * N;
  float cb = 0.f;
#pragma unroll
  for (int e = 0; e < EN; ++e) {
    Bv[e] = __bfloat162float(Bp[lane + 32 * e]);
    Cv[e] = __bfloat162float(Cp[lane + 32 * e]);
    cb += Bv[e] * Cv[e];
    dBacc[e] = 0.f;
    dCacc[e] = 0.f;
  }
  cb = warp_sum(cb);
  for (int r = 0; r < rep; ++r) {
    const int h = hb * rep + r;
    const long long row = bl * a.H + h, row_rev = bl_rev * a.H + h;
    const bf16* xp = reinterpret_cast<const bf16*>(a.x) + row * P;
    const bf16* dyp = reinterpret_cast<const bf16*>(a.dy) + row * P;
    const bf16* yp = reinterpret_cast<const bf16*>(a.y) + row * P;
    const bf16* dxr = reinterpret_cast<const bf16*>(a.dx_rev) + row_rev * P;
    float xv[EP], dyv[EP], dxo[EP];
    float dyx = 0.f, xdx = 0.f, dyy = 0.f;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      xv[e] = __bfloat162float(xp[lane + 32 * e]);
      dyv[e] = __bfloat162float(dyp[lane + 32 * e]);
      dxo[e] = __bfloat162float(dxr[lane + 32 * e]);
      dyx += dyv[e] * xv[e];
      xdx += xv[e] * dxo[e];
      dyy += dyv[e] * __bfloat162float(yp[lane + 32 * e]);
    }
    dyx = warp_sum(dyx); xdx = warp_sum(xdx); dyy = warp_sum(dyy);
    const float go = a.g_off[row], gd = a.g_diag[row];
    bf16* dxp = reinterpret_cast<bf16*>(a.dx) + row * P;
#pragma unroll
    for (int e = 0; e < EP; ++e) dxp[lane + 32 * e] = __float2bfloat16_rn(go * dxo[e] + gd * cb * dyv[e]);
    const bf16* dBr = reinterpret_cast<const bf16*>(a.dB_rev) + row_rev * N;
    const bf16* dCh = reinterpret_cast<const bf16*>(a.dC_heads) + row * N;
#pragma unroll
    for (int e = 0; e < EN; ++e) {
      dBacc[e] += go * __bfloat162float(dBr[lane + 32 * e]) + gd * dyx * Cv[e];
      dCacc[e] += __bfloat162float(dCh[lane + 32 * e]);
    }
    if (lane == 0) {
      a.d_goff[row] = xdx;
      a.d_gdiag[row] = cb * dyx;
      a.inner[row] = dyy - gd * cb * dyx - go * xdx;   // row sum of the off-diagonal pairs minus their column sum
    }
  }
  bf16* dBp = reinterpret_cast<bf16*>(a.dB) + (bl * a.Hb + hb) * N;
  bf16* dCp = reinterpret_cast<bf16*>(a.dC) + (bl * a.Hb + hb) * N;
#pragma unroll
  for (int e = 0; e < EN; ++e) {
    dBp[lane + 32 * e] = __float2bfloat16_rn(dBacc[e]);
    dCp[lane + 32 * e] = __float2bfloat16_rn(dCacc[e]);
  }
}

void check(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

void ssd_flip_time(const void* src, void* dst, int batch, int L, long long row_bytes, cudaStream_t s) {
  if (row_bytes % 16 != 0) throw std::runtime_error("ssd_flip_time: rows must be multiples of 16 bytes");
  const int vpr = (int)(row_bytes / 16);
  const long long total = (long long)batch * L * vpr;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  flip_time_kernel<<<blocks, 256, 0, s>>>((const uint4*)src, (uint4*)dst, L, vpr, total);
  check("ssd_flip_time");
}

void ssd_bwd_post(const SsdPostArgs& a) {
  if (a.H % a.Hb != 0) throw std::runtime_error("ssd_bwd_post: heads must be a multiple of the B / C groups");
  const long long warps = (long long)a.batch * a.L * a.Hb;
  const int blocks = (int)((warps * 32 + 255) / 256);
  if (a.P == 64 && a.N == 64) ssd_bwd_post_kernel<2, 2><<<blocks, 256, 0, a.stream>>>(a);
  else if (a.P == 64 && a.N == 128) ssd_bwd_post_kernel<2, 4><<<blocks, 256, 0, a.stream>>>(a);
  else if (a.P == 128 && a.N == 64) ssd_bwd_post_kernel<4, 2><<<blocks, 256, 0, a.stream>>>(a);
  else if (a.P == 128 && a.N == 128) ssd_bwd_post_kernel<4, 4><<<blocks, 256, 0, a.stream>>>(a);
  else throw std::runtime_error("ssd_bwd_post: N and P must be 64 or 128");
  check("ssd_bwd_post");
}

}  // namespace b200
