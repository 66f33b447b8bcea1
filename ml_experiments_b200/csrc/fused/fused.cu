// Memory-bound fused kernels of the GPT step: RMSNorm (+ residual mixing), QK-norm + RoPE + value mixing,
// embedding gather / scatter-add, fp8 casts, soft-capped cross entropy, Adam and Muon element-wise parts.
// One warp owns one row wherever a row reduction is needed; all global accesses are 16-byte vectors.
#include "fused.h"

#include "common/per_device.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void ld4(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
__device__ __forceinline__ void ld4(const bf16* p, float (&f)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
}
__device__ __forceinline__ void st4(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void st4(bf16* p, const float (&f)[4]) {
  uint2 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
  h[0] = __floats2bfloat162_rn(f[0], f[1]);
  h[1] = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ void round8(float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16_rn(f[i]));
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

constexpr int kRowThreads = 256;  // 8 rows per block
inline int row_blocks(int R) { return (R + 7) / 8; }

// ---------------------------------------------------------------------------------------------- RMSNorm
template <int NCH>
__global__ void __launch_bounds__(kRowThreads)
mix_norm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ x0, const bf16* __restrict__ skip,
                    const float* __restrict__ lam, const float* __restrict__ skip_w, bf16* __restrict__ x_mix,
                    bf16* __restrict__ xn, int R, int C, float eps) {
  const int row = (blockIdx.x * kRowThreads + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  const long long base = (long long)row * C;
  const float l0 = (x0 && lam) ? lam[0] : 1.f, l1 = (x0 && lam) ? lam[1] : 0.f;
  const float w = (skip && skip_w) ? skip_w[0] : 0.f;
  float v[NCH][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (lane + 32 * k) * 8;
    if (c < C) {
      load8(x + base + c, v[k]);
      if (skip) {
        float s8[8];
        load8(skip + base + c, s8);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = fmaf(w, s8[i], v[k][i]);
      }
      if (x0) {
        float z8[8];
        load8(x0 + base + c, z8);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = l0 * v[k][i] + l1 * z8[i];
      }
      if (x_mix) {
        round8(v[k]);
        store8(x_mix + base + c, v[k]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[k][i], v[k][i], ss);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / C + eps);
  if (xn) {
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = (lane + 32 * k) * 8;
      if (c < C) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] *= r;
        store8(xn + base + c, v[k]);
      }
    }
  }
}

template <int NCH>
__global__ void __launch_bounds__(kRowThreads)
norm_bwd_add_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ dres,
                    bf16* __restrict__ out, int R, int C, float eps) {
  const int row = (blockIdx.x * kRowThreads + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  const long long base = (long long)row * C;
  float xv[NCH][8], gv[NCH][8];
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (lane + 32 * k) * 8;
    if (c < C) {
      load8(x + base + c, xv[k]);
      load8(dy + base + c, gv[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss = fmaf(xv[k][i], xv[k][i], ss);
        dot = fmaf(xv[k][i], gv[k][i], dot);
      }
    }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss / C + eps);
  const float coef = dot * r * r * r / C;  // mean(dy * y) * r / |x| scaling folded: dx = r*dy - x * coef
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (lane + 32 * k) * 8;
    if (c < C) {
      float o[8];
      if (dres) load8(dres + base + c, o);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += r * gv[k][i] - xv[k][i] * coef;
      store8(out + base + c, o);
    }
  }
}

template <int NCH>
__global__ void __launch_bounds__(kRowThreads)
mix_bwd_kernel(const bf16* __restrict__ dmix, const bf16* __restrict__ x, const bf16* __restrict__ x0,
               const bf16* __restrict__ skip, const float* __restrict__ lam, const float* __restrict__ skip_w,
               bf16* __restrict__ dx, bf16* __restrict__ dskip, float* __restrict__ dx0_acc, float* __restrict__ dlam,
               float* __restrict__ dskip_w, const bf16* __restrict__ dx_add, int R, int C) {
  __shared__ float red[3][kRowThreads / 32];
  const int warp_in_block = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const float l0 = lam[0], l1 = lam[1];
  const float w = (skip && skip_w) ? skip_w[0] : 0.f;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  for (int row = blockIdx.x * (kRowThreads / 32) + warp_in_block; row < R; row += gridDim.x * (kRowThreads / 32)) {
    const long long base = (long long)row * C;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = (lane + 32 * k) * 8;
      if (c < C) {
        float g[8], xv[8], zv[8], sv[8], o[8];
        load8(dmix + base + c, g);
        load8(x + base + c, xv);
        load8(x0 + base + c, zv);
        if (skip) {
          load8(skip + base + c, sv);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a2 = fmaf(l0 * g[i], sv[i], a2);
            xv[i] = fmaf(w, sv[i], xv[i]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = l0 * w * g[i];
          store8(dskip + base + c, o);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a0 = fmaf(g[i], xv[i], a0);
          a1 = fmaf(g[i], zv[i], a1);
          o[i] = l0 * g[i];
        }
        if (dx_add) {   // a second gradient of the same activation (the U-net skip path), added before the rounding
          float av[8];
          load8(dx_add + base + c, av);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += av[i];
        }
        store8(dx + base + c, o);
        float4* acc = reinterpret_cast<float4*>(dx0_acc + base + c);
        float4 p0 = acc[0], p1 = acc[1];
        p0.x = fmaf(l1, g[0], p0.x); p0.y = fmaf(l1, g[1], p0.y); p0.z = fmaf(l1, g[2], p0.z); p0.w = fmaf(l1, g[3], p0.w);
        p1.x = fmaf(l1, g[4], p1.x); p1.y = fmaf(l1, g[5], p1.y); p1.z = fmaf(l1, g[6], p1.z); p1.w = fmaf(l1, g[7], p1.w);
        acc[0] = p0; acc[1] = p1;
      }
    }
  }
  a0 = warp_sum(a0); a1 = warp_sum(a1); a2 = warp_sum(a2);
  if (lane == 0) { red[0][warp_in_block] = a0; red[1][warp_in_block] = a1; red[2][warp_in_block] = a2; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float t = 0.f;
    for (int i = 0; i < kRowThreads / 32; ++i) t += red[threadIdx.x][i];
    if (threadIdx.x == 0) atomicAdd(&dlam[0], t);
    else if (threadIdx.x == 1) atomicAdd(&dlam[1], t);
    else if (skip && dskip_w) atomicAdd(dskip_w, t);
  }
}

// ---------------------------------------------------------------------------------------------- QK-norm + RoPE + value mix
// A (token, slot) row of D elements (slot in [0, 3H): q heads, k heads, v heads) is owned by D/16 adjacent lanes;
// every lane holds 8 elements of the first half and the 8 partner elements of the second half (16-byte accesses).
// Sum over the LPR adjacent lanes that own one row. Rows of one warp may take different branches (q/k versus v
// slots), so the shuffle names only the lanes of its own row group.
template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
  const unsigned lane = threadIdx.x & 31u;
  const unsigned mask = (LPR == 32 ? 0xffffffffu : ((1u << LPR) - 1u)) << (lane & ~unsigned(LPR - 1));
#pragma unroll
  for (int s = LPR / 2; s > 0; s >>= 1) v += __shfl_xor_sync(mask, v, s);
  return v;
}
__device__ __forceinline__ void load8f(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <int D>
__global__ void __launch_bounds__(256)
qkv_post_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ ve, const float* __restrict__ lam,
                    const float* __restrict__ cs, const float* __restrict__ sn, bf16* __restrict__ out, int T, int H,
                    float eps) {
  constexpr int LPR = D / 16;
  const long long row = ((long long)blockIdx.x * 256 + threadIdx.x) / LPR;
  const int sub = threadIdx.x % LPR;
  const bool active = row < (long long)T * 3 * H;
  const long long rr = active ? row : 0;
  const int t = (int)(rr / (3 * H));
  const int slot = (int)(rr % (3 * H));
  const bf16* src = qkv + rr * D;
  bf16* dst = out + rr * D;
  float a[8], b[8];
  load8(src + sub * 8, a);
  load8(src + D / 2 + sub * 8, b);
  if (slot < 2 * H) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + b[i] * b[i];
    ss = group_sum<LPR>(ss);
    const float r = rsqrtf(ss / D + eps);
    float c[8], s8[8], y1[8], y2[8];
    load8f(cs + (long long)t * (D / 2) + sub * 8, c);
    load8f(sn + (long long)t * (D / 2) + sub * 8, s8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // the reference normalises in bf16, then rotates in fp32
      const float x1 = __bfloat162float(__float2bfloat16_rn(a[i] * r));
      const float x2 = __bfloat162float(__float2bfloat16_rn(b[i] * r));
      y1[i] = x1 * c[i] + x2 * s8[i];
      y2[i] = -x1 * s8[i] + x2 * c[i];
    }
    if (active) { store8(dst + sub * 8, y1); store8(dst + D / 2 + sub * 8, y2); }
  } else {
    const float l0 = lam[0], l1 = lam[1];
    const int hv = slot - 2 * H;
    if (ve) {
      const bf16* vs = ve + ((long long)t * H + hv) * D;
      float e1[8], e2[8];
      load8(vs + sub * 8, e1);
      load8(vs + D / 2 + sub * 8, e2);
#pragma unroll
      for (int i = 0; i < 8; ++i) { a[i] = l0 * a[i] + l1 * e1[i]; b[i] = l0 * b[i] + l1 * e2[i]; }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) { a[i] *= l0; b[i] *= l0; }
    }
    if (active) { store8(dst + sub * 8, a); store8(dst + D / 2 + sub * 8, b); }
  }
}

template <int D>
__global__ void __launch_bounds__(256)
qkv_post_bwd_kernel(const float* __restrict__ dq, const bf16* __restrict__ dk, const bf16* __restrict__ dv,
                    const bf16* __restrict__ qkv, const bf16* __restrict__ ve, const float* __restrict__ lam,
                    const float* __restrict__ cs, const float* __restrict__ sn, bf16* __restrict__ dqkv,
                    bf16* __restrict__ dve, float* __restrict__ dlam, int T, int H, float eps) {
  constexpr int LPR = D / 16;
  __shared__ float red[2][8];
  const int sub = threadIdx.x % LPR;
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const long long total = (long long)T * 3 * H;
  const long long ngroups = (total * LPR + 255) / 256;   // 256-thread groups of rows; a block walks them with a stride
  float s0 = 0.f, s1 = 0.f;                              // so that the two sums cost one atomic per block, not per group
  for (long long grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
    const long long row = (grp * 256 + threadIdx.x) / LPR;
    const bool active = row < total;
    const long long rr = active ? row : 0;
    const int t = (int)(rr / (3 * H));
    const int slot = (int)(rr % (3 * H));
    const bf16* src = qkv + rr * D;
    bf16* dst = dqkv + rr * D;
    float a[8], b[8], ga[8], gb[8];
    load8(src + sub * 8, a);
    load8(src + D / 2 + sub * 8, b);
    if (slot < 2 * H) {
      const int hh = slot < H ? slot : slot - H;
      const long long g0 = ((long long)t * H + hh) * D;
      float y1[8], y2[8], c[8], s8[8];
      if (slot < H) { load8f(dq + g0 + sub * 8, y1); load8f(dq + g0 + D / 2 + sub * 8, y2); }
      else { load8(dk + g0 + sub * 8, y1); load8(dk + g0 + D / 2 + sub * 8, y2); }
      load8f(cs + (long long)t * (D / 2) + sub * 8, c);
      load8f(sn + (long long)t * (D / 2) + sub * 8, s8);
      float ss = 0.f, dot = 0.f;
  #pragma unroll
      for (int i = 0; i < 8; ++i) {
        ga[i] = y1[i] * c[i] - y2[i] * s8[i];  // transpose of the rotation
        gb[i] = y1[i] * s8[i] + y2[i] * c[i];
        ss += a[i] * a[i] + b[i] * b[i];
        dot += a[i] * ga[i] + b[i] * gb[i];
      }
      ss = group_sum<LPR>(ss);
      dot = group_sum<LPR>(dot);
      const float r = rsqrtf(ss / D + eps);
      const float coef = dot * r * r * r / D;
  #pragma unroll
      for (int i = 0; i < 8; ++i) { ga[i] = r * ga[i] - a[i] * coef; gb[i] = r * gb[i] - b[i] * coef; }
      if (active) { store8(dst + sub * 8, ga); store8(dst + D / 2 + sub * 8, gb); }
    } else {
      const int hv = slot - 2 * H;
      const long long g0 = ((long long)t * H + hv) * D;
      const float l0 = lam[0], l1 = lam[1];
      load8(dv + g0 + sub * 8, ga);
      load8(dv + g0 + D / 2 + sub * 8, gb);
      float o1[8], o2[8];
  #pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (active) s0 += ga[i] * a[i] + gb[i] * b[i];
        o1[i] = l0 * ga[i];
        o2[i] = l0 * gb[i];
      }
      if (active) { store8(dst + sub * 8, o1); store8(dst + D / 2 + sub * 8, o2); }
      if (ve) {
        float e1[8], e2[8];
        load8(ve + g0 + sub * 8, e1);
        load8(ve + g0 + D / 2 + sub * 8, e2);
  #pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (active) s1 += ga[i] * e1[i] + gb[i] * e2[i];
          o1[i] = l1 * ga[i];
          o2[i] = l1 * gb[i];
        }
        if (dve && active) { store8(dve + g0 + sub * 8, o1); store8(dve + g0 + D / 2 + sub * 8, o2); }
      }
    }
  }
  s0 = warp_sum(s0);
  s1 = warp_sum(s1);
  if (lane == 0) { red[0][wib] = s0; red[1][wib] = s1; }
  __syncthreads();
  if (threadIdx.x < 2) {
    float tsum = 0.f;
    for (int i = 0; i < 8; ++i) tsum += red[threadIdx.x][i];
    if (tsum != 0.f) atomicAdd(&dlam[threadIdx.x], tsum);
  }
}

// ---------------------------------------------------------------------------------------------- embeddings
template <int NCH>
__global__ void __launch_bounds__(kRowThreads)
embed_gather_kernel(const int* __restrict__ idx, const bf16* __restrict__ table, bf16* __restrict__ out, int T, int C,
                    int normalize, float eps) {
  const int row = (blockIdx.x * kRowThreads + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const bf16* src = table + (long long)idx[row] * C;
  bf16* dst = out + (long long)row * C;
  float v[NCH][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (lane + 32 * k) * 8;
    if (c < C) {
      load8(src + c, v[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[k][i], v[k][i], ss);
    }
  }
  float r = 1.f;
  if (normalize) {
    ss = warp_sum(ss);
    r = rsqrtf(ss / C + eps);
  }
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (lane + 32 * k) * 8;
    if (c < C) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[k][i] *= r;
      store8(dst + c, v[k]);
    }
  }
}

// grad_table[idx[t]] += src[t] (+ src2[t]): one 16-byte vector atomic per four channels.
template <typename TS>
__global__ void embed_scatter_add_kernel(const int* __restrict__ idx, const TS* __restrict__ src,
                                         const TS* __restrict__ src2, float* __restrict__ grad_table, int T, int C) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cq = C / 4;
  if (i >= (long long)T * cq) return;
  const int t = (int)(i / cq), c = (int)(i % cq) * 4;
  float f[4];
  ld4(src + (long long)t * C + c, f);
  if (src2) {
    float h[4];
    ld4(src2 + (long long)t * C + c, h);
#pragma unroll
    for (int k = 0; k < 4; ++k) f[k] += h[k];
  }
  atomicAdd(reinterpret_cast<float4*>(grad_table + (long long)idx[t] * C + c), make_float4(f[0], f[1], f[2], f[3]));
}

// ---------------------------------------------------------------------------------------------- document bounds
// doc_start[i] = last position <= i whose token equals `bos` (position 0 always starts a document);
// doc_end[i] = first such position > i, or T. One block per 1024 tokens: starts inside the tile are located with warp
// ballots; a token whose document begins (ends) outside the tile takes the block's carry, which the block finds by
// scanning backwards (forwards) from the tile edge 1024 tokens at a time until a start turns up.
__global__ void __launch_bounds__(1024)
doc_bounds_kernel(const long long* __restrict__ tokens, long long bos, int* __restrict__ doc_start,
                  int* __restrict__ doc_end, int T) {
  __shared__ int s_last[32], s_first[32], s_carry[2];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int t0 = blockIdx.x * 1024, i = t0 + tid;
  const bool flag = i < T && (i == 0 || tokens[i] == bos);
  const unsigned m = __ballot_sync(0xffffffffu, flag);
  if (lane == 0) {
    s_last[w] = m ? t0 + w * 32 + 31 - __clz(m) : -1;
    s_first[w] = m ? t0 + w * 32 + __ffs(m) - 1 : T;
  }
  if (tid == 0) s_carry[0] = -1, s_carry[1] = T;
  __syncthreads();
  // carries: block-parallel search outside the tile, only as far as the neighbouring start. Every thread reads the
  // carry, then a barrier, then the (uniform) exit test: no warp can publish a hit before all have read.
  for (int base = t0 - 1024;; base -= 1024) {   // backwards
    const int c = s_carry[0];
    __syncthreads();
    if (c >= 0 || base <= -1024) break;
    const int j = base + tid;
    const bool f = j >= 0 && (j == 0 || tokens[j] == bos);
    const unsigned mm = __ballot_sync(0xffffffffu, f);
    if (lane == 0 && mm) atomicMax(&s_carry[0], base + w * 32 + 31 - __clz(mm));
    __syncthreads();
  }
  for (int base = t0 + 1024;; base += 1024) {   // forwards
    const int c = s_carry[1];
    __syncthreads();
    if (c < T || base >= T) break;
    const int j = base + tid;
    const bool f = j < T && tokens[j] == bos;
    const unsigned mm = __ballot_sync(0xffffffffu, f);
    if (lane == 0 && mm) atomicMin(&s_carry[1], base + w * 32 + __ffs(mm) - 1);
    __syncthreads();
  }
  if (i >= T) return;
  // last start <= i: own warp (lanes <= lane), else earlier warps of the tile, else the carry
  const unsigned lo = m & (0xffffffffu >> (31 - lane));
  int st = lo ? t0 + w * 32 + 31 - __clz(lo) : -1;
  for (int q = w - 1; st < 0 && q >= 0; --q) st = s_last[q];
  if (st < 0) st = s_carry[0];
  doc_start[i] = max(st, 0);
  // first start > i
  const unsigned hi = lane == 31 ? 0u : (m & (0xffffffffu << (lane + 1)));
  int en = hi ? t0 + w * 32 + __ffs(hi) - 1 : T;
  for (int q = w + 1; en >= T && q < 32; ++q) en = s_first[q];
  if (en >= T) en = s_carry[1];
  doc_end[i] = min(en, T);
}

// ---------------------------------------------------------------------------------------------- fp8 cast
template <typename TI>
__global__ void cast_fp8_kernel(const TI* __restrict__ x, uint8_t* __restrict__ out, float scale, long long n,
                                int out_kind) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const __nv_fp8_interpretation_t kind = out_kind ? __NV_E5M2 : __NV_E4M3;
  if (i + 8 <= n) {
    float f[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = (float)x[i + k] * scale;
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      w0 |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f[2 * k], f[2 * k + 1]), __NV_SATFINITE, kind) << (16 * k);
      w1 |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f[4 + 2 * k], f[5 + 2 * k]), __NV_SATFINITE, kind) << (16 * k);
    }
    *reinterpret_cast<uint2*>(out + i) = make_uint2(w0, w1);
  } else {
    for (long long k = i; k < n; ++k) out[k] = __nv_cvt_float_to_fp8((float)x[k] * scale, __NV_SATFINITE, kind);
  }
}

// ---------------------------------------------------------------------------------------------- soft-capped CE
// One block per row. z = cap * sigmoid(x / div) is bounded by cap (30), so exp(z) needs no running maximum.
// The kernel is bound by the SFU (tanh + exp per element and pass). With CACHE the first pass keeps exp(z) of the whole
// row in shared memory as bf16 (2 bytes per column; two 1024-thread blocks, i.e. two rows, per SM at a 50k vocabulary); the gradient pass
// then reads neither the logits nor evaluates tanh / exp again: sigmoid = log(e) / cap costs one SFU op instead of two,
// and the 0.4 % rounding of e moves the sigmoid by 1e-4.
bool g_ce_cache = true;   // measured 49152 x 50304: 2.32 ms cached, 2.55 ms recomputed

template <bool CACHE>
__global__ void __launch_bounds__(CACHE ? 1024 : 512)
softcap_ce_kernel(const bf16* __restrict__ logits, const long long* __restrict__ targets,
                  float* __restrict__ loss_rows, uint8_t* __restrict__ grad, int grad_is_bf16, int T, int V, long long ld,
                  float cap, float inv_div, float shift, float loss_scale, float grad_scale,
                  const float* __restrict__ mtp_w, int n_predict) {
  // z = cap * sigmoid((x + shift) / div); loss_row = sum_k w_k (lse - z[target[row + k]]) over the rows that exist
  // (multi-token prediction: row r also predicts the targets of the next n_predict - 1 rows), w = {1} by default.
  constexpr int MAXP = 4;
  extern __shared__ __align__(16) uint8_t s_cache_raw[];
  bf16* s_cache = reinterpret_cast<bf16*>(s_cache_raw);     // [V] exp(z) of this row
  __shared__ float red[32];
  __shared__ float s_total;
  const int row = blockIdx.x;
  const bf16* x = logits + (long long)row * ld;
  int tg[MAXP];
  float wk[MAXP], wsum = 0.f;
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    const bool on = k < n_predict && row + k < T;
    const int t = on ? (int)targets[row + k] : -1;
    const float w = on ? (mtp_w ? mtp_w[k] : 1.f) : 0.f;
    wsum += w;                                    // the probability term counts every existing row's weight
    const bool valid = t >= 0 && t < V && w > 0.f;
    tg[k] = valid ? t : -1;
    wk[k] = valid ? w : 0.f;
  }
  const bool single_ignored = (n_predict == 1 && tg[0] < 0);  // an ignored position contributes nothing at all
  if (single_ignored) wsum = 0.f;
  const int nch = V / 8;
  const float L2E = 1.4426950408889634f;
  const float ta = 0.5f * inv_div, tb = shift * ta, zc = 0.5f * cap * L2E;
  float sum = 0.f;
  for (int ci = threadIdx.x; ci < nch; ci += blockDim.x) {
    float f[8];
    load8(x + ci * 8, f);
    float e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float th = tanhf(fmaf(f[i], ta, tb));   // sigmoid = 0.5 * th + 0.5: one MUFU under fast-math
      e[i] = exp2f(fmaf(th, zc, zc));               // exp(cap * sigmoid)
      sum += e[i];
    }
    if constexpr (CACHE) store8(s_cache + ci * 8, e);   // read back by the same thread: no barrier needed for the cache
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_total = t;
  }
  __syncthreads();
  const float total = s_total;
  const float lse = logf(total);
  if (threadIdx.x == 0) {
    float loss = 0.f;
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      if (tg[k] >= 0) {
        const float sg = 0.5f * tanhf(0.5f * (__bfloat162float(x[tg[k]]) + shift) * inv_div) + 0.5f;
        loss += wk[k] * (lse - cap * sg);
      }
    }
    loss_rows[row] = loss * loss_scale;
  }
  if (!grad) return;
  const float c1 = wsum / total;                       // probability term: wsum * exp(z) / total
  const float gs = grad_scale * cap * inv_div;         // d z / d x = cap / div * sg * (1 - sg)
  const float inv_cap_l2e = 1.f / (cap * L2E);
  for (int ci = threadIdx.x; ci < nch; ci += blockDim.x) {
    float f[8], g[8], dd[8];
    if constexpr (CACHE) load8(s_cache + ci * 8, f);
    else load8(x + ci * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float ev;
      if constexpr (CACHE) {
        ev = f[i];
        const float sg = __log2f(ev) * inv_cap_l2e;
        dd[i] = fmaf(-sg, sg, sg) * gs;
      } else {
        const float th = tanhf(fmaf(f[i], ta, tb));
        ev = exp2f(fmaf(th, zc, zc));
        dd[i] = fmaf(-th, th, 1.f) * (0.25f * gs);     // sg * (1 - sg) = (1 - th^2) / 4
      }
      g[i] = ev * c1 * dd[i];
    }
    // the one-hot terms touch at most MAXP columns of the row: test the chunk, not every element
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      const unsigned rel = (unsigned)(tg[k] - ci * 8);
      if (rel < 8u) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if ((unsigned)i == rel) g[i] -= wk[k] * dd[i];
      }
    }
    if (grad_is_bf16) {
      store8(reinterpret_cast<bf16*>(grad) + (long long)row * ld + ci * 8, g);
    } else {
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        w0 |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(g[2 * k], g[2 * k + 1]), __NV_SATFINITE, __NV_E5M2) << (16 * k);
        w1 |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(g[4 + 2 * k], g[5 + 2 * k]), __NV_SATFINITE, __NV_E5M2) << (16 * k);
      }
      *reinterpret_cast<uint2*>(grad + (long long)row * ld + ci * 8) = make_uint2(w0, w1);
    }
  }
}

// ---------------------------------------------------------------------------------------------- optimizer pieces
__device__ __forceinline__ void adam_one(float& pi, float gi, float& mi, float& vi, float lr, float b1, float b2, float eps,
                                         float wd, float bias1, float inv_sqrt_bias2) {
  mi = b1 * mi + (1.f - b1) * gi;
  vi = b2 * vi + (1.f - b2) * gi * gi;
  pi -= lr * wd * pi;
  const float denom = sqrtf(vi) * inv_sqrt_bias2 + eps;
  pi -= (lr / bias1) * mi / denom;
}

// VEC = 4: four consecutive elements per thread with 8 / 16-byte accesses (all pointers 16-byte aligned); VEC = 1 otherwise.
// shadow_kind: 0 none, 1 bf16 copy of the new parameter, 2 e4m3 copy of (new parameter * shadow_scale): the
// low-precision operand that the next forward GEMM reads is produced in the same pass as the update.
template <typename TP, typename TG, int VEC>
__global__ void adam_kernel(TP* __restrict__ p, const TG* __restrict__ g, float* __restrict__ m,
                            float* __restrict__ v, long long n, float lr, float b1, float b2, float eps, float wd,
                            float bias1, float bias2, float grad_scale, void* __restrict__ shadow, int shadow_kind,
                            float shadow_scale) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= n) return;
  const float isb2 = rsqrtf(bias2);
  if (VEC == 4 && i + 4 <= n) {
    float pf[4], gf[4], mf[4], vf[4];
    ld4(p + i, pf); ld4(g + i, gf); ld4(m + i, mf); ld4(v + i, vf);
#pragma unroll
    for (int k = 0; k < 4; ++k) adam_one(pf[k], gf[k] * grad_scale, mf[k], vf[k], lr, b1, b2, eps, wd, bias1, isb2);
    st4(m + i, mf); st4(v + i, vf); st4(p + i, pf);
    if (shadow_kind == 1) {
      st4(reinterpret_cast<bf16*>(shadow) + i, pf);
    } else if (shadow_kind == 2) {
      const uint32_t w =
          (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(pf[0] * shadow_scale, pf[1] * shadow_scale), __NV_SATFINITE, __NV_E4M3) |
          ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(pf[2] * shadow_scale, pf[3] * shadow_scale), __NV_SATFINITE, __NV_E4M3) << 16);
      *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(shadow) + i) = w;
    }
    return;
  }
  for (long long j = i; j < n && j < i + VEC; ++j) {
    float pi = (float)p[j], mi = m[j], vi = v[j];
    adam_one(pi, (float)g[j] * grad_scale, mi, vi, lr, b1, b2, eps, wd, bias1, isb2);
    m[j] = mi;
    v[j] = vi;
    p[j] = (TP)pi;
    if (shadow_kind == 1) reinterpret_cast<bf16*>(shadow)[j] = __float2bfloat16(pi);
    else if (shadow_kind == 2)
      reinterpret_cast<uint8_t*>(shadow)[j] = __nv_cvt_float_to_fp8(pi * shadow_scale, __NV_SATFINITE, __NV_E4M3);
  }
}

// grid (blocks per matrix, matrices): matrix blockIdx.y of the contiguous stacks g / buf / out [nmat][n], one sum of
// squares per matrix. Four elements per thread (`vec`) when n % 4 == 0 and the stacks are 16-byte aligned.
__global__ void muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ buf, bf16* __restrict__ out,
                                     float* __restrict__ sumsq, long long n, float mu, int nesterov,
                                     float grad_scale, int vec) {
  __shared__ float red[8];
  const long long off = (long long)blockIdx.y * n;
  g += off; buf += off; out += off;
  float acc = 0.f;
  if (vec) {
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
      float gv[4], bv[4], uv[4];
      ld4(g + i, gv);
      ld4(buf + i, bv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gi = gv[k] * grad_scale;
        bv[k] = mu * bv[k] + (1.f - mu) * gi;
        const float u = nesterov ? (1.f - mu) * gi + mu * bv[k] : bv[k];
        uv[k] = __bfloat162float(__float2bfloat16_rn(u));
        acc = fmaf(uv[k], uv[k], acc);
      }
      st4(buf + i, bv);
      st4(out + i, uv);
    }
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
      const float gi = g[i] * grad_scale;
      const float b = mu * buf[i] + (1.f - mu) * gi;
      buf[i] = b;
      const float u = nesterov ? (1.f - mu) * gi + mu * b : b;
      const bf16 ub = __float2bfloat16_rn(u);
      out[i] = ub;
      const float uf = __bfloat162float(ub);
      acc = fmaf(uf, uf, acc);
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    atomicAdd(sumsq + blockIdx.y, t);
  }
}

__global__ void scale_by_inv_norm_kernel(bf16* __restrict__ x, const float* __restrict__ sumsq, long long n,
                                         float eps) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float s = 1.f / (sqrtf(sumsq[0]) + eps);
  x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * s);
}

__global__ void axpy_kernel(float* __restrict__ p, const bf16* __restrict__ u, bf16* __restrict__ p_bf16, long long n,
                            float alpha) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = fmaf(alpha, __bfloat162float(u[i]), p[i]);
  p[i] = v;
  if (p_bf16) p_bf16[i] = __float2bfloat16_rn(v);
}

int pick_nch(int C) {
  if (C % 8 != 0) throw std::runtime_error("row kernels need the row length to be a multiple of 8");
  const int nch = (C + 255) / 256;
  if (nch <= 3) return 3;
  if (nch <= 4) return 4;
  if (nch <= 8) return 8;
  throw std::runtime_error("row kernels support row lengths up to 2048");
}

#define DISPATCH_NCH(C, CALL)            \
  switch (pick_nch(C)) {                 \
    case 3: { constexpr int N_ = 3; CALL; break; } \
    case 4: { constexpr int N_ = 4; CALL; break; } \
    default: { constexpr int N_ = 8; CALL; break; } \
  }

}  // namespace

void rmsnorm_fwd(const void* x, void* y, int R, int C, float eps, cudaStream_t s) {
  mix_norm_fwd(x, nullptr, nullptr, nullptr, nullptr, nullptr, y, R, C, eps, s);
}

void mix_norm_fwd(const void* x, const void* x0, const void* skip, const float* lam, const float* skip_w,
                  void* x_mix, void* xn, int R, int C, float eps, cudaStream_t s) {
  DISPATCH_NCH(C, (mix_norm_fwd_kernel<N_><<<row_blocks(R), kRowThreads, 0, s>>>(
                      (const bf16*)x, (const bf16*)x0, (const bf16*)skip, lam, skip_w, (bf16*)x_mix, (bf16*)xn, R, C, eps)));
  check("mix_norm_fwd");
}

void norm_bwd_add(const void* dy, const void* x, const void* dres, void* out, int R, int C, float eps,
                  cudaStream_t s) {
  DISPATCH_NCH(C, (norm_bwd_add_kernel<N_><<<row_blocks(R), kRowThreads, 0, s>>>((const bf16*)dy, (const bf16*)x,
                                                                                 (const bf16*)dres, (bf16*)out, R, C, eps)));
  check("norm_bwd_add");
}

void mix_bwd(const void* dmix, const void* x, const void* x0, const void* skip, const float* lam,
             const float* skip_w, void* dx, void* dskip, float* dx0_acc, float* dlam, float* dskip_w, const void* dx_add,
             int R, int C, cudaStream_t s) {
  const int blocks = 148 * 4;
  DISPATCH_NCH(C, (mix_bwd_kernel<N_><<<blocks, kRowThreads, 0, s>>>((const bf16*)dmix, (const bf16*)x, (const bf16*)x0,
                                                                    (const bf16*)skip, lam, skip_w, (bf16*)dx,
                                                                    (bf16*)dskip, dx0_acc, dlam, dskip_w, (const bf16*)dx_add, R, C)));
  check("mix_bwd");
}

void qkv_post_fwd(const void* qkv, const void* ve, const float* lam, const float* cos, const float* sin, void* out,
                  int T, int H, int D, float eps, cudaStream_t s) {
  const long long rows = (long long)T * 3 * H;
  const int rpb = 256 / (D / 16);
  const int blocks = (int)((rows + rpb - 1) / rpb);
  if (D == 128) qkv_post_fwd_kernel<128><<<blocks, 256, 0, s>>>((const bf16*)qkv, (const bf16*)ve, lam, cos, sin, (bf16*)out, T, H, eps);
  else if (D == 64) qkv_post_fwd_kernel<64><<<blocks, 256, 0, s>>>((const bf16*)qkv, (const bf16*)ve, lam, cos, sin, (bf16*)out, T, H, eps);
  else throw std::runtime_error("qkv_post: head_dim must be 64 or 128");
  check("qkv_post_fwd");
}

void qkv_post_bwd(const float* dq, const void* dk, const void* dv, const void* qkv, const void* ve,
                  const float* lam, const float* cos, const float* sin, void* dqkv, void* dve, float* dlam, int T,
                  int H, int D, float eps, cudaStream_t s) {
  const long long rows = (long long)T * 3 * H;
  const int rpb = 256 / (D / 16);
  int blocks = (int)((rows + rpb - 1) / rpb);
  if (blocks > 148 * 4) blocks = 148 * 4;     // 64 registers: four resident blocks of 256 threads per SM
  if (D == 128) qkv_post_bwd_kernel<128><<<blocks, 256, 0, s>>>(dq, (const bf16*)dk, (const bf16*)dv, (const bf16*)qkv, (const bf16*)ve, lam, cos, sin, (bf16*)dqkv, (bf16*)dve, dlam, T, H, eps);
  else if (D == 64) qkv_post_bwd_kernel<64><<<blocks, 256, 0, s>>>(dq, (const bf16*)dk, (const bf16*)dv, (const bf16*)qkv, (const bf16*)ve, lam, cos, sin, (bf16*)dqkv, (bf16*)dve, dlam, T, H, eps);
  else throw std::runtime_error("qkv_post: head_dim must be 64 or 128");
  check("qkv_post_bwd");
}

void embed_gather(const int* idx, const void* table, void* out, int T, int C, int normalize, float eps,
                  cudaStream_t s) {
  DISPATCH_NCH(C, (embed_gather_kernel<N_><<<row_blocks(T), kRowThreads, 0, s>>>(idx, (const bf16*)table, (bf16*)out, T, C, normalize, eps)));
  check("embed_gather");
}

void embed_scatter_add(const int* idx, const void* src, const void* src2, int src_is_f32, float* grad_table, int T, int C,
                       cudaStream_t s) {
  if (C % 4 != 0) throw std::runtime_error("embed_scatter_add: C must be a multiple of 4");
  const long long n = (long long)T * (C / 4);
  const int blocks = (int)((n + 255) / 256);
  if (src_is_f32) embed_scatter_add_kernel<float><<<blocks, 256, 0, s>>>(idx, (const float*)src, (const float*)src2, grad_table, T, C);
  else embed_scatter_add_kernel<bf16><<<blocks, 256, 0, s>>>(idx, (const bf16*)src, (const bf16*)src2, grad_table, T, C);
  check("embed_scatter_add");
}

void doc_bounds(const long long* tokens, long long bos, int* doc_start, int* doc_end, int T, cudaStream_t s) {
  if (T <= 0) return;
  doc_bounds_kernel<<<(T + 1023) / 1024, 1024, 0, s>>>(tokens, bos, doc_start, doc_end, T);
  check("doc_bounds");
}

void cast_fp8(const void* x, void* out, float scale, long long n, int in_kind, int out_kind, cudaStream_t s) {
  const long long thr = (n + 7) / 8;
  const int blocks = (int)((thr + 255) / 256);
  if (in_kind == 0) cast_fp8_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)x, (uint8_t*)out, scale, n, out_kind);
  else cast_fp8_kernel<float><<<blocks, 256, 0, s>>>((const float*)x, (uint8_t*)out, scale, n, out_kind);
  check("cast_fp8");
}

void softcap_ce_set_cache(bool on) { g_ce_cache = on; }

void softcap_ce(const void* logits, const long long* targets, float* loss_rows, void* grad, int grad_is_bf16, int T,
                int V, long long ld, float cap, float div, float shift, float loss_scale, float grad_scale,
                const float* mtp_w, int n_predict, cudaStream_t s) {
  if (V % 8 != 0 || ld % 8 != 0) throw std::runtime_error("softcap_ce: vocabulary and row pitch must be multiples of 8");
  if (n_predict < 1 || n_predict > 4) throw std::runtime_error("softcap_ce: 1 to 4 prediction offsets");
  const size_t cache_bytes = (size_t)V * 2;
  if (grad && g_ce_cache && cache_bytes <= 110 * 1024) {   // two rows per SM
    static PerDeviceOnce attr;   // the shared-memory opt-in is a per-device attribute
    int dev = 0;
    if (attr.pending(&dev)) {
      cudaFuncSetAttribute(softcap_ce_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
      attr.done(dev);
    }
    softcap_ce_kernel<true><<<T, 1024, cache_bytes, s>>>((const bf16*)logits, targets, loss_rows, (uint8_t*)grad, grad_is_bf16,
                                                        T, V, ld, cap, 1.f / div, shift, loss_scale, grad_scale, mtp_w,
                                                        n_predict);
  } else {
    softcap_ce_kernel<false><<<T, 512, 0, s>>>((const bf16*)logits, targets, loss_rows, (uint8_t*)grad, grad_is_bf16, T, V,
                                               ld, cap, 1.f / div, shift, loss_scale, grad_scale, mtp_w, n_predict);
  }
  check("softcap_ce");
}

void adam_step(void* p, int p_is_bf16, const void* g, int g_is_bf16, float* m, float* v, long long n, float lr,
               float beta1, float beta2, float eps, float wd, float bias1, float bias2, float grad_scale,
               void* shadow, int shadow_kind, float shadow_scale, cudaStream_t s) {
  bool vec = (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0 && n >= 4;
  if (shadow_kind && ((uintptr_t)shadow & 7)) vec = false;
#define ADAM_LAUNCH(TP, TG)                                                                                          \
  do {                                                                                                               \
    if (vec)                                                                                                         \
      adam_kernel<TP, TG, 4><<<(int)((n + 1023) / 1024), 256, 0, s>>>((TP*)p, (const TG*)g, m, v, n, lr, beta1, beta2, \
                                                                      eps, wd, bias1, bias2, grad_scale, shadow,     \
                                                                      shadow_kind, shadow_scale);                    \
    else                                                                                                             \
      adam_kernel<TP, TG, 1><<<(int)((n + 255) / 256), 256, 0, s>>>((TP*)p, (const TG*)g, m, v, n, lr, beta1, beta2, \
                                                                    eps, wd, bias1, bias2, grad_scale, shadow,       \
                                                                    shadow_kind, shadow_scale);                      \
  } while (0)
  if (p_is_bf16 && g_is_bf16) ADAM_LAUNCH(bf16, bf16);
  else if (p_is_bf16) ADAM_LAUNCH(bf16, float);
  else if (g_is_bf16) ADAM_LAUNCH(float, bf16);
  else ADAM_LAUNCH(float, float);
#undef ADAM_LAUNCH
  check("adam_step");
}

void muon_momentum(const float* g, float* buf, void* out_bf16, float* sumsq, long long n, int nmat, float mu,
                   int nesterov, float grad_scale, cudaStream_t s) {
  if (nmat <= 0 || n <= 0) return;
  int blocks = (int)((n / 4 + 255) / 256) + 1;
  const int cap = (148 * 8 + nmat - 1) / nmat;
  if (blocks > cap) blocks = cap;
  const int vec = (n & 3) == 0 && ((((uintptr_t)g | (uintptr_t)buf) & 15) == 0) && (((uintptr_t)out_bf16 & 7) == 0);
  muon_momentum_kernel<<<dim3(blocks, nmat), 256, 0, s>>>(g, buf, (bf16*)out_bf16, sumsq, n, mu, nesterov, grad_scale, vec);
  check("muon_momentum");
}

void scale_by_inv_norm(void* x_bf16, const float* sumsq, long long n, float eps, cudaStream_t s) {
  const int blocks = (int)((n + 255) / 256);
  scale_by_inv_norm_kernel<<<blocks, 256, 0, s>>>((bf16*)x_bf16, sumsq, n, eps);
  check("scale_by_inv_norm");
}

void axpy_bf16_to_f32(float* p, const void* u_bf16, void* p_bf16, long long n, float alpha, cudaStream_t s) {
  const int blocks = (int)((n + 255) / 256);
  axpy_kernel<<<blocks, 256, 0, s>>>(p, (const bf16*)u_bf16, (bf16*)p_bf16, n, alpha);
  check("axpy_bf16_to_f32");
}

}  // namespace b200
