// See fused_taps.h. A group of LPR adjacent lanes owns one (b, l, h) row and each lane keeps CPL = D / LPR channels
// (8 where the head dimension allows: 16-byte row loads, and the per-tap index arithmetic is shared by more channels). Taps are processed LPR at a time: lane j of the group evaluates the tap formula of tap
// s0 + j (so the transcendental work is done once per tap, not once per lane), then the group walks the LPR taps,
// broadcasting (weight, position) by shuffle and gathering the two value rows. In the backward the owner lane of a tap
// turns the two reduced dot products into the gradients of the row's scalars; kernel-table gradients accumulate in
// shared memory and leave the block coalesced.
#include "fused_taps.h"

#include <cuda_bf16.h>

#include <cstdint>
#include <stdexcept>
#include <string>

namespace b200 {
namespace {
using bf16 = __nv_bfloat16;
constexpr int KMAX = 64;

template <int CPL>
struct Vec {
  float v[CPL];
};
template <int CPL>
__device__ __forceinline__ Vec<CPL> vzero() {
  Vec<CPL> r;
#pragma unroll
  for (int i = 0; i < CPL; ++i) r.v[i] = 0.f;
  return r;
}
template <int CPL>
__device__ __forceinline__ Vec<CPL> vload(const bf16* p) {
  Vec<CPL> r;
  if (CPL == 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      r.v[2 * i] = f.x;
      r.v[2 * i + 1] = f.y;
    }
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      r.v[2 * i] = f.x;
      r.v[2 * i + 1] = f.y;
    }
  }
  return r;
}
template <int CPL>
__device__ __forceinline__ void vstore(bf16* p, const Vec<CPL>& a) {
  uint32_t w[CPL / 2];
#pragma unroll
  for (int i = 0; i < CPL / 2; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a.v[2 * i], a.v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  if (CPL == 8) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  else *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
}
template <int CPL>
__device__ __forceinline__ float vdot(const Vec<CPL>& a, const Vec<CPL>& b) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < CPL; ++i) s += a.v[i] * b.v[i];
  return s;
}
template <int CPL>
__device__ __forceinline__ void vaxpy2(Vec<CPL>& acc, float wa, const Vec<CPL>& a, float wc, const Vec<CPL>& c) {
#pragma unroll
  for (int i = 0; i < CPL; ++i) acc.v[i] += wa * a.v[i] + wc * c.v[i];
}
template <int CPL>
__device__ __forceinline__ void scatter_row(float* dst, float wgt, const Vec<CPL>& g) {
#pragma unroll
  for (int i = 0; i < CPL; i += 4)
    atomicAdd(reinterpret_cast<float4*>(dst + i), make_float4(wgt * g.v[i], wgt * g.v[i + 1], wgt * g.v[i + 2], wgt * g.v[i + 3]));
}
template <int LPR>
__device__ __forceinline__ unsigned group_mask() {
  const unsigned lane = threadIdx.x & 31u;
  return (LPR == 32 ? 0xffffffffu : ((1u << LPR) - 1u)) << (lane & ~unsigned(LPR - 1));
}
template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
  const unsigned mask = group_mask<LPR>();
#pragma unroll
  for (int s = LPR / 2; s > 0; s >>= 1) v += __shfl_xor_sync(mask, v, s);
  return v;
}
template <int LPR>
__device__ __forceinline__ float group_bcast(float v, int j) {
  return __shfl_sync(group_mask<LPR>(), v, j, LPR);
}

struct Lerp {
  int lo;
  float wh, v, slope;
};
// table value at t in [0, 1] (K entries), with the slope d v / d t
__device__ __forceinline__ Lerp lerp_table(const float* kr, int K, float t) {
  Lerp r;
  const float idx = fminf(fmaxf(t, 0.f), 1.f) * (float)(K - 1);
  r.lo = min((int)idx, K - 2);
  r.wh = idx - (float)r.lo;
  const float a = kr[r.lo], b = kr[r.lo + 1];
  r.v = a * (1.f - r.wh) + b * r.wh;
  r.slope = (t >= 0.f && t <= 1.f) ? (b - a) * (float)(K - 1) : 0.f;
  return r;
}

struct Row {
  long long row, bl;
  int b, l, h, sub;
  bool active;
};
// A block owns 256 / LPR consecutive positions of ONE (batch, head): neighbouring positions sample neighbouring rows, so
// the floor row of one is the ceil row of the next and the pair of loads hits L1 instead of L2.
template <int LPR>
__device__ __forceinline__ Row locate(int B, int L, int H) {
  constexpr int RPB = 256 / LPR;
  const int nt = (L + RPB - 1) / RPB;
  Row r;
  const int tile = blockIdx.x % nt;
  r.h = (blockIdx.x / nt) % H;
  r.b = blockIdx.x / (nt * H);
  r.sub = threadIdx.x % LPR;
  const int l = tile * RPB + threadIdx.x / LPR;
  r.active = l < L;
  r.l = r.active ? l : L - 1;
  r.bl = (long long)r.b * L + r.l;
  r.row = r.bl * H + r.h;
  return r;
}
template <int LPR>
__device__ __forceinline__ void store_dkern(float* __restrict__ dkern, const float* s_dk, int L, int H, int K) {
  constexpr int RPB = 256 / LPR;
  const int nt = (L + RPB - 1) / RPB;
  const int tile = blockIdx.x % nt, h = (blockIdx.x / nt) % H, b = blockIdx.x / (nt * H);
  for (int i = threadIdx.x; i < RPB * K; i += 256) {
    const int l = tile * RPB + i / K;
    if (l < L) dkern[(((long long)b * L + l) * H + h) * K + i % K] = s_dk[i];
  }
}

struct Bil {
  int fl, ce;
  float fr;
};
__device__ __forceinline__ Bil bilinear(float p, int L) {
  Bil r;
  const float pc = fminf(fmaxf(p, 0.f), (float)L - 1.001f);
  r.fl = min((int)pc, max(L - 2, 0));
  r.ce = min(r.fl + 1, L - 1);
  r.fr = pc - (float)r.fl;
  return r;
}

// Walks the n <= LPR taps held one per lane (weight w, position p), UNR at a time (the row loads of UNR taps are issued
// together); taps of weight zero are not loaded.
constexpr int UNR = 1;  // measured: 2 and 4 lose more to the lower occupancy (64 / 99 registers) than the batched loads win
template <int LPR, int CPL>
__device__ __forceinline__ void gather_taps(Vec<CPL>& acc, float w, float p, int n, const bf16* xb, int L, long long rs) {
  for (int j0 = 0; j0 < n; j0 += UNR) {
    float wj[UNR];
    Bil bi[UNR];
    Vec<CPL> a[UNR], c[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const int j = j0 + u;
      const float wb = group_bcast<LPR>(w, j & (LPR - 1)), pb = group_bcast<LPR>(p, j & (LPR - 1));
      wj[u] = j < n ? wb : 0.f;
      bi[u] = bilinear(pb, L);
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      a[u] = c[u] = vzero<CPL>();
      if (wj[u] != 0.f) {
        a[u] = vload<CPL>(xb + bi[u].fl * rs);
        c[u] = vload<CPL>(xb + bi[u].ce * rs);
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) vaxpy2<CPL>(acc, wj[u] * (1.f - bi[u].fr), a[u], wj[u] * bi[u].fr, c[u]);
  }
}


// ------------------------------------------------------------------------------------------------ telephone
template <int LPR, int CPL>
__global__ void __launch_bounds__(256)
tele_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ freq, const float* __restrict__ phase,
                const float* __restrict__ kern, const float* __restrict__ expo, bf16* __restrict__ out, int B, int L, int H,
                int K, int half, float max_rec) {
  constexpr int D = LPR * CPL;
  const Row r = locate<LPR>(B, L, H);
  const float f = freq[r.row], ph = phase[r.row], e = expo[r.bl];
  const float* kr = kern + r.row * K;
  const bf16* xb = x + (long long)r.b * L * H * D + r.h * D + r.sub * CPL;
  const float invL = 1.f / (float)L, inv_rec = 1.f / max_rec;
  Vec<CPL> acc = vzero<CPL>();
  for (int s0 = -half; s0 <= half; s0 += LPR) {
    const int s = s0 + r.sub;
    float w = 0.f, p = 0.f;
    if (s <= half) {
      const float rel = (float)s * f, ar = fabsf(rel);
      p = (float)r.l + rel + ph;
      if (p >= 0.f && p < (float)L) w = lerp_table(kr, K, ar * inv_rec).v * exp2f(-e * log2f(1.f + ar * invL));
    }
    const int n = min(LPR, half - s0 + 1);
    gather_taps<LPR, CPL>(acc, w, p, n, xb, L, (long long)H * D);
  }
  if (r.active) vstore<CPL>(out + r.row * D + r.sub * CPL, acc);
}

template <int LPR, int CPL>
__global__ void __launch_bounds__(256)
tele_bwd_kernel(const bf16* __restrict__ x, const float* __restrict__ freq, const float* __restrict__ phase,
                const float* __restrict__ kern, const float* __restrict__ expo, const bf16* __restrict__ dout,
                float* __restrict__ dx, float* __restrict__ dfreq, float* __restrict__ dphase, float* __restrict__ dkern,
                float* __restrict__ dexpo_h, int B, int L, int H, int K, int half, float max_rec) {
  constexpr int D = LPR * CPL;
  constexpr int RPB = 256 / LPR;
  extern __shared__ float s_dk[];  // [RPB][K]
  for (int i = threadIdx.x; i < RPB * K; i += 256) s_dk[i] = 0.f;
  __syncthreads();
  const Row r = locate<LPR>(B, L, H);
  const float f = freq[r.row], ph = phase[r.row], e = expo[r.bl];
  const float* kr = kern + r.row * K;
  float* dk = s_dk + (threadIdx.x / LPR) * K;
  const bf16* xb = x + (long long)r.b * L * H * D + r.h * D + r.sub * CPL;
  float* dxb = dx + (long long)r.b * L * H * D + r.h * D + r.sub * CPL;
  const float invL = 1.f / (float)L, inv_rec = 1.f / max_rec, hi = (float)L - 1.001f;
  const Vec<CPL> g = vload<CPL>(dout + r.row * D + r.sub * CPL);
  float df = 0.f, dph = 0.f, de = 0.f;
  for (int s0 = -half; s0 <= half; s0 += LPR) {
    const int s = s0 + r.sub;
    float w = 0.f, p = 0.f, kv = 0.f, pw = 0.f, rel = 0.f, base = 1.f;
    Lerp lt;
    lt.lo = 0; lt.wh = 0.f; lt.v = 0.f; lt.slope = 0.f;
    bool valid = false;
    if (s <= half) {
      rel = (float)s * f;
      const float ar = fabsf(rel);
      p = (float)r.l + rel + ph;
      valid = p >= 0.f && p < (float)L;
      if (valid) {
        lt = lerp_table(kr, K, ar * inv_rec);
        kv = lt.v;
        base = 1.f + ar * invL;
        pw = exp2f(-e * log2f(base));
        w = kv * pw;
      }
    }
    const int n = min(LPR, half - s0 + 1);
    float my_sa = 0.f, my_sc = 0.f, my_fr = 0.f;
    const long long rs = (long long)H * D;
    for (int j0 = 0; j0 < n; j0 += UNR) {
      float wj[UNR];
      bool vj[UNR];
      Bil bi[UNR];
      Vec<CPL> a[UNR], c[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int j = j0 + u, src = j & (LPR - 1);
        const float vb = group_bcast<LPR>(valid ? 1.f : 0.f, src), wb = group_bcast<LPR>(w, src), pb = group_bcast<LPR>(p, src);
        vj[u] = j < n && vb != 0.f;
        wj[u] = wb;
        bi[u] = bilinear(pb, L);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        a[u] = c[u] = vzero<CPL>();
        if (vj[u]) {
          a[u] = vload<CPL>(xb + bi[u].fl * rs);
          c[u] = vload<CPL>(xb + bi[u].ce * rs);
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const float sa = group_sum<LPR>(vdot<CPL>(g, a[u])), sc = group_sum<LPR>(vdot<CPL>(g, c[u]));
        if (r.sub == j0 + u) { my_sa = sa; my_sc = sc; my_fr = bi[u].fr; }
        if (r.active && vj[u] && wj[u] != 0.f) {
          scatter_row<CPL>(dxb + bi[u].fl * rs, wj[u] * (1.f - bi[u].fr), g);
          if (bi[u].fr != 0.f) scatter_row<CPL>(dxb + bi[u].ce * rs, wj[u] * bi[u].fr, g);
        }
      }
    }
    if (valid && r.active) {  // scalar gradients of this lane's own tap
      const float dW = my_sa * (1.f - my_fr) + my_sc * my_fr;
      const float dP = (p >= 0.f && p <= hi) ? w * (my_sc - my_sa) : 0.f;
      const float dkv = dW * pw;
      atomicAdd(&dk[lt.lo], dkv * (1.f - lt.wh));
      atomicAdd(&dk[lt.lo + 1], dkv * lt.wh);
      const float dpw = dW * kv;
      de += dpw * pw * (-logf(base));
      float dar = dkv * lt.slope * inv_rec + dpw * pw * (-e) * invL / base;
      const float sgn = rel > 0.f ? 1.f : (rel < 0.f ? -1.f : 0.f);
      const float drel = dar * sgn + dP;
      df += drel * (float)s;
      dph += dP;
    }
  }
  df = group_sum<LPR>(df);
  dph = group_sum<LPR>(dph);
  de = group_sum<LPR>(de);
  if (r.active && r.sub == 0) {
    dfreq[r.row] = df;
    dphase[r.row] = dph;
    dexpo_h[r.row] = de;
  }
  __syncthreads();
  store_dkern<LPR>(dkern, s_dk, L, H, K);
}

// ------------------------------------------------------------------------------------------------ adaptive local conv
struct AlcTap {
  float base, rk, ex, r, p;
  Lerp lt;
  bool valid;
};
__device__ __forceinline__ AlcTap alc_tap(const float* kr, int K, int s, float inv_hw, float pc0, int L) {
  AlcTap t;
  t.r = fabsf((float)s) * inv_hw;
  t.p = pc0 + (float)s;
  t.valid = t.p >= 0.f && t.p < (float)L;
  t.lt = lerp_table(kr, K, t.r);
  t.rk = fmaxf(t.lt.v, 0.f) + 1.f;
  t.ex = __expf(-t.r * t.r);
  t.base = t.valid ? t.rk * t.ex : 0.f;
  return t;
}

template <int LPR, int CPL>
__global__ void __launch_bounds__(256)
alc_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ half_w, const float* __restrict__ center,
               const float* __restrict__ kern, bf16* __restrict__ out, int B, int L, int H, int K, int half) {
  constexpr int D = LPR * CPL;
  const Row r = locate<LPR>(B, L, H);
  const float inv_hw = 1.f / half_w[r.row], pc0 = (float)r.l + center[r.row];
  const float* kr = kern + r.row * K;
  const bf16* xb = x + (long long)r.b * L * H * D + r.h * D + r.sub * CPL;
  float sum = 0.f;
  for (int s = -half + r.sub; s <= half; s += LPR) sum += alc_tap(kr, K, s, inv_hw, pc0, L).base;
  const float inv_norm = 1.f / fmaxf(group_sum<LPR>(sum), 1.f);
  Vec<CPL> acc = vzero<CPL>();
  for (int s0 = -half; s0 <= half; s0 += LPR) {
    const int s = s0 + r.sub;
    float w = 0.f, p = 0.f;
    if (s <= half) {
      const AlcTap t = alc_tap(kr, K, s, inv_hw, pc0, L);
      w = t.base * inv_norm;
      p = t.p;
    }
    const int n = min(LPR, half - s0 + 1);
    gather_taps<LPR, CPL>(acc, w, p, n, xb, L, (long long)H * D);
  }
  if (r.active) vstore<CPL>(out + r.row * D + r.sub * CPL, acc);
}

// shared memory: [RPB][K] kernel gradients, then [RPB][SP] per-tap dW (SP = 2*half+1)
template <int LPR, int CPL>
__global__ void __launch_bounds__(256)
alc_bwd_kernel(const bf16* __restrict__ x, const float* __restrict__ half_w, const float* __restrict__ center,
               const float* __restrict__ kern, const bf16* __restrict__ dout, float* __restrict__ dx,
               float* __restrict__ dhalf_w, float* __restrict__ dcenter, float* __restrict__ dkern, int B, int L, int H,
               int K, int half) {
  constexpr int D = LPR * CPL;
  constexpr int RPB = 256 / LPR;
  extern __shared__ float s_mem[];
  const int SP = 2 * half + 1;
  float* s_dk = s_mem;
  float* s_dw = s_mem + RPB * K;
  for (int i = threadIdx.x; i < RPB * K; i += 256) s_dk[i] = 0.f;
  __syncthreads();
  const Row r = locate<LPR>(B, L, H);
  const float hw = half_w[r.row], inv_hw = 1.f / hw, pc0 = (float)r.l + center[r.row];
  const float* kr = kern + r.row * K;
  float* dk = s_dk + (threadIdx.x / LPR) * K;
  float* dw = s_dw + (threadIdx.x / LPR) * SP;
  const bf16* xb = x + (long long)r.b * L * H * D + r.h * D + r.sub * CPL;
  float* dxb = dx + (long long)r.b * L * H * D + r.h * D + r.sub * CPL;
  const float hi = (float)L - 1.001f;
  const Vec<CPL> g = vload<CPL>(dout + r.row * D + r.sub * CPL);
  float sum = 0.f;
  for (int s = -half + r.sub; s <= half; s += LPR) sum += alc_tap(kr, K, s, inv_hw, pc0, L).base;
  sum = group_sum<LPR>(sum);
  const float inv_norm = 1.f / fmaxf(sum, 1.f);
  float dc = 0.f, G = 0.f;
  // pass 1: gathers -> per-tap dW (shared), dx atomics, centre gradient, G = sum_j dW_j w_j
  for (int s0 = -half; s0 <= half; s0 += LPR) {
    const int s = s0 + r.sub;
    float w = 0.f, p = 0.f;
    if (s <= half) {
      const AlcTap t = alc_tap(kr, K, s, inv_hw, pc0, L);
      w = t.base * inv_norm;
      p = t.p;
    }
    const int n = min(LPR, half - s0 + 1);
    const long long rs = (long long)H * D;
    for (int j0 = 0; j0 < n; j0 += UNR) {
      float wj[UNR], pj[UNR];
      bool vj[UNR];
      Bil bi[UNR];
      Vec<CPL> a[UNR], c[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int j = j0 + u, src = j & (LPR - 1);
        wj[u] = group_bcast<LPR>(w, src);
        pj[u] = group_bcast<LPR>(p, src);
        vj[u] = j < n && pj[u] >= 0.f && pj[u] < (float)L;
        bi[u] = bilinear(pj[u], L);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        a[u] = c[u] = vzero<CPL>();
        if (vj[u]) {
          a[u] = vload<CPL>(xb + bi[u].fl * rs);
          c[u] = vload<CPL>(xb + bi[u].ce * rs);
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const float sa = group_sum<LPR>(vdot<CPL>(g, a[u])), sc = group_sum<LPR>(vdot<CPL>(g, c[u]));
        const float dWj = sa * (1.f - bi[u].fr) + sc * bi[u].fr;  // zero for a tap outside the sequence
        if (r.sub == j0 + u && j0 + u < n) {
          G += dWj * wj[u];
          if (vj[u] && pj[u] <= hi) dc += wj[u] * (sc - sa);
          dw[s0 + j0 + u + half] = dWj;
        }
        if (r.active && vj[u] && wj[u] != 0.f) {
          scatter_row<CPL>(dxb + bi[u].fl * rs, wj[u] * (1.f - bi[u].fr), g);
          if (bi[u].fr != 0.f) scatter_row<CPL>(dxb + bi[u].ce * rs, wj[u] * bi[u].fr, g);
        }
      }
    }
  }
  G = group_sum<LPR>(G);
  dc = group_sum<LPR>(dc);
  __syncwarp(group_mask<LPR>());
  // pass 2: per-tap gradients of the kernel table and of the half window
  const float corr = sum > 1.f ? G : 0.f;
  float dhw = 0.f;
  for (int s = -half + r.sub; s <= half; s += LPR) {
    const AlcTap t = alc_tap(kr, K, s, inv_hw, pc0, L);
    if (!t.valid) continue;
    const float dbase = (dw[s + half] - corr) * inv_norm;
    const float dkv = t.lt.v > 0.f ? dbase * t.ex : 0.f;
    atomicAdd(&dk[t.lt.lo], dkv * (1.f - t.lt.wh));
    atomicAdd(&dk[t.lt.lo + 1], dkv * t.lt.wh);
    const float dr = dbase * t.rk * t.ex * (-2.f * t.r) + dkv * t.lt.slope;
    dhw += dr * (-t.r * inv_hw);
  }
  dhw = group_sum<LPR>(dhw);
  if (r.active && r.sub == 0) {
    dhalf_w[r.row] = dhw;
    dcenter[r.row] = dc;
  }
  __syncthreads();
  store_dkern<LPR>(dkern, s_dk, L, H, K);
}

void chk(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void check_dims(int D, int K, int half) {
  if (K < 2 || K > KMAX) throw std::runtime_error("fused taps: kernel table size must be in [2, 64]");
  if (half < 0 || half > 4096) throw std::runtime_error("fused taps: half tap count out of range");
  (void)D;
}

#define DISPATCH_LPR(D, ...)                                                              \
  switch (D) {                                                                            \
    case 8: { constexpr int LPR_ = 2, CPL_ = 4; __VA_ARGS__; break; }                          \
    case 16: { constexpr int LPR_ = 2, CPL_ = 8; __VA_ARGS__; break; }                         \
    case 32: { constexpr int LPR_ = 4, CPL_ = 8; __VA_ARGS__; break; }                         \
    case 64: { constexpr int LPR_ = 8, CPL_ = 8; __VA_ARGS__; break; }                         \
    case 128: { constexpr int LPR_ = 16, CPL_ = 8; __VA_ARGS__; break; }                       \
    default: throw std::runtime_error("fused taps: head_dim must be 8, 16, 32, 64 or 128"); \
  }
// The backward kernels keep 4 channels per lane: with 8, each 16-byte vector reduction of a lane group covers only
// every other 16 bytes of the row (two instructions per row), and the atomic path, the bottleneck of the backward,
// measured 1.4-1.6x slower (telephone 16.1 vs 10.4 ms, adaptive conv 4.1 vs 3.0 ms on the classifier layer).
#define DISPATCH_LPR_BWD(D, ...)                                                          \
  switch (D) {                                                                            \
    case 8: { constexpr int LPR_ = 2, CPL_ = 4; __VA_ARGS__; break; }                          \
    case 16: { constexpr int LPR_ = 4, CPL_ = 4; __VA_ARGS__; break; }                         \
    case 32: { constexpr int LPR_ = 8, CPL_ = 4; __VA_ARGS__; break; }                         \
    case 64: { constexpr int LPR_ = 16, CPL_ = 4; __VA_ARGS__; break; }                        \
    case 128: { constexpr int LPR_ = 32, CPL_ = 4; __VA_ARGS__; break; }                       \
    default: throw std::runtime_error("fused taps: head_dim must be 8, 16, 32, 64 or 128"); \
  }
template <typename Kern>
void opt_in_smem(Kern k, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) throw std::runtime_error(std::string("fused taps: shared memory opt-in: ") + cudaGetErrorString(e));
  }
}
}  // namespace

void tele_fused_fwd(const void* x, const float* freq, const float* phase, const float* kern, const float* expo, void* out,
                    int B, int L, int H, int D, int K, int half, float max_rec, cudaStream_t s) {
  check_dims(D, K, half);
  DISPATCH_LPR(D, {
    const int rpb = 256 / LPR_;
    const long long nblk = (long long)B * H * ((L + rpb - 1) / rpb);
    tele_fwd_kernel<LPR_, CPL_><<<(unsigned)nblk, 256, 0, s>>>((const bf16*)x, freq, phase, kern, expo, (bf16*)out, B, L, H, K, half, max_rec);
  });
  chk("tele_fused_fwd");
}

void tele_fused_bwd(const void* x, const float* freq, const float* phase, const float* kern, const float* expo,
                    const void* dout, float* dx, float* dfreq, float* dphase, float* dkern, float* dexpo_h, int B, int L,
                    int H, int D, int K, int half, float max_rec, cudaStream_t s) {
  check_dims(D, K, half);
  DISPATCH_LPR_BWD(D, {
    const int rpb = 256 / LPR_;
    const long long nblk = (long long)B * H * ((L + rpb - 1) / rpb);
    const size_t smem = (size_t)rpb * K * sizeof(float);
    tele_bwd_kernel<LPR_, CPL_><<<(unsigned)nblk, 256, smem, s>>>((const bf16*)x, freq, phase, kern, expo, (const bf16*)dout, dx,
                                                                               dfreq, dphase, dkern, dexpo_h, B, L, H, K, half, max_rec);
  });
  chk("tele_fused_bwd");
}

void alc_fused_fwd(const void* x, const float* half_w, const float* center, const float* kern, void* out, int B, int L,
                   int H, int D, int K, int half, cudaStream_t s) {
  check_dims(D, K, half);
  DISPATCH_LPR(D, {
    const int rpb = 256 / LPR_;
    const long long nblk = (long long)B * H * ((L + rpb - 1) / rpb);
    alc_fwd_kernel<LPR_, CPL_><<<(unsigned)nblk, 256, 0, s>>>((const bf16*)x, half_w, center, kern, (bf16*)out, B, L, H, K, half);
  });
  chk("alc_fused_fwd");
}

void alc_fused_bwd(const void* x, const float* half_w, const float* center, const float* kern, const void* dout, float* dx,
                   float* dhalf_w, float* dcenter, float* dkern, int B, int L, int H, int D, int K, int half, cudaStream_t s) {
  check_dims(D, K, half);
  if (half > 64) throw std::runtime_error("adaptive local conv: at most 129 taps");
  DISPATCH_LPR_BWD(D, {
    const int rpb = 256 / LPR_;
    const long long nblk = (long long)B * H * ((L + rpb - 1) / rpb);
    const size_t smem = (size_t)rpb * (K + 2 * half + 1) * sizeof(float);
    auto kernel = alc_bwd_kernel<LPR_, CPL_>;
    opt_in_smem(kernel, smem);
    kernel<<<(unsigned)nblk, 256, smem, s>>>((const bf16*)x, half_w, center, kern, (const bf16*)dout, dx, dhalf_w, dcenter,
                                                                dkern, B, L, H, K, half);
  });
  chk("alc_fused_bwd");
}

}  // namespace b200
