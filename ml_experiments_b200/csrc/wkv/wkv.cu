// RWKV-4 and RWKV-5 time-mixing kernels, forward and backward. The recurrences are those of the reference's scalar
// kernels (zoology/mixers/rwkv/v4/wkv_cuda.cu, rwkv/v5/wkv5_cuda.cu) restated:
//  * WKV-4 keeps the running numerator / denominator divided by e^o (o = running maximum exponent) so nothing
//    overflows. One thread per (batch, channel) with the channel fastest: every step of a warp reads 32 consecutive
//    channels. The backward keeps its per-step intermediates in a caller-provided scratch buffer (no T limit, no
//    per-thread stack arrays).
//  * WKV-5 is linear attention with a per-key-channel decay. A block owns one (batch, head); thread x holds one row or
//    column of the N x N state in registers. The backward runs three sweeps: forward in time for gr, gu and gw (gw
//    from the derivative state dS_{t+1} = S_t + w dS_t), backward in time for gk (rows of the adjoint state) and
//    again for gv (columns).
#include "wkv.h"

#include <cuda_bf16.h>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;
__device__ __forceinline__ float ldf(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ldf(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr float MIN_VALUE = -1e38f;

template <typename F>
__global__ void wkv4_fwd_kernel(const F* __restrict__ k, const F* __restrict__ v, const float* __restrict__ w_,
                                const float* __restrict__ u_, F* __restrict__ y, int B, int T, int C) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * C) return;
  const int b = idx / C, c = idx % C;
  const float w = w_[c], u = u_[c];
  float p = 0.f, q = 0.f, o = MIN_VALUE;
  long long off = (long long)b * T * C + c;
  for (int t = 0; t < T; ++t, off += C) {
    const float kt = ldf(k, off), vt = ldf(v, off);
    float no = fmaxf(o, u + kt);
    float a = __expf(o - no), e = __expf(u + kt - no);
    stf(y, off, (a * p + e * vt) / (a * q + e));
    no = fmaxf(w + o, kt);
    a = __expf(w + o - no);
    e = __expf(kt - no);
    p = a * p + e * vt;
    q = a * q + e;
    o = no;
  }
}

template <typename F>
__global__ void wkv4_bwd_kernel(const F* __restrict__ k, const F* __restrict__ v, const float* __restrict__ w_,
                                const float* __restrict__ u_, const F* __restrict__ gy, F* __restrict__ gk,
                                F* __restrict__ gv, float* __restrict__ gw, float* __restrict__ gu,
                                float* __restrict__ scratch, int B, int T, int C) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * C) return;
  const int b = idx / C, c = idx % C;
  const float w = w_[c], u = u_[c];
  const long long plane = (long long)B * T * C, base = (long long)b * T * C + c;
  float* sy = scratch;              // y_t
  float* sz = scratch + plane;      // 1 / denominator
  float* se = scratch + 2 * plane;  // exponent of the current token's term
  float gwa = 0.f, gua = 0.f, p = 0.f, q = 0.f, dpdw = 0.f, dqdw = 0.f, o = MIN_VALUE;
  long long off = base;
  for (int t = 0; t < T; ++t, off += C) {
    const float kt = ldf(k, off), vt = ldf(v, off), g = ldf(gy, off);
    float no = fmaxf(o, kt + u);
    float a = __expf(o - no), e = __expf(kt + u - no);
    const float iden = 1.f / (a * q + e), yt = (a * p + e * vt) * iden;
    sy[off] = yt;
    sz[off] = iden;
    se[off] = kt + u - no;
    gwa += g * (dpdw - dqdw * yt) * iden * a;
    gua += g * (vt - yt) * e * iden;
    no = fmaxf(w + o, kt);
    a = __expf(w + o - no);
    e = __expf(kt - no);
    dpdw = a * (p + dpdw);
    dqdw = a * (q + dqdw);
    p = a * p + e * vt;
    q = a * q + e;
    o = no;
  }
  float gp = 0.f, gq = 0.f;
  o = MIN_VALUE;
  off = base + (long long)(T - 1) * C;
  for (int t = T - 1; t >= 0; --t, off -= C) {
    const float kt = ldf(k, off), vt = ldf(v, off), g = ldf(gy, off);
    const float yt = sy[off], iden = sz[off], ze = se[off];
    float a = g * iden * __expf(ze);
    float e = __expf(kt + o);
    stf(gk, off, a * (vt - yt) + e * (gp * vt + gq));
    stf(gv, off, a + e * gp);
    const float no = fmaxf(w + o, ze - kt - u);
    a = __expf(w + o - no);
    e = g * iden * __expf(ze - kt - u - no);
    gp = a * gp + e;
    gq = a * gq - e * yt;
    o = no;
  }
  gw[(long long)b * C + c] = gwa;
  gu[(long long)b * C + c] = gua;
}

// ---------------------------------------------------------------------------------------------------------- WKV-5
template <typename F, int N>
__global__ void __launch_bounds__(N) wkv5_fwd_kernel(const F* __restrict__ r, const F* __restrict__ k,
                                                     const F* __restrict__ v, const float* __restrict__ w_,
                                                     const float* __restrict__ u_, F* __restrict__ y, int T, int H) {
  const int b = blockIdx.x / H, h = blockIdx.x % H, i = threadIdx.x, C = H * N;
  __shared__ __align__(16) float rs[N], ks[N], ws[N], us[N];
  ws[i] = w_[h * N + i];
  us[i] = u_[h * N + i];
  float S[N];
#pragma unroll
  for (int j = 0; j < N; ++j) S[j] = 0.f;
  long long off = (long long)b * T * C + h * N + i;
  for (int t = 0; t < T; ++t, off += C) {
    __syncthreads();
    rs[i] = ldf(r, off);
    ks[i] = ldf(k, off);
    __syncthreads();
    const float vt = ldf(v, off);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float x = ks[j] * vt;
      acc = fmaf(rs[j], fmaf(us[j], x, S[j]), acc);
      S[j] = fmaf(S[j], ws[j], x);
    }
    stf(y, off, acc);
  }
}

template <typename F, int N>
__global__ void __launch_bounds__(N) wkv5_bwd_kernel(const F* __restrict__ r, const F* __restrict__ k,
                                                     const F* __restrict__ v, const float* __restrict__ w_,
                                                     const float* __restrict__ u_, const F* __restrict__ gy,
                                                     F* __restrict__ gr, F* __restrict__ gk, F* __restrict__ gv,
                                                     float* __restrict__ gw, float* __restrict__ gu, int T, int H) {
  const int b = blockIdx.x / H, h = blockIdx.x % H, x = threadIdx.x, C = H * N;
  __shared__ __align__(16) float sa[N], sb[N], ws[N], us[N];
  ws[x] = w_[h * N + x];
  us[x] = u_[h * N + x];
  const float w = w_[h * N + x], u = u_[h * N + x];
  const long long first = (long long)b * T * C + h * N + x, last = first + (long long)(T - 1) * C;
  float S[N];
  // sweep 1 (forward in time, thread = key channel j): gr_t[j], gu[j], gw[j]; S = row j of the state, dS = dS/dw
  {
    float dS[N];
#pragma unroll
    for (int i = 0; i < N; ++i) S[i] = dS[i] = 0.f;
    float gua = 0.f, gwa = 0.f;
    long long off = first;
    for (int t = 0; t < T; ++t, off += C) {
      __syncthreads();
      sa[x] = ldf(v, off);
      sb[x] = ldf(gy, off);
      __syncthreads();
      const float kt = ldf(k, off), rt = ldf(r, off);
      float grs = 0.f, gus = 0.f, gws = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float kv = kt * sa[i], g = sb[i];
        grs = fmaf(fmaf(u, kv, S[i]), g, grs);
        gus = fmaf(kv, g, gus);
        gws = fmaf(dS[i], g, gws);
        dS[i] = fmaf(w, dS[i], S[i]);
        S[i] = fmaf(w, S[i], kv);
      }
      stf(gr, off, grs);
      gua = fmaf(rt, gus, gua);
      gwa = fmaf(rt, gws, gwa);
    }
    gu[(long long)b * C + h * N + x] = gua;
    gw[(long long)b * C + h * N + x] = gwa;
  }
  // sweep 2 (backward in time, thread = key channel j): gk_t[j]; S = row j of the adjoint state G
#pragma unroll
  for (int i = 0; i < N; ++i) S[i] = 0.f;
  {
    long long off = last;
    for (int t = T - 1; t >= 0; --t, off -= C) {
      __syncthreads();
      sa[x] = ldf(v, off);
      sb[x] = ldf(gy, off);
      __syncthreads();
      const float rt = ldf(r, off);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float rg = rt * sb[i];
        acc = fmaf(fmaf(u, rg, S[i]), sa[i], acc);
        S[i] = fmaf(S[i], w, rg);
      }
      stf(gk, off, acc);
    }
  }
  // sweep 3 (backward in time, thread = value channel i): gv_t[i]; S = column i of the adjoint state
#pragma unroll
  for (int j = 0; j < N; ++j) S[j] = 0.f;
  {
    long long off = last;
    for (int t = T - 1; t >= 0; --t, off -= C) {
      __syncthreads();
      sa[x] = ldf(r, off);
      sb[x] = ldf(k, off);
      __syncthreads();
      const float g = ldf(gy, off);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float rg = g * sa[j];
        acc = fmaf(fmaf(us[j], rg, S[j]), sb[j], acc);
        S[j] = fmaf(S[j], ws[j], rg);
      }
      stf(gv, off, acc);
    }
  }
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename F>
void wkv5_fwd_t(const void* r, const void* k, const void* v, const float* w, const float* u, void* y, int B, int T, int H,
                int N, cudaStream_t s) {
  const F *rr = (const F*)r, *kk = (const F*)k, *vv = (const F*)v;
  if (N == 32) wkv5_fwd_kernel<F, 32><<<B * H, 32, 0, s>>>(rr, kk, vv, w, u, (F*)y, T, H);
  else if (N == 64) wkv5_fwd_kernel<F, 64><<<B * H, 64, 0, s>>>(rr, kk, vv, w, u, (F*)y, T, H);
  else if (N == 128) wkv5_fwd_kernel<F, 128><<<B * H, 128, 0, s>>>(rr, kk, vv, w, u, (F*)y, T, H);
  else throw std::runtime_error("wkv5: head size must be 32, 64 or 128");
}

template <typename F>
void wkv5_bwd_t(const void* r, const void* k, const void* v, const float* w, const float* u, const void* gy, void* gr,
                void* gk, void* gv, float* gw, float* gu, int B, int T, int H, int N, cudaStream_t s) {
  const F *rr = (const F*)r, *kk = (const F*)k, *vv = (const F*)v, *gg = (const F*)gy;
  if (N == 32) wkv5_bwd_kernel<F, 32><<<B * H, 32, 0, s>>>(rr, kk, vv, w, u, gg, (F*)gr, (F*)gk, (F*)gv, gw, gu, T, H);
  else if (N == 64) wkv5_bwd_kernel<F, 64><<<B * H, 64, 0, s>>>(rr, kk, vv, w, u, gg, (F*)gr, (F*)gk, (F*)gv, gw, gu, T, H);
  else if (N == 128) wkv5_bwd_kernel<F, 128><<<B * H, 128, 0, s>>>(rr, kk, vv, w, u, gg, (F*)gr, (F*)gk, (F*)gv, gw, gu, T, H);
  else throw std::runtime_error("wkv5: head size must be 32, 64 or 128");
}

}  // namespace

void wkv4_fwd(const void* k, const void* v, const float* w, const float* u, void* y, bool io_bf16, int B, int T, int C,
              cudaStream_t s) {
  const int threads = 128, blocks = (B * C + threads - 1) / threads;
  if (io_bf16) wkv4_fwd_kernel<bf16><<<blocks, threads, 0, s>>>((const bf16*)k, (const bf16*)v, w, u, (bf16*)y, B, T, C);
  else wkv4_fwd_kernel<float><<<blocks, threads, 0, s>>>((const float*)k, (const float*)v, w, u, (float*)y, B, T, C);
  check("wkv4_fwd");
}

void wkv4_bwd(const void* k, const void* v, const float* w, const float* u, const void* gy, void* gk, void* gv, float* gw,
              float* gu, float* scratch, bool io_bf16, int B, int T, int C, cudaStream_t s) {
  const int threads = 128, blocks = (B * C + threads - 1) / threads;
  if (io_bf16)
    wkv4_bwd_kernel<bf16><<<blocks, threads, 0, s>>>((const bf16*)k, (const bf16*)v, w, u, (const bf16*)gy, (bf16*)gk,
                                                     (bf16*)gv, gw, gu, scratch, B, T, C);
  else
    wkv4_bwd_kernel<float><<<blocks, threads, 0, s>>>((const float*)k, (const float*)v, w, u, (const float*)gy, (float*)gk,
                                                      (float*)gv, gw, gu, scratch, B, T, C);
  check("wkv4_bwd");
}

void wkv5_fwd(const void* r, const void* k, const void* v, const float* w, const float* u, void* y, bool io_bf16, int B,
              int T, int H, int N, cudaStream_t s) {
  if (io_bf16) wkv5_fwd_t<bf16>(r, k, v, w, u, y, B, T, H, N, s);
  else wkv5_fwd_t<float>(r, k, v, w, u, y, B, T, H, N, s);
  check("wkv5_fwd");
}

void wkv5_bwd(const void* r, const void* k, const void* v, const float* w, const float* u, const void* gy, void* gr,
              void* gk, void* gv, float* gw, float* gu, bool io_bf16, int B, int T, int H, int N, cudaStream_t s) {
  if (io_bf16) wkv5_bwd_t<bf16>(r, k, v, w, u, gy, gr, gk, gv, gw, gu, B, T, H, N, s);
  else wkv5_bwd_t<float>(r, k, v, w, u, gy, gr, gk, gv, gw, gu, B, T, H, N, s);
  check("wkv5_bwd");
}

}  // namespace b200
