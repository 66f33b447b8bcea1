// Local window attention (K <= 64 taps around every position, per-tap additive bias), forward and backward.
//
// A block owns 128 consecutive positions of one (batch, head); one thread per position. The K / V rows the block needs
// (128 + K - 1 of them) are staged once in shared memory as bf16 with an odd word stride, so that the 32 threads of a
// warp, which read 32 consecutive rows at the same column, never collide. Scores live in a [K][128] shared scratch
// (column = thread), the query or the output accumulator in registers. The backward is two kernels: per query
// (dS = P (dP - sum P dP), written out as dbias, and dq), then per key (dk, dv gathered from the dS / P / q / dout rows
// of the queries whose window covers the key), so no atomics are needed and the result is deterministic.
// This replaces the reference's one-program-per-(b, l, h) Triton kernels (models/triton_scatter.py:346-579), which
// recompute the scores three times and scatter dk / dv with atomics.
#include "window_attn.h"

#include <cuda_bf16.h>

#include <cstdint>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;
constexpr int TB = 128;  // positions per block

__device__ __forceinline__ float2 ld2(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }

// rows [row0, row0 + nrows) of a [B][L][H][D] tensor (one head) into shared memory, zero outside [0, L)
template <int D>
__device__ __forceinline__ void stage_rows(bf16* dst, const bf16* __restrict__ src, int b, int h, int row0, int nrows, int L,
                                           int H, int stride) {
  constexpr int VPR = D / 8;  // 16-byte vectors per row
  for (int i = threadIdx.x; i < nrows * VPR; i += TB) {
    const int r = i / VPR, c = (i % VPR) * 8, l = row0 + r;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (l >= 0 && l < L) val = *reinterpret_cast<const uint4*>(src + (((long long)b * L + l) * H + h) * D + c);
    // the shared row stride is odd in words, so rows are only 4-byte aligned: store as four words
    uint32_t* d32 = reinterpret_cast<uint32_t*>(dst + r * stride + c);
    d32[0] = val.x; d32[1] = val.y; d32[2] = val.z; d32[3] = val.w;
  }
}

template <int D>
__global__ void __launch_bounds__(TB) window_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                        const bf16* __restrict__ v, const float* __restrict__ bias,
                                                        bf16* __restrict__ out, float* __restrict__ P, float scale, int L,
                                                        int H, int K) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int STR = D + 2;  // bf16 per shared row: (D + 2) / 2 words is odd for D in {16, 32, 64}
  const int rows = TB + K - 1, padl = (K - 1) / 2;
  bf16* ks = reinterpret_cast<bf16*>(smem);
  bf16* vs = ks + rows * STR;
  float* sc = reinterpret_cast<float*>(vs + rows * STR);  // [K][TB]
  const int h = blockIdx.y, b = blockIdx.z, l0 = blockIdx.x * TB, t = threadIdx.x, l = l0 + t;
  stage_rows<D>(ks, k, b, h, l0 - padl, rows, L, H, STR);
  stage_rows<D>(vs, v, b, h, l0 - padl, rows, L, H, STR);
  __syncthreads();
  if (l >= L) return;
  const long long row = (((long long)b * L + l) * H + h);
  float reg[D];
  {
    const bf16* qp = q + row * D;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 f = ld2(qp + d);
      reg[d] = f.x * scale;
      reg[d + 1] = f.y * scale;
    }
  }
  float m = -3.0e38f;
  for (int w = 0; w < K; ++w) {
    const bf16* kr = ks + (t + w) * STR;
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 f = ld2(kr + d);
      s = fmaf(reg[d], f.x, s);
      s = fmaf(reg[d + 1], f.y, s);
    }
    s += bias[row * K + w];
    sc[w * TB + t] = s;
    m = fmaxf(m, s);
  }
  float denom = 0.f;
#pragma unroll
  for (int d = 0; d < D; ++d) reg[d] = 0.f;
  for (int w = 0; w < K; ++w) {
    const float p = __expf(sc[w * TB + t] - m);
    sc[w * TB + t] = p;
    denom += p;
    const bf16* vr = vs + (t + w) * STR;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 f = ld2(vr + d);
      reg[d] = fmaf(p, f.x, reg[d]);
      reg[d + 1] = fmaf(p, f.y, reg[d + 1]);
    }
  }
  const float inv = 1.f / denom;
  for (int w = 0; w < K; ++w) P[row * K + w] = sc[w * TB + t] * inv;
  bf16* op = out + row * D;
#pragma unroll
  for (int d = 0; d < D; d += 2)
    *reinterpret_cast<__nv_bfloat162*>(op + d) = __floats2bfloat162_rn(reg[d] * inv, reg[d + 1] * inv);
}

// per query: dS (= dbias) and dq
template <int D>
__global__ void __launch_bounds__(TB) window_bwd_q_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                          const float* __restrict__ P, const bf16* __restrict__ dout,
                                                          bf16* __restrict__ dq, float* __restrict__ dS, float scale, int L,
                                                          int H, int K) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int STR = D + 2;
  const int rows = TB + K - 1, padl = (K - 1) / 2;
  bf16* ks = reinterpret_cast<bf16*>(smem);
  bf16* vs = ks + rows * STR;
  float* sc = reinterpret_cast<float*>(vs + rows * STR);
  const int h = blockIdx.y, b = blockIdx.z, l0 = blockIdx.x * TB, t = threadIdx.x, l = l0 + t;
  stage_rows<D>(ks, k, b, h, l0 - padl, rows, L, H, STR);
  stage_rows<D>(vs, v, b, h, l0 - padl, rows, L, H, STR);
  __syncthreads();
  if (l >= L) return;
  const long long row = (((long long)b * L + l) * H + h);
  float reg[D];
  {
    const bf16* gp = dout + row * D;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 f = ld2(gp + d);
      reg[d] = f.x;
      reg[d + 1] = f.y;
    }
  }
  float delta = 0.f;
  for (int w = 0; w < K; ++w) {
    const bf16* vr = vs + (t + w) * STR;
    float dp = 0.f;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 f = ld2(vr + d);
      dp = fmaf(reg[d], f.x, dp);
      dp = fmaf(reg[d + 1], f.y, dp);
    }
    sc[w * TB + t] = dp;
    delta = fmaf(P[row * K + w], dp, delta);
  }
#pragma unroll
  for (int d = 0; d < D; ++d) reg[d] = 0.f;
  for (int w = 0; w < K; ++w) {
    const float ds = P[row * K + w] * (sc[w * TB + t] - delta);
    dS[row * K + w] = ds;
    const bf16* kr = ks + (t + w) * STR;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 f = ld2(kr + d);
      reg[d] = fmaf(ds, f.x, reg[d]);
      reg[d + 1] = fmaf(ds, f.y, reg[d + 1]);
    }
  }
  bf16* op = dq + row * D;
#pragma unroll
  for (int d = 0; d < D; d += 2)
    *reinterpret_cast<__nv_bfloat162*>(op + d) = __floats2bfloat162_rn(reg[d] * scale, reg[d + 1] * scale);
}

// per key j: dk[j] = scale * sum_w dS[i][w] q[i],  dv[j] = sum_w P[i][w] dout[i]  with  i = j + padl - w
template <int D>
__global__ void __launch_bounds__(TB) window_bwd_kv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ dout,
                                                           const float* __restrict__ P, const float* __restrict__ dS,
                                                           bf16* __restrict__ dk, bf16* __restrict__ dv, float scale, int L,
                                                           int H, int K) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int STR = D + 2;
  const int rows = TB + K - 1, padl = (K - 1) / 2, wstr = K | 1;
  bf16* qs = reinterpret_cast<bf16*>(smem);
  bf16* gs = qs + rows * STR;
  float* ps = reinterpret_cast<float*>(gs + rows * STR);  // [rows][wstr]
  float* ds = ps + rows * wstr;
  const int h = blockIdx.y, b = blockIdx.z, j0 = blockIdx.x * TB, t = threadIdx.x, j = j0 + t;
  const int i_lo = j0 + padl - (K - 1);  // first query row whose window reaches this block's keys
  stage_rows<D>(qs, q, b, h, i_lo, rows, L, H, STR);
  stage_rows<D>(gs, dout, b, h, i_lo, rows, L, H, STR);
  for (int idx = threadIdx.x; idx < rows * K; idx += TB) {
    const int r = idx / K, w = idx % K, i = i_lo + r;
    const bool ok = i >= 0 && i < L;
    const long long off = ((((long long)b * L + i) * H + h)) * K + w;
    ps[r * wstr + w] = ok ? P[off] : 0.f;
    ds[r * wstr + w] = ok ? dS[off] : 0.f;
  }
  __syncthreads();
  if (j >= L) return;
  float ak[D], av[D];
#pragma unroll
  for (int d = 0; d < D; ++d) ak[d] = av[d] = 0.f;
  for (int w = 0; w < K; ++w) {
    const int r = t + (K - 1) - w;
    const float sd = ds[r * wstr + w], sp = ps[r * wstr + w];
    const bf16 *qr = qs + r * STR, *gr = gs + r * STR;
#pragma unroll
    for (int d = 0; d < D; d += 2) {
      const float2 fq = ld2(qr + d), fg = ld2(gr + d);
      ak[d] = fmaf(sd, fq.x, ak[d]);
      ak[d + 1] = fmaf(sd, fq.y, ak[d + 1]);
      av[d] = fmaf(sp, fg.x, av[d]);
      av[d + 1] = fmaf(sp, fg.y, av[d + 1]);
    }
  }
  const long long row = (((long long)b * L + j) * H + h);
#pragma unroll
  for (int d = 0; d < D; d += 2) {
    *reinterpret_cast<__nv_bfloat162*>(dk + row * D + d) = __floats2bfloat162_rn(ak[d] * scale, ak[d + 1] * scale);
    *reinterpret_cast<__nv_bfloat162*>(dv + row * D + d) = __floats2bfloat162_rn(av[d], av[d + 1]);
  }
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

size_t smem_qk(int D, int K) {
  const int rows = TB + K - 1, str = D + 2;
  return (size_t)2 * rows * str * 2 + (size_t)K * TB * 4;
}
size_t smem_kv(int D, int K) {
  const int rows = TB + K - 1, str = D + 2;
  return (size_t)2 * rows * str * 2 + (size_t)2 * rows * (K | 1) * 4;
}

template <typename Kern>
void set_smem(Kern kern, size_t bytes) {
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

#define B200_WINDOW_DISPATCH(D_, CALL)                                         \
  switch (D_) {                                                                \
    case 16: { constexpr int DD = 16; CALL; break; }                           \
    case 32: { constexpr int DD = 32; CALL; break; }                           \
    case 64: { constexpr int DD = 64; CALL; break; }                           \
    default: throw std::runtime_error("window_attn: head dim must be 16, 32 or 64"); \
  }

void window_attn_fwd(const void* q, const void* k, const void* v, const float* bias, void* out, float* P, float scale,
                     int B, int L, int H, int D, int K, cudaStream_t s) {
  if (K < 1 || K > 64) throw std::runtime_error("window_attn: window must have 1..64 taps");
  dim3 grid((L + TB - 1) / TB, H, B);
  const size_t sm = smem_qk(D, K);
  B200_WINDOW_DISPATCH(D, (set_smem(window_fwd_kernel<DD>, sm),
                           window_fwd_kernel<DD><<<grid, TB, sm, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, bias,
                                                                      (bf16*)out, P, scale, L, H, K)));
  check("window_attn_fwd");
}

void window_attn_bwd(const void* q, const void* k, const void* v, const float* P, const void* dout, void* dq, void* dk,
                     void* dv, float* dbias, float scale, int B, int L, int H, int D, int K, cudaStream_t s) {
  if (K < 1 || K > 64) throw std::runtime_error("window_attn: window must have 1..64 taps");
  dim3 grid((L + TB - 1) / TB, H, B);
  const size_t sm1 = smem_qk(D, K), sm2 = smem_kv(D, K);
  B200_WINDOW_DISPATCH(D, (set_smem(window_bwd_q_kernel<DD>, sm1),
                           window_bwd_q_kernel<DD><<<grid, TB, sm1, s>>>((const bf16*)k, (const bf16*)v, P, (const bf16*)dout,
                                                                         (bf16*)dq, dbias, scale, L, H, K)));
  check("window_attn_bwd (queries)");
  B200_WINDOW_DISPATCH(D, (set_smem(window_bwd_kv_kernel<DD>, sm2),
                           window_bwd_kv_kernel<DD><<<grid, TB, sm2, s>>>((const bf16*)q, (const bf16*)dout, P, dbias,
                                                                          (bf16*)dk, (bf16*)dv, scale, L, H, K)));
  check("window_attn_bwd (keys)");
}

}  // namespace b200
