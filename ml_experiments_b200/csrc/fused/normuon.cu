// NorMuon update kernels: variance reduction of the orthogonalised update and the cautious weight-decay /
// parameter update with an optional 16-bit mantissa extension of bf16 parameters.
//
// For a stack v [nmat][R][C] (bf16 or fp32) the reference computes (modded-nanogpt/train_gpt.py:764-775):
//   v_mean  = mean(v^2) along the reduced side (per row when red_cols, per column otherwise)
//   v_norm  = sqrt(sum(v_mean) * red_size)                        (Frobenius norm of the matrix)
//   second  = lerp(second, v_mean, 1 - beta2) ;  step = rsqrt(max(second, 1e-10))
//   v_new   = sqrt(sum(v_mean * red_size * step^2)) ;  scale = step * v_norm / max(v_new, 1e-10)
//   v      *= scale                                               (broadcast along the reduced side)
// and then (:744-760)  p -= p * [v * p >= 0] * wd * lr + v * lr  in fp32, where a bf16 parameter is widened by a
// uint16 "mantissa" buffer holding the low half of its fp32 value.
//
// Three launches: (1) sums of squares per row / column, (2) one block per matrix turns them into the per-row / column
// scale and updates the second-moment buffer, (3) the update kernel applies scale, decay and step in one pass over p
// and v, so the scaled update is never written to memory.
#include "fused.h"

#include <cuda_bf16.h>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;

template <typename T>
__device__ __forceinline__ float ldf(const T* p) { return (float)(*p); }

// stat[m][r] = sum_c v[m][r][c]^2 : one warp per row
template <typename T>
__global__ void nm_row_sumsq_kernel(const T* __restrict__ v, float* __restrict__ stat, int rows_total, int C) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows_total) return;
  const T* x = v + (long long)row * C;
  float acc = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float f = ldf(x + c);
    acc = fmaf(f, f, acc);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) stat[row] = acc;
}

// stat[m][c] = sum_r v[m][r][c]^2 : block (32 columns x 8 row-lanes), grid (C/32, nmat)
template <typename T>
__global__ void nm_col_sumsq_kernel(const T* __restrict__ v, float* __restrict__ stat, int R, int C) {
  __shared__ float red[8][33];
  const int m = blockIdx.y;
  const int c = blockIdx.x * 32 + threadIdx.x;
  const T* x = v + (long long)m * R * C;
  float acc = 0.f;
  if (c < C)
    for (int r = threadIdx.y; r < R; r += 8) {
      const float f = ldf(x + (long long)r * C + c);
      acc = fmaf(f, f, acc);
    }
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i][threadIdx.x];
    stat[(long long)m * C + c] = t;
  }
}

__device__ float block_sum(float x, float* sh) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) x += __shfl_xor_sync(0xffffffffu, x, s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = x;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += sh[i];
  __syncthreads();
  return t;
}

// One block per matrix. stat: sums of squares (n_stat entries per matrix, each over red_size elements); on exit stat
// holds the scale of every row / column. second: running second moment, same shape as stat.
__global__ void nm_scale_kernel(float* __restrict__ stat, float* __restrict__ second, int n_stat, int red_size,
                                float beta2) {
  __shared__ float sh[32];
  float* st = stat + (long long)blockIdx.x * n_stat;
  float* sm = second + (long long)blockIdx.x * n_stat;
  const float inv_red = 1.f / red_size;
  float sum_mean = 0.f, sum_scaled = 0.f;
  for (int i = threadIdx.x; i < n_stat; i += blockDim.x) {
    const float mean = st[i] * inv_red;
    const float s2 = sm[i] + (1.f - beta2) * (mean - sm[i]);       // lerp(second, mean, 1 - beta2)
    sm[i] = s2;
    const float step = rsqrtf(fmaxf(s2, 1e-10f));
    sum_mean += mean;
    sum_scaled += mean * red_size * step * step;
  }
  const float tot_mean = block_sum(sum_mean, sh);
  const float tot_scaled = block_sum(sum_scaled, sh);
  const float v_norm = sqrtf(tot_mean * red_size);
  const float ratio = v_norm / fmaxf(sqrtf(tot_scaled), 1e-10f);
  for (int i = threadIdx.x; i < n_stat; i += blockDim.x) st[i] = rsqrtf(fmaxf(sm[i], 1e-10f)) * ratio;
}

// p -= p * [u * p >= 0] * wd_lr + u * lr with u = v * scale ; grid (blocks, nmat). TP: float or bf16 (+ mantissa).
// lr / wd_lr may differ per matrix (lr_mat / wd_mat non-null: values per matrix).
template <typename TP, typename TV>
__global__ void nm_update_kernel(TP* __restrict__ p, unsigned short* __restrict__ mant, const TV* __restrict__ v,
                                 const float* __restrict__ scale, int R, int C, int scale_per_row, float lr, float wd_lr,
                                 const float* __restrict__ lr_mat, const float* __restrict__ wd_mat) {
  const int m = blockIdx.y;
  const long long n = (long long)R * C;
  const long long base = (long long)m * n;
  const float lr_m = lr_mat ? lr_mat[m] : lr;
  const float wd_m = wd_mat ? wd_mat[m] : wd_lr;
  const float* sc = scale ? scale + (long long)m * (scale_per_row ? R : C) : nullptr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / C), c = (int)(i - (long long)r * C);
    float u = (float)v[base + i];
    if (sc) u *= sc[scale_per_row ? r : c];
    float pf;
    if constexpr (sizeof(TP) == 2) {
      const unsigned int hi = (unsigned int)(*reinterpret_cast<const unsigned short*>(p + base + i));
      const unsigned int lo = mant ? (unsigned int)mant[base + i] : 0u;
      pf = __uint_as_float((hi << 16) | lo);
    } else {
      pf = (float)p[base + i];
    }
    const float mask = (u * pf >= 0.f) ? 1.f : 0.f;
    pf = pf - pf * mask * wd_m - u * lr_m;
    if constexpr (sizeof(TP) == 2) {
      const unsigned int raw = __float_as_uint(pf);
      if (mant) {
        *reinterpret_cast<unsigned short*>(p + base + i) = (unsigned short)(raw >> 16);   // truncation: the rest lives in mant
        mant[base + i] = (unsigned short)(raw & 0xffffu);
      } else {
        p[base + i] = (TP)__float2bfloat16_rn(pf);
      }
    } else {
      p[base + i] = (TP)pf;
    }
  }
}

void chk(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}


// Adam with the cautious weight decay of the combined optimizer (modded-nanogpt/train_gpt.py:654-691): moments in fp32,
//   upd = m / (sqrt(v) + eps) * step_size;  upd += p * [upd * p > 0] * wd_lr;  p -= upd      (one pass over p, g, m, v)
template <typename TP, typename TG>
__global__ void adam_cautious_kernel(TP* __restrict__ p, const TG* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                     long long n, float b1, float b2, float eps, float step_size, float wd_lr) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gi = ldf(g + i), pi = ldf(p + i);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    float upd = mi / (sqrtf(vi) + eps) * step_size;
    if (upd * pi > 0.f) upd += pi * wd_lr;
    p[i] = (TP)(pi - upd);
  }
}

}  // namespace

void adam_cautious(void* p, int p_is_bf16, const void* g, int g_is_bf16, float* m, float* v, long long n, float b1, float b2,
                   float eps, float step_size, float wd_lr, cudaStream_t s) {
  if (n <= 0) return;
  long long bl = (n + 255) / 256;
  if (bl > 148 * 16) bl = 148 * 16;
#define AC(TP, TG) adam_cautious_kernel<TP, TG><<<(int)bl, 256, 0, s>>>((TP*)p, (const TG*)g, m, v, n, b1, b2, eps, step_size, wd_lr)
  if (p_is_bf16 && g_is_bf16) AC(bf16, bf16);
  else if (p_is_bf16) AC(bf16, float);
  else if (g_is_bf16) AC(float, bf16);
  else AC(float, float);
#undef AC
  chk("adam_cautious");
}

void normuon_scales(const void* v, int v_is_bf16, float* stat, float* second, int nmat, int R, int C, int red_cols,
                    float beta2, cudaStream_t s) {
  if (nmat <= 0) return;
  if (red_cols) {
    const int rows = nmat * R;
    const int blocks = (rows * 32 + 255) / 256;
    if (v_is_bf16) nm_row_sumsq_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)v, stat, rows, C);
    else           nm_row_sumsq_kernel<float><<<blocks, 256, 0, s>>>((const float*)v, stat, rows, C);
  } else {
    dim3 grid((C + 31) / 32, nmat), block(32, 8);
    if (v_is_bf16) nm_col_sumsq_kernel<bf16><<<grid, block, 0, s>>>((const bf16*)v, stat, R, C);
    else           nm_col_sumsq_kernel<float><<<grid, block, 0, s>>>((const float*)v, stat, R, C);
  }
  chk("normuon sums of squares");
  nm_scale_kernel<<<nmat, 256, 0, s>>>(stat, second, red_cols ? R : C, red_cols ? C : R, beta2);
  chk("normuon scale");
}

void normuon_update(void* p, int p_is_bf16, unsigned short* mant, const void* v, int v_is_bf16, const float* scale,
                    int nmat, int R, int C, int scale_per_row, float lr, float wd_lr, const float* lr_mat,
                    const float* wd_mat, cudaStream_t s) {
  if (nmat <= 0) return;
  const long long n = (long long)R * C;
  int bx = (int)((n + 255) / 256);
  const int cap = (148 * 8 + nmat - 1) / nmat;
  if (bx > cap) bx = cap;
  dim3 grid(bx, nmat);
#define NM_UPD(TP, TV) \
  nm_update_kernel<TP, TV><<<grid, 256, 0, s>>>((TP*)p, mant, (const TV*)v, scale, R, C, scale_per_row, lr, wd_lr, lr_mat, wd_mat)
  if (p_is_bf16 && v_is_bf16) NM_UPD(bf16, bf16);
  else if (p_is_bf16) NM_UPD(bf16, float);
  else if (v_is_bf16) NM_UPD(float, bf16);
  else NM_UPD(float, float);
#undef NM_UPD
  chk("normuon update");
}

}  // namespace b200
