// MRA block-sparse kernels: sampled dense-dense product, block-sparse x dense product (plain and transposed) and the
// per-row maximum over a row's listed blocks. One CUDA block per listed 32 x 32 tile; the two 32 x D operand tiles are
// staged in shared memory (row stride padded to D + 1 words: conflict-free for both access patterns) and every thread
// produces a 1 x 4 strip. Rows that several listed tiles share accumulate with fp32 atomics (spmm) or an ordered-integer
// atomicMax (rowmax). Counterparts of the reference's fp32 kernels (zoology/mixers/mra/cuda/cuda_kernel.cu), which keep
// operands in a transposed [D][32] layout; here tensors stay [L][D] as the model produces them.
#include "mra.h"

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

constexpr int BS = 32;

__global__ void __launch_bounds__(256) sddmm_kernel(const float* __restrict__ Q, const float* __restrict__ K,
                                                    const int* __restrict__ indices, float* __restrict__ S, int Lq, int Lk,
                                                    int D, int nblk) {
  extern __shared__ float sm[];
  const int b = blockIdx.y, n = blockIdx.x, kbn = Lk / BS, str = D + 1;
  const int idx = indices[(long long)b * nblk + n], qb = idx / kbn, kb = idx % kbn;
  float* qs = sm;
  float* ks = sm + BS * str;
  const float* qg = Q + ((long long)b * Lq + qb * BS) * D;
  const float* kg = K + ((long long)b * Lk + kb * BS) * D;
  for (int i = threadIdx.x; i < BS * D; i += 256) {
    const int r = i / D, c = i % D;
    qs[r * str + c] = qg[i];
    ks[r * str + c] = kg[i];
  }
  __syncthreads();
  const int i = threadIdx.x / 8, j0 = (threadIdx.x % 8) * 4;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int d = 0; d < D; ++d) {
    const float qv = qs[i * str + d];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = fmaf(qv, ks[(j0 + u) * str + d], acc[u]);
  }
  float* out = S + (((long long)b * nblk + n) * BS + i) * BS + j0;
  *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

template <bool T>
__global__ void __launch_bounds__(256) spmm_kernel(const float* __restrict__ P, const int* __restrict__ indices,
                                                   const float* __restrict__ V, float* __restrict__ out, int Lq, int Lk, int D,
                                                   int nblk) {
  extern __shared__ float sm[];
  const int b = blockIdx.y, n = blockIdx.x, kbn = Lk / BS;
  const int idx = indices[(long long)b * nblk + n], qb = idx / kbn, kb = idx % kbn;
  float* ps = sm;             // [32][33]
  float* vs = sm + BS * 33;   // [32][D]
  const float* pg = P + ((long long)b * nblk + n) * BS * BS;
  // plain: rows of V come from the key block, results go to the query block; transposed: the other way round
  const int src_blk = T ? qb : kb, dst_blk = T ? kb : qb, Lsrc = T ? Lq : Lk, Ldst = T ? Lk : Lq;
  const float* vg = V + ((long long)b * Lsrc + src_blk * BS) * D;
  for (int i = threadIdx.x; i < BS * BS; i += 256) ps[(i / BS) * 33 + (i % BS)] = pg[i];
  for (int i = threadIdx.x; i < BS * D; i += 256) vs[i] = vg[i];
  __syncthreads();
  float* og = out + ((long long)b * Ldst + dst_blk * BS) * D;
  for (int e = threadIdx.x; e < BS * D; e += 256) {
    const int r = e / D, c = e % D;
    float acc = 0.f;
#pragma unroll 8
    for (int j = 0; j < BS; ++j) acc = fmaf(T ? ps[j * 33 + r] : ps[r * 33 + j], vs[j * D + c], acc);
    atomicAdd(og + e, acc);
  }
}

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  // ordered-integer trick: non-negative floats compare like ints, negative ones like reversed unsigned ints
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__global__ void __launch_bounds__(256) rowmax_kernel(const float* __restrict__ S, const int* __restrict__ indices,
                                                     float* __restrict__ m, int Lq, int Lk, int nblk) {
  const int b = blockIdx.y, n = blockIdx.x, kbn = Lk / BS;
  const int qb = indices[(long long)b * nblk + n] / kbn;
  const float* sg = S + ((long long)b * nblk + n) * BS * BS;
  const int i = threadIdx.x / 8, j0 = (threadIdx.x % 8) * 4;
  const float4 v = *reinterpret_cast<const float4*>(sg + i * BS + j0);
  float mx = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
  if ((threadIdx.x & 7) == 0) atomic_max_float(m + (long long)b * Lq + qb * BS + i, mx);
}

void check(const char* what, int D = 4) {
  if (D % 4 != 0 || D > 256 || D < 4) throw std::runtime_error("mra: head dim must be a multiple of 4, at most 256");
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

void mra_sddmm(const float* Q, const float* K, const int* indices, float* S, int B, int Lq, int Lk, int D, int nblk, cudaStream_t s) {
  check("mra (before sddmm)", D);
  const size_t sm = (size_t)2 * BS * (D + 1) * sizeof(float);
  cudaFuncSetAttribute(sddmm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  sddmm_kernel<<<dim3(nblk, B), 256, sm, s>>>(Q, K, indices, S, Lq, Lk, D, nblk);
  check("mra_sddmm");
}

void mra_spmm(const float* P, const int* indices, const float* V, float* out, int B, int Lq, int Lk, int D, int nblk, bool transposed,
              cudaStream_t s) {
  check("mra (before spmm)", D);
  const size_t sm = (size_t)(BS * 33 + BS * D) * sizeof(float);
  if (transposed) {
    cudaFuncSetAttribute(spmm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    spmm_kernel<true><<<dim3(nblk, B), 256, sm, s>>>(P, indices, V, out, Lq, Lk, D, nblk);
  } else {
    cudaFuncSetAttribute(spmm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    spmm_kernel<false><<<dim3(nblk, B), 256, sm, s>>>(P, indices, V, out, Lq, Lk, D, nblk);
  }
  check("mra_spmm");
}

void mra_rowmax(const float* S, const int* indices, float* m, int B, int Lq, int Lk, int nblk, cudaStream_t s) {
  rowmax_kernel<<<dim3(nblk, B), 256, 0, s>>>(S, indices, m, Lq, Lk, nblk);
  check("mra_rowmax");
}

}  // namespace b200
