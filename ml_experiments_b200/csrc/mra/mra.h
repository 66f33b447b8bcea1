// Block-sparse attention primitives for MRA (multi-resolution attention), 32 x 32 blocks, fp32, torch-free interface.
// A "block list" is indices[b][n] = q_block * num_k_blocks + k_block for n < nblk.
//   sddmm : S[b][n][i][j] = Q[b][qb*32 + i][:] . K[b][kb*32 + j][:]                     (Q [B][Lq][D], K [B][Lk][D])
//   spmm  : out[b][qb*32 + i][:] += sum_j P[b][n][i][j] * V[b][kb*32 + j][:]             (out [B][Lq][D], zero it first)
//           transposed: out[b][kb*32 + j][:] += sum_i P[b][n][i][j] * X[b][qb*32 + i][:] (out [B][Lk][D])
//   rowmax: m[b][qb*32 + i] = max over the listed blocks of that row and j of S           (m [B][Lq], preset to -inf)
// D must be a multiple of 4 and at most 256.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
void mra_sddmm(const float* Q, const float* K, const int* indices, float* S, int B, int Lq, int Lk, int D, int nblk, cudaStream_t s);
void mra_spmm(const float* P, const int* indices, const float* V, float* out, int B, int Lq, int Lk, int D, int nblk, bool transposed,
              cudaStream_t s);
void mra_rowmax(const float* S, const int* indices, float* m, int B, int Lq, int Lk, int nblk, cudaStream_t s);
}  // namespace b200
