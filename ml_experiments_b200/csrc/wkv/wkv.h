// RWKV time-mixing recurrences (torch-free interface). Channel-last tensors, fp32 or bf16 I/O (io_bf16), fp32 math.
//
// WKV-4 (per channel c, decay w[c] < 0, bonus u[c]):
//   y_t = (sum_{s<t} e^{(t-1-s) w + k_s} v_s + e^{u + k_t} v_t) / (sum_{s<t} e^{(t-1-s) w + k_s} + e^{u + k_t})
//   k, v, y, gy, gk, gv : [B][T][C];  w, u : fp32 [C];  gw, gu : fp32 [B][C] (the caller sums over B; gw is d/dw)
//   scratch : fp32 [3][B][T][C] (backward only)
// WKV-5 (per head of size N, decay w[h][j] in (0, 1), bonus u[h][j], state S[j][i]):
//   y_t[i] = sum_j r_t[j] (u[j] k_t[j] v_t[i] + S_t[j][i]);   S_{t+1}[j][i] = w[j] S_t[j][i] + k_t[j] v_t[i]
//   r, k, v, y, gy, gr, gk, gv : [B][T][H*N];  w, u : fp32 [H][N];  gw, gu : fp32 [B][H*N] (gw is d/dw)
//   N must be 32, 64 or 128.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

void wkv4_fwd(const void* k, const void* v, const float* w, const float* u, void* y, bool io_bf16, int B, int T, int C,
              cudaStream_t s);
void wkv4_bwd(const void* k, const void* v, const float* w, const float* u, const void* gy, void* gk, void* gv, float* gw,
              float* gu, float* scratch, bool io_bf16, int B, int T, int C, cudaStream_t s);

void wkv5_fwd(const void* r, const void* k, const void* v, const float* w, const float* u, void* y, bool io_bf16, int B,
              int T, int H, int N, cudaStream_t s);
void wkv5_bwd(const void* r, const void* k, const void* v, const float* w, const float* u, const void* gy, void* gr,
              void* gk, void* gv, float* gw, float* gu, bool io_bf16, int B, int T, int H, int N, cudaStream_t s);

}  // namespace b200
