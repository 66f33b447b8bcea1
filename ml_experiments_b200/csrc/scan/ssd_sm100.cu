// Chunked scan for state-space layers with one scalar decay per head ("SSD" form; Mamba-2, the trapezoidal SSMMixer3) on
// tcgen05 tensor cores with the running state resident in tensor memory.
//
// Per (batch b, head h) the recurrence over time t, with state S [N x P], inputs x_t [P], maps B_t, C_t [N]:
//     S_t = a_t S_{t-1} + g_t B_t (x) x_t  (+ look-back term folded into the weights, see below)        y_t = C_t . S_t
// is evaluated 128 steps at a time. With cs = inclusive cumulative sum of log a inside the chunk:
//     G  = C B^T                                  (128 x 128, K = N)          tcgen05.mma  #1
//     M  = G o [j <= i] exp(cs_i - cs_j) w_ij     (threads: TMEM -> registers -> bf16 -> shared memory)
//     Y  = M x                                    (128 x P,   K = 128)        tcgen05.mma  #2
//     Z  = C S_prev                               (128 x P,   K = N)          tcgen05.mma  #3   (state of the previous chunks;
//                                                                                  issued after M is built, into G's columns)
//     y_i = Y_i + exp(cs_i) Z_i                   (epilogue)
//     S  = exp(cs_end) S + (B o exp(cs_end - cs_j) w_j)^T x      (N x P, K = 128, accumulated in TMEM)   tcgen05.mma  #4
// One CTA owns one (b, h) and walks its chunks in order, so the state never leaves the chip: fp32 in tensor memory for
// the accumulation, a bf16 copy in shared memory as the B operand of #3. Nothing of size L x N x P and no per-chunk
// state tensor exists in global memory (the reference pipelines write both).
//
// Weights: w_ij = g_off[j] for j < i and g_diag[i] for j = i; the state uses g_off. With the plain recurrence both are
// gamma. The trapezoidal look-back  + beta_t B_{t-1} (x) x_{t-1}  becomes g_off[j] = gamma_j + beta_{j+1} / a_{j+1}
// (the host passes it; beyond the sequence end the second term is 0), g_diag = gamma: the look-back of step j+1 is the
// same outer product B_j (x) x_j entering one step later and not decayed by a_{j+1}.
//
// Shapes: chunk = 128 steps (L % 128 == 0), N in {64, 128}, P in {64, 128}; bf16 inputs, fp32 state. Other shapes are
// served by the PyTorch formulation.
#include "ssd.h"

#include <cuda_bf16.h>

#include <stdexcept>
#include <string>

#include "../common/per_device.h"
#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace b200 {
namespace {

struct SsdParams {
  int L, H, Hb;             // sequence length, heads, heads of B / C (H % Hb == 0: grouped B / C)
  int nchunks;
  const float* log_a;       // [b, L, H]
  const float* g_off;       // [b, L, H]
  const float* g_diag;      // [b, L, H]
  __nv_bfloat16* y;         // [b, L, H, P]
  const float* init_state;  // [b, H, N, P] or null
  float* final_state;       // [b, H, N, P] or null
  float* chunk_states;      // [b, H, nchunks, N, P] or null: the state after every chunk
  int* status;
};

__device__ __forceinline__ void cta_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (*abort_flag) return;
  if (!mbar_wait(bar, parity, status, code)) *abort_flag = 1;
}

// 128 threads: thread t owns time step t of the chunk (rows of G / M / Y / Z) and, for t < N, row t of the state.
template <int N, int P>
__global__ void __launch_bounds__(128, (128 + 2 * P) <= 256 ? 2 : 1)
ssd_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const SsdParams p) {
  constexpr int Q = 128;
  constexpr int NSN = N / 64, NSP = P / 64;        // 128-byte spans along N and along P
  constexpr int C_BYTES = NSN * Q * 128;           // C chunk  [Q][N]  (K-major A of #1 and #3)
  constexpr int B_BYTES = NSN * Q * 128;           // B chunk  [Q][N]  (K-major B of #1, MN-major A of #4)
  constexpr int X_BYTES = NSP * Q * 128;           // x chunk  [Q][P]  (MN-major B of #2 and #4)
  constexpr int M_BYTES = 2 * Q * 128;             // M        [Q][Q]  (K-major A of #2)
  constexpr int S_BYTES = NSP * N * 128;           // state    [N][P]  bf16 (MN-major B of #3)
  // Z = C S_prev reuses the columns of G: G has been read into registers (to build M) before #3 is issued. With P = 64
  // that makes 256 tensor-memory columns per CTA, so two CTAs share an SM and hide each other's load / barrier latency.
  constexpr uint32_t G_COL = 0, Z_COL = 0, Y_COL = 128, S_COL = 128 + P;
  constexpr uint32_t TMEM_COLS = (128 + 2 * P) <= 256 ? 256 : 512;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sC = smem;
  uint8_t* sB = sC + C_BYTES;
  // #4 is issued at M = 128 whatever N is: with N = 64 the upper half of its A operand falls on the x tile that follows
  // B in shared memory (valid memory, finite or not: those accumulator rows are never read)
  uint8_t* sX = sB + B_BYTES;
  uint8_t* sM = sX + X_BYTES;
  uint8_t* sS = sM + M_BYTES;
  float* s_cs = reinterpret_cast<float*>(sS + S_BYTES);     // [128] inclusive cumulative log-decay
  float* s_warp = s_cs + Q;                                  // [4] warp totals of the scan
  float* s_g = s_warp + 4;                                   // [128] off-diagonal weights g_off of the chunk
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_g + Q);
  uint64_t* bar_load = bars;       // C, B, x of the current chunk have landed
  uint64_t* bar_g = bars + 1;      // #1 done
  uint64_t* bar_y = bars + 2;      // #2, #3 and #4 done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (status_poisoned(p.status)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x;
  const int b = bh / p.H, h = bh % p.H;
  const int hb = h / (p.H / p.Hb);

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_g, 1);
    mbar_init(bar_y, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  auto load_chunk = [&](int c) {
    const int row0 = b * p.L + c * Q;
    mbar_arrive_expect_tx(bar_load, C_BYTES + B_BYTES + X_BYTES);
    for (int s = 0; s < NSN; ++s) {
      tma_load_3d(sC + s * Q * 128, &tmC, bar_load, s * 64, row0, hb);
      tma_load_3d(sB + s * Q * 128, &tmB, bar_load, s * 64, row0, hb);
    }
    for (int s = 0; s < NSP; ++s) tma_load_3d(sX + s * Q * 128, &tmX, bar_load, s * 64, row0, h);
  };

  // ---- initial state: fp32 into tensor memory, bf16 into shared memory
  const bool has_init = p.init_state != nullptr;
  if (has_init && tid < N) {
    const float* src = p.init_state + ((long long)bh * N + tid) * P;
    uint8_t* srow = sS + tid * 128;
#pragma unroll
    for (int cblk = 0; cblk < P / 32; ++cblk) {
      uint32_t v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(src[cblk * 32 + i]);
      tmem_st_32x32b_x32(tmem_base + lane_off + S_COL + cblk * 32, v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = cblk * 32 + j * 8;
        const uint4 u = make_uint4(pack_bf16x2(src[col], src[col + 1]), pack_bf16x2(src[col + 2], src[col + 3]),
                                   pack_bf16x2(src[col + 4], src[col + 5]), pack_bf16x2(src[col + 6], src[col + 7]));
        *reinterpret_cast<uint4*>(srow + (col / 64) * (N * 128) + ((((col % 64) / 8) ^ (tid & 7)) << 4)) = u;
      }
    }
    tmem_st_wait();
  }
  if (tid == 0) load_chunk(0);
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t idesc_g = make_idesc(FMT_BF16, FMT_BF16, 0, 0, 128, 128);   // C B^T
  const uint32_t idesc_y = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, P);     // M x and C S: B operand MN-major
  const uint32_t idesc_s = make_idesc(FMT_BF16, FMT_BF16, 1, 1, 128, P);     // (B o w)^T x: both MN-major
  const uint32_t ca = smem_u32(sC), ba = smem_u32(sB), xa = smem_u32(sX), ma = smem_u32(sM), sa = smem_u32(sS);

  for (int c = 0; c < p.nchunks; ++c) {
    const bool have_state = has_init || c > 0;
    cta_wait(bar_load, c & 1, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
    if (tid == 32 && c + 1 < p.nchunks) {
      // the operand buffers are single (two CTAs share an SM instead): the next chunk's loads can only be issued when
      // this chunk's products are done, so at least have their tiles waiting in L2 by then
      const int row1 = b * p.L + (c + 1) * Q;
      for (int s = 0; s < NSN; ++s) {
        tma_prefetch_3d(&tmC, s * 64, row1, hb);
        tma_prefetch_3d(&tmB, s * 64, row1, hb);
      }
      for (int s = 0; s < NSP; ++s) tma_prefetch_3d(&tmX, s * 64, row1, h);
    }
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < N / 16; ++ks) {   // #1: G = C B^T
        const uint64_t ad = make_smem_desc_sw128(ca + (ks / 4) * (Q * 128) + (ks % 4) * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(ba + (ks / 4) * (Q * 128) + (ks % 4) * 32, 16, 1024);
        tc_mma_f16(tmem_base + G_COL, ad, bd, idesc_g, ks != 0);
      }
      tc_commit(bar_g);
    }
    __syncwarp();

    // ---- cumulative log-decay of the chunk (overlaps the two products above)
    const long long t_glob = ((long long)b * p.L + c * Q + tid) * p.H + h;
    float la = p.log_a[t_glob];
    const float goff = p.g_off[t_glob], gdiag = p.g_diag[t_glob];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, la, s);
      if (lane >= s) la += up;
    }
    if (lane == 31) s_warp[warp] = la;
    s_g[tid] = goff;
    __syncthreads();
    float cs = la;
    for (int w = 0; w < warp; ++w) cs += s_warp[w];
    const float cs_end = s_warp[0] + s_warp[1] + s_warp[2] + s_warp[3];
    s_cs[tid] = cs;
    __syncthreads();

    cta_wait(bar_g, c & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();

    // ---- B rows scaled in place by exp(cs_end - cs_j) * g_off[j]: the A operand of #4 (B is no longer needed by #1)
    {
      const float wj = __expf(cs_end - cs) * goff;
#pragma unroll
      for (int s = 0; s < NSN; ++s) {
        uint4* row = reinterpret_cast<uint4*>(sB + s * Q * 128 + tid * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 u = row[j];
          float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
          row[j] = make_uint4(pack_bf16x2(a0.x * wj, a0.y * wj), pack_bf16x2(a1.x * wj, a1.y * wj),
                              pack_bf16x2(a2.x * wj, a2.y * wj), pack_bf16x2(a3.x * wj, a3.y * wj));
        }
      }
    }
    // ---- the state in tensor memory decays over the whole chunk before #4 adds to it
    if (have_state && tid < N) {
      const float dec = __expf(cs_end);
#pragma unroll
      for (int cblk = 0; cblk < P / 32; ++cblk) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_off + S_COL + cblk * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * dec);
        tmem_st_32x32b_x32(tmem_base + lane_off + S_COL + cblk * 32, v);
      }
      tmem_st_wait();
    }
    // ---- M = G o decay mask o weights, row tid, written K-major (two 64-column spans, 128-byte swizzle)
    {
      uint8_t* mrow = sM + tid * 128;
#pragma unroll
      for (int cblk = 0; cblk < 4; ++cblk) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_off + G_COL + cblk * 32, v);
        tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int j = cblk * 32 + i;
          float m = 0.f;
          if (j < tid) m = __expf(cs - s_cs[j]) * s_g[j];
          else if (j == tid) m = gdiag;
          e[i] = __uint_as_float(v[i]) * m;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int col = cblk * 32 + k * 8;
          const uint4 u = make_uint4(pack_bf16x2(e[8 * k], e[8 * k + 1]), pack_bf16x2(e[8 * k + 2], e[8 * k + 3]),
                                     pack_bf16x2(e[8 * k + 4], e[8 * k + 5]), pack_bf16x2(e[8 * k + 6], e[8 * k + 7]));
          *reinterpret_cast<uint4*>(mrow + (col / 64) * (Q * 128) + ((((col % 64) / 8) ^ (tid & 7)) << 4)) = u;
        }
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < Q / 16; ++ks) {   // #2: Y = M x
        const uint64_t ad = make_smem_desc_sw128(ma + (ks / 4) * (Q * 128) + (ks % 4) * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(xa + ks * 2048, Q * 128, 1024);
        tc_mma_f16(tmem_base + Y_COL, ad, bd, idesc_y, ks != 0);
      }
      if (have_state) {
#pragma unroll
        for (int ks = 0; ks < N / 16; ++ks) {   // #3: Z = C S_prev (into the columns G occupied)
          const uint64_t ad = make_smem_desc_sw128(ca + (ks / 4) * (Q * 128) + (ks % 4) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sa + ks * 2048, N * 128, 1024);
          tc_mma_f16(tmem_base + Z_COL, ad, bd, idesc_y, ks != 0);
        }
      }
#pragma unroll
      for (int ks = 0; ks < Q / 16; ++ks) {   // #4: S += (B o w)^T x
        const uint64_t ad = make_smem_desc_sw128(ba + ks * 2048, Q * 128, 1024);
        const uint64_t bd = make_smem_desc_sw128(xa + ks * 2048, Q * 128, 1024);
        tc_mma_f16(tmem_base + S_COL, ad, bd, idesc_s, (have_state || ks != 0) ? 1u : 0u);
      }
      tc_commit(bar_y);
    }
    __syncwarp();
    cta_wait(bar_y, c & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();
    if (tid == 0 && c + 1 < p.nchunks) load_chunk(c + 1);   // every operand buffer of this chunk is free now

    // ---- epilogue: y_i = Y_i + exp(cs_i) Z_i
    {
      const float ei = __expf(cs);
      __nv_bfloat16* yrow = p.y + (((long long)b * p.L + c * Q + tid) * p.H + h) * P;
#pragma unroll
      for (int cblk = 0; cblk < P / 32; ++cblk) {
        uint32_t vy[32], vz[32];
        tmem_ld_32x32b_x32(tmem_base + lane_off + Y_COL + cblk * 32, vy);
        if (have_state) tmem_ld_32x32b_x32(tmem_base + lane_off + Z_COL + cblk * 32, vz);
        tmem_ld_wait();
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(vy[i]) + (have_state ? ei * __uint_as_float(vz[i]) : 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          reinterpret_cast<uint4*>(yrow + cblk * 32)[j] =
              make_uint4(pack_bf16x2(o[8 * j], o[8 * j + 1]), pack_bf16x2(o[8 * j + 2], o[8 * j + 3]),
                         pack_bf16x2(o[8 * j + 4], o[8 * j + 5]), pack_bf16x2(o[8 * j + 6], o[8 * j + 7]));
      }
    }
    // ---- bf16 copy of the new state for #3 of the next chunk; after the last chunk the fp32 state goes to memory
    if (tid < N) {
      const bool last = c + 1 == p.nchunks;
      uint8_t* srow = sS + tid * 128;
      float* fin = (last && p.final_state) ? p.final_state + ((long long)bh * N + tid) * P : nullptr;
      float* cst = p.chunk_states ? p.chunk_states + (((long long)bh * p.nchunks + c) * N + tid) * P : nullptr;
#pragma unroll
      for (int cblk = 0; cblk < P / 32; ++cblk) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_off + S_COL + cblk * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          float* dst = which == 0 ? fin : cst;
          if (!dst) continue;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + cblk * 32 + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                          __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        }
        if (!last) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int col = cblk * 32 + j * 8;
            const uint4 u = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                                       pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                                       pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                                       pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
            *reinterpret_cast<uint4*>(srow + (col / 64) * (N * 128) + ((((col % 64) / 8) ^ (tid & 7)) << 4)) = u;
          }
        }
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
  }

  if (*abort_flag && tid == 0) {  // let loads still in flight land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int N, int P>
void launch(const SsdArgs& a) {
  constexpr int Q = 128;
  const int smem = 2 * (N / 64) * Q * 128 + (P / 64) * Q * 128 + 2 * Q * 128 + (P / 64) * N * 128 + (2 * Q + 4) * 4 + 64 + 1024;
  // rows of x / B / C are (batch, time) pairs: batch stride = L * (time stride), so (b, t) folds into one coordinate
  CUtensorMap tx = make_tmap_3d(a.x, TmapDtype::BF16, (uint64_t)P, (uint64_t)a.batch * a.L, (uint64_t)a.H, (uint64_t)a.H * P * 2,
                                (uint64_t)P * 2, 64, Q, true);
  CUtensorMap tb = make_tmap_3d(a.B, TmapDtype::BF16, (uint64_t)N, (uint64_t)a.batch * a.L, (uint64_t)a.Hb, (uint64_t)a.Hb * N * 2,
                                (uint64_t)N * 2, 64, Q, true);
  CUtensorMap tc = make_tmap_3d(a.C, TmapDtype::BF16, (uint64_t)N, (uint64_t)a.batch * a.L, (uint64_t)a.Hb, (uint64_t)a.Hb * N * 2,
                                (uint64_t)N * 2, 64, Q, true);
  auto kern = ssd_fwd_kernel<N, P>;
  static PerDeviceOnce cfg;
  int dev = 0;
  if (cfg.pending(&dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) throw std::runtime_error(std::string("ssd: cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    cfg.done(dev);
  }
  SsdParams p;
  p.L = a.L; p.H = a.H; p.Hb = a.Hb; p.nchunks = a.L / Q;
  p.log_a = a.log_a; p.g_off = a.g_off; p.g_diag = a.g_diag;
  p.y = reinterpret_cast<__nv_bfloat16*>(a.y);
  p.init_state = a.init_state; p.final_state = a.final_state; p.chunk_states = a.chunk_states; p.status = a.status;
  kern<<<a.batch * a.H, 128, smem, a.stream>>>(tx, tb, tc, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("ssd launch: ") + cudaGetErrorString(e));
}

}  // namespace

bool ssd_fwd_supported(int L, int H, int Hb, int N, int P) {
  return L > 0 && L % 128 == 0 && (N == 64 || N == 128) && (P == 64 || P == 128) && Hb > 0 && H % Hb == 0;
}

void ssd_fwd_sm100(const SsdArgs& a) {
  if (!ssd_fwd_supported(a.L, a.H, a.Hb, a.N, a.P)) throw std::runtime_error("ssd: unsupported shape (L % 128, N and P in {64, 128})");
  if (a.N == 64 && a.P == 64) launch<64, 64>(a);
  else if (a.N == 64) launch<64, 128>(a);
  else if (a.P == 64) launch<128, 64>(a);
  else launch<128, 128>(a);
}

}  // namespace b200
