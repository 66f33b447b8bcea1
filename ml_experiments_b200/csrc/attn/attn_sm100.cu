// Flash attention forward / backward for sm_100a: every product runs on tcgen05.mma with the
// accumulators in tensor memory, operands are staged by TMA into 128B-swizzled shared memory.
//
// Masking model (the one the GPT trainers need): causal, restricted to the query's document
// (per-token doc_start / doc_end), and a sliding window counted in 128-token blocks.
//
// forward  : one CTA = 128 queries x one head, key/value tiles of 64; S = Q·Kᵀ (K-major operands),
//            P staged in shared memory, O_part = P·V with V consumed MN-major straight from its
//            [token][d] tile. Two CTAs per SM so one CTA's softmax overlaps the other's MMAs.
// backward : one CTA = 128 keys x one head, looping over 64-query tiles; Sᵀ = K·Qᵀ and dPᵀ = V·dOᵀ are
//            formed transposed so that Pᵀ / dSᵀ rows are owned by one thread each and feed
//            dV += Pᵀ·dO, dK += dSᵀ·Q (TMEM-resident accumulators) and dQᵀ = Kᵀ·dSᵀ, which is
//            added into an fp32 dQ buffer by TMA reduce-add.
#include "../common/per_device.h"
#include "attn.h"

#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace b200 {
namespace {

struct KP {
  int T, H;
  float sl2;    // softmax scale * log2(e)
  float scale;  // softmax scale
  int window_blocks;
  const int* doc_start;
  const int* doc_end;
  __nv_bfloat16* o; long long ld_o;
  __nv_bfloat16* dk; long long ld_dk;
  __nv_bfloat16* dv; long long ld_dv;
  float* lse;
  const float* delta;
  int* status;
};

// Bounded wait shared by all threads of a CTA: once any thread times out, `*abort_flag` makes every later
// wait in the CTA return at once, so control flow stays convergent and the kernel terminates.
__device__ __forceinline__ void cta_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                         int code) {
  if (*abort_flag) return;
  if (!mbar_wait(bar, parity, status, code)) *abort_flag = 1;
}

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
// The output accumulator stays in tensor memory across key tiles (PV MMAs accumulate in place). The running
// maximum is only raised when a tile exceeds it by more than 2^8, so the TMEM read-scale-write of the accumulator
// is rare; probabilities are then at most 2^8, well inside bf16 / fp32 range.
template <int D>
__global__ void __launch_bounds__(128, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const KP p) {
  constexpr int NS = D / 64;  // 128-byte spans along the head dimension
  constexpr int BQ = 128, BKV = 64;
  constexpr int Q_BYTES = NS * BQ * 128;
  constexpr int KV_BYTES = NS * BKV * 128;
  constexpr int P_BYTES = BQ * 128;
  constexpr uint32_t S_COL = 0, O_COL = 64;
  constexpr uint32_t TMEM_COLS = (64 + D) <= 128 ? 128 : 256;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;           // 2 buffers
  uint8_t* sV = sK + 2 * KV_BYTES;      // 2 buffers
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* bar_q = bars;
  uint64_t* bar_k = bars + 1;  // [2]
  uint64_t* bar_v = bars + 3;  // [2]
  uint64_t* bar_s = bars + 5;
  uint64_t* bar_o = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (status_poisoned(p.status)) return;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;  // late (long-context) tiles first
  const int h = blockIdx.y;
  const int q0 = qb * BQ;
  const int q = q0 + tid;
  const bool row_ok = q < p.T;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&bar_k[i], 1); mbar_init(&bar_v[i], 1); }
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
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

  const int ds = row_ok ? p.doc_start[q] : q;
  const int ds_last = p.doc_start[min(q0 + BQ, p.T) - 1];
  int kv_lo = p.doc_start[q0] & ~(BKV - 1);
  if (p.window_blocks > 0) kv_lo = max(kv_lo, (qb - p.window_blocks + 1) * 128);
  kv_lo = max(kv_lo, 0);
  const int kv_hi = min(q0 + BQ, p.T);
  const int nblk = (kv_hi - kv_lo + BKV - 1) / BKV;

  const uint32_t idesc_s = make_idesc(FMT_BF16, FMT_BF16, 0, 0, 128, BKV);
  const uint32_t idesc_o = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, D);

  auto load_k = [&](int j) {
    const int b = j & 1;
    mbar_arrive_expect_tx(&bar_k[b], KV_BYTES);
    for (int s = 0; s < NS; ++s) tma_load_3d(sK + b * KV_BYTES + s * BKV * 128, &tmK, &bar_k[b], s * 64, kv_lo + j * BKV, h);
  };
  auto load_v = [&](int j) {
    const int b = j & 1;
    mbar_arrive_expect_tx(&bar_v[b], KV_BYTES);
    for (int s = 0; s < NS; ++s) tma_load_3d(sV + b * KV_BYTES + s * BKV * 128, &tmV, &bar_v[b], s * 64, kv_lo + j * BKV, h);
  };
  auto issue_s = [&](int j) {
    const int b = j & 1;
    cta_wait(&bar_k[b], (j >> 1) & 1, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
    tc_fence_after_sync();
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + b * KV_BYTES);
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint64_t ad = make_smem_desc_sw128(qa + (ks / 4) * (BQ * 128) + (ks % 4) * 32, 16, 1024);
      const uint64_t bd = make_smem_desc_sw128(ka + (ks / 4) * (BKV * 128) + (ks % 4) * 32, 16, 1024);
      tc_mma_f16(tmem_base + S_COL, ad, bd, idesc_s, ks != 0);
    }
    tc_commit(bar_s);
  };

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_q, Q_BYTES);
    for (int s = 0; s < NS; ++s) tma_load_3d(sQ + s * BQ * 128, &tmQ, bar_q, s * 64, q0, h);
    load_k(0);
    load_v(0);
    if (nblk > 1) load_k(1);
    cta_wait(bar_q, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
    issue_s(0);
  }
  __syncwarp();

  float m_run = -INFINITY, l = 0.f;

  for (int jb = 0; jb < nblk; ++jb) {
    const int buf = jb & 1;
    const int kvb = kv_lo + jb * BKV;
    cta_wait(bar_s, jb & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);  // S(jb) done => PV(jb-1) done as well
    tc_fence_after_sync();
    if (tid == 0 && jb + 1 < nblk) load_v(jb + 1);
    __syncwarp();

    const bool need_mask = (kvb + BKV - 1 > q0) || (kvb < ds_last);
    float sc[BKV];
    float mblk = -INFINITY;
#pragma unroll
    for (int c = 0; c < BKV / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + S_COL + c * 32, v);
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kvb + c * 32 + i;
          const float s = (kv >= ds && kv <= q) ? __uint_as_float(v[i]) * p.sl2 : -INFINITY;
          sc[c * 32 + i] = s;
          mblk = fmaxf(mblk, s);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(v[i]) * p.sl2;
          sc[c * 32 + i] = s;
          mblk = fmaxf(mblk, s);
        }
      }
    }
    float alpha = 1.f;
    bool rescale = false;
    if (mblk > m_run + 8.f) {
      alpha = exp2f(m_run - mblk);  // m_run == -inf gives 0
      m_run = mblk;
      rescale = jb > 0;
    }
    const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
    float lsum = 0.f;
    uint8_t* prow = sP + tid * 128;
#pragma unroll
    for (int j = 0; j < BKV / 8; ++j) {
      float e[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        e[i] = exp2f(sc[8 * j + i] - m_use);
        lsum += e[i];
      }
      uint4 u = make_uint4(pack_bf16x2(e[0], e[1]), pack_bf16x2(e[2], e[3]), pack_bf16x2(e[4], e[5]),
                           pack_bf16x2(e[6], e[7]));
      *reinterpret_cast<uint4*>(prow + ((j ^ (tid & 7)) << 4)) = u;
    }
    l = l * alpha + lsum;
    if (__any_sync(0xffffffffu, rescale)) {  // rare: bring this warp's accumulator rows to the new maximum
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_off + O_COL + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
        tmem_st_32x32b_x32(tmem_base + lane_off + O_COL + c * 32, v);
      }
      tmem_st_wait();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      cta_wait(&bar_v[buf], (jb >> 1) & 1, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      tc_fence_after_sync();
      const uint32_t pa = smem_u32(sP), va = smem_u32(sV + buf * KV_BYTES);
#pragma unroll
      for (int ks = 0; ks < BKV / 16; ++ks) {
        const uint64_t ad = make_smem_desc_sw128(pa + ks * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(va + ks * 2048, BKV * 128, 1024);
        tc_mma_f16(tmem_base + O_COL, ad, bd, idesc_o, (jb | ks) != 0);
      }
      if (jb + 1 < nblk) {
        issue_s(jb + 1);
        if (jb + 2 < nblk) load_k(jb + 2);  // its buffer held K(jb), which S(jb) has finished reading
      } else {
        tc_commit(bar_o);
      }
    }
    __syncwarp();
  }

  cta_wait(bar_o, 0, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
  tc_fence_after_sync();
  {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* orow = p.o + (long long)q * p.ld_o + h * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + O_COL + c * 32, v);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 u = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]) * inv, __uint_as_float(v[8 * j + 1]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * j + 2]) * inv, __uint_as_float(v[8 * j + 3]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * j + 4]) * inv, __uint_as_float(v[8 * j + 5]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * j + 6]) * inv, __uint_as_float(v[8 * j + 7]) * inv));
          reinterpret_cast<uint4*>(orow + c * 32)[j] = u;
        }
      }
    }
    if (row_ok) p.lse[(long long)h * p.T + q] = m_run + log2f(l);
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

// ------------------------------------------------------------------------------------------------
// delta[h][t] = sum_d O[t,h,d] * dO[t,h,d]
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ld_o,
                                  const __nv_bfloat16* __restrict__ d_o, long long ld_do, float* __restrict__ delta,
                                  int T, int H) {
  // one warp per (t, h)
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * H) return;
  const int t = gw / H, h = gw % H;
  const __nv_bfloat16* a = o + (long long)t * ld_o + h * D;
  const __nv_bfloat16* b = d_o + (long long)t * ld_do + h * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + i));
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[(long long)h * T + t] = acc;
}

// Same with 16-byte loads: D / 8 adjacent lanes own a row, a warp covers 32 / (D / 8) rows (needs 16-byte aligned rows).
template <int D>
__global__ void attn_delta_vec_kernel(const __nv_bfloat16* __restrict__ o, long long ld_o,
                                      const __nv_bfloat16* __restrict__ d_o, long long ld_do,
                                      float* __restrict__ delta, int T, int H) {
  constexpr int LPR = D / 8;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
  const int sub = threadIdx.x % LPR;
  float acc = 0.f;
  int t = 0, h = 0;
  const bool on = row < (long long)T * H;
  if (on) {
    t = (int)(row / H), h = (int)(row % H);
    const uint4 ua = *reinterpret_cast<const uint4*>(o + (long long)t * ld_o + h * D + sub * 8);
    const uint4 ub = *reinterpret_cast<const uint4*>(d_o + (long long)t * ld_do + h * D + sub * 8);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
      acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
    }
  }
#pragma unroll
  for (int s = LPR / 2; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (on && sub == 0) delta[(long long)h * T + t] = acc;
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
// 8 warps: warps w and w+4 share TMEM lane quarter (w & 3) and split the columns of every accumulator in halves.
template <int D>
__global__ void __launch_bounds__(256, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, const KP p) {
  constexpr int NS = D / 64;
  constexpr int BKV = 128, BQ = 64;
  constexpr int KV_BYTES = NS * BKV * 128;  // K or V tile
  constexpr int Q_BYTES = NS * BQ * 128;    // Q or dO tile
  constexpr int PT_BYTES = BKV * 128;       // Pᵀ or dSᵀ: 128 key rows x 64 queries
  constexpr int DQ_BYTES = BQ * D * 4;      // fp32 staging of one dQ tile
  constexpr uint32_t ST_COL = 0, DPT_COL = 64, DV_COL = 128, DK_COL = 128 + D, DQT_COL = 128 + 2 * D;
  constexpr uint32_t TMEM_COLS = (128 + 2 * D + 64) <= 256 ? 256 : 512;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KV_BYTES;
  constexpr int NQB = 3;              // Q / dO buffers
  uint8_t* sQ = sV + KV_BYTES;
  uint8_t* sdO = sQ + NQB * Q_BYTES;
  uint8_t* sPT = sdO + NQB * Q_BYTES;
  uint8_t* sdST = sPT + PT_BYTES;
  float* sdQ = reinterpret_cast<float*>(sdST + PT_BYTES);
  float2* s_ld_all = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(sdQ) + DQ_BYTES);  // [2][64] {lse, delta}, double-buffered over query tiles
  int* s_ds_all = reinterpret_cast<int*>(s_ld_all + 2 * BQ);      // [2][64] document start of each query
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_ds_all + 2 * BQ);
  uint64_t* bar_kv = bars;
  uint64_t* bar_q = bars + 1;  // [3]
  uint64_t* bar_m1 = bars + 4;   // S / dP of a tile are in TMEM
  uint64_t* bar_m2 = bars + 5;   // dV / dK of a tile are accumulated: its P / dS staging and its Q / dO buffer are free
  uint64_t* bar_dq = bars + 6;   // dQ of a tile is in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (status_poisoned(p.status)) return;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int quarter = warp & 3;
  const int half = warp >> 2;
  const int r = quarter * 32 + lane;  // accumulator row owned by this thread
  const int jb = blockIdx.x;
  const int h = blockIdx.y;
  const int kv0 = jb * BKV;
  const int kv = kv0 + r;
  // The single-thread issue work is spread over four warps so that no warp carries all of it on top of its share of the
  // exponentials: S / dP products, the products that follow the exponentials, the dQ bulk reductions, the Q / dO loads.
  const bool issue_sdp = tid == 0, issue_grad = tid == 32, issue_red = tid == 64, issue_load = tid == 96;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(&bar_q[0], 1);
    mbar_init(&bar_q[1], 1);
    mbar_init(&bar_q[2], 1);
    mbar_init(bar_m1, 1);
    mbar_init(bar_m2, 1);
    mbar_init(bar_dq, 1);
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
  const uint32_t lane_off = uint32_t(quarter * 32) << 16;

  // query range that can see any key of this tile
  const int last_kv = min(kv0 + BKV, p.T) - 1;
  int q_hi = p.doc_end[last_kv];
  if (p.window_blocks > 0) q_hi = min(q_hi, (jb + p.window_blocks) * 128);
  q_hi = min(q_hi, p.T);
  const int q_lo = kv0;
  const int ntile = (q_hi - q_lo + BQ - 1) / BQ;

  const uint32_t idesc_st = make_idesc(FMT_BF16, FMT_BF16, 0, 0, 128, BQ);   // K·Qᵀ, V·dOᵀ
  const uint32_t idesc_dv = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, D);    // Pᵀ·dO, dSᵀ·Q   (B MN-major)
  const uint32_t idesc_dq = make_idesc(FMT_BF16, FMT_BF16, 1, 1, 128, BQ);   // Kᵀ·dSᵀ         (A, B MN-major)

  // One thread issues every TMA load and MMA; the tensor pipe runs them in issue order. Per query tile:
  //   S, dP of tile it+1   issued as soon as every thread has copied tile it's S / dP out of TMEM: they run while the CTA
  //                        does the exponentials of tile it;
  //   dQ of tile it        issued right after the exponentials, on its own barrier: the CTA stages and reduces dQ while
  //   dV, dK of tile it    are still accumulating; their barrier is only waited for in the next iteration, before the
  //                        P / dS staging buffers are overwritten.
  // Q / dO tiles are triple-buffered so that the load of tile it+2 never waits for a buffer.
  auto issue_s_dp = [&](int buf) {
    const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
    const uint32_t qa = smem_u32(sQ + buf * Q_BYTES), doa = smem_u32(sdO + buf * Q_BYTES);
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint64_t ad = make_smem_desc_sw128(ka + (ks / 4) * (BKV * 128) + (ks % 4) * 32, 16, 1024);
      const uint64_t bd = make_smem_desc_sw128(qa + (ks / 4) * (BQ * 128) + (ks % 4) * 32, 16, 1024);
      tc_mma_f16(tmem_base + ST_COL, ad, bd, idesc_st, ks != 0);
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const uint64_t ad = make_smem_desc_sw128(va + (ks / 4) * (BKV * 128) + (ks % 4) * 32, 16, 1024);
      const uint64_t bd = make_smem_desc_sw128(doa + (ks / 4) * (BQ * 128) + (ks % 4) * 32, 16, 1024);
      tc_mma_f16(tmem_base + DPT_COL, ad, bd, idesc_st, ks != 0);
    }
    tc_commit(bar_m1);
  };
  auto load_q_do = [&](int buf, int q0) {
    mbar_arrive_expect_tx(&bar_q[buf], 2 * Q_BYTES);
    for (int s = 0; s < NS; ++s) {
      tma_load_3d(sQ + buf * Q_BYTES + s * BQ * 128, &tmQ, &bar_q[buf], s * 64, q0, h);
      tma_load_3d(sdO + buf * Q_BYTES + s * BQ * 128, &tmdO, &bar_q[buf], s * 64, q0, h);
    }
  };

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_kv, 2 * KV_BYTES);
    for (int s = 0; s < NS; ++s) {
      tma_load_3d(sK + s * BKV * 128, &tmK, bar_kv, s * 64, kv0, h);
      tma_load_3d(sV + s * BKV * 128, &tmV, bar_kv, s * 64, kv0, h);
    }
    if (ntile > 0) {
      load_q_do(0, q_lo);
      if (ntile > 1) load_q_do(1, q_lo + BQ);
      if (ntile > 2) load_q_do(2, q_lo + 2 * BQ);
      cta_wait(bar_kv, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      cta_wait(&bar_q[0], 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      tc_fence_after_sync();
      issue_s_dp(0);
    }
  }

  // per-query scalars (lse, delta, document start) of the next tile are fetched one iteration ahead
  float2 nxt_ld = make_float2(INFINITY, 0.f);
  int nxt_ds = 0x7fffffff;
  auto fetch_scalars = [&](int q0) {
    const int qq = q0 + tid;
    const bool okq = qq < p.T;
    nxt_ld = make_float2(okq ? p.lse[(long long)h * p.T + qq] : INFINITY, okq ? p.delta[(long long)h * p.T + qq] : 0.f);
    nxt_ds = okq ? p.doc_start[qq] : 0x7fffffff;
  };
  if (tid < BQ && ntile > 0) {
    fetch_scalars(q_lo);
    s_ld_all[tid] = nxt_ld;
    s_ds_all[tid] = nxt_ds;
  }

  for (int it = 0; it < ntile; ++it) {
    const int buf = it % NQB;
    const int qt0 = q_lo + it * BQ;
    const float2* s_ld = s_ld_all + (it & 1) * BQ;
    const int* s_ds = s_ds_all + (it & 1) * BQ;
    if (tid < BQ && it + 1 < ntile) fetch_scalars(qt0 + BQ);  // loads stay in flight until the stores at the end of the iteration
    __syncthreads();  // s_ld / s_ds of this tile visible (written in the prologue or at the end of the previous iteration)
    cta_wait(bar_m1, it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();
    uint32_t sv[32], dv_[32];
    tmem_ld_32x32b_x32(tmem_base + lane_off + ST_COL + half * 32, sv);
    tmem_ld_32x32b_x32(tmem_base + lane_off + DPT_COL + half * 32, dv_);
    tmem_ld_wait();
    tc_fence_before_sync();
    __syncthreads();  // every thread holds its S / dP values: the TMEM columns may be overwritten
    if (issue_sdp && it + 1 < ntile) {
      cta_wait(&bar_q[(it + 1) % NQB], ((it + 1) / NQB) & 1, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      tc_fence_after_sync();
      issue_s_dp((it + 1) % NQB);
    }
    if (it > 0) {  // dV / dK of the previous tile: frees the P / dS staging and that tile's Q / dO buffer
      cta_wait(bar_m2, (it - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
      tc_fence_after_sync();
      if (issue_load && it + 2 < ntile) load_q_do((it + 2) % NQB, qt0 + 2 * BQ);
    }

    // masks are needed only where the tile touches the causal diagonal, a document boundary or the sequence end
    const bool need_mask = (qt0 < kv0 + BKV) || (s_ds[BQ - 1] > kv0) || (kv0 + BKV > p.T) || (qt0 + BQ > p.T);
    {
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const int qi = half * 32 + i;
        const float2 ld0 = s_ld[qi], ld1 = s_ld[qi + 1];
        float p0 = exp2f(fmaf(__uint_as_float(sv[i]), p.sl2, -ld0.x));
        float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), p.sl2, -ld1.x));
        if (need_mask) {
          const int qq = qt0 + qi;
          if (!((qq >= kv) && (kv >= s_ds[qi]) && (kv < p.T))) p0 = 0.f;
          if (!((qq + 1 >= kv) && (kv >= s_ds[qi + 1]) && (kv < p.T))) p1 = 0.f;
        }
        pp[i >> 1] = pack_bf16x2(p0, p1);
        dd[i >> 1] = pack_bf16x2(p0 * (__uint_as_float(dv_[i]) - ld0.y), p1 * (__uint_as_float(dv_[i + 1]) - ld1.y));
      }
      uint8_t* prow = sPT + r * 128;
      uint8_t* drow = sdST + r * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        *reinterpret_cast<uint4*>(prow + (((half * 4 + j) ^ (r & 7)) << 4)) = make_uint4(pp[4 * j], pp[4 * j + 1], pp[4 * j + 2], pp[4 * j + 3]);
        *reinterpret_cast<uint4*>(drow + (((half * 4 + j) ^ (r & 7)) << 4)) = make_uint4(dd[4 * j], dd[4 * j + 1], dd[4 * j + 2], dd[4 * j + 3]);
      }
    }
    if (issue_red) tma_store_wait_read<0>();  // the previous tile's reduce-add has drained the dQ staging buffer; the barrier
                                              // below orders this before every thread's staging stores of this tile
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (issue_grad) {
      tc_fence_after_sync();
      const uint32_t pa = smem_u32(sPT), dsa = smem_u32(sdST), ka = smem_u32(sK);
      const uint32_t qa = smem_u32(sQ + buf * Q_BYTES), doa = smem_u32(sdO + buf * Q_BYTES);
#pragma unroll
      for (int ks = 0; ks < BKV / 16; ++ks) {  // dQᵀ = Kᵀ · dSᵀ
        const uint64_t ad = make_smem_desc_sw128(ka + ks * 2048, BKV * 128, 1024);
        const uint64_t bd = make_smem_desc_sw128(dsa + ks * 2048, BKV * 128, 1024);
        tc_mma_f16(tmem_base + DQT_COL, ad, bd, idesc_dq, ks != 0);
      }
      tc_commit(bar_dq);
#pragma unroll
      for (int ks = 0; ks < BQ / 16; ++ks) {  // dV += Pᵀ · dO
        const uint64_t ad = make_smem_desc_sw128(pa + ks * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(doa + ks * 2048, BQ * 128, 1024);
        tc_mma_f16(tmem_base + DV_COL, ad, bd, idesc_dv, (it | ks) != 0);
      }
#pragma unroll
      for (int ks = 0; ks < BQ / 16; ++ks) {  // dK += dSᵀ · Q
        const uint64_t ad = make_smem_desc_sw128(dsa + ks * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(qa + ks * 2048, BQ * 128, 1024);
        tc_mma_f16(tmem_base + DK_COL, ad, bd, idesc_dv, (it | ks) != 0);
      }
      tc_commit(bar_m2);
    }
    cta_wait(bar_dq, it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();
    // dQᵀ row (= head-dim index r), this warp's half of the query columns -> staging[q][r], then one bulk reduce-add
    // into the fp32 accumulator (reductions issued element by element from registers measured 25 % slower)
    if (r < D) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + DQT_COL + half * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) sdQ[(half * 32 + i) * D + r] = __uint_as_float(v[i]) * p.scale;
    }
    fence_proxy_async_smem();
    if (tid < BQ && it + 1 < ntile) {
      s_ld_all[((it + 1) & 1) * BQ + tid] = nxt_ld;
      s_ds_all[((it + 1) & 1) * BQ + tid] = nxt_ds;
    }
    tc_fence_before_sync();
    __syncthreads();  // dQ columns of TMEM are free for the next tile; the staged dQ tile is complete
    if (issue_red) {
      tma_reduce_add_3d(&tmdQ, sdQ, 0, qt0, h);
      tma_store_commit();
    }
  }

  // final: dV, dK rows; each warp writes its half of the head dimension
  if (ntile > 0) cta_wait(bar_m2, (ntile - 1) & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
  tc_fence_after_sync();
  if (ntile > 0) {
    __nv_bfloat16* dvrow = p.dv + (long long)kv * p.ld_dv + h * D + half * (D / 2);
    __nv_bfloat16* dkrow = p.dk + (long long)kv * p.ld_dk + h * D + half * (D / 2);
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + DV_COL + half * (D / 2) + c * 32, v);
      tmem_ld_wait();
      if (kv < p.T) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 u = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                               pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                               pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                               pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
          reinterpret_cast<uint4*>(dvrow + c * 32)[j] = u;
        }
      }
      tmem_ld_32x32b_x32(tmem_base + lane_off + DK_COL + half * (D / 2) + c * 32, v);
      tmem_ld_wait();
      if (kv < p.T) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 u = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]) * p.scale, __uint_as_float(v[8 * j + 1]) * p.scale),
                               pack_bf16x2(__uint_as_float(v[8 * j + 2]) * p.scale, __uint_as_float(v[8 * j + 3]) * p.scale),
                               pack_bf16x2(__uint_as_float(v[8 * j + 4]) * p.scale, __uint_as_float(v[8 * j + 5]) * p.scale),
                               pack_bf16x2(__uint_as_float(v[8 * j + 6]) * p.scale, __uint_as_float(v[8 * j + 7]) * p.scale));
          reinterpret_cast<uint4*>(dkrow + c * 32)[j] = u;
        }
      }
    }
  } else if (kv < p.T) {
    // no query tile attends this key tile: its gradients are zero (the caller does not pre-zero dk / dv)
    __nv_bfloat16* dvrow = p.dv + (long long)kv * p.ld_dv + h * D + half * (D / 2);
    __nv_bfloat16* dkrow = p.dk + (long long)kv * p.ld_dk + h * D + half * (D / 2);
#pragma unroll
    for (int j = 0; j < D / 16; ++j) {
      reinterpret_cast<uint4*>(dvrow)[j] = make_uint4(0u, 0u, 0u, 0u);
      reinterpret_cast<uint4*>(dkrow)[j] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (issue_red) tma_store_wait_all<0>();
  if (tid == 0) {
    if (*abort_flag) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

CUtensorMap qkv_map(const void* base, int T, int H, int D, long long ld, int rows) {
  return make_tmap_3d(base, TmapDtype::BF16, (uint64_t)D, (uint64_t)T, (uint64_t)H, (uint64_t)ld * 2, (uint64_t)D * 2, 64,
                      (uint32_t)rows, true);
}

KP make_kp(const AttnArgs& a) {
  KP p;
  p.T = a.T; p.H = a.H;
  p.scale = a.scale;
  p.sl2 = a.scale * 1.4426950408889634f;
  p.window_blocks = a.window_blocks;
  p.doc_start = a.doc_start; p.doc_end = a.doc_end;
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o); p.ld_o = a.ld_o;
  p.dk = reinterpret_cast<__nv_bfloat16*>(a.dk); p.ld_dk = a.ld_dk;
  p.dv = reinterpret_cast<__nv_bfloat16*>(a.dv); p.ld_dv = a.ld_dv;
  p.lse = a.lse; p.delta = a.delta;
  p.status = a.status;
  return p;
}

void check_common(const AttnArgs& a) {
  if (a.D != 64 && a.D != 128) throw std::runtime_error("attention: head_dim must be 64 or 128");
  if (a.T <= 0 || a.H <= 0) throw std::runtime_error("attention: empty problem");
  if (!a.doc_start || !a.doc_end) throw std::runtime_error("attention: doc_start / doc_end are required");
}

template <typename K>
void set_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) throw std::runtime_error(std::string("attention: cudaFuncSetAttribute: ") + cudaGetErrorString(e));
}

void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <int D>
void fwd_impl(const AttnArgs& a) {
  constexpr int NS = D / 64;
  // no alignment slack: the dynamic shared-memory window is declared 1024-byte aligned, and two CTAs must fit per SM
  const int smem = NS * 128 * 128 + 4 * NS * 64 * 128 + 128 * 128 + 96;
  CUtensorMap tq = qkv_map(a.q, a.T, a.H, D, a.ld_q, 128);
  CUtensorMap tk = qkv_map(a.k, a.T, a.H, D, a.ld_k, 64);
  CUtensorMap tv = qkv_map(a.v, a.T, a.H, D, a.ld_v, 64);
  auto kern = attn_fwd_kernel<D>;
  static PerDeviceOnce cfg;   // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  if (cfg.pending(&dev)) { set_smem(kern, smem); cfg.done(dev); }
  dim3 grid((a.T + 127) / 128, a.H);
  kern<<<grid, 128, smem, a.stream>>>(tq, tk, tv, make_kp(a));
  check_launch("attn_fwd launch");
}

template <int D>
void bwd_impl(const AttnArgs& a) {
  constexpr int NS = D / 64;
  const int smem = 2 * NS * 128 * 128 + 6 * NS * 64 * 128 + 2 * 128 * 128 + 64 * D * 4 + 6 * 64 * 4 + 96 + 1024;
  CUtensorMap tq = qkv_map(a.q, a.T, a.H, D, a.ld_q, 64);
  CUtensorMap tk = qkv_map(a.k, a.T, a.H, D, a.ld_k, 128);
  CUtensorMap tv = qkv_map(a.v, a.T, a.H, D, a.ld_v, 128);
  CUtensorMap tdo = qkv_map(a.d_o, a.T, a.H, D, a.ld_do, 64);
  CUtensorMap tdq = make_tmap_3d(a.dq_acc, TmapDtype::F32, (uint64_t)D, (uint64_t)a.T, (uint64_t)a.H,
                                 (uint64_t)a.ld_dq * 4, (uint64_t)D * 4, (uint32_t)D, 64, false);
  auto kern = attn_bwd_kernel<D>;
  static PerDeviceOnce cfg;   // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  if (cfg.pending(&dev)) { set_smem(kern, smem); cfg.done(dev); }
  dim3 grid((a.T + 127) / 128, a.H);
  kern<<<grid, 256, smem, a.stream>>>(tq, tk, tv, tdo, tdq, make_kp(a));
  check_launch("attn_bwd launch");
}

}  // namespace

void attn_fwd_sm100(const AttnArgs& a) {
  check_common(a);
  if (a.D == 128) fwd_impl<128>(a); else fwd_impl<64>(a);
}

void attn_delta_sm100(const AttnArgs& a) {
  check_common(a);
  const long long warps = (long long)a.T * a.H;
  const int threads = 256;
  const int blocks = (int)((warps * 32 + threads - 1) / threads);
  auto* o = reinterpret_cast<const __nv_bfloat16*>(a.o);
  auto* d_o = reinterpret_cast<const __nv_bfloat16*>(a.d_o);
  const bool aligned = (((uintptr_t)o | (uintptr_t)d_o) & 15) == 0 && a.ld_o % 8 == 0 && a.ld_do % 8 == 0;
  if (aligned) {
    const long long lanes = warps * (a.D / 8);
    const int vblocks = (int)((lanes + threads - 1) / threads);
    if (a.D == 128) attn_delta_vec_kernel<128><<<vblocks, threads, 0, a.stream>>>(o, a.ld_o, d_o, a.ld_do, a.delta, a.T, a.H);
    else            attn_delta_vec_kernel<64><<<vblocks, threads, 0, a.stream>>>(o, a.ld_o, d_o, a.ld_do, a.delta, a.T, a.H);
  } else if (a.D == 128) {
    attn_delta_kernel<128><<<blocks, threads, 0, a.stream>>>(o, a.ld_o, d_o, a.ld_do, a.delta, a.T, a.H);
  } else {
    attn_delta_kernel<64><<<blocks, threads, 0, a.stream>>>(o, a.ld_o, d_o, a.ld_do, a.delta, a.T, a.H);
  }
  check_launch("attn_delta launch");
}

void attn_bwd_sm100(const AttnArgs& a) {
  check_common(a);
  // dQᵀ = Kᵀ·dSᵀ puts the head dimension on the MMA M axis, always issued at M = 128. With head_dim 64 the upper 64
  // rows of the A operand fall on the V tile that follows K in shared memory; their accumulator rows are never read.
  if (a.D == 128) bwd_impl<128>(a); else bwd_impl<64>(a);
}

}  // namespace b200

// ------------------------------------------------------------------------------------------------
// Allocation-free entry point (see attn_noalloc.h): the delta scratch is a fixed array in the library image.
// ------------------------------------------------------------------------------------------------
#include "attn_noalloc.h"

static __device__ __align__(256) float g_noalloc_delta[B200_ATTN_NOALLOC_MAX_HT];

namespace {
thread_local std::string t_noalloc_error;
// Device address of the scratch array, per device ordinal. Two host threads that make the first call on one device
// both store the same value.
std::atomic<float*> g_noalloc_delta_addr[64];
}  // namespace

extern "C" const char* b200_attn_bwd_noalloc_error(void) { return t_noalloc_error.c_str(); }

extern "C" int b200_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                     const float* lse, float* dq_acc, void* dk, void* dv, const int* doc_start,
                                     const int* doc_end, int T, int H, int D, long long ld_q, long long ld_k,
                                     long long ld_v, long long ld_o, long long ld_do, long long ld_dq, long long ld_dk,
                                     long long ld_dv, float scale, int window_blocks, int* status,
                                     cudaStream_t stream) {
  try {
    if (!q || !k || !v || !o || !d_o || !lse || !dq_acc || !dk || !dv || !doc_start || !doc_end || T <= 0 || H <= 0) {
      t_noalloc_error = "null pointer or empty problem";
      return -1;
    }
    if (D != 128 && D != 64) {
      t_noalloc_error = "head_dim must be 64 or 128";
      return -1;
    }
    if ((long long)T * H > (long long)B200_ATTN_NOALLOC_MAX_HT) {
      t_noalloc_error = "H * T exceeds the built-in scratch (B200_ATTN_NOALLOC_MAX_HT floats)";
      return -2;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
      t_noalloc_error = "cannot determine the current device";
      return -3;
    }
    float* scratch = g_noalloc_delta_addr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
      // Once per device, with that device current: in host code the array's name is only a handle, the address a
      // kernel can use has to be asked for.
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_delta);
      if (e != cudaSuccess || ptr == nullptr) {
        t_noalloc_error = std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e);
        return -3;
      }
      scratch = static_cast<float*>(ptr);
      g_noalloc_delta_addr[dev].store(scratch, std::memory_order_release);
    }
    b200::AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.o = const_cast<void*>(o); a.d_o = d_o;
    a.dq_acc = dq_acc; a.dk = dk; a.dv = dv;
    a.lse = const_cast<float*>(lse);
    a.delta = scratch;
    a.doc_start = doc_start; a.doc_end = doc_end;
    a.T = T; a.H = H; a.D = D;
    a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v; a.ld_o = ld_o; a.ld_do = ld_do; a.ld_dq = ld_dq; a.ld_dk = ld_dk;
    a.ld_dv = ld_dv;
    a.scale = scale; a.window_blocks = window_blocks; a.status = status; a.stream = stream;
    b200::attn_delta_sm100(a);
    b200::attn_bwd_sm100(a);
    return 0;
  } catch (const std::exception& ex) {
    t_noalloc_error = ex.what();
    return -3;
  }
}
