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
  uint64_t* bar_kv = bars + 1;  // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;  // late (long-context) tiles first
  const int h = blockIdx.y;
  const int q0 = qb * BQ;
  const int q = q0 + tid;
  const bool row_ok = q < p.T;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
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
  int kv_lo = p.doc_start[q0] & ~(BKV - 1);
  if (p.window_blocks > 0) kv_lo = max(kv_lo, (qb - p.window_blocks + 1) * 128);
  kv_lo = max(kv_lo, 0);
  const int kv_hi = min(q0 + BQ, p.T);
  const int nblk = (kv_hi - kv_lo + BKV - 1) / BKV;

  const uint32_t idesc_s = make_idesc(FMT_BF16, FMT_BF16, 0, 0, 128, BKV);
  const uint32_t idesc_o = make_idesc(FMT_BF16, FMT_BF16, 0, 1, 128, D);

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_q, Q_BYTES);
    for (int s = 0; s < NS; ++s) tma_load_3d(sQ + s * BQ * 128, &tmQ, bar_q, s * 64, q0, h);
    mbar_arrive_expect_tx(&bar_kv[0], 2 * KV_BYTES);
    for (int s = 0; s < NS; ++s) {
      tma_load_3d(sK + s * BKV * 128, &tmK, &bar_kv[0], s * 64, kv_lo, h);
      tma_load_3d(sV + s * BKV * 128, &tmV, &bar_kv[0], s * 64, kv_lo, h);
    }
  }

  float o[D];
#pragma unroll
  for (int i = 0; i < D; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int jb = 0; jb < nblk; ++jb) {
    const int buf = jb & 1;
    const int kvb = kv_lo + jb * BKV;
    if (tid == 0) {
      if (jb + 1 < nblk) {  // prefetch the next key/value tile (its buffer was released by bar_o of block jb-1)
        const int nb = buf ^ 1;
        mbar_arrive_expect_tx(&bar_kv[nb], 2 * KV_BYTES);
        for (int s = 0; s < NS; ++s) {
          tma_load_3d(sK + nb * KV_BYTES + s * BKV * 128, &tmK, &bar_kv[nb], s * 64, kvb + BKV, h);
          tma_load_3d(sV + nb * KV_BYTES + s * BKV * 128, &tmV, &bar_kv[nb], s * 64, kvb + BKV, h);
        }
      }
      if (jb == 0) cta_wait(bar_q, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      cta_wait(&bar_kv[buf], (jb >> 1) & 1, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      tc_fence_after_sync();
      const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + buf * KV_BYTES);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint64_t ad = make_smem_desc_sw128(qa + (ks / 4) * (BQ * 128) + (ks % 4) * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(ka + (ks / 4) * (BKV * 128) + (ks % 4) * 32, 16, 1024);
        tc_mma_f16(tmem_base + S_COL, ad, bd, idesc_s, ks != 0);
      }
      tc_commit(bar_s);
    }
    __syncwarp();
    cta_wait(bar_s, jb & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();

    float sc[BKV];
    float mblk = -INFINITY;
#pragma unroll
    for (int c = 0; c < BKV / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + S_COL + c * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int kv = kvb + c * 32 + i;
        const float s = (kv >= ds && kv <= q) ? __uint_as_float(v[i]) * p.sl2 : -INFINITY;
        sc[c * 32 + i] = s;
        mblk = fmaxf(mblk, s);
      }
    }
    const float m_new = fmaxf(m, mblk);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = exp2f(m - m_use);
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
    m = m_new;
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t pa = smem_u32(sP), va = smem_u32(sV + buf * KV_BYTES);
#pragma unroll
      for (int ks = 0; ks < BKV / 16; ++ks) {
        const uint64_t ad = make_smem_desc_sw128(pa + ks * 32, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(va + ks * 2048, BKV * 128, 1024);
        tc_mma_f16(tmem_base + O_COL, ad, bd, idesc_o, ks != 0);
      }
      tc_commit(bar_o);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] *= alpha;
    cta_wait(bar_o, jb & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + O_COL + c * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(v[i]);
    }
    tc_fence_before_sync();
  }

  if (row_ok) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* orow = p.o + (long long)q * p.ld_o + h * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      uint4 u = make_uint4(pack_bf16x2(o[8 * j] * inv, o[8 * j + 1] * inv), pack_bf16x2(o[8 * j + 2] * inv, o[8 * j + 3] * inv),
                           pack_bf16x2(o[8 * j + 4] * inv, o[8 * j + 5] * inv), pack_bf16x2(o[8 * j + 6] * inv, o[8 * j + 7] * inv));
      reinterpret_cast<uint4*>(orow)[j] = u;
    }
    p.lse[(long long)h * p.T + q] = m + log2f(l);
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

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128, 1)
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
  uint8_t* sQ = sV + KV_BYTES;        // 2 buffers
  uint8_t* sdO = sQ + 2 * Q_BYTES;    // 2 buffers
  uint8_t* sPT = sdO + 2 * Q_BYTES;
  uint8_t* sdST = sPT + PT_BYTES;
  float* sdQ = reinterpret_cast<float*>(sdST + PT_BYTES);
  float* s_lse = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sdQ) + DQ_BYTES);  // [64]
  float* s_delta = s_lse + BQ;
  int* s_ds = reinterpret_cast<int*>(s_delta + BQ);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_ds + BQ);
  uint64_t* bar_kv = bars;
  uint64_t* bar_q = bars + 1;  // [2]
  uint64_t* bar_m1 = bars + 3;
  uint64_t* bar_m2 = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int jb = blockIdx.x;
  const int h = blockIdx.y;
  const int kv0 = jb * BKV;
  const int kv = kv0 + tid;

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(&bar_q[0], 1);
    mbar_init(&bar_q[1], 1);
    mbar_init(bar_m1, 1);
    mbar_init(bar_m2, 1);
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

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_kv, 2 * KV_BYTES);
    for (int s = 0; s < NS; ++s) {
      tma_load_3d(sK + s * BKV * 128, &tmK, bar_kv, s * 64, kv0, h);
      tma_load_3d(sV + s * BKV * 128, &tmV, bar_kv, s * 64, kv0, h);
    }
    if (ntile > 0) {
      mbar_arrive_expect_tx(&bar_q[0], 2 * Q_BYTES);
      for (int s = 0; s < NS; ++s) {
        tma_load_3d(sQ + s * BQ * 128, &tmQ, &bar_q[0], s * 64, q_lo, h);
        tma_load_3d(sdO + s * BQ * 128, &tmdO, &bar_q[0], s * 64, q_lo, h);
      }
    }
  }

  for (int it = 0; it < ntile; ++it) {
    const int buf = it & 1;
    const int qt0 = q_lo + it * BQ;
    if (tid < BQ) {
      const int qq = qt0 + tid;
      const bool okq = qq < p.T;
      s_lse[tid] = okq ? p.lse[(long long)h * p.T + qq] : INFINITY;
      s_delta[tid] = okq ? p.delta[(long long)h * p.T + qq] : 0.f;
      s_ds[tid] = okq ? p.doc_start[qq] : 0x7fffffff;
    }
    if (tid == 0) {
      if (it + 1 < ntile) {  // prefetch next Q / dO tile; its buffer was released by bar_m2 of tile it-1
        const int nb = buf ^ 1;
        mbar_arrive_expect_tx(&bar_q[nb], 2 * Q_BYTES);
        for (int s = 0; s < NS; ++s) {
          tma_load_3d(sQ + nb * Q_BYTES + s * BQ * 128, &tmQ, &bar_q[nb], s * 64, qt0 + BQ, h);
          tma_load_3d(sdO + nb * Q_BYTES + s * BQ * 128, &tmdO, &bar_q[nb], s * 64, qt0 + BQ, h);
        }
      }
      if (it == 0) cta_wait(bar_kv, 0, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      cta_wait(&bar_q[buf], (it >> 1) & 1, abort_flag, p.status, ERR_WAIT_SMEM_FULL);
      tc_fence_after_sync();
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
    }
    __syncthreads();  // s_lse / s_delta / s_ds visible; also orders the previous tile's staging reads
    cta_wait(bar_m1, it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();

    uint8_t* prow = sPT + tid * 128;
    uint8_t* drow = sdST + tid * 128;
#pragma unroll
    for (int c = 0; c < BQ / 32; ++c) {
      uint32_t sv[32], dv_[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + ST_COL + c * 32, sv);
      tmem_ld_32x32b_x32(tmem_base + lane_off + DPT_COL + c * 32, dv_);
      tmem_ld_wait();
      float pr[32], dsv[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int qi = c * 32 + i;
        const int qq = qt0 + qi;
        const bool valid = (qq >= kv) && (kv >= s_ds[qi]) && (kv < p.T);
        const float pv = valid ? exp2f(__uint_as_float(sv[i]) * p.sl2 - s_lse[qi]) : 0.f;
        pr[i] = pv;
        dsv[i] = pv * (__uint_as_float(dv_[i]) - s_delta[qi]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u = make_uint4(pack_bf16x2(pr[8 * j], pr[8 * j + 1]), pack_bf16x2(pr[8 * j + 2], pr[8 * j + 3]),
                             pack_bf16x2(pr[8 * j + 4], pr[8 * j + 5]), pack_bf16x2(pr[8 * j + 6], pr[8 * j + 7]));
        *reinterpret_cast<uint4*>(prow + (((c * 4 + j) ^ (tid & 7)) << 4)) = u;
        uint4 w = make_uint4(pack_bf16x2(dsv[8 * j], dsv[8 * j + 1]), pack_bf16x2(dsv[8 * j + 2], dsv[8 * j + 3]),
                             pack_bf16x2(dsv[8 * j + 4], dsv[8 * j + 5]), pack_bf16x2(dsv[8 * j + 6], dsv[8 * j + 7]));
        *reinterpret_cast<uint4*>(drow + (((c * 4 + j) ^ (tid & 7)) << 4)) = w;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t pa = smem_u32(sPT), dsa = smem_u32(sdST), ka = smem_u32(sK);
      const uint32_t qa = smem_u32(sQ + buf * Q_BYTES), doa = smem_u32(sdO + buf * Q_BYTES);
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
#pragma unroll
      for (int ks = 0; ks < BKV / 16; ++ks) {  // dQᵀ = Kᵀ · dSᵀ
        const uint64_t ad = make_smem_desc_sw128(ka + ks * 2048, BKV * 128, 1024);
        const uint64_t bd = make_smem_desc_sw128(dsa + ks * 2048, BKV * 128, 1024);
        tc_mma_f16(tmem_base + DQT_COL, ad, bd, idesc_dq, ks != 0);
      }
      tc_commit(bar_m2);
      tma_store_wait_read<0>();  // previous tile's reduce-add has drained the staging buffer
    }
    __syncthreads();
    cta_wait(bar_m2, it & 1, abort_flag, p.status, ERR_WAIT_TMEM_FULL);
    tc_fence_after_sync();
    // dQᵀ row (= head-dim index tid) -> staging[q][tid]
    if (tid < D) {
#pragma unroll
      for (int c = 0; c < BQ / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_off + DQT_COL + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sdQ[(c * 32 + i) * D + tid] = __uint_as_float(v[i]) * p.scale;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tma_reduce_add_3d(&tmdQ, sdQ, 0, qt0, h);
      tma_store_commit();
    }
  }

  // final: dV, dK rows
  tc_fence_after_sync();
  if (ntile > 0 && kv < p.T) {
    __nv_bfloat16* dvrow = p.dv + (long long)kv * p.ld_dv + h * D;
    __nv_bfloat16* dkrow = p.dk + (long long)kv * p.ld_dk + h * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + lane_off + DV_COL + c * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u = make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                             pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                             pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                             pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
        reinterpret_cast<uint4*>(dvrow + c * 32)[j] = u;
      }
      tmem_ld_32x32b_x32(tmem_base + lane_off + DK_COL + c * 32, v);
      tmem_ld_wait();
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
  if (tid == 0) {
    tma_store_wait_all<0>();
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
  const int smem = NS * 128 * 128 + 4 * NS * 64 * 128 + 128 * 128 + 64;
  CUtensorMap tq = qkv_map(a.q, a.T, a.H, D, a.ld_q, 128);
  CUtensorMap tk = qkv_map(a.k, a.T, a.H, D, a.ld_k, 64);
  CUtensorMap tv = qkv_map(a.v, a.T, a.H, D, a.ld_v, 64);
  auto kern = attn_fwd_kernel<D>;
  static bool cfg = false;
  if (!cfg) { set_smem(kern, smem); cfg = true; }
  dim3 grid((a.T + 127) / 128, a.H);
  kern<<<grid, 128, smem, a.stream>>>(tq, tk, tv, make_kp(a));
  check_launch("attn_fwd launch");
}

template <int D>
void bwd_impl(const AttnArgs& a) {
  constexpr int NS = D / 64;
  const int smem = 2 * NS * 128 * 128 + 4 * NS * 64 * 128 + 2 * 128 * 128 + 64 * D * 4 + 3 * 64 * 4 + 64 + 1024;
  CUtensorMap tq = qkv_map(a.q, a.T, a.H, D, a.ld_q, 64);
  CUtensorMap tk = qkv_map(a.k, a.T, a.H, D, a.ld_k, 128);
  CUtensorMap tv = qkv_map(a.v, a.T, a.H, D, a.ld_v, 128);
  CUtensorMap tdo = qkv_map(a.d_o, a.T, a.H, D, a.ld_do, 64);
  CUtensorMap tdq = make_tmap_3d(a.dq_acc, TmapDtype::F32, (uint64_t)D, (uint64_t)a.T, (uint64_t)a.H,
                                 (uint64_t)a.ld_dq * 4, (uint64_t)D * 4, (uint32_t)D, 64, false);
  auto kern = attn_bwd_kernel<D>;
  static bool cfg = false;
  if (!cfg) { set_smem(kern, smem); cfg = true; }
  dim3 grid((a.T + 127) / 128, a.H);
  kern<<<grid, 128, smem, a.stream>>>(tq, tk, tv, tdo, tdq, make_kp(a));
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
  if (a.D == 128) attn_delta_kernel<128><<<blocks, threads, 0, a.stream>>>(o, a.ld_o, d_o, a.ld_do, a.delta, a.T, a.H);
  else            attn_delta_kernel<64><<<blocks, threads, 0, a.stream>>>(o, a.ld_o, d_o, a.ld_do, a.delta, a.T, a.H);
  check_launch("attn_delta launch");
}

void attn_bwd_sm100(const AttnArgs& a) {
  check_common(a);
  // dQᵀ = Kᵀ·dSᵀ puts the head dimension on the MMA M axis, which this kernel issues at M = 128 only.
  if (a.D != 128) throw std::runtime_error("attention backward: head_dim must be 128");
  bwd_impl<128>(a);
}

}  // namespace b200
