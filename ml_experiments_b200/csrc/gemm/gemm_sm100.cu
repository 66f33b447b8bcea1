// Persistent, warp-specialised GEMM for sm_100a.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor -> 128B-swizzled shared-memory stages)
//   warp 1      : MMA issuer    (one thread issues tcgen05.mma; accumulators live in tensor memory)
//   warps 2..5  : epilogue      (tcgen05.ld -> fused epilogue -> swizzled staging -> TMA store / reduce-add)
//
// Two TMEM accumulators (2 x BN columns) let the epilogue of tile i overlap the main loop of tile
// i+1. Operands may be K-major or MN-major (selected per operand through the shared-memory
// descriptor and the instruction descriptor), so forward (A·Wᵀ), data-gradient (dY·W) and
// weight-gradient (dYᵀ·X) products all run without a transpose pass. bf16 and fp8 (e4m3/e5m2)
// inputs, fp32 accumulation, bf16 or fp32 output, batched, optional split-K by TMA reduce-add.
#include "../common/per_device.h"
#include "gemm.h"

#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"
#include "../common/tmap.h"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int kThreads = 192;
constexpr int kStagingBytes = 4 * 2 * 4096;  // 4 epilogue warps x 2 buffers x (32 rows x 128 B)

struct KParams {
  int M, N, K;
  int batch, splits;
  int k_per_split;  // multiple of the stage depth
  int tiles_m, tiles_n, total_tiles;
  uint32_t idesc;
  int epi;
  int out_f32;
  int reduce_add;
  float alpha, beta;
  const __nv_bfloat16* aux;
  long long ld_aux, stride_aux;
  int* status;
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = BM * 128;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes + kStagingBytes;
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4 + 8) * 8 + 16 + 1024;  // + alignment slack
};

template <int BN, int STAGES, int AMN, int BMN, int ESZ>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux, const KParams p) {
  using L = SmemLayout<BN, STAGES>;
  constexpr int BK = 128 / ESZ;         // elements along K per stage (one 128-byte swizzle span)
  constexpr int UMMA_K = 32 / ESZ;      // elements along K per tcgen05.mma
  constexpr int KSTEPS = BK / UMMA_K;   // 4
  constexpr int MN_SPAN = 128 / ESZ;    // elements per 128-byte span along M/N (MN-major operands)
  constexpr int CHUNK_BYTES = BK * 128; // one MN-major box: BK k-rows x 128 B
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * L::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* aux_bar = tempty_bar + 2;  // [4 epilogue warps][2 staging buffers]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux_bar + 8);

  if (status_poisoned(p.status)) return;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    for (int a = 0; a < 8; ++a) mbar_init(&aux_bar[a], 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmAux);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        int r = t;
        const int nt = r % p.tiles_n; r /= p.tiles_n;  // N fastest: concurrent CTAs share one A panel through L2
        const int mt = r % p.tiles_m; r /= p.tiles_m;
        const int sp = r % p.splits;
        const int b = r / p.splits;
        const int m0 = mt * BM, n0 = nt * BN;
        const int kbeg = sp * p.k_per_split;
        const int kend = min(p.K, kbeg + p.k_per_split);
        const int nkb = (kend - kbeg + BK - 1) / BK;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ERR_WAIT_SMEM_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + stage * L::kStageBytes;
          uint8_t* sB = sA + L::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
          const int k0 = kbeg + kb * BK;
          if (AMN == 0) {
            tma_load_3d(sA, &tmA, &full_bar[stage], k0, m0, b);
          } else {
#pragma unroll
            for (int c = 0; c < BM / MN_SPAN; ++c)
              tma_load_3d(sA + c * CHUNK_BYTES, &tmA, &full_bar[stage], m0 + c * MN_SPAN, k0, b);
          }
          if (BMN == 0) {
            tma_load_3d(sB, &tmB, &full_bar[stage], k0, n0, b);
          } else {
#pragma unroll
            for (int c = 0; c < BN / MN_SPAN; ++c)
              tma_load_3d(sB + c * CHUNK_BYTES, &tmB, &full_bar[stage], n0 + c * MN_SPAN, k0, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Give loads that are still in flight a bounded time (1 ms) to land before shared memory is released.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        int r = t / (p.tiles_m * p.tiles_n);
        const int sp = r % p.splits;
        const int kbeg = sp * p.k_per_split;
        const int kend = min(p.K, kbeg + p.k_per_split);
        const int nkb = (kend - kbeg + BK - 1) / BK;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t b_addr = a_addr + L::kABytes;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const uint64_t adesc = AMN ? make_smem_desc_sw128(a_addr + ks * UMMA_K * 128, CHUNK_BYTES, 1024)
                                       : make_smem_desc_sw128(a_addr + ks * 32, 16, 1024);
            const uint64_t bdesc = BMN ? make_smem_desc_sw128(b_addr + ks * UMMA_K * 128, CHUNK_BYTES, 1024)
                                       : make_smem_desc_sw128(b_addr + ks * 32, 16, 1024);
            if (ESZ == 2) tc_mma_f16(d_tmem, adesc, bdesc, p.idesc, (kb | ks) != 0);
            else          tc_mma_f8(d_tmem, adesc, bdesc, p.idesc, (kb | ks) != 0);
          }
          tc_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tfull_bar[acc]);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* my_staging = staging + (warp - 2) * 8192;
    int buf = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const int out_cols_per_buf = p.out_f32 ? 32 : 64;
    // bf16 output with an aux operand: the aux tile is brought by TMA into the (swizzled) staging buffer, combined in
    // place by the thread that owns the row, and the same buffer is then stored - no uncoalesced per-row global loads.
    const bool aux_tma = (p.epi == EPI_AXPBY || p.epi == EPI_RELU2_BWD) && !p.out_f32 && !p.reduce_add;
    uint64_t* my_aux_bar = aux_bar + (warp - 2) * 2;
    uint32_t aux_phase0 = 0, aux_phase1 = 0;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      int r = t;
      const int nt = r % p.tiles_n; r /= p.tiles_n;
      const int mt = r % p.tiles_m; r /= p.tiles_m;
      const int b = r / p.splits;
      const int m0 = mt * BM, n0 = nt * BN;
      const int row = m0 + q * 32 + lane;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      if (aux_tma) {
        const int ngroups = min(BN / 64, (p.N - n0 + 63) / 64);
        auto issue_aux = [&](int g, int bsel) {
          if (lane == 0) {
            tma_store_wait_read<0>();  // the store that last used this buffer has drained it
            mbar_arrive_expect_tx(&my_aux_bar[bsel], 4096);
            tma_load_3d(my_staging + bsel * 4096, &tmAux, &my_aux_bar[bsel], n0 + g * 64, m0 + q * 32, b);
          }
        };
        issue_aux(0, buf);
        for (int g = 0; g < ngroups && ok; ++g) {
          if (g + 1 < ngroups) issue_aux(g + 1, buf ^ 1);
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + g * 64, v0);
          tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + g * 64 + 32, v1);
          tmem_ld_wait();
          const uint32_t ph = buf ? aux_phase1 : aux_phase0;
          if (!mbar_wait(&my_aux_bar[buf], ph, p.status, ERR_WAIT_SMEM_FULL)) { ok = false; break; }
          if (buf) aux_phase1 ^= 1; else aux_phase0 ^= 1;
          uint8_t* rowp = my_staging + buf * 4096 + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4* cell = reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4));
            const uint4 u = *cell;
            float a[8], f[8];
            float2 x0 = unpack_bf16x2(u.x), x1 = unpack_bf16x2(u.y), x2 = unpack_bf16x2(u.z), x3 = unpack_bf16x2(u.w);
            a[0] = x0.x; a[1] = x0.y; a[2] = x1.x; a[3] = x1.y; a[4] = x2.x; a[5] = x2.y; a[6] = x3.x; a[7] = x3.y;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float accv = __uint_as_float(j < 4 ? v0[8 * j + i] : v1[8 * (j - 4) + i]) * p.alpha;
              f[i] = (p.epi == EPI_AXPBY) ? fmaf(p.beta, a[i], accv) : accv * 2.f * sqrtf(a[i]);
            }
            *cell = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmC, my_staging + buf * 4096, n0 + g * 64, m0 + q * 32, b);
            tma_store_commit();
          }
          buf ^= 1;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      }
      const __nv_bfloat16* aux_row =
          p.aux ? p.aux + (long long)b * p.stride_aux + (long long)row * p.ld_aux : nullptr;
      int filled = 0;      // columns written into the current staging buffer
      int buf_col0 = n0;   // first output column of the current staging buffer
      const bool use_aux = (p.epi == EPI_AXPBY || p.epi == EPI_RELU2_BWD);
      const bool aux_vec = use_aux && row < p.M && ((p.ld_aux & 7) == 0);
      uint4 aux_next[4];
      auto fetch_aux = [&](int c) {  // 32 bf16 of this thread's row, columns n0+c .. n0+c+31
        const int col = n0 + c;
        if (aux_vec && col + 32 <= p.N) {
          const uint4* src = reinterpret_cast<const uint4*>(aux_row + col);
#pragma unroll
          for (int i = 0; i < 4; ++i) aux_next[i] = __ldg(src + i);
        } else {
          __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(aux_next);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            e[i] = (row < p.M && col + i < p.N) ? aux_row[col + i] : __float2bfloat16(0.f);
        }
      };
      if (use_aux) fetch_aux(0);
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= p.N) break;
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + c, v);
        uint4 aux_cur[4];
        if (use_aux) {
#pragma unroll
          for (int i = 0; i < 4; ++i) aux_cur[i] = aux_next[i];
          if (c + 32 < BN && n0 + c + 32 < p.N) fetch_aux(c + 32);  // in flight while this chunk is processed
        }
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]) * p.alpha;
        if (p.epi == EPI_RELU2) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { float rr = fmaxf(f[i], 0.f); f[i] = rr * rr; }
        } else if (use_aux) {
          float a[32];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 u = aux_cur[i];
            float2 x0 = unpack_bf16x2(u.x), x1 = unpack_bf16x2(u.y), x2 = unpack_bf16x2(u.z), x3 = unpack_bf16x2(u.w);
            a[8 * i + 0] = x0.x; a[8 * i + 1] = x0.y; a[8 * i + 2] = x1.x; a[8 * i + 3] = x1.y;
            a[8 * i + 4] = x2.x; a[8 * i + 5] = x2.y; a[8 * i + 6] = x3.x; a[8 * i + 7] = x3.y;
          }
          if (p.epi == EPI_AXPBY) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = fmaf(p.beta, a[i], f[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = f[i] * 2.f * sqrtf(a[i]);
          }
        }
        // ---- stage into 128B-swizzled shared memory (row = lane, 16-byte chunk j stored at j ^ (lane & 7))
        if (filled == 0) {
          if (lane == 0) tma_store_wait_read<1>();  // the store that last used this buffer has drained it
          __syncwarp();
          buf_col0 = n0 + c;
        }
        uint8_t* rowp = my_staging + buf * 4096 + lane * 128;
        if (p.out_f32) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 u = make_uint4(__float_as_uint(f[4 * j]), __float_as_uint(f[4 * j + 1]),
                                 __float_as_uint(f[4 * j + 2]), __float_as_uint(f[4 * j + 3]));
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = u;
          }
        } else {
          const int h = filled >> 5;  // 0 or 1: which half of the 64-column buffer
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 u = make_uint4(pack_bf16x2(f[8 * j], f[8 * j + 1]), pack_bf16x2(f[8 * j + 2], f[8 * j + 3]),
                                 pack_bf16x2(f[8 * j + 4], f[8 * j + 5]), pack_bf16x2(f[8 * j + 6], f[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + (((h * 4 + j) ^ (lane & 7)) << 4)) = u;
          }
        }
        filled += 32;
        if (filled == out_cols_per_buf) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (p.reduce_add) tma_reduce_add_3d(&tmC, my_staging + buf * 4096, buf_col0, m0 + q * 32, b);
            else              tma_store_3d(&tmC, my_staging + buf * 4096, buf_col0, m0 + q * 32, b);
            tma_store_commit();
          }
          buf ^= 1;
          filled = 0;
        }
      }
      // accumulator fully read: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (filled != 0) {  // partially filled buffer at a ragged N edge (columns beyond N are clipped by TMA)
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (p.reduce_add) tma_reduce_add_3d(&tmC, my_staging + buf * 4096, buf_col0, m0 + q * 32, b);
          else              tma_store_3d(&tmC, my_staging + buf * 4096, buf_col0, m0 + q * 32, b);
          tma_store_commit();
        }
        buf ^= 1;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int BN, int STAGES, int AMN, int BMN, int ESZ>
void launch(const GemmArgs& a, const KParams& kp, const CUtensorMap& tA, const CUtensorMap& tB,
            const CUtensorMap& tC, const CUtensorMap& tX, int grid) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_kernel<BN, STAGES, AMN, BMN, ESZ>;
  static PerDeviceOnce configured;   // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  if (configured.pending(&dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) throw std::runtime_error(std::string("gemm: cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    configured.done(dev);
  }
  kern<<<grid, kThreads, L::kTotal, a.stream>>>(tA, tB, tC, tX, kp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm launch: ") + cudaGetErrorString(e));
}

template <int BN, int STAGES, int ESZ>
void dispatch_major(const GemmArgs& a, const KParams& kp, const CUtensorMap& tA, const CUtensorMap& tB,
                    const CUtensorMap& tC, const CUtensorMap& tX, int grid) {
  if (!a.a_mn && !a.b_mn) launch<BN, STAGES, 0, 0, ESZ>(a, kp, tA, tB, tC, tX, grid);
  else if (!a.a_mn && a.b_mn) launch<BN, STAGES, 0, 1, ESZ>(a, kp, tA, tB, tC, tX, grid);
  else if (a.a_mn && !a.b_mn) launch<BN, STAGES, 1, 0, ESZ>(a, kp, tA, tB, tC, tX, grid);
  else launch<BN, STAGES, 1, 1, ESZ>(a, kp, tA, tB, tC, tX, grid);
}

int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace

void gemm_sm100(const GemmArgs& a) {
  const int esz = (a.a_dtype == GEMM_BF16) ? 2 : 1;
  const int esz_b = (a.b_dtype == GEMM_BF16) ? 2 : 1;
  if (esz != esz_b) throw std::runtime_error("gemm: A and B must both be bf16 or both be fp8");
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) throw std::runtime_error("gemm: empty problem");
  if (a.c_dtype != GEMM_BF16 && a.c_dtype != GEMM_F32) throw std::runtime_error("gemm: C must be bf16 or fp32");
  const int splits = a.split_k < 1 ? 1 : a.split_k;
  const bool reduce_add = (splits > 1) || a.accumulate;
  if (reduce_add && a.c_dtype != GEMM_F32) throw std::runtime_error("gemm: split-K / accumulate needs fp32 C");
  if (splits > 1 && !a.accumulate && a.ldc != a.N) throw std::runtime_error("gemm: split-K needs a dense C (ldc == N)");
  if (splits > 1 && a.epilogue != EPI_NONE) throw std::runtime_error("gemm: split-K supports only the plain epilogue");
  if ((a.epilogue == EPI_AXPBY || a.epilogue == EPI_RELU2_BWD) && a.aux == nullptr)
    throw std::runtime_error("gemm: this epilogue needs aux");

  const int BN = a.N > 128 ? 256 : 128;
  const int BK = 128 / esz;
  const int span = 128 / esz;
  const TmapDtype in_dt = esz == 2 ? TmapDtype::BF16 : TmapDtype::U8;
  const uint64_t nb = (uint64_t)a.batch;

  CUtensorMap tA, tB, tC;
  if (!a.a_mn) tA = make_tmap_3d(a.A, in_dt, a.K, a.M, nb, a.lda * esz, a.stride_a * esz, BK, BM, true);
  else         tA = make_tmap_3d(a.A, in_dt, a.M, a.K, nb, a.lda * esz, a.stride_a * esz, span, BK, true);
  if (!a.b_mn) tB = make_tmap_3d(a.B, in_dt, a.K, a.N, nb, a.ldb * esz, a.stride_b * esz, BK, BN, true);
  else         tB = make_tmap_3d(a.B, in_dt, a.N, a.K, nb, a.ldb * esz, a.stride_b * esz, span, BK, true);
  const int osz = a.c_dtype == GEMM_F32 ? 4 : 2;
  tC = make_tmap_3d(a.C, a.c_dtype == GEMM_F32 ? TmapDtype::F32 : TmapDtype::BF16, a.N, a.M, nb, a.ldc * osz,
                    a.stride_c * osz, 128 / osz, 32, true);

  CUtensorMap tX = tC;  // aux tile map (bf16 [batch][M][N]); only dereferenced by the aux epilogues
  if (a.aux != nullptr && (a.ldaux % 8) == 0)
    tX = make_tmap_3d(a.aux, TmapDtype::BF16, a.N, a.M, nb, a.ldaux * 2, a.stride_aux * 2, 64, 32, true);
  else if (a.aux != nullptr)
    throw std::runtime_error("gemm: aux row pitch must be a multiple of 8 elements");

  KParams kp;
  kp.M = a.M; kp.N = a.N; kp.K = a.K;
  kp.batch = a.batch; kp.splits = splits;
  int kps = (a.K + splits - 1) / splits;
  kps = (kps + BK - 1) / BK * BK;
  kp.k_per_split = kps;
  // drop splits that would start beyond K
  while (kp.splits > 1 && (long long)(kp.splits - 1) * kps >= a.K) kp.splits--;
  kp.tiles_m = (a.M + BM - 1) / BM;
  kp.tiles_n = (a.N + BN - 1) / BN;
  kp.total_tiles = kp.tiles_m * kp.tiles_n * kp.splits * a.batch;
  auto fmt = [](int dt) -> uint32_t { return dt == GEMM_BF16 ? FMT_BF16 : (dt == GEMM_E4M3 ? FMT_E4M3 : FMT_E5M2); };
  kp.idesc = make_idesc(fmt(a.a_dtype), fmt(a.b_dtype), a.a_mn ? 1 : 0, a.b_mn ? 1 : 0, BM, BN);
  kp.epi = a.epilogue;
  kp.out_f32 = a.c_dtype == GEMM_F32;
  kp.reduce_add = reduce_add ? 1 : 0;
  kp.alpha = a.alpha; kp.beta = a.beta;
  kp.aux = reinterpret_cast<const __nv_bfloat16*>(a.aux);
  kp.ld_aux = a.ldaux; kp.stride_aux = a.stride_aux;
  kp.status = a.status;

  if (splits > 1 && !a.accumulate) {
    // split-K partial sums are combined by reduce-add into C, which therefore starts from zero
    if (a.batch == 1 || a.stride_c == (long long)a.M * a.ldc) {
      cudaMemsetAsync(a.C, 0, (size_t)a.batch * a.M * a.ldc * osz, a.stream);
    } else {
      for (int b = 0; b < a.batch; ++b)
        cudaMemsetAsync((char*)a.C + (size_t)b * a.stride_c * osz, 0, (size_t)a.M * a.ldc * osz, a.stream);
    }
  }

  int grid = a.max_ctas > 0 ? a.max_ctas : num_sms();
  if (grid > kp.total_tiles) grid = kp.total_tiles;

  if (esz == 2) {
    if (BN == 256) dispatch_major<256, 4, 2>(a, kp, tA, tB, tC, tX, grid);
    else           dispatch_major<128, 6, 2>(a, kp, tA, tB, tC, tX, grid);
  } else {
    if (BN == 256) dispatch_major<256, 4, 1>(a, kp, tA, tB, tC, tX, grid);
    else           dispatch_major<128, 6, 1>(a, kp, tA, tB, tC, tX, grid);
  }
}

}  // namespace b200
