// S6 (Mamba-1) selective scan, forward and backward.
//
//   dt_t[d]  = softplus(delta_t[d] + delta_bias[d])            (both optional: plain delta when softplus is off)
//   h_t[d,n] = exp(dt_t[d] * A[d,n]) * h_{t-1}[d,n] + dt_t[d] * B_t[n] * u_t[d]
//   y_t[d]   = sum_n C_t[n] * h_t[d,n] + D[d] * u_t[d] ;   out = y * silu(z)
//
// Thread mapping: a block owns 32 channels; lane = channel, warp = QS of the 16 states in registers (QS = 4: four warps
// per block, QS = 2: eight warps per block, twice the warps per SM to hide the exp / FMA latency of the recurrence).
// B_t / C_t are then warp-uniform shared-memory broadcasts, dt / u loads are conflict-free, the forward needs no
// shuffles at all (the four partial sums over states meet in shared memory), and the backward's dB_t / dC_t, which sum
// over channels, are 8 values reduced across the 32 lanes with a halving butterfly (9 shuffles for all 8).
// Time is processed in tiles of 16 steps. The forward stores the state at the start of every tile; the backward walks
// the tiles in reverse, recomputes the 16 states of a tile into registers from that checkpoint and runs the adjoint
// recurrence. The gate (silu(z)), the softplus of delta and its bias are applied inside both kernels, so no
// elementwise pass is left outside. dB / dC leave as deterministic partial sums per 32-channel block
// [B][ceil(Din/32)][L][N] that the caller adds up.
//
// Semantics follow selective_scan_ref of the reference (zoology/mixers/mamba_ssm/ops/selective_scan_interface.py:91-157)
// with real A and input-dependent B and C shared across channels.
#include "s6_scan.h"

#include <cuda_bf16.h>

#include <cstdint>

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;
constexpr int NS = 16;    // states per channel
constexpr int CB = 32;    // channels per block (= lanes)
constexpr int SUB = 16;   // time steps per tile and per state checkpoint
int g_fwd_qs = 2, g_bwd_qs = 4;  // measured on 8 x 4096 x 2048: forward 0.72 ms at 2 (0.80 at 4); backward 2.6 ms at 4 (5.5 at 2: spills)

// State checkpoints are stored in groups of four states whatever QS the kernels run with:
// [B][tiles][4][Din][4]; a thread's QS states (first state n0 = w * QS) are contiguous in it.
__device__ __forceinline__ long long state_off(int b, int nsub, int tile, int n0, int Din, int d) {
  return ((((long long)b * nsub + tile) * 4 + (n0 >> 2)) * Din + d) * 4 + (n0 & 3);
}

template <int QS>
struct Shape {
  static constexpr int NW = NS / QS;          // warps per block
  static constexpr int NT = 32 * NW;          // threads per block
  static constexpr int RPT = SUB / NW;        // rows of a [16][32] tile staged per thread
  static constexpr int BCPT = SUB * NS / NT;  // B (and C) elements staged per thread
};

// QS consecutive floats as one vector access
template <int QS>
__device__ __forceinline__ void ldv(float (&o)[QS], const float* p) {
  if constexpr (QS == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w;
  } else {
    const float2 v = *reinterpret_cast<const float2*>(p);
    o[0] = v.x, o[1] = v.y;
  }
}
template <int QS>
__device__ __forceinline__ void stv(float* p, const float (&o)[QS]) {
  if constexpr (QS == 4) *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  else *reinterpret_cast<float2*>(p) = make_float2(o[0], o[1]);
}
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Request a line into L1 (and L2) without holding a register for it.
__device__ __forceinline__ void prefetch_near(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ float ld(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

template <int QS>
struct FwdSmem {
  float dt[SUB][CB];
  float u[SUB][CB];
  float B[SUB][NS];
  float C[SUB][NS];
  float yp[NS / QS][SUB][CB];
};

// grid (ceil(Din / 32), batch), 32 * 16 / QS threads. DT = element type of delta (fp32 or bf16).
template <typename DT, int QS>
__global__ void __launch_bounds__(Shape<QS>::NT, 1024 / Shape<QS>::NT)
s6_fwd_kernel(const bf16* __restrict__ u, const DT* __restrict__ delta, const float* __restrict__ delta_bias,
              int softplus, const float* __restrict__ A, const float* __restrict__ Bm, const float* __restrict__ Cm,
              const float* __restrict__ Dv, const bf16* __restrict__ z, bf16* __restrict__ y_pre,
              bf16* __restrict__ out, float* __restrict__ state, int L, int Din) {
  constexpr int NW = Shape<QS>::NW, NT = Shape<QS>::NT, RPT = Shape<QS>::RPT, BCPT = Shape<QS>::BCPT;
  __shared__ __align__(16) FwdSmem<QS> s;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int b = blockIdx.y, d0 = blockIdx.x * CB, d = d0 + lane;
  const bool dok = d < Din;
  const int nsub = (L + SUB - 1) / SUB;
  float h[QS], a2[QS];
#pragma unroll
  for (int k = 0; k < QS; ++k) {
    h[k] = 0.f;
    a2[k] = dok ? A[(long long)d * NS + w * QS + k] * LOG2E : 0.f;
  }
  const float bias = (dok && delta_bias) ? delta_bias[d] : 0.f;
  const float dsk = (dok && Dv) ? Dv[d] : 0.f;
  // staging registers for the next tile: the thread covers rows w + NW * j of the [16][32] tiles and BCPT B / C elements
  float pdt[RPT], pu[RPT], pz[RPT], pB[BCPT], pC[BCPT];
  auto fetch = [&](int tile) {
    const int t0 = tile * SUB;
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int t = t0 + w + NW * j;
      const bool ok = dok && t < L;
      const long long off = ((long long)b * L + t) * Din + d;
      pdt[j] = ok ? ld(delta, off) : 0.f;
      pu[j] = ok ? __bfloat162float(u[off]) : 0.f;
      pz[j] = (ok && z) ? __bfloat162float(z[off]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < BCPT; ++j) {
      const int i = tid + NT * j, t = t0 + i / NS;
      const long long off = ((long long)b * L + t) * NS + (i % NS);
      pB[j] = t < L ? Bm[off] : 0.f;
      pC[j] = t < L ? Cm[off] : 0.f;
    }
  };
  fetch(0);
  for (int tile = 0; tile < nsub; ++tile) {
    const int t0 = tile * SUB;
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int t = w + NW * j;
      float dtv = pdt[j];
      if (softplus) dtv = (dok && t0 + t < L) ? softplusf(dtv + bias) : 0.f;
      s.dt[t][lane] = dtv;
      s.u[t][lane] = pu[j];
    }
#pragma unroll
    for (int j = 0; j < BCPT; ++j) {
      const int i = tid + NT * j;
      s.B[i / NS][i % NS] = pB[j];
      s.C[i / NS][i % NS] = pC[j];
    }
    float zc[RPT];  // this tile's gate inputs (the staging registers are about to be refilled)
#pragma unroll
    for (int j = 0; j < RPT; ++j) zc[j] = pz[j];
    __syncthreads();
    if (tile + 1 < nsub) fetch(tile + 1);
    if (state && dok)
      stv<QS>(&state[state_off(b, nsub, tile, w * QS, Din, d)], h);
#pragma unroll
    for (int t = 0; t < SUB; ++t) {
      const float dt = s.dt[t][lane], dtu = dt * s.u[t][lane];
      float bb[QS], cc[QS];
      ldv<QS>(bb, &s.B[t][w * QS]);
      ldv<QS>(cc, &s.C[t][w * QS]);
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < QS; ++k) {
        h[k] = fmaf(ex2(dt * a2[k]), h[k], dtu * bb[k]);
        y = fmaf(h[k], cc[k], y);
      }
      s.yp[w][t][lane] = y;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int t = w + NW * j;
      if (dok && t0 + t < L) {
        const long long off = ((long long)b * L + t0 + t) * Din + d;
        float yv = dsk * s.u[t][lane];
#pragma unroll
        for (int q = 0; q < NW; ++q) yv += s.yp[q][t][lane];
        if (y_pre) y_pre[off] = __float2bfloat16_rn(yv);
        float o = yv;
        if (z) o = yv * zc[j] * sigmoidf(zc[j]);
        out[off] = __float2bfloat16_rn(o);
      }
    }
    __syncthreads();
  }
}

template <int QS>
struct BwdSmem {
  float dt[SUB][CB];
  float u[SUB][CB];
  float dy[SUB][CB];
  float B[SUB][NS];
  float C[SUB][NS];
  float dB[SUB][NS];
  float dC[SUB][NS];
  float pddt[NS / QS][SUB][CB];
  float pdu[NS / QS][SUB][CB];
};

// Sum each of 8 per-lane values over the 32 lanes; afterwards every lane holds the total of value
// ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1).
__device__ __forceinline__ float reduce8(const float (&v)[8], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float r[4], q[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = b4 ? v[i] : v[i + 4], keep = b4 ? v[i + 4] : v[i];
    r[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = b3 ? r[i] : r[i + 2], keep = b3 ? r[i + 2] : r[i];
    q[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  const float send = b2 ? q[0] : q[1], keep = b2 ? q[1] : q[0];
  float p = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  p += __shfl_xor_sync(0xffffffffu, p, 2);
  p += __shfl_xor_sync(0xffffffffu, p, 1);
  return p;
}

// Same for 4 per-lane values: afterwards every lane holds the total of value ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1).
__device__ __forceinline__ float reduce4(const float (&v)[4], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8;
  float r[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = b4 ? v[i] : v[i + 2], keep = b4 ? v[i + 2] : v[i];
    r[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
  const float send = b3 ? r[0] : r[1], keep = b3 ? r[1] : r[0];
  float p = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  p += __shfl_xor_sync(0xffffffffu, p, 4);
  p += __shfl_xor_sync(0xffffffffu, p, 2);
  p += __shfl_xor_sync(0xffffffffu, p, 1);
  return p;
}

// One tile's inputs exactly as they lie in memory: filled by 16-byte cp.async copies one tile ahead of its use, so the
// backward never waits for global memory at the start of a tile (the walk over the sequence is serial per block, and
// that wait was its largest stall).
template <typename DT>
struct RawTile {
  DT delta[SUB][CB];
  bf16 u[SUB][CB];
  bf16 dout[SUB][CB];
  bf16 z[SUB][CB];
  bf16 yp[SUB][CB];
  float B[SUB][NS];
  float C[SUB][NS];
  float st[4][CB][4];   // the state checkpoint of the tile: [group of four states][channel][state in group]
};

// 16 bytes global -> shared; `bytes` (0..16) of them are read, the rest of the destination is zero-filled
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int bytes) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// grid (ceil(Din / 32), batch), 32 * 16 / QS threads. dout is the gradient of `out`; with z given the gate's backward is applied
// here (dy = dout * silu(z), dz = dout * y_pre * silu'(z)).
template <typename DT, int QS>
__global__ void __launch_bounds__(Shape<QS>::NT, 4)
s6_bwd_kernel(const bf16* __restrict__ u, const DT* __restrict__ delta, const float* __restrict__ delta_bias,
              int softplus, const float* __restrict__ A, const float* __restrict__ Bm, const float* __restrict__ Cm,
              const float* __restrict__ Dv, const bf16* __restrict__ z, const bf16* __restrict__ y_pre,
              const bf16* __restrict__ dout, const float* __restrict__ state, bf16* __restrict__ du,
              DT* __restrict__ ddelta, float* __restrict__ dA, float* __restrict__ dB_part,
              float* __restrict__ dC_part, float* __restrict__ dD, bf16* __restrict__ dz,
              float* __restrict__ ddelta_bias, int L, int Din, int piped) {
  constexpr int NW = Shape<QS>::NW, NT = Shape<QS>::NT, RPT = Shape<QS>::RPT, BCPT = Shape<QS>::BCPT;
  __shared__ __align__(16) BwdSmem<QS> s;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int b = blockIdx.y, d0 = blockIdx.x * CB, d = d0 + lane, nblk = gridDim.x;
  const bool dok = d < Din;
  const int nsub = (L + SUB - 1) / SUB;
  float ar[QS], a2[QS], cr[QS], dAa[QS];
#pragma unroll
  for (int k = 0; k < QS; ++k) {
    ar[k] = dok ? A[(long long)d * NS + w * QS + k] : 0.f;
    a2[k] = ar[k] * LOG2E;
    cr[k] = 0.f;
    dAa[k] = 0.f;
  }
  const float bias = (dok && delta_bias) ? delta_bias[d] : 0.f;
  const float dsk = (dok && Dv) ? Dv[d] : 0.f;
  float dDa = 0.f, dbias = 0.f;
  // two RawTile buffers in dynamic shared memory; the host passes piped = 0 (and no dynamic memory) when rows are not
  // 16-byte aligned (Din % 8 != 0) or the variant's static arrays leave no room for them
  extern __shared__ __align__(16) unsigned char s6_dyn_smem[];
  RawTile<DT>* raw = reinterpret_cast<RawTile<DT>*>(s6_dyn_smem);
  auto issue_tile = [&](int tile, int buf) {
    RawTile<DT>& r = raw[buf];
    const int t0 = tile * SUB;
    constexpr int CPR = CB * (int)sizeof(bf16) / 16;       // chunks per bf16 row (4)
    constexpr int DPR = CB * (int)sizeof(DT) / 16;         // chunks per delta row (4 or 8)
    constexpr int N16 = SUB * CPR, ND = SUB * DPR, NBC = SUB * NS * 4 / 16, NST = 4 * CB * 4 * 4 / 16;
    const int nz = z ? N16 : 0;
    const int total = ND + 2 * N16 + 2 * nz + 2 * NBC + NST;
    for (int c = tid; c < total; c += NT) {
      int i = c;
      if (i < ND) {
        const int row = i / DPR, part = i % DPR, per = 16 / (int)sizeof(DT), ch = d0 + part * per;
        const int ok = (t0 + row < L) ? max(0, min(16, (Din - ch) * (int)sizeof(DT))) : 0;
        cp_async16(&r.delta[row][part * per], delta + ((long long)b * L + min(t0 + row, L - 1)) * Din + min(ch, Din - per), ok);
        continue;
      }
      i -= ND;
      if (i < 2 * N16 + 2 * nz) {
        const int which = i / N16, j = i % N16, row = j / CPR, part = j % CPR, ch = d0 + part * 8;
        const int ok = (t0 + row < L) ? max(0, min(16, (Din - ch) * 2)) : 0;
        const bf16* src = which == 0 ? u : which == 1 ? dout : which == 2 ? z : y_pre;
        bf16* dst = which == 0 ? &r.u[row][part * 8] : which == 1 ? &r.dout[row][part * 8] : which == 2 ? &r.z[row][part * 8] : &r.yp[row][part * 8];
        cp_async16(dst, src + ((long long)b * L + min(t0 + row, L - 1)) * Din + min(ch, Din - 8), ok);
        continue;
      }
      i -= 2 * N16 + 2 * nz;
      if (i < 2 * NBC) {
        const int which = i / NBC, j = i % NBC, row = j / 4, part = j % 4;
        const int ok = (t0 + row < L) ? 16 : 0;
        const float* src = (which == 0 ? Bm : Cm) + ((long long)b * L + min(t0 + row, L - 1)) * NS + part * 4;
        cp_async16(which == 0 ? &r.B[row][part * 4] : &r.C[row][part * 4], src, ok);
        continue;
      }
      i -= 2 * NBC;
      {
        const int g = i / CB, chn = i % CB;
        const int ok = (d0 + chn < Din) ? 16 : 0;
        cp_async16(&r.st[g][chn][0], &state[state_off(b, nsub, tile, g * 4, Din, min(d0 + chn, Din - 1))], ok);
      }
    }
    cp_async_commit();
  };
  if (piped) issue_tile(nsub - 1, 0);
  for (int tile = nsub - 1; tile >= 0; --tile) {
    const int t0 = tile * SUB;
    const int buf = (nsub - 1 - tile) & 1;
    if (piped) {
      if (tile > 0) { issue_tile(tile - 1, buf ^ 1); cp_async_wait<1>(); }
      else cp_async_wait<0>();
      __syncthreads();   // this tile's copies, issued by all threads, are visible to all
    }
    const RawTile<DT>& rt = raw[buf];
    float sp[RPT];  // d softplus / d raw for the rows this thread stages (and writes back)
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int t = w + NW * j;
      const bool ok = dok && t0 + t < L;
      const long long off = ((long long)b * L + t0 + t) * Din + d;
      float dtv = ok ? (piped ? (float)rt.delta[t][lane] : ld(delta, off)) : 0.f;
      sp[j] = 1.f;
      if (softplus) {
        const float raw = dtv + bias;
        sp[j] = raw > 20.f ? 1.f : sigmoidf(raw);
        dtv = ok ? softplusf(raw) : 0.f;
      }
      float g = ok ? __bfloat162float(piped ? rt.dout[t][lane] : dout[off]) : 0.f;
      if (z && ok) {
        const float zv = __bfloat162float(piped ? rt.z[t][lane] : z[off]), sg = sigmoidf(zv);
        if (dz) dz[off] = __float2bfloat16_rn(g * __bfloat162float(piped ? rt.yp[t][lane] : y_pre[off]) * sg * (1.f + zv * (1.f - sg)));
        g *= zv * sg;
      }
      s.dt[t][lane] = dtv;
      s.u[t][lane] = ok ? __bfloat162float(piped ? rt.u[t][lane] : u[off]) : 0.f;
      s.dy[t][lane] = g;
    }
#pragma unroll
    for (int j = 0; j < BCPT; ++j) {
      const int i = tid + NT * j, t = t0 + i / NS;
      const long long off = ((long long)b * L + t) * NS + (i % NS);
      s.B[i / NS][i % NS] = t < L ? (piped ? rt.B[i / NS][i % NS] : Bm[off]) : 0.f;
      s.C[i / NS][i % NS] = t < L ? (piped ? rt.C[i / NS][i % NS] : Cm[off]) : 0.f;
    }
    float h0[QS];
#pragma unroll
    for (int k = 0; k < QS; ++k) h0[k] = 0.f;
    if (dok) {
      if (piped) ldv<QS>(h0, &rt.st[(w * QS) >> 2][lane][(w * QS) & 3]);
      else ldv<QS>(h0, &state[state_off(b, nsub, tile, w * QS, Din, d)]);
    }
    __syncthreads();
    if (tile > 0 && !piped) {  // warm L1 with the rows of the tile processed next (one tile earlier in time)
#pragma unroll
      for (int j = 0; j < RPT; ++j) {
        const long long off = ((long long)b * L + t0 - SUB + w + NW * j) * Din + d;
        if (dok) {
          prefetch_near(delta + off);
          prefetch_near(u + off);
          prefetch_near(dout + off);
          if (z) {
            prefetch_near(z + off);
            prefetch_near(y_pre + off);
          }
        }
      }
      if (dok) prefetch_near(&state[state_off(b, nsub, tile - 1, w * QS, Din, d)]);
      if (tid < 2 * SUB) {
        const long long off = ((long long)b * L + t0 - SUB + (tid >> 1)) * NS;
        prefetch_near((tid & 1) ? Cm + off : Bm + off);
      }
    }
    float hs[SUB][QS];
    {
      float hh[QS];
#pragma unroll
      for (int k = 0; k < QS; ++k) hh[k] = h0[k];
#pragma unroll
      for (int t = 0; t < SUB; ++t) {
        const float dt = s.dt[t][lane], dtu = dt * s.u[t][lane];
        float bb[QS];
        ldv<QS>(bb, &s.B[t][w * QS]);
#pragma unroll
        for (int k = 0; k < QS; ++k) {
          hh[k] = fmaf(ex2(dt * a2[k]), hh[k], dtu * bb[k]);
          hs[t][k] = hh[k];
        }
      }
    }
#pragma unroll
    for (int t = SUB - 1; t >= 0; --t) {
      const float dt = s.dt[t][lane], uu = s.u[t][lane], gy = s.dy[t][lane], dtu = dt * uu;
      float bb[QS], cc[QS];
      ldv<QS>(bb, &s.B[t][w * QS]);
      ldv<QS>(cc, &s.C[t][w * QS]);
      float v[2 * QS], ddt_p = 0.f, du_p = 0.f;
#pragma unroll
      for (int k = 0; k < QS; ++k) {
        const float gh = fmaf(cc[k], gy, cr[k]);  // dL/dh_t
        const float hprev = t > 0 ? hs[t - 1][k] : h0[k];
        const float gha = gh * ex2(dt * a2[k]);
        dAa[k] = fmaf(gha * hprev, dt, dAa[k]);
        ddt_p = fmaf(gha * hprev, ar[k], ddt_p);
        du_p = fmaf(gh, bb[k], du_p);
        v[k] = gh * dtu;
        v[QS + k] = gy * hs[t][k];
        cr[k] = gha;
      }
      s.pddt[w][t][lane] = fmaf(du_p, uu, ddt_p);  // d(dt * B * u) / d dt = B * u
      s.pdu[w][t][lane] = du_p * dt;
      if constexpr (QS == 4) {
        const float p = reduce8(v, lane);
        if ((lane & 3) == 0) {
          const int idx = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
          if (idx < 4) s.dB[t][w * QS + idx] = p;
          else s.dC[t][w * QS + idx - 4] = p;
        }
      } else {
        const float p = reduce4(v, lane);
        if ((lane & 7) == 0) {
          const int idx = ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1);
          if (idx < 2) s.dB[t][w * QS + idx] = p;
          else s.dC[t][w * QS + idx - 2] = p;
        }
      }
      if (w == 0) dDa = fmaf(gy, uu, dDa);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int t = w + NW * j;
      if (dok && t0 + t < L) {
        const long long off = ((long long)b * L + t0 + t) * Din + d;
        float g = 0.f, gu = dsk * s.dy[t][lane];
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          g += s.pddt[q][t][lane];
          gu += s.pdu[q][t][lane];
        }
        g *= sp[j];
        st(ddelta, off, g);
        dbias += g;
        du[off] = __float2bfloat16_rn(gu);
      }
    }
#pragma unroll
    for (int j = 0; j < BCPT; ++j) {
      const int i = tid + NT * j, t = t0 + i / NS;
      if (t < L) {
        const long long off = ((((long long)b * nblk + blockIdx.x) * L) + t) * NS + (i % NS);
        dB_part[off] = s.dB[i / NS][i % NS];
        dC_part[off] = s.dC[i / NS][i % NS];
      }
    }
    __syncthreads();
  }
  if (dok) {
#pragma unroll
    for (int k = 0; k < QS; ++k) atomicAdd(&dA[(long long)d * NS + w * QS + k], dAa[k]);
    if (w == 0 && dD) atomicAdd(&dD[d], dDa);
    if (ddelta_bias) atomicAdd(&ddelta_bias[d], dbias);
  }
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

int s6_channel_blocks(int Din) { return (Din + CB - 1) / CB; }
int s6_num_chunks(int L) { return (L + SUB - 1) / SUB; }

void s6_set_states_per_thread(int fwd_qs, int bwd_qs) {
  if ((fwd_qs != 2 && fwd_qs != 4) || (bwd_qs != 2 && bwd_qs != 4))
    throw std::runtime_error("s6_scan: states per thread must be 2 or 4");
  g_fwd_qs = fwd_qs;
  g_bwd_qs = bwd_qs;
}

#define S6_FWD(DT, QS)                                                                                               \
  s6_fwd_kernel<DT, QS><<<grid, Shape<QS>::NT, 0, st>>>((const bf16*)u, (const DT*)delta, delta_bias, softplus ? 1 : 0, \
                                                        A, Bm, Cm, Dv, (const bf16*)z, (bf16*)y_pre, (bf16*)out, state, L, Din)
#define S6_BWD(DT, QS)                                                                                               \
  s6_bwd_kernel<DT, QS><<<grid, Shape<QS>::NT, piped ? 2 * sizeof(RawTile<DT>) : 0, st>>>((const bf16*)u, (const DT*)delta, delta_bias, softplus ? 1 : 0, \
                                                        A, Bm, Cm, Dv, (const bf16*)z, (const bf16*)y_pre,            \
                                                        (const bf16*)dout, state, (bf16*)du, (DT*)ddelta, dA, dB_part, \
                                                        dC_part, dD, (bf16*)dz, ddelta_bias, L, Din, piped)

void s6_scan_fwd(const void* u, const void* delta, bool delta_bf16, const float* delta_bias, bool softplus,
                 const float* A, const float* Bm, const float* Cm, const float* Dv, const void* z, void* y_pre, void* out,
                 float* state, int batch, int L, int Din, int N, cudaStream_t st) {
  if (N != NS) throw std::runtime_error("s6_scan: state dimension must be 16");
  dim3 grid(s6_channel_blocks(Din), batch);
  const bool q2 = g_fwd_qs == 2;
  if (delta_bf16) {
    if (q2) S6_FWD(bf16, 2); else S6_FWD(bf16, 4);
  } else {
    if (q2) S6_FWD(float, 2); else S6_FWD(float, 4);
  }
  check("s6_scan_fwd");
}

void s6_scan_bwd(const void* u, const void* delta, bool delta_bf16, const float* delta_bias, bool softplus,
                 const float* A, const float* Bm, const float* Cm, const float* Dv, const void* z, const void* y_pre,
                 const void* dout, const float* state, void* du, void* ddelta, float* dA, float* dB_part, float* dC_part,
                 float* dD, void* dz, float* ddelta_bias, int batch, int L, int Din, int N, cudaStream_t st) {
  if (N != NS) throw std::runtime_error("s6_scan: state dimension must be 16");
  if (z && !y_pre) throw std::runtime_error("s6_scan_bwd: the gate's backward needs y_pre");
  dim3 grid(s6_channel_blocks(Din), batch);
  const bool q2 = g_bwd_qs == 2;
  // input tiles are copied one tile ahead when the rows allow 16-byte copies (static + dynamic shared memory of the
  // four-states-per-thread variant stays under the 48 KB that need no opt-in)
  const int piped = (!q2 && Din % 8 == 0) ? 1 : 0;
  if (delta_bf16) {
    if (q2) S6_BWD(bf16, 2); else S6_BWD(bf16, 4);
  } else {
    if (q2) S6_BWD(float, 2); else S6_BWD(float, 4);
  }
  check("s6_scan_bwd");
}

}  // namespace b200
