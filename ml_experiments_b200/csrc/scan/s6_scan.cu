// S6 (Mamba-1) selective scan, forward and backward.
//
//   dt_t[d]  = softplus(delta_t[d] + delta_bias[d])            (both optional: plain delta when softplus is off)
//   h_t[d,n] = exp(dt_t[d] * A[d,n]) * h_{t-1}[d,n] + dt_t[d] * B_t[n] * u_t[d]
//   y_t[d]   = sum_n C_t[n] * h_t[d,n] + D[d] * u_t[d] ;   out = y * silu(z)
//
// Thread mapping: a block owns 32 channels; lane = channel, warp = one quarter of the 16 states (4 states in registers).
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
constexpr int QS = 4;     // states per thread
constexpr int CB = 32;    // channels per block (= lanes)
constexpr int SUB = 16;   // time steps per tile and per state checkpoint
constexpr int NT = 128;   // threads per block
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ float ld(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

struct FwdSmem {
  float dt[SUB][CB];
  float u[SUB][CB];
  float B[SUB][NS];
  float C[SUB][NS];
  float yp[NS / QS][SUB][CB];
};

// grid (ceil(Din / 32), batch), 128 threads. DT = element type of delta (fp32 or bf16).
template <typename DT>
__global__ void __launch_bounds__(NT, 8)
s6_fwd_kernel(const bf16* __restrict__ u, const DT* __restrict__ delta, const float* __restrict__ delta_bias,
              int softplus, const float* __restrict__ A, const float* __restrict__ Bm, const float* __restrict__ Cm,
              const float* __restrict__ Dv, const bf16* __restrict__ z, bf16* __restrict__ y_pre,
              bf16* __restrict__ out, float* __restrict__ state, int L, int Din) {
  __shared__ __align__(16) FwdSmem s;
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
  // staging registers for the next tile: the thread covers rows w + 4j of the [16][32] tiles and two B / C elements
  float pdt[SUB / 4], pu[SUB / 4], pz[SUB / 4], pB[2], pC[2];
  auto fetch = [&](int tile) {
    const int t0 = tile * SUB;
#pragma unroll
    for (int j = 0; j < SUB / 4; ++j) {
      const int t = t0 + w + 4 * j;
      const bool ok = dok && t < L;
      const long long off = ((long long)b * L + t) * Din + d;
      pdt[j] = ok ? ld(delta, off) : 0.f;
      pu[j] = ok ? __bfloat162float(u[off]) : 0.f;
      pz[j] = (ok && z) ? __bfloat162float(z[off]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
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
    for (int j = 0; j < SUB / 4; ++j) {
      const int t = w + 4 * j;
      float dtv = pdt[j];
      if (softplus) dtv = (dok && t0 + t < L) ? softplusf(dtv + bias) : 0.f;
      s.dt[t][lane] = dtv;
      s.u[t][lane] = pu[j];
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + NT * j;
      s.B[i / NS][i % NS] = pB[j];
      s.C[i / NS][i % NS] = pC[j];
    }
    float zc[SUB / 4];  // this tile's gate inputs (the staging registers are about to be refilled)
#pragma unroll
    for (int j = 0; j < SUB / 4; ++j) zc[j] = pz[j];
    __syncthreads();
    if (tile + 1 < nsub) fetch(tile + 1);
    if (state && dok)
      *reinterpret_cast<float4*>(&state[((((long long)b * nsub + tile) * (NS / QS) + w) * Din + d) * QS]) =
          make_float4(h[0], h[1], h[2], h[3]);
#pragma unroll
    for (int t = 0; t < SUB; ++t) {
      const float dt = s.dt[t][lane], dtu = dt * s.u[t][lane];
      const float4 b4 = *reinterpret_cast<const float4*>(&s.B[t][w * QS]);
      const float4 c4 = *reinterpret_cast<const float4*>(&s.C[t][w * QS]);
      const float bb[QS] = {b4.x, b4.y, b4.z, b4.w}, cc[QS] = {c4.x, c4.y, c4.z, c4.w};
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
    for (int j = 0; j < SUB / 4; ++j) {
      const int t = w + 4 * j;
      if (dok && t0 + t < L) {
        const long long off = ((long long)b * L + t0 + t) * Din + d;
        const float yv = s.yp[0][t][lane] + s.yp[1][t][lane] + s.yp[2][t][lane] + s.yp[3][t][lane] + dsk * s.u[t][lane];
        if (y_pre) y_pre[off] = __float2bfloat16_rn(yv);
        float o = yv;
        if (z) o = yv * zc[j] * sigmoidf(zc[j]);
        out[off] = __float2bfloat16_rn(o);
      }
    }
    __syncthreads();
  }
}

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

// grid (ceil(Din / 32), batch), 128 threads. dout is the gradient of `out`; with z given the gate's backward is applied
// here (dy = dout * silu(z), dz = dout * y_pre * silu'(z)).
template <typename DT>
__global__ void __launch_bounds__(NT, 4)
s6_bwd_kernel(const bf16* __restrict__ u, const DT* __restrict__ delta, const float* __restrict__ delta_bias,
              int softplus, const float* __restrict__ A, const float* __restrict__ Bm, const float* __restrict__ Cm,
              const float* __restrict__ Dv, const bf16* __restrict__ z, const bf16* __restrict__ y_pre,
              const bf16* __restrict__ dout, const float* __restrict__ state, bf16* __restrict__ du,
              DT* __restrict__ ddelta, float* __restrict__ dA, float* __restrict__ dB_part,
              float* __restrict__ dC_part, float* __restrict__ dD, bf16* __restrict__ dz,
              float* __restrict__ ddelta_bias, int L, int Din) {
  __shared__ __align__(16) BwdSmem s;
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
  for (int tile = nsub - 1; tile >= 0; --tile) {
    const int t0 = tile * SUB;
    float sp[SUB / 4];  // d softplus / d raw for the rows this thread stages (and writes back)
#pragma unroll
    for (int j = 0; j < SUB / 4; ++j) {
      const int t = w + 4 * j;
      const bool ok = dok && t0 + t < L;
      const long long off = ((long long)b * L + t0 + t) * Din + d;
      float dtv = ok ? ld(delta, off) : 0.f;
      sp[j] = 1.f;
      if (softplus) {
        const float raw = dtv + bias;
        sp[j] = raw > 20.f ? 1.f : sigmoidf(raw);
        dtv = ok ? softplusf(raw) : 0.f;
      }
      float g = ok ? __bfloat162float(dout[off]) : 0.f;
      if (z && ok) {
        const float zv = __bfloat162float(z[off]), sg = sigmoidf(zv);
        if (dz) dz[off] = __float2bfloat16_rn(g * __bfloat162float(y_pre[off]) * sg * (1.f + zv * (1.f - sg)));
        g *= zv * sg;
      }
      s.dt[t][lane] = dtv;
      s.u[t][lane] = ok ? __bfloat162float(u[off]) : 0.f;
      s.dy[t][lane] = g;
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + NT * j, t = t0 + i / NS;
      const long long off = ((long long)b * L + t) * NS + (i % NS);
      s.B[i / NS][i % NS] = t < L ? Bm[off] : 0.f;
      s.C[i / NS][i % NS] = t < L ? Cm[off] : 0.f;
    }
    float4 h04 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (dok)
      h04 = *reinterpret_cast<const float4*>(&state[((((long long)b * nsub + tile) * (NS / QS) + w) * Din + d) * QS]);
    const float h0[QS] = {h04.x, h04.y, h04.z, h04.w};
    __syncthreads();
    if (tile > 0) {  // warm L2 with the rows of the tile processed next (one tile earlier in time)
#pragma unroll
      for (int j = 0; j < SUB / 4; ++j) {
        const long long off = ((long long)b * L + t0 - SUB + w + 4 * j) * Din + d;
        if (dok) {
          prefetch_l2(delta + off);
          prefetch_l2(u + off);
          prefetch_l2(dout + off);
          if (z) {
            prefetch_l2(z + off);
            prefetch_l2(y_pre + off);
          }
        }
      }
      if (dok) prefetch_l2(&state[((((long long)b * nsub + tile - 1) * (NS / QS) + w) * Din + d) * QS]);
      if (tid < 2 * SUB) {
        const long long off = ((long long)b * L + t0 - SUB + (tid >> 1)) * NS;
        prefetch_l2((tid & 1) ? Cm + off : Bm + off);
      }
    }
    float hs[SUB][QS];
    {
      float hh[QS] = {h0[0], h0[1], h0[2], h0[3]};
#pragma unroll
      for (int t = 0; t < SUB; ++t) {
        const float dt = s.dt[t][lane], dtu = dt * s.u[t][lane];
        const float4 b4 = *reinterpret_cast<const float4*>(&s.B[t][w * QS]);
        const float bb[QS] = {b4.x, b4.y, b4.z, b4.w};
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
      const float4 b4 = *reinterpret_cast<const float4*>(&s.B[t][w * QS]);
      const float4 c4 = *reinterpret_cast<const float4*>(&s.C[t][w * QS]);
      const float bb[QS] = {b4.x, b4.y, b4.z, b4.w}, cc[QS] = {c4.x, c4.y, c4.z, c4.w};
      float v[8], ddt_p = 0.f, du_p = 0.f;
#pragma unroll
      for (int k = 0; k < QS; ++k) {
        const float gh = fmaf(cc[k], gy, cr[k]);  // dL/dh_t
        const float hprev = t > 0 ? hs[t - 1][k] : h0[k];
        const float gha = gh * ex2(dt * a2[k]);
        dAa[k] = fmaf(gha * hprev, dt, dAa[k]);
        ddt_p = fmaf(gha * hprev, ar[k], ddt_p);
        du_p = fmaf(gh, bb[k], du_p);
        v[k] = gh * dtu;
        v[4 + k] = gy * hs[t][k];
        cr[k] = gha;
      }
      s.pddt[w][t][lane] = fmaf(du_p, uu, ddt_p);  // d(dt * B * u) / d dt = B * u
      s.pdu[w][t][lane] = du_p * dt;
      const float p = reduce8(v, lane);
      if ((lane & 3) == 0) {
        const int idx = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
        if (idx < 4) s.dB[t][w * QS + idx] = p;
        else s.dC[t][w * QS + idx - 4] = p;
      }
      if (w == 0) dDa = fmaf(gy, uu, dDa);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < SUB / 4; ++j) {
      const int t = w + 4 * j;
      if (dok && t0 + t < L) {
        const long long off = ((long long)b * L + t0 + t) * Din + d;
        const float g = (s.pddt[0][t][lane] + s.pddt[1][t][lane] + s.pddt[2][t][lane] + s.pddt[3][t][lane]) * sp[j];
        st(ddelta, off, g);
        dbias += g;
        du[off] = __float2bfloat16_rn(s.pdu[0][t][lane] + s.pdu[1][t][lane] + s.pdu[2][t][lane] + s.pdu[3][t][lane] +
                                      dsk * s.dy[t][lane]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
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

void s6_scan_fwd(const void* u, const void* delta, bool delta_bf16, const float* delta_bias, bool softplus,
                 const float* A, const float* Bm, const float* Cm, const float* Dv, const void* z, void* y_pre, void* out,
                 float* state, int batch, int L, int Din, int N, cudaStream_t st) {
  if (N != NS) throw std::runtime_error("s6_scan: state dimension must be 16");
  dim3 grid(s6_channel_blocks(Din), batch);
  if (delta_bf16)
    s6_fwd_kernel<bf16><<<grid, NT, 0, st>>>((const bf16*)u, (const bf16*)delta, delta_bias, softplus ? 1 : 0, A, Bm, Cm, Dv,
                                             (const bf16*)z, (bf16*)y_pre, (bf16*)out, state, L, Din);
  else
    s6_fwd_kernel<float><<<grid, NT, 0, st>>>((const bf16*)u, (const float*)delta, delta_bias, softplus ? 1 : 0, A, Bm, Cm, Dv,
                                              (const bf16*)z, (bf16*)y_pre, (bf16*)out, state, L, Din);
  check("s6_scan_fwd");
}

void s6_scan_bwd(const void* u, const void* delta, bool delta_bf16, const float* delta_bias, bool softplus,
                 const float* A, const float* Bm, const float* Cm, const float* Dv, const void* z, const void* y_pre,
                 const void* dout, const float* state, void* du, void* ddelta, float* dA, float* dB_part, float* dC_part,
                 float* dD, void* dz, float* ddelta_bias, int batch, int L, int Din, int N, cudaStream_t st) {
  if (N != NS) throw std::runtime_error("s6_scan: state dimension must be 16");
  if (z && !y_pre) throw std::runtime_error("s6_scan_bwd: the gate's backward needs y_pre");
  dim3 grid(s6_channel_blocks(Din), batch);
  if (delta_bf16)
    s6_bwd_kernel<bf16><<<grid, NT, 0, st>>>((const bf16*)u, (const bf16*)delta, delta_bias, softplus ? 1 : 0, A, Bm, Cm, Dv,
                                             (const bf16*)z, (const bf16*)y_pre, (const bf16*)dout, state, (bf16*)du,
                                             (bf16*)ddelta, dA, dB_part, dC_part, dD, (bf16*)dz, ddelta_bias, L, Din);
  else
    s6_bwd_kernel<float><<<grid, NT, 0, st>>>((const bf16*)u, (const float*)delta, delta_bias, softplus ? 1 : 0, A, Bm, Cm, Dv,
                                              (const bf16*)z, (const bf16*)y_pre, (const bf16*)dout, state, (bf16*)du,
                                              (float*)ddelta, dA, dB_part, dC_part, dD, (bf16*)dz, ddelta_bias, L, Din);
  check("s6_scan_bwd");
}

}  // namespace b200
