// MIMO-Jacobi state iteration: every iteration of
//     H <- alpha * diffuse(H) + [ it == 0 ? inj_0 : (1 - gamma) * alpha * inj_{it-1} + gamma * inj_it ]
//     inj_it = mix( rot(B, (it + 1) * theta) * x_r ),     diffuse = depthwise 3-tap convolution along the sequence (+ bias)
// in ONE launch, followed by the gated readout  rot(C, n * theta) * H_n  (optionally mixed as sum / difference of the two
// state halves). The reference runs this loop as ~10 PyTorch operators per iteration plus two Triton kernels for the
// rotation and the decay step (src/heuristic_secrets/models/scatter_attention.py:1458-1482, triton_scatter.py:582-667),
// i.e. n_iters round trips of the [batch, R, L, N] state through HBM.
//
// Forward: a CTA owns a window of W sequence positions of one (batch, r) pair, W = tile + 2 * (n_iters - 1): the state
// of the window lives in shared memory (two buffers) for the whole loop; after iteration i the outermost i - 1 positions
// on each side are stale (their neighbours were outside the window), which is exactly the halo, so the tile in the
// middle is exact after n_iters iterations. Threads hold their positions' constants (B, alpha, cos / sin of theta) in
// registers; the rotation angle advances by one complex multiplication per iteration. A thread owns a "quad" of
// channels {2q, 2q+1, 2q+N/2, 2q+1+N/2}: two rotation pairs whose members are also partners of the sum / difference
// mixes, so both mixes are register-local. Nothing but the inputs is read and nothing but the outputs (and, for
// training, the per-iteration states) is written.
//
// Backward: the same windows walked in reverse, one CTA per (window, batch) looping over r so that the gradients of the
// maps shared by all r (theta, alpha, gamma) accumulate in registers. dL/dH_it on the window is propagated through the
// adjoint stencil in shared memory; the parameter gradients of the tile read the saved states.
#include "jacobi.h"

#include "common/per_device.h"

#include <stdexcept>
#include <string>

namespace b200 {
namespace {

constexpr int kThreads = 512;

template <int N, int ITEMS>
struct Geo {
  static constexpr int NQ = N / 4;            // quads per position
  static constexpr int PPI = kThreads / NQ;   // positions covered by one item step of the block
  static constexpr int W = PPI * ITEMS;       // window
  static constexpr int H2 = N / 2;
};

__device__ __forceinline__ void rot(float c, float s, float x0, float x1, float& y0, float& y1) {
  y0 = x0 * c - x1 * s;
  y1 = x0 * s + x1 * c;
}
// adjoint (transpose) of rot
__device__ __forceinline__ void rot_t(float c, float s, float g0, float g1, float& d0, float& d1) {
  d0 = g0 * c + g1 * s;
  d1 = -g0 * s + g1 * c;
}

template <int N, int ITEMS>
__global__ void __launch_bounds__(kThreads) jacobi_fwd_kernel(const JacobiArgs p) {
  using G = Geo<N, ITEMS>;
  extern __shared__ float sm[];
  float* Hc = sm;
  float* Hn = sm + G::W * N;
  const int t = threadIdx.x, q = t % G::NQ, wq = t / G::NQ;
  const int b = blockIdx.z, r = blockIdx.y;
  const int halo = p.n_iters - 1, TL = G::W - 2 * halo;
  const int l0 = blockIdx.x * TL - halo;
  const int ch[4] = {2 * q, 2 * q + 1, 2 * q + G::H2, 2 * q + 1 + G::H2};
  float cw[4][3], cb[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int k = 0; k < 3; ++k) cw[j][k] = p.conv_w[ch[j] * 3 + k];
    cb[j] = p.conv_b[ch[j]];
  }
  const bool di = p.inj_lambda != nullptr;
  const float lam_i = di ? *p.inj_lambda : 0.f;

  float Bq[ITEMS][4], al[ITEMS][4], c1[ITEMS][2], s1[ITEMS][2], c[ITEMS][2], s[ITEMS][2], prev[ITEMS][4], xr[ITEMS], gm[ITEMS];
  bool valid[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int w = k * G::PPI + wq, l = l0 + w;
    valid[k] = l >= 0 && l < p.L;
#pragma unroll
    for (int j = 0; j < 4; ++j) { Bq[k][j] = 0.f; al[k][j] = 0.f; prev[k][j] = 0.f; }
    c1[k][0] = c1[k][1] = 1.f; s1[k][0] = s1[k][1] = 0.f; xr[k] = 0.f; gm[k] = 0.f;
    if (valid[k]) {
      const long long bb = (long long)b * p.b_sb + (long long)r * p.b_sr + (long long)l * p.b_sl;
      const long long row = (long long)b * p.L + l;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        Bq[k][j] = p.Bm[bb + (long long)ch[j] * p.b_sn];
        al[k][j] = p.alpha[row * N + ch[j]];
      }
      sincosf(p.theta[row * G::H2 + q], &s1[k][0], &c1[k][0]);
      sincosf(p.theta[row * G::H2 + q + G::NQ], &s1[k][1], &c1[k][1]);
      xr[k] = p.xr[(long long)b * p.x_sb + (long long)r * p.x_sr + (long long)l * p.x_sl];
      gm[k] = p.gamma[row];
    }
    c[k][0] = c[k][1] = 1.f; s[k][0] = s[k][1] = 0.f;
  }
  for (int i = t; i < G::W * N; i += kThreads) Hc[i] = 0.f;
  __syncthreads();

  for (int it = 0; it < p.n_iters; ++it) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int w = k * G::PPI + wq, l = l0 + w;
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {  // angle (it + 1) * theta
        const float cn = c[k][pr] * c1[k][pr] - s[k][pr] * s1[k][pr];
        s[k][pr] = s[k][pr] * c1[k][pr] + c[k][pr] * s1[k][pr];
        c[k][pr] = cn;
      }
      float rb[4], inj[4];
      rot(c[k][0], s[k][0], Bq[k][0], Bq[k][1], rb[0], rb[1]);
      rot(c[k][1], s[k][1], Bq[k][2], Bq[k][3], rb[2], rb[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) rb[j] *= xr[k];
      if (di) {
        inj[0] = rb[0] - lam_i * rb[2]; inj[1] = rb[1] - lam_i * rb[3];
        inj[2] = rb[0] + lam_i * rb[2]; inj[3] = rb[1] + lam_i * rb[3];
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) inj[j] = rb[j];
      }
      const bool own = w >= halo && w < halo + TL && l < p.L;
      float hn[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float hm = w > 0 ? Hc[(w - 1) * N + ch[j]] : 0.f;
        const float h0 = Hc[w * N + ch[j]];
        const float hp = w < G::W - 1 ? Hc[(w + 1) * N + ch[j]] : 0.f;
        const float cv = cw[j][0] * hm + cw[j][1] * h0 + cw[j][2] * hp + cb[j];
        float v = al[k][j] * cv + (it == 0 ? inj[j] : (1.f - gm[k]) * al[k][j] * prev[k][j] + gm[k] * inj[j]);
        if (!valid[k]) v = 0.f;  // outside the sequence: the zero padding of the convolution
        hn[j] = v;
        prev[k][j] = inj[j];
      }
      *reinterpret_cast<float2*>(Hn + w * N + ch[0]) = make_float2(hn[0], hn[1]);
      *reinterpret_cast<float2*>(Hn + w * N + ch[2]) = make_float2(hn[2], hn[3]);
      if (p.Hs && own) {
        float* dst = p.Hs + ((((long long)it * p.batch + b) * p.R + r) * p.L + l) * N;
        *reinterpret_cast<float2*>(dst + ch[0]) = make_float2(hn[0], hn[1]);
        *reinterpret_cast<float2*>(dst + ch[2]) = make_float2(hn[2], hn[3]);
      }
    }
    __syncthreads();
    float* tmp = Hc; Hc = Hn; Hn = tmp;
  }

  // gated readout of the tile: rot(C, n * theta) * H_n, written in the layout the output projection reads
  const bool dr = p.ro_lambda != nullptr;
  const float lam_r = dr ? *p.ro_lambda : 0.f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int w = k * G::PPI + wq, l = l0 + w;
    if (!(w >= halo && w < halo + TL && l < p.L)) continue;
    const long long cbase = (long long)b * p.c_sb + (long long)r * p.c_sr + (long long)l * p.c_sl;
    float Cq[4], rc[4], g[4], o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) Cq[j] = p.Cm[cbase + (long long)ch[j] * p.c_sn];
    rot(c[k][0], s[k][0], Cq[0], Cq[1], rc[0], rc[1]);
    rot(c[k][1], s[k][1], Cq[2], Cq[3], rc[2], rc[3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) g[j] = rc[j] * Hc[w * N + ch[j]];
    if (dr) {
      o[0] = g[0] - lam_r * g[2]; o[1] = g[1] - lam_r * g[3];
      o[2] = g[0] + lam_r * g[2]; o[3] = g[1] + lam_r * g[3];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = g[j];
    }
    float* dst = p.gated + (((long long)b * p.L + l) * p.R + r) * N;
    *reinterpret_cast<float2*>(dst + ch[0]) = make_float2(o[0], o[1]);
    *reinterpret_cast<float2*>(dst + ch[2]) = make_float2(o[2], o[3]);
  }
}

// sum over the NQ consecutive lanes that share a position (NQ is a power of two <= 32)
template <int NQ>
__device__ __forceinline__ float quad_group_sum(float v) {
#pragma unroll
  for (int o = NQ / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int N, int ITEMS>
__global__ void __launch_bounds__(kThreads) jacobi_bwd_kernel(const JacobiArgs p) {
  using G = Geo<N, ITEMS>;
  extern __shared__ float sm[];
  float* A0 = sm;               // alpha * dL/dH of the window, two buffers used in alternation
  float* A1 = sm + G::W * N;
  const int t = threadIdx.x, q = t % G::NQ, wq = t / G::NQ;
  const int b = blockIdx.y;
  const int n = p.n_iters, halo = n - 1, TL = G::W - 2 * halo;
  const int l0 = blockIdx.x * TL - halo;
  const int ch[4] = {2 * q, 2 * q + 1, 2 * q + G::H2, 2 * q + 1 + G::H2};
  float cw[4][3], cb[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int k = 0; k < 3; ++k) cw[j][k] = p.conv_w[ch[j] * 3 + k];
    cb[j] = p.conv_b[ch[j]];
  }
  const bool di = p.inj_lambda != nullptr, dr = p.ro_lambda != nullptr;
  const float lam_i = di ? *p.inj_lambda : 0.f, lam_r = dr ? *p.ro_lambda : 0.f;

  // constants and accumulators shared by all r
  float al[ITEMS][4], c1[ITEMS][2], s1[ITEMS][2], gm[ITEMS];
  float d_al[ITEMS][4], d_th[ITEMS][2], d_gm[ITEMS];
  bool valid[ITEMS], own[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int w = k * G::PPI + wq, l = l0 + w;
    valid[k] = l >= 0 && l < p.L;
    own[k] = w >= halo && w < halo + TL && l < p.L;
#pragma unroll
    for (int j = 0; j < 4; ++j) { al[k][j] = 0.f; d_al[k][j] = 0.f; }
    c1[k][0] = c1[k][1] = 1.f; s1[k][0] = s1[k][1] = 0.f; gm[k] = 0.f;
    d_th[k][0] = d_th[k][1] = 0.f; d_gm[k] = 0.f;
    if (valid[k]) {
      const long long row = (long long)b * p.L + l;
#pragma unroll
      for (int j = 0; j < 4; ++j) al[k][j] = p.alpha[row * N + ch[j]];
      sincosf(p.theta[row * G::H2 + q], &s1[k][0], &c1[k][0]);
      sincosf(p.theta[row * G::H2 + q + G::NQ], &s1[k][1], &c1[k][1]);
      gm[k] = p.gamma[row];
    }
  }
  float d_cw[4][3], d_cb[4], d_lam_i = 0.f, d_lam_r = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { d_cb[j] = 0.f; d_cw[j][0] = d_cw[j][1] = d_cw[j][2] = 0.f; }

  for (int r = 0; r < p.R; ++r) {
    float Bq[ITEMS][4], c[ITEMS][2], s[ITEMS][2], Gq[ITEMS][4], carry[ITEMS][4], dB[ITEMS][4], xr[ITEMS], d_xr[ITEMS];
    // ---- readout adjoint on the whole window: dL/dH_n, and the gradient of C on the tile
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int w = k * G::PPI + wq, l = l0 + w;
#pragma unroll
      for (int j = 0; j < 4; ++j) { Bq[k][j] = 0.f; Gq[k][j] = 0.f; carry[k][j] = 0.f; dB[k][j] = 0.f; }
      xr[k] = 0.f; d_xr[k] = 0.f;
      c[k][0] = c[k][1] = 1.f; s[k][0] = s[k][1] = 0.f;
#pragma unroll
      for (int pr = 0; pr < 2; ++pr)
        for (int i = 0; i < n; ++i) {  // angle n * theta by the same recurrence as the forward
          const float cn = c[k][pr] * c1[k][pr] - s[k][pr] * s1[k][pr];
          s[k][pr] = s[k][pr] * c1[k][pr] + c[k][pr] * s1[k][pr];
          c[k][pr] = cn;
        }
      if (!valid[k]) continue;
      const long long bb = (long long)b * p.b_sb + (long long)r * p.b_sr + (long long)l * p.b_sl;
      const long long cbase = (long long)b * p.c_sb + (long long)r * p.c_sr + (long long)l * p.c_sl;
      float Cq[4], rc[4], dgt[4], dg[4], Hn[4];
      const float* hsrc = p.Hs + ((((long long)(n - 1) * p.batch + b) * p.R + r) * p.L + l) * N;
      const float* gsrc = p.dgated + (((long long)b * p.L + l) * p.R + r) * N;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        Bq[k][j] = p.Bm[bb + (long long)ch[j] * p.b_sn];
        Cq[j] = p.Cm[cbase + (long long)ch[j] * p.c_sn];
        dgt[j] = gsrc[ch[j]];
        Hn[j] = hsrc[ch[j]];
      }
      xr[k] = p.xr[(long long)b * p.x_sb + (long long)r * p.x_sr + (long long)l * p.x_sl];
      rot(c[k][0], s[k][0], Cq[0], Cq[1], rc[0], rc[1]);
      rot(c[k][1], s[k][1], Cq[2], Cq[3], rc[2], rc[3]);
      if (dr) {
        dg[0] = dgt[0] + dgt[2]; dg[1] = dgt[1] + dgt[3];
        dg[2] = lam_r * (dgt[2] - dgt[0]); dg[3] = lam_r * (dgt[3] - dgt[1]);
        if (own[k]) d_lam_r += rc[2] * Hn[2] * (dgt[2] - dgt[0]) + rc[3] * Hn[3] * (dgt[3] - dgt[1]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) dg[j] = dgt[j];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) Gq[k][j] = dg[j] * rc[j];
      if (own[k]) {
        float dcr[4], dC[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) dcr[j] = dg[j] * Hn[j];
        rot_t(c[k][0], s[k][0], dcr[0], dcr[1], dC[0], dC[1]);
        rot_t(c[k][1], s[k][1], dcr[2], dcr[3], dC[2], dC[3]);
        d_th[k][0] += (float)n * (-dcr[0] * rc[1] + dcr[1] * rc[0]);
        d_th[k][1] += (float)n * (-dcr[2] * rc[3] + dcr[3] * rc[2]);
        float* dst = p.dCm + ((((long long)b * p.R + r) * p.L + l) * N);
        *reinterpret_cast<float2*>(dst + ch[0]) = make_float2(dC[0], dC[1]);
        *reinterpret_cast<float2*>(dst + ch[2]) = make_float2(dC[2], dC[3]);
      }
    }
    // ---- iterations in reverse; Gq = dL/dH_{it+1}
    for (int it = n - 1; it >= 0; --it) {
      float* A = (it & 1) ? A1 : A0;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const int w = k * G::PPI + wq, l = l0 + w;
        float aG[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) aG[j] = valid[k] ? al[k][j] * Gq[k][j] : 0.f;
        *reinterpret_cast<float2*>(A + w * N + ch[0]) = make_float2(aG[0], aG[1]);
        *reinterpret_cast<float2*>(A + w * N + ch[2]) = make_float2(aG[2], aG[3]);
        if (own[k]) {
          if (it > 1) {   // the states the next (earlier) iteration reads: ask for their lines now, no register held
            const float* nxt = p.Hs + ((((long long)(it - 2) * p.batch + b) * p.R + r) * p.L + l) * N;
            asm volatile("prefetch.global.L1 [%0];" ::"l"(nxt + ch[0]));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(nxt + ch[2]));
          }
          // injections of this iteration (angle (it+1) theta) and of the previous one (angle it * theta)
          float rb[4], rbp[4], inj[4], injp[4];
          rot(c[k][0], s[k][0], Bq[k][0], Bq[k][1], rb[0], rb[1]);
          rot(c[k][1], s[k][1], Bq[k][2], Bq[k][3], rb[2], rb[3]);
          float cp[2], sp[2];
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            cp[pr] = c[k][pr] * c1[k][pr] + s[k][pr] * s1[k][pr];
            sp[pr] = s[k][pr] * c1[k][pr] - c[k][pr] * s1[k][pr];
          }
          rot(cp[0], sp[0], Bq[k][0], Bq[k][1], rbp[0], rbp[1]);
          rot(cp[1], sp[1], Bq[k][2], Bq[k][3], rbp[2], rbp[3]);
          if (di) {
            inj[0] = (rb[0] - lam_i * rb[2]) * xr[k]; inj[1] = (rb[1] - lam_i * rb[3]) * xr[k];
            inj[2] = (rb[0] + lam_i * rb[2]) * xr[k]; inj[3] = (rb[1] + lam_i * rb[3]) * xr[k];
            injp[0] = (rbp[0] - lam_i * rbp[2]) * xr[k]; injp[1] = (rbp[1] - lam_i * rbp[3]) * xr[k];
            injp[2] = (rbp[0] + lam_i * rbp[2]) * xr[k]; injp[3] = (rbp[1] + lam_i * rbp[3]) * xr[k];
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) { inj[j] = rb[j] * xr[k]; injp[j] = rbp[j] * xr[k]; }
          }
          // state entering this iteration (H_it; zero for it == 0) at l - 1, l, l + 1
          float dinj[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float hm = 0.f, h0 = 0.f, hp = 0.f;
            if (it > 0) {
              const float* hs = p.Hs + ((((long long)(it - 1) * p.batch + b) * p.R + r) * p.L + l) * N + ch[j];
              h0 = hs[0];
              if (l > 0) hm = hs[-N];
              if (l < p.L - 1) hp = hs[N];
            }
            const float cv = cw[j][0] * hm + cw[j][1] * h0 + cw[j][2] * hp + cb[j];
            const float g = Gq[k][j];
            d_al[k][j] += g * (cv + (it > 0 ? (1.f - gm[k]) * injp[j] : 0.f));
            if (it > 0) d_gm[k] += g * (inj[j] - al[k][j] * injp[j]);
            dinj[j] = (it == 0 ? 1.f : gm[k]) * g + carry[k][j];
            carry[k][j] = it > 0 ? (1.f - gm[k]) * al[k][j] * g : 0.f;
            d_cw[j][0] += aG[j] * hm; d_cw[j][1] += aG[j] * h0; d_cw[j][2] += aG[j] * hp;
            d_cb[j] += aG[j];
          }
          float di_[4];  // gradient of rot(B) * x_r (before the sum / difference mix)
          if (di) {
            di_[0] = dinj[0] + dinj[2]; di_[1] = dinj[1] + dinj[3];
            di_[2] = lam_i * (dinj[2] - dinj[0]); di_[3] = lam_i * (dinj[3] - dinj[1]);
            d_lam_i += rb[2] * xr[k] * (dinj[2] - dinj[0]) + rb[3] * xr[k] * (dinj[3] - dinj[1]);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) di_[j] = dinj[j];
          }
          float drb[4], dBt[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) { drb[j] = di_[j] * xr[k]; d_xr[k] += di_[j] * rb[j]; }
          rot_t(c[k][0], s[k][0], drb[0], drb[1], dBt[0], dBt[1]);
          rot_t(c[k][1], s[k][1], drb[2], drb[3], dBt[2], dBt[3]);
#pragma unroll
          for (int j = 0; j < 4; ++j) dB[k][j] += dBt[j];
          d_th[k][0] += (float)(it + 1) * (-drb[0] * rb[1] + drb[1] * rb[0]);
          d_th[k][1] += (float)(it + 1) * (-drb[2] * rb[3] + drb[3] * rb[2]);
        } else {
          // carry of positions outside the tile is never used; keep the recurrence state consistent anyway
#pragma unroll
          for (int j = 0; j < 4; ++j) carry[k][j] = 0.f;
        }
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {  // angle it * theta for the next (earlier) iteration
          const float cn = c[k][pr] * c1[k][pr] + s[k][pr] * s1[k][pr];
          s[k][pr] = s[k][pr] * c1[k][pr] - c[k][pr] * s1[k][pr];
          c[k][pr] = cn;
        }
      }
      __syncthreads();
      if (it > 0) {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const int w = k * G::PPI + wq;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float am = w > 0 ? A[(w - 1) * N + ch[j]] : 0.f;
            const float a0 = A[w * N + ch[j]];
            const float ap = w < G::W - 1 ? A[(w + 1) * N + ch[j]] : 0.f;
            Gq[k][j] = cw[j][0] * ap + cw[j][1] * a0 + cw[j][2] * am;
          }
        }
      }
    }
    __syncthreads();  // the buffer written by the last iteration is rewritten by the next r only after everyone read it
    // ---- per-r outputs of the tile
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int w = k * G::PPI + wq, l = l0 + w;
      const float sx = quad_group_sum<G::NQ>(own[k] ? d_xr[k] : 0.f);
      if (!own[k]) continue;
      float* dst = p.dBm + ((((long long)b * p.R + r) * p.L + l) * N);
      *reinterpret_cast<float2*>(dst + ch[0]) = make_float2(dB[k][0], dB[k][1]);
      *reinterpret_cast<float2*>(dst + ch[2]) = make_float2(dB[k][2], dB[k][3]);
      if (q == 0) p.dxr[((long long)b * p.R + r) * p.L + l] = sx;
    }
  }
  // ---- outputs shared by all r
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int w = k * G::PPI + wq, l = l0 + w;
    const float sg = quad_group_sum<G::NQ>(own[k] ? d_gm[k] : 0.f);
    if (!own[k]) continue;
    const long long row = (long long)b * p.L + l;
    *reinterpret_cast<float2*>(p.dalpha + row * N + ch[0]) = make_float2(d_al[k][0], d_al[k][1]);
    *reinterpret_cast<float2*>(p.dalpha + row * N + ch[2]) = make_float2(d_al[k][2], d_al[k][3]);
    p.dtheta[row * G::H2 + q] = d_th[k][0];
    p.dtheta[row * G::H2 + q + G::NQ] = d_th[k][1];
    if (q == 0) p.dgamma[row] = sg;
  }
  // ---- diffusion taps, bias and mix weights: block sums, then one atomic per value and block
  __syncthreads();
  float* red = sm;  // [kThreads][18]
  float* mine = red + t * 18;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    mine[j * 4 + 0] = d_cw[j][0]; mine[j * 4 + 1] = d_cw[j][1]; mine[j * 4 + 2] = d_cw[j][2]; mine[j * 4 + 3] = d_cb[j];
  }
  mine[16] = d_lam_i; mine[17] = d_lam_r;
  __syncthreads();
  if (t < G::NQ * 16) {
    const int qq = t / 16, e = t % 16;
    float acc = 0.f;
    for (int i = qq; i < kThreads; i += G::NQ) acc += red[i * 18 + e];
    const int j = e / 4, k = e % 4;
    const int chn = (j & 1) + 2 * qq + (j >= 2 ? G::H2 : 0);
    if (k < 3) atomicAdd(p.dconv_w + chn * 3 + k, acc);
    else atomicAdd(p.dconv_b + chn, acc);
  }
  if (t < 2 && p.dlam) {
    const int e = 16 + t;
    float acc = 0.f;
    for (int i = 0; i < kThreads; ++i) acc += red[i * 18 + e];
    atomicAdd(p.dlam + (e - 16), acc);
  }
}

constexpr int kFwdItems = 4, kBwdItems = 2;

template <int N>
void launch_fwd(const JacobiArgs& a) {
  using G = Geo<N, kFwdItems>;
  const int TL = G::W - 2 * (a.n_iters - 1);
  const size_t smem = 2ull * G::W * N * sizeof(float);
  static PerDeviceOnce cfg;   // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  if (cfg.pending(&dev)) {
    cudaFuncSetAttribute(jacobi_fwd_kernel<N, kFwdItems>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cfg.done(dev);
  }
  dim3 grid((a.L + TL - 1) / TL, a.R, a.batch);
  jacobi_fwd_kernel<N, kFwdItems><<<grid, kThreads, smem, a.stream>>>(a);
}

template <int N>
void launch_bwd(const JacobiArgs& a) {
  using G = Geo<N, kBwdItems>;
  const int TL = G::W - 2 * (a.n_iters - 1);
  size_t smem = 2ull * G::W * N * sizeof(float);
  const size_t red = (size_t)kThreads * 18 * sizeof(float);
  if (smem < red) smem = red;
  static PerDeviceOnce cfg;
  int dev = 0;
  if (cfg.pending(&dev)) {
    cudaFuncSetAttribute(jacobi_bwd_kernel<N, kBwdItems>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cfg.done(dev);
  }
  dim3 grid((a.L + TL - 1) / TL, a.batch);
  jacobi_bwd_kernel<N, kBwdItems><<<grid, kThreads, smem, a.stream>>>(a);
}

void check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

bool jacobi_supported(int N, int n_iters) {
  if (N != 16 && N != 32 && N != 64 && N != 128) return false;
  if (n_iters < 1) return false;
  const int w_bwd = kThreads / (N / 4) * kBwdItems;   // the narrower of the two windows
  return w_bwd - 2 * (n_iters - 1) >= w_bwd / 4;
}

void jacobi_fwd(const JacobiArgs& a) {
  if (!jacobi_supported(a.N, a.n_iters)) throw std::runtime_error("jacobi_fwd: unsupported state size / iteration count");
  switch (a.N) {
    case 16: launch_fwd<16>(a); break;
    case 32: launch_fwd<32>(a); break;
    case 64: launch_fwd<64>(a); break;
    default: launch_fwd<128>(a); break;
  }
  check_launch("jacobi_fwd");
}

void jacobi_bwd(const JacobiArgs& a) {
  if (!jacobi_supported(a.N, a.n_iters)) throw std::runtime_error("jacobi_bwd: unsupported state size / iteration count");
  switch (a.N) {
    case 16: launch_bwd<16>(a); break;
    case 32: launch_bwd<32>(a); break;
    case 64: launch_bwd<64>(a); break;
    default: launch_bwd<128>(a); break;
  }
  check_launch("jacobi_bwd");
}

}  // namespace b200
