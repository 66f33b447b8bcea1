// Memory-bound fused kernels of the GPT training step (torch-free interface). All tensors are
// row-major and dense unless a leading dimension is given; "bf16" pointers are __nv_bfloat16.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {

// y = x * rsqrt(mean(x^2) + eps)                                  x, y : [R][C]
void rmsnorm_fwd(const void* x, void* y, int R, int C, float eps, cudaStream_t s);

// x_mix = lam[0] * (x + skip_w[0] * skip) + lam[1] * x0 ;  xn = rmsnorm(x_mix)
// skip / skip_w may be null (no skip term); x0 may be null (then lam is ignored and x_mix = x (+skip)).
void mix_norm_fwd(const void* x, const void* x0, const void* skip, const float* lam, const float* skip_w,
                  void* x_mix, void* xn, int R, int C, float eps, cudaStream_t s);

// out = dres + d/dx[ rmsnorm(x) ] applied to dy     (dres may be null)
void norm_bwd_add(const void* dy, const void* x, const void* dres, void* out, int R, int C, float eps,
                  cudaStream_t s);

// Backward of the mix above given dmix = dL/dx_mix:
//   dx = lam0 * dmix ; dskip = lam0 * skip_w * dmix ; dx0_acc += lam1 * dmix  (fp32 accumulator)
//   dlam[0] += sum(dmix * (x + skip_w*skip)) ; dlam[1] += sum(dmix * x0) ; dskip_w += sum(lam0 * dmix * skip)
void mix_bwd(const void* dmix, const void* x, const void* x0, const void* skip, const float* lam,
             const float* skip_w, void* dx, void* dskip, float* dx0_acc, float* dlam, float* dskip_w, const void* dx_add,
             int R, int C, cudaStream_t s);   // dx_add (bf16, optional) is added to dx before it is rounded

// qkv [T][3][H][D] -> out [T][3][H][D]:  q,k <- rope(rmsnorm_head(q,k)) ; v <- lam[0]*v + lam[1]*ve
// cos/sin : fp32 [>=T][D/2], position = row index. ve ([T][H*D]) may be null.
void qkv_post_fwd(const void* qkv, const void* ve, const float* lam, const float* cos, const float* sin, void* out,
                  int T, int H, int D, float eps, cudaStream_t s);

// dq : fp32 [T][H][D] ; dk, dv : bf16 [T][H][D] ; writes dqkv [T][3][H][D] (bf16), dve [T][H*D] (bf16, nullable),
// accumulates dlam[2] (fp32).
void qkv_post_bwd(const float* dq, const void* dk, const void* dv, const void* qkv, const void* ve,
                  const float* lam, const float* cos, const float* sin, void* dqkv, void* dve, float* dlam, int T,
                  int H, int D, float eps, cudaStream_t s);

// out[t] = table[idx[t]]  (bf16 rows of C elements); normalize != 0 applies rmsnorm to each gathered row.
void embed_gather(const int* idx, const void* table, void* out, int T, int C, int normalize, float eps,
                  cudaStream_t s);
// grad_table[idx[t]] += src[t] (+ src2[t] when given)   (16-byte fp32 vector atomics; src bf16 or fp32 by src_is_f32)
void embed_scatter_add(const int* idx, const void* src, const void* src2, int src_is_f32, float* grad_table, int T, int C,
                       cudaStream_t s);

// out = fp8(x * scale) ; in_kind: 0 = bf16, 1 = fp32 ; out_kind: 0 = e4m3, 1 = e5m2
// Per-token document bounds of a packed token stream: doc_start[i] = last position <= i holding `bos` (position 0
// always starts a document), doc_end[i] = first such position > i, or T.
void doc_bounds(const long long* tokens, long long bos, int* doc_start, int* doc_end, int T, cudaStream_t s);
void cast_fp8(const void* x, void* out, float scale, long long n, int in_kind, int out_kind, cudaStream_t s);

// Soft-capped cross entropy over bf16 logits [T][V]:  z = cap * sigmoid(logit / div),
// z = cap * sigmoid((logit + shift) / div).
// loss_rows[t] = sum_k w_k (logsumexp(z_t) - z_t[target_{t+k}]) * loss_scale over k < n_predict with t + k < T (w = mtp_w,
// {1} when null: plain next-token loss); grad (e5m2) = dL/dlogit * grad_scale.
// Targets outside [0, V) are ignored (with n_predict = 1: zero loss and gradient). grad may be null (evaluation).
// grad_is_bf16 selects a bf16 gradient buffer instead of e5m2.
// Keep exp(z) of the row in shared memory between the two passes (one SFU op less per element, half the occupancy).
void softcap_ce_set_cache(bool on);
void softcap_ce(const void* logits, const long long* targets, float* loss_rows, void* grad, int grad_is_bf16, int T,
                int V, long long ld, float cap, float div, float shift, float loss_scale, float grad_scale,
                const float* mtp_w, int n_predict, cudaStream_t s);

// ---- optimizer pieces -------------------------------------------------------------------------
// Adam (bias-corrected, decoupled weight decay wd*lr) over n elements. p : fp32 or bf16 (p_is_bf16);
// g : fp32 or bf16 (g_is_bf16) ; m, v : fp32. lr, step-dependent corrections are passed as scalars.
// shadow (optional): the low-precision copy of the updated parameter that the forward GEMMs read, written in the
// same pass: shadow_kind 1 = bf16, 2 = e4m3 of (p * shadow_scale), 0 = none.
void adam_step(void* p, int p_is_bf16, const void* g, int g_is_bf16, float* m, float* v, long long n, float lr,
               float beta1, float beta2, float eps, float wd, float bias1, float bias2, float grad_scale,
               void* shadow, int shadow_kind, float shadow_scale, cudaStream_t s);

// Muon momentum: buf = mu*buf + (1-mu)*g ; u = nesterov ? (1-mu)*g + mu*buf : buf ; out_bf16 = u ; also
// accumulates sum(u^2) into sumsq[0] (fp32) for the Frobenius normalisation.
void muon_momentum(const float* g, float* buf, void* out_bf16, float* sumsq, long long n, int nmat, float mu,
                   int nesterov, float grad_scale, cudaStream_t s);   // stacks [nmat][n], sumsq [nmat]
// x_bf16 *= 1 / (sqrt(sumsq[0]) + eps)
void scale_by_inv_norm(void* x_bf16, const float* sumsq, long long n, float eps, cudaStream_t s);
// p (fp32) += alpha * u (bf16) ; optionally also writes the bf16 copy p_bf16 used by the forward GEMMs
void axpy_bf16_to_f32(float* p, const void* u_bf16, void* p_bf16, long long n, float alpha, cudaStream_t s);

// ---- RMS norm + rotary of the current speedrun GPT (norm_rope.cu): x [batch, T, H, D] bf16 with element strides st
// (between tokens; batch entries are T * st apart) and sh (between heads), tables [T_max, tab_w] bf16 (tab_w = D, or 2 D
// for the paired-head layout), y / dx / dy contiguous [batch * T * H, D], rstd [batch * T * H].
void norm_rope_fwd(const void* x, long long st, long long sh, const void* f1, const void* f2, int tab_w, void* y, float* rstd,
                   long long rows, int H, int T, int D, float eps, cudaStream_t s);
void norm_rope_bwd(const void* x, long long st, long long sh, const void* f1, const void* f2, int tab_w, const float* rstd,
                   const void* dy, void* dx, long long rows, int H, int T, int D, cudaStream_t s);

// ---- row-scaled add and three-term linear combination (rowops.cu); all activations bf16
void rowscale_add_fwd(const void* a, long long st, long long sh, const void* g, const void* b, void* out, long long rows, int H,
                      int D, cudaStream_t s);
void rowscale_add_bwd(const void* g, const void* b, const void* dout, void* db, void* dg, long long rows, int D, cudaStream_t s);
void lincomb3_fwd(const void* x, const void* y, const void* z, const float* c, void* out, long long n, cudaStream_t s);
void lincomb3_bwd(const void* x, const void* y, const void* z, const float* c, const void* dout, void* dx, void* dy, void* dz,
                  float* dc, long long n, cudaStream_t s);

// ---- NorMuon (normuon.cu) ---------------------------------------------------------------------
// v : stack [nmat][R][C] (bf16 or fp32). red_cols != 0: statistics per row (reduced over the C columns), else per column.
// stat : scratch [nmat][R or C], receives the per-row / per-column scale; second : running second moment, same shape.
void normuon_scales(const void* v, int v_is_bf16, float* stat, float* second, int nmat, int R, int C, int red_cols,
                    float beta2, cudaStream_t s);
// p -= p * [u * p >= 0] * wd_lr + u * lr with u = v * scale (scale may be null). p fp32, or bf16 with an optional
// uint16 mantissa buffer (p and mant together are one fp32 number). lr_mat / wd_mat (optional): values per matrix.
void adam_cautious(void* p, int p_is_bf16, const void* g, int g_is_bf16, float* m, float* v, long long n, float b1, float b2,
                   float eps, float step_size, float wd_lr, cudaStream_t s);
void normuon_update(void* p, int p_is_bf16, unsigned short* mant, const void* v, int v_is_bf16, const float* scale,
                    int nmat, int R, int C, int scale_per_row, float lr, float wd_lr, const float* lr_mat,
                    const float* wd_mat, cudaStream_t s);

}  // namespace b200
