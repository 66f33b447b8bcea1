// torch op registrations (namespace b200). The .cu files are torch-free; this file adapts
// at::Tensor arguments to their plain C++ launch structs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include "attn/attn.h"
#include "comm/comm.h"
#include "fused/fused.h"
#include "gather/gather_conv.h"
#include "gather/fused_taps.h"
#include "fused/norm_act.h"
#include "gemm/gemm.h"
#include "mra/mra.h"
#include "scan/s6_scan.h"
#include "scan/jacobi.h"
#include "scan/ssd.h"
#include "window/window_attn.h"
#include "wkv/wkv.h"

namespace {

using at::Tensor;

int gemm_dtype(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return b200::GEMM_BF16;
    case at::kFloat8_e4m3fn: return b200::GEMM_E4M3;
    case at::kFloat8_e5m2: return b200::GEMM_E5M2;
    case at::kFloat: return b200::GEMM_F32;
    default: TORCH_CHECK(false, "b200::gemm: unsupported dtype ", t.scalar_type());
  }
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// c = epilogue(a @ b^T) with per-operand majorness; see csrc/gemm/gemm.h.
void gemm(const Tensor& a, const Tensor& b, Tensor c, const c10::optional<Tensor>& aux, bool a_mn, bool b_mn,
          int64_t epilogue, double alpha, double beta, int64_t split_k, bool accumulate, Tensor status) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "b200::gemm needs CUDA tensors");
  TORCH_CHECK(a.dim() == b.dim() && a.dim() == c.dim() && (a.dim() == 2 || a.dim() == 3), "gemm: rank 2 or 3");
  TORCH_CHECK(a.stride(-1) == 1 && b.stride(-1) == 1 && c.stride(-1) == 1, "gemm: innermost stride must be 1");
  const c10::cuda::CUDAGuard guard(a.device());
  b200::GemmArgs g;
  const int d = a.dim();
  g.batch = d == 3 ? (int)a.size(0) : 1;
  g.M = (int)c.size(-2);
  g.N = (int)c.size(-1);
  g.K = (int)(a_mn ? a.size(-2) : a.size(-1));
  TORCH_CHECK((a_mn ? a.size(-1) : a.size(-2)) == g.M, "gemm: A does not match C rows");
  TORCH_CHECK((b_mn ? b.size(-1) : b.size(-2)) == g.N, "gemm: B does not match C cols");
  TORCH_CHECK((b_mn ? b.size(-2) : b.size(-1)) == g.K, "gemm: A and B disagree on K");
  if (d == 3) TORCH_CHECK(b.size(0) == g.batch && c.size(0) == g.batch, "gemm: batch mismatch");
  g.A = a.data_ptr(); g.B = b.data_ptr(); g.C = c.data_ptr();
  g.lda = a.stride(-2); g.ldb = b.stride(-2); g.ldc = c.stride(-2);
  g.stride_a = d == 3 ? a.stride(0) : 0;
  g.stride_b = d == 3 ? b.stride(0) : 0;
  g.stride_c = d == 3 ? c.stride(0) : 0;
  g.a_mn = a_mn; g.b_mn = b_mn;
  g.a_dtype = gemm_dtype(a); g.b_dtype = gemm_dtype(b); g.c_dtype = gemm_dtype(c);
  TORCH_CHECK(g.a_dtype != b200::GEMM_F32 && g.b_dtype != b200::GEMM_F32, "gemm: inputs must be bf16 or fp8");
  if (aux.has_value()) {
    const Tensor& x = *aux;
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.stride(-1) == 1 && x.dim() == d, "gemm: aux must be bf16");
    TORCH_CHECK(x.size(-2) == g.M && x.size(-1) == g.N, "gemm: aux shape");
    g.aux = x.data_ptr(); g.ldaux = x.stride(-2); g.stride_aux = d == 3 ? x.stride(0) : 0;
  }
  g.epilogue = (int)epilogue; g.alpha = (float)alpha; g.beta = (float)beta;
  g.split_k = (int)split_k; g.accumulate = accumulate;
  g.status = status.data_ptr<int>();
  g.stream = cur_stream();
  b200::gemm_sm100(g);
}


// ---------------------------------------------------------------------------------------------- attention
void fill_thd(const Tensor& t, const char* name, int T, int H, int D) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 3, name, ": expected a CUDA [T, H, D] tensor");
  TORCH_CHECK(t.size(0) == T && t.size(1) == H && t.size(2) == D, name, ": shape mismatch");
  TORCH_CHECK(t.stride(2) == 1 && t.stride(1) == D, name, ": heads must be contiguous (stride(1) == D, stride(2) == 1)");
}

void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor o, Tensor lse, const Tensor& doc_start,
              const Tensor& doc_end, double scale, int64_t window_blocks, Tensor status) {
  const c10::cuda::CUDAGuard guard(q.device());
  b200::AttnArgs a;
  a.T = (int)q.size(0); a.H = (int)q.size(1); a.D = (int)q.size(2);
  fill_thd(q, "q", a.T, a.H, a.D); fill_thd(k, "k", a.T, a.H, a.D); fill_thd(v, "v", a.T, a.H, a.D);
  fill_thd(o, "o", a.T, a.H, a.D);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 &&
              o.scalar_type() == at::kBFloat16, "attention tensors must be bf16");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == (int64_t)a.T * a.H, "lse: fp32 [H, T]");
  TORCH_CHECK(doc_start.scalar_type() == at::kInt && doc_end.scalar_type() == at::kInt && doc_start.numel() == a.T &&
              doc_end.numel() == a.T, "doc_start / doc_end: int32 [T]");
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
  a.ld_q = q.stride(0); a.ld_k = k.stride(0); a.ld_v = v.stride(0); a.ld_o = o.stride(0);
  a.lse = lse.data_ptr<float>();
  a.doc_start = doc_start.data_ptr<int>(); a.doc_end = doc_end.data_ptr<int>();
  a.scale = (float)scale; a.window_blocks = (int)window_blocks;
  a.status = status.data_ptr<int>(); a.stream = cur_stream();
  b200::attn_fwd_sm100(a);
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o,
              const Tensor& lse, Tensor delta, Tensor dq_acc, Tensor dk, Tensor dv, const Tensor& doc_start,
              const Tensor& doc_end, double scale, int64_t window_blocks, Tensor status) {
  const c10::cuda::CUDAGuard guard(q.device());
  b200::AttnArgs a;
  a.T = (int)q.size(0); a.H = (int)q.size(1); a.D = (int)q.size(2);
  fill_thd(q, "q", a.T, a.H, a.D); fill_thd(k, "k", a.T, a.H, a.D); fill_thd(v, "v", a.T, a.H, a.D);
  fill_thd(o, "o", a.T, a.H, a.D); fill_thd(d_o, "do", a.T, a.H, a.D);
  fill_thd(dq_acc, "dq_acc", a.T, a.H, a.D); fill_thd(dk, "dk", a.T, a.H, a.D); fill_thd(dv, "dv", a.T, a.H, a.D);
  TORCH_CHECK(dq_acc.scalar_type() == at::kFloat, "dq_acc must be fp32 (zero-initialised accumulator)");
  TORCH_CHECK(dk.scalar_type() == at::kBFloat16 && dv.scalar_type() == at::kBFloat16 && d_o.scalar_type() == at::kBFloat16,
              "dk, dv, do must be bf16");
  TORCH_CHECK(delta.scalar_type() == at::kFloat && delta.is_contiguous() && delta.numel() == (int64_t)a.T * a.H, "delta: fp32 [H, T]");
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = const_cast<void*>(o.data_ptr());
  a.d_o = d_o.data_ptr(); a.dq_acc = dq_acc.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
  a.ld_q = q.stride(0); a.ld_k = k.stride(0); a.ld_v = v.stride(0); a.ld_o = o.stride(0); a.ld_do = d_o.stride(0);
  a.ld_dq = dq_acc.stride(0); a.ld_dk = dk.stride(0); a.ld_dv = dv.stride(0);
  a.lse = const_cast<float*>(lse.data_ptr<float>()); a.delta = delta.data_ptr<float>();
  a.doc_start = doc_start.data_ptr<int>(); a.doc_end = doc_end.data_ptr<int>();
  a.scale = (float)scale; a.window_blocks = (int)window_blocks;
  a.status = status.data_ptr<int>(); a.stream = cur_stream();
  b200::attn_delta_sm100(a);
  b200::attn_bwd_sm100(a);
}

// ---------------------------------------------------------------------------------------------- fused row kernels
const void* optp(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
const float* optf(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }
void chk_bf16c(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), n, ": contiguous bf16 CUDA tensor expected");
}

void mix_norm_fwd(const Tensor& x, const c10::optional<Tensor>& x0, const c10::optional<Tensor>& skip,
                  const c10::optional<Tensor>& lam, const c10::optional<Tensor>& skip_w,
                  const c10::optional<Tensor>& x_mix, const c10::optional<Tensor>& xn, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x");
  const int C = (int)x.size(-1), R = (int)(x.numel() / C);
  b200::mix_norm_fwd(x.data_ptr(), optp(x0), optp(skip), optf(lam), optf(skip_w),
                     x_mix.has_value() ? x_mix->data_ptr() : nullptr, xn.has_value() ? xn->data_ptr() : nullptr, R, C,
                     (float)eps, cur_stream());
}

void norm_bwd_add(const Tensor& dy, const Tensor& x, const c10::optional<Tensor>& dres, Tensor out, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(dy, "dy"); chk_bf16c(x, "x"); chk_bf16c(out, "out");
  const int C = (int)x.size(-1), R = (int)(x.numel() / C);
  b200::norm_bwd_add(dy.data_ptr(), x.data_ptr(), optp(dres), out.data_ptr(), R, C, (float)eps, cur_stream());
}

void mix_bwd(const Tensor& dmix, const Tensor& x, const Tensor& x0, const c10::optional<Tensor>& skip,
             const Tensor& lam, const c10::optional<Tensor>& skip_w, Tensor dx, const c10::optional<Tensor>& dskip,
             Tensor dx0_acc, Tensor dlam, const c10::optional<Tensor>& dskip_w, const c10::optional<Tensor>& dx_add) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(dmix, "dmix"); chk_bf16c(x, "x"); chk_bf16c(x0, "x0"); chk_bf16c(dx, "dx");
  if (dx_add.has_value()) {
    chk_bf16c(*dx_add, "dx_add");
    TORCH_CHECK(dx_add->numel() == x.numel(), "dx_add: same size as x");
  }
  TORCH_CHECK(dx0_acc.scalar_type() == at::kFloat && dx0_acc.is_contiguous(), "dx0_acc: contiguous fp32");
  const int C = (int)x.size(-1), R = (int)(x.numel() / C);
  b200::mix_bwd(dmix.data_ptr(), x.data_ptr(), x0.data_ptr(), optp(skip), lam.data_ptr<float>(), optf(skip_w),
                dx.data_ptr(), dskip.has_value() ? dskip->data_ptr() : nullptr, dx0_acc.data_ptr<float>(),
                dlam.data_ptr<float>(), dskip_w.has_value() ? dskip_w->data_ptr<float>() : nullptr, optp(dx_add), R, C, cur_stream());
}

void qkv_post_fwd(const Tensor& qkv, const c10::optional<Tensor>& ve, const Tensor& lam, const Tensor& cos,
                  const Tensor& sin, Tensor out, int64_t H, int64_t D, double eps) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  chk_bf16c(qkv, "qkv"); chk_bf16c(out, "out");
  const int T = (int)(qkv.numel() / (3 * H * D));
  TORCH_CHECK(cos.scalar_type() == at::kFloat && cos.size(0) >= T && cos.size(1) == D / 2 && cos.is_contiguous(), "cos table");
  TORCH_CHECK(sin.scalar_type() == at::kFloat && sin.size(0) >= T && sin.size(1) == D / 2 && sin.is_contiguous(), "sin table");
  b200::qkv_post_fwd(qkv.data_ptr(), optp(ve), lam.data_ptr<float>(), cos.data_ptr<float>(), sin.data_ptr<float>(),
                     out.data_ptr(), T, (int)H, (int)D, (float)eps, cur_stream());
}

void qkv_post_bwd(const Tensor& dq, const Tensor& dk, const Tensor& dv, const Tensor& qkv,
                  const c10::optional<Tensor>& ve, const Tensor& lam, const Tensor& cos, const Tensor& sin,
                  Tensor dqkv, const c10::optional<Tensor>& dve, Tensor dlam, int64_t H, int64_t D, double eps) {
  const c10::cuda::CUDAGuard guard(qkv.device());
  chk_bf16c(qkv, "qkv"); chk_bf16c(dk, "dk"); chk_bf16c(dv, "dv"); chk_bf16c(dqkv, "dqkv");
  TORCH_CHECK(dq.scalar_type() == at::kFloat && dq.is_contiguous(), "dq: contiguous fp32");
  const int T = (int)(qkv.numel() / (3 * H * D));
  b200::qkv_post_bwd(dq.data_ptr<float>(), dk.data_ptr(), dv.data_ptr(), qkv.data_ptr(), optp(ve),
                     lam.data_ptr<float>(), cos.data_ptr<float>(), sin.data_ptr<float>(), dqkv.data_ptr(),
                     dve.has_value() ? dve->data_ptr() : nullptr, dlam.data_ptr<float>(), T, (int)H, (int)D, (float)eps,
                     cur_stream());
}

void embed_gather(const Tensor& idx, const Tensor& table, Tensor out, bool normalize, double eps) {
  const c10::cuda::CUDAGuard guard(table.device());
  chk_bf16c(table, "table"); chk_bf16c(out, "out");
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous(), "idx: contiguous int32");
  b200::embed_gather(idx.data_ptr<int>(), table.data_ptr(), out.data_ptr(), (int)idx.numel(), (int)table.size(1),
                     normalize, (float)eps, cur_stream());
}

void embed_scatter_add(const Tensor& idx, const Tensor& src, Tensor grad_table, const c10::optional<Tensor>& src2) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous() && src.is_contiguous(), "embed_scatter_add: layout");
  TORCH_CHECK(grad_table.scalar_type() == at::kFloat && grad_table.is_contiguous(), "grad_table: contiguous fp32");
  const bool f32 = src.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || src.scalar_type() == at::kBFloat16, "src: fp32 or bf16");
  if (src2.has_value())
    TORCH_CHECK(src2->scalar_type() == src.scalar_type() && src2->is_contiguous() && src2->sizes() == src.sizes(), "src2: same dtype and shape as src");
  b200::embed_scatter_add(idx.data_ptr<int>(), src.data_ptr(), src2.has_value() ? src2->data_ptr() : nullptr, f32, grad_table.data_ptr<float>(), (int)idx.numel(),
                          (int)grad_table.size(1), cur_stream());
}

void softcap_ce_set_cache(bool on, const Tensor& like) {
  (void)like;
  b200::softcap_ce_set_cache(on);
}

void doc_bounds(const Tensor& tokens, int64_t bos, Tensor doc_start, Tensor doc_end) {
  const c10::cuda::CUDAGuard guard(tokens.device());
  TORCH_CHECK(tokens.scalar_type() == at::kLong && tokens.is_contiguous() && tokens.dim() == 1, "doc_bounds: tokens int64 [T]");
  TORCH_CHECK(doc_start.scalar_type() == at::kInt && doc_end.scalar_type() == at::kInt && doc_start.is_contiguous() &&
              doc_end.is_contiguous() && doc_start.numel() == tokens.numel() && doc_end.numel() == tokens.numel(),
              "doc_bounds: doc_start / doc_end int32 [T]");
  b200::doc_bounds(reinterpret_cast<const long long*>(tokens.data_ptr<int64_t>()), (long long)bos,
                   doc_start.data_ptr<int>(), doc_end.data_ptr<int>(), (int)tokens.numel(), cur_stream());
}

void cast_fp8(const Tensor& x, Tensor out, double scale) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && x.numel() == out.numel(), "cast_fp8: layout");
  const int in_kind = x.scalar_type() == at::kBFloat16 ? 0 : 1;
  TORCH_CHECK(in_kind == 0 || x.scalar_type() == at::kFloat, "cast_fp8: input must be bf16 or fp32");
  const int out_kind = out.scalar_type() == at::kFloat8_e4m3fn ? 0 : 1;
  TORCH_CHECK(out_kind == 0 || out.scalar_type() == at::kFloat8_e5m2, "cast_fp8: output must be e4m3fn or e5m2");
  b200::cast_fp8(x.data_ptr(), out.data_ptr(), (float)scale, x.numel(), in_kind, out_kind, cur_stream());
}

void softcap_ce(const Tensor& logits, const Tensor& targets, Tensor loss_rows, const c10::optional<Tensor>& grad,
                double cap, double div, double loss_scale, double grad_scale, double shift, const c10::optional<Tensor>& mtp_w) {
  const c10::cuda::CUDAGuard guard(logits.device());
  if (mtp_w.has_value()) TORCH_CHECK(mtp_w->is_cuda() && mtp_w->scalar_type() == at::kFloat && mtp_w->is_contiguous() && mtp_w->numel() >= 1 && mtp_w->numel() <= 4, "mtp_w: fp32 [1..4]");
  TORCH_CHECK(logits.dim() == 2 && logits.scalar_type() == at::kBFloat16 && logits.stride(1) == 1, "logits: bf16 [T, V]");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous(), "targets: int64");
  TORCH_CHECK(loss_rows.scalar_type() == at::kFloat && loss_rows.numel() == logits.size(0), "loss_rows: fp32 [T]");
  int grad_bf16 = 0;
  if (grad.has_value()) {
    grad_bf16 = grad->scalar_type() == at::kBFloat16;
    TORCH_CHECK(grad_bf16 || grad->scalar_type() == at::kFloat8_e5m2, "grad: bf16 or e5m2");
    TORCH_CHECK(grad->stride(0) == logits.stride(0) && grad->stride(1) == 1, "grad must share the logits layout");
  }
  b200::softcap_ce(logits.data_ptr(), targets.data_ptr<int64_t>() ? (const long long*)targets.data_ptr<int64_t>() : nullptr,
                   loss_rows.data_ptr<float>(), grad.has_value() ? grad->data_ptr() : nullptr, grad_bf16,
                   (int)logits.size(0), (int)logits.size(1), logits.stride(0), (float)cap, (float)div, (float)shift, (float)loss_scale,
                   (float)grad_scale, mtp_w.has_value() ? mtp_w->data_ptr<float>() : nullptr, mtp_w.has_value() ? (int)mtp_w->numel() : 1,
                   cur_stream());
}

void adam_step(Tensor p, const Tensor& g, Tensor m, Tensor v, double lr, double beta1, double beta2, double eps,
               double wd, double bias1, double bias2, double grad_scale, const c10::optional<Tensor>& shadow,
               double shadow_scale) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adam_step: contiguous");
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "adam_step: fp32 m/v");
  const bool pb = p.scalar_type() == at::kBFloat16;
  const bool gb = g.scalar_type() == at::kBFloat16;
  TORCH_CHECK(pb || p.scalar_type() == at::kFloat, "adam_step: p must be fp32 or bf16");
  TORCH_CHECK(gb || g.scalar_type() == at::kFloat, "adam_step: g must be fp32 or bf16");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "adam_step: size mismatch");
  int kind = 0;
  void* sh = nullptr;
  if (shadow.has_value()) {
    TORCH_CHECK(shadow->is_contiguous() && shadow->numel() == p.numel(), "adam_step: shadow must be contiguous and of p's size");
    kind = shadow->scalar_type() == at::kBFloat16 ? 1 : shadow->scalar_type() == at::kFloat8_e4m3fn ? 2 : 0;
    TORCH_CHECK(kind != 0, "adam_step: shadow must be bf16 or float8_e4m3fn");
    sh = shadow->data_ptr();
  }
  b200::adam_step(p.data_ptr(), pb, g.data_ptr(), gb, m.data_ptr<float>(), v.data_ptr<float>(), p.numel(), (float)lr,
                  (float)beta1, (float)beta2, (float)eps, (float)wd, (float)bias1, (float)bias2, (float)grad_scale, sh,
                  kind, (float)shadow_scale, cur_stream());
}

void muon_momentum(const Tensor& g, Tensor buf, Tensor out, Tensor sumsq, double mu, bool nesterov, double grad_scale) {
  const c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_contiguous() && buf.is_contiguous() && out.is_contiguous(), "muon_momentum: contiguous");
  TORCH_CHECK(g.scalar_type() == at::kFloat && buf.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16 &&
              sumsq.scalar_type() == at::kFloat, "muon_momentum: dtypes");
  const int64_t nmat = sumsq.numel();   // g, buf, out are stacks of nmat equally sized matrices
  TORCH_CHECK(nmat >= 1 && g.numel() % nmat == 0 && buf.numel() == g.numel() && out.numel() == g.numel() && sumsq.is_contiguous(),
              "muon_momentum: g, buf, out [nmat, n] with sumsq [nmat]");
  b200::muon_momentum(g.data_ptr<float>(), buf.data_ptr<float>(), out.data_ptr(), sumsq.data_ptr<float>(), g.numel() / nmat,
                      (int)nmat, (float)mu, nesterov, (float)grad_scale, cur_stream());
}

void scale_by_inv_norm(Tensor x, const Tensor& sumsq, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x");
  b200::scale_by_inv_norm(x.data_ptr(), sumsq.data_ptr<float>(), x.numel(), (float)eps, cur_stream());
}

void axpy_bf16_to_f32(Tensor p, const Tensor& u, const c10::optional<Tensor>& p_bf16, double alpha) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.scalar_type() == at::kFloat && p.is_contiguous() && u.is_contiguous() && u.scalar_type() == at::kBFloat16 &&
              u.numel() == p.numel(), "axpy: p fp32, u bf16, same numel");
  b200::axpy_bf16_to_f32(p.data_ptr<float>(), u.data_ptr(), p_bf16.has_value() ? p_bf16->data_ptr() : nullptr, p.numel(),
                         (float)alpha, cur_stream());
}


void adam_cautious(Tensor p, const Tensor& g, Tensor m, Tensor v, double b1, double b2, double eps, double step_size, double wd_lr) {
  const c10::cuda::CUDAGuard guard(p.device());
  const bool pb = p.scalar_type() == at::kBFloat16, gb = g.scalar_type() == at::kBFloat16;
  TORCH_CHECK(p.is_cuda() && p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adam_cautious: contiguous CUDA tensors");
  TORCH_CHECK((pb || p.scalar_type() == at::kFloat) && (gb || g.scalar_type() == at::kFloat), "adam_cautious: p, g bf16 or fp32");
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(),
              "adam_cautious: fp32 moments of p's size");
  b200::adam_cautious(p.data_ptr(), pb, g.data_ptr(), gb, m.data_ptr<float>(), v.data_ptr<float>(), p.numel(), (float)b1, (float)b2, (float)eps,
                      (float)step_size, (float)wd_lr, cur_stream());
}

void normuon_scales(const Tensor& v, Tensor stat, Tensor second, bool red_cols, double beta2) {
  const c10::cuda::CUDAGuard guard(v.device());
  TORCH_CHECK(v.dim() == 3 && v.is_contiguous(), "normuon_scales: v [nmat, R, C] contiguous");
  const bool vb = v.scalar_type() == at::kBFloat16;
  TORCH_CHECK(vb || v.scalar_type() == at::kFloat, "normuon_scales: v bf16 or fp32");
  const int64_t nmat = v.size(0), R = v.size(1), C = v.size(2), ns = red_cols ? R : C;
  TORCH_CHECK(stat.scalar_type() == at::kFloat && second.scalar_type() == at::kFloat && stat.is_contiguous() &&
              second.is_contiguous() && stat.numel() == nmat * ns && second.numel() == nmat * ns,
              "normuon_scales: stat / second fp32 with one entry per row (red_cols) or column");
  b200::normuon_scales(v.data_ptr(), vb, stat.data_ptr<float>(), second.data_ptr<float>(), (int)nmat, (int)R, (int)C, red_cols,
                       (float)beta2, cur_stream());
}

void normuon_update(Tensor p, const c10::optional<Tensor>& mant, const Tensor& v, const c10::optional<Tensor>& scale,
                    bool scale_per_row, double lr, double wd_lr, const c10::optional<Tensor>& lr_mat,
                    const c10::optional<Tensor>& wd_mat) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(v.dim() == 3 && v.is_contiguous() && p.is_contiguous() && p.numel() == v.numel(), "normuon_update: p, v [nmat, R, C]");
  const bool pb = p.scalar_type() == at::kBFloat16, vb = v.scalar_type() == at::kBFloat16;
  TORCH_CHECK((pb || p.scalar_type() == at::kFloat) && (vb || v.scalar_type() == at::kFloat), "normuon_update: bf16 or fp32");
  unsigned short* mp = nullptr;
  if (mant.has_value()) {
    TORCH_CHECK(pb && mant->is_contiguous() && mant->numel() == p.numel() && mant->element_size() == 2, "normuon_update: mantissa is a 16-bit buffer of a bf16 p");
    mp = reinterpret_cast<unsigned short*>(mant->data_ptr());
  }
  const int64_t nmat = v.size(0), R = v.size(1), C = v.size(2);
  const float* sp = nullptr;
  if (scale.has_value()) {
    TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->is_contiguous() && scale->numel() == nmat * (scale_per_row ? R : C), "normuon_update: scale");
    sp = scale->data_ptr<float>();
  }
  auto per_mat = [&](const c10::optional<Tensor>& t) -> const float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == nmat && t->is_cuda(), "normuon_update: per-matrix values fp32 [nmat] on the device");
    return t->data_ptr<float>();
  };
  b200::normuon_update(p.data_ptr(), pb, mp, v.data_ptr(), vb, sp, (int)nmat, (int)R, (int)C, scale_per_row, (float)lr, (float)wd_lr,
                       per_mat(lr_mat), per_mat(wd_mat), cur_stream());
}

// ---------------------------------------------------------------------------------------------- peer-memory collectives
b200::PeerPtrs to_peers(at::IntArrayRef ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && (int)ptrs.size() <= b200::kMaxWorld, "peer pointer list: 1..", b200::kMaxWorld, " entries");
  b200::PeerPtrs pp;
  for (int i = 0; i < b200::kMaxWorld; ++i) pp.p[i] = nullptr;
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]));
  return pp;
}

void comm_signal(at::IntArrayRef peer_flags, int64_t rank, int64_t channel, int64_t epoch, const Tensor& like) {
  const c10::cuda::CUDAGuard guard(like.device());
  b200::comm_signal(to_peers(peer_flags), (int)peer_flags.size(), (int)rank, (int)channel, (int)epoch, cur_stream());
}

void comm_wait(const Tensor& flags, int64_t world, int64_t channel, int64_t epoch, Tensor status) {
  const c10::cuda::CUDAGuard guard(flags.device());
  b200::comm_wait(flags.data_ptr<int>(), (int)world, (int)channel, (int)epoch, status.data_ptr<int>(), cur_stream());
}

void muon_rs_momentum(at::IntArrayRef grad_ptrs, int64_t elem_off, int64_t nmat, int64_t mat_elems, Tensor mom,
                      Tensor u_out, Tensor sumsq, double mu, bool nesterov, const Tensor& flags, int64_t channel,
                      int64_t epoch, Tensor status) {
  const c10::cuda::CUDAGuard guard(mom.device());
  TORCH_CHECK(mom.scalar_type() == at::kFloat && mom.is_contiguous() && mom.numel() >= nmat * mat_elems, "mom: fp32 shard");
  TORCH_CHECK(u_out.scalar_type() == at::kBFloat16 && u_out.is_contiguous() && u_out.numel() >= nmat * mat_elems, "u_out: bf16 shard");
  TORCH_CHECK(sumsq.scalar_type() == at::kFloat && sumsq.numel() >= nmat, "sumsq: fp32 [nmat]");
  b200::muon_rs_momentum(to_peers(grad_ptrs), (int)grad_ptrs.size(), elem_off, (int)nmat, mat_elems, mom.data_ptr<float>(),
                         u_out.data_ptr(), sumsq.data_ptr<float>(), (float)mu, nesterov, flags.data_ptr<int>(), (int)channel,
                         (int)epoch, status.data_ptr<int>(), cur_stream());
}

void adam_shard(at::IntArrayRef grad_ptrs, at::IntArrayRef param_ptrs, int64_t rank, int64_t lo, int64_t hi, int64_t dtype,
                Tensor m, Tensor v, double lr, double beta1, double beta2, double eps, double wd, double bias1, double bias2,
                const Tensor& flags, at::IntArrayRef peer_flags, int64_t channel, int64_t epoch, Tensor status,
                int64_t max_blocks) {
  const c10::cuda::CUDAGuard guard(m.device());
  TORCH_CHECK(grad_ptrs.size() == param_ptrs.size() && grad_ptrs.size() == peer_flags.size(), "adam_shard: one pointer per rank");
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && m.is_contiguous() && v.is_contiguous() &&
              m.numel() >= hi - lo && v.numel() >= hi - lo, "adam_shard: m, v fp32 of at least the owned range");
  b200::adam_shard(to_peers(grad_ptrs), to_peers(param_ptrs), (int)grad_ptrs.size(), (int)rank, lo, hi, (int)dtype,
                   m.data_ptr<float>(), v.data_ptr<float>(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd,
                   (float)bias1, (float)bias2, flags.data_ptr<int>(), to_peers(peer_flags), (int)channel, (int)epoch,
                   status.data_ptr<int>(), (int)max_blocks, cur_stream());
}

void stack_scale_by_inv_norm(Tensor x, const Tensor& sumsq, int64_t nmat, int64_t mat_elems, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x");
  b200::stack_scale_by_inv_norm(x.data_ptr(), sumsq.data_ptr<float>(), (int)nmat, mat_elems, (float)eps, cur_stream());
}

void ag_push(const Tensor& src, at::IntArrayRef u_full_ptrs, int64_t rank, int64_t dst_off, at::IntArrayRef peer_flags,
             int64_t channel, int64_t epoch, int64_t slot) {
  const c10::cuda::CUDAGuard guard(src.device());
  chk_bf16c(src, "src");
  b200::ag_push(src.data_ptr(), to_peers(u_full_ptrs), (int)u_full_ptrs.size(), (int)rank, dst_off, src.numel(),
                to_peers(peer_flags), (int)channel, (int)epoch, (int)slot, cur_stream());
}

void ag_wait_apply(Tensor p, const Tensor& u, const c10::optional<Tensor>& p_bf16, double alpha, int64_t world,
                   const Tensor& flags, int64_t channel, int64_t epoch, Tensor status) {
  const c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.scalar_type() == at::kFloat && p.is_contiguous() && u.scalar_type() == at::kBFloat16 && u.is_contiguous() &&
              u.numel() >= p.numel(), "ag_wait_apply: p fp32, u bf16");
  b200::ag_wait_apply(p.data_ptr<float>(), u.data_ptr(), p_bf16.has_value() ? p_bf16->data_ptr() : nullptr, p.numel(),
                      (float)alpha, (int)world, flags.data_ptr<int>(), (int)channel, (int)epoch, status.data_ptr<int>(),
                      cur_stream());
}

void allreduce_mean_multimem(int64_t mc_ptr, int64_t world, int64_t rank, int64_t n, int64_t dtype, const Tensor& flags,
                             at::IntArrayRef peer_flags, int64_t channel, int64_t epoch, Tensor status) {
  const c10::cuda::CUDAGuard guard(flags.device());
  b200::allreduce_mean_multimem(reinterpret_cast<void*>(mc_ptr), (int)world, (int)rank, n, (int)dtype, flags.data_ptr<int>(),
                                to_peers(peer_flags), (int)channel, (int)epoch, status.data_ptr<int>(), cur_stream());
}

void allreduce_mean(at::IntArrayRef buf_ptrs, int64_t rank, int64_t n, int64_t dtype, const Tensor& flags,
                    at::IntArrayRef peer_flags, int64_t channel, int64_t epoch, Tensor status) {
  const c10::cuda::CUDAGuard guard(flags.device());
  b200::allreduce_mean(to_peers(buf_ptrs), (int)buf_ptrs.size(), (int)rank, n, (int)dtype, flags.data_ptr<int>(),
                       to_peers(peer_flags), (int)channel, (int)epoch, status.data_ptr<int>(), cur_stream());
}


// ---------------------------------------------------------------------------------------------- S6 selective scan
void s6_set_states_per_thread(int64_t fwd_qs, int64_t bwd_qs, const Tensor& like) {
  (void)like;  // only selects the CUDA dispatch key
  b200::s6_set_states_per_thread((int)fwd_qs, (int)bwd_qs);
}

static void jacobi_fill(b200::JacobiArgs& a, const Tensor& Bm, const Tensor& Cm, const Tensor& theta, const Tensor& xr, const Tensor& alpha,
                        const Tensor& gamma, const Tensor& conv_w, const Tensor& conv_b, const c10::optional<Tensor>& inj_lambda,
                        const c10::optional<Tensor>& ro_lambda, int64_t n_iters) {
  TORCH_CHECK(Bm.dim() == 4 && Cm.dim() == 4 && Bm.sizes() == Cm.sizes(), "jacobi: B / C maps [batch, R, L, N] (any strides)");
  a.batch = (int)Bm.size(0); a.R = (int)Bm.size(1); a.L = (int)Bm.size(2); a.N = (int)Bm.size(3); a.n_iters = (int)n_iters;
  const int64_t rows = (int64_t)a.batch * a.L;
  for (const Tensor* t : {&Bm, &Cm, &theta, &xr, &alpha, &gamma, &conv_w, &conv_b})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat, "jacobi: fp32 CUDA tensors");
  TORCH_CHECK(theta.is_contiguous() && theta.numel() == rows * (a.N / 2), "jacobi: theta [batch, L, N/2] contiguous");
  TORCH_CHECK(alpha.is_contiguous() && alpha.numel() == rows * a.N, "jacobi: alpha [batch, L, N] contiguous");
  TORCH_CHECK(gamma.is_contiguous() && gamma.numel() == rows, "jacobi: gamma [batch, L] contiguous");
  TORCH_CHECK(xr.dim() == 3 && xr.size(0) == a.batch && xr.size(1) == a.R && xr.size(2) == a.L, "jacobi: x_r [batch, R, L] (any strides)");
  TORCH_CHECK(conv_w.is_contiguous() && conv_w.numel() == 3 * a.N && conv_b.is_contiguous() && conv_b.numel() == a.N, "jacobi: taps [N, 3], bias [N]");
  a.Bm = Bm.data_ptr<float>(); a.b_sb = Bm.stride(0); a.b_sr = Bm.stride(1); a.b_sl = Bm.stride(2); a.b_sn = Bm.stride(3);
  a.Cm = Cm.data_ptr<float>(); a.c_sb = Cm.stride(0); a.c_sr = Cm.stride(1); a.c_sl = Cm.stride(2); a.c_sn = Cm.stride(3);
  a.theta = theta.data_ptr<float>(); a.alpha = alpha.data_ptr<float>(); a.gamma = gamma.data_ptr<float>();
  a.xr = xr.data_ptr<float>(); a.x_sb = xr.stride(0); a.x_sr = xr.stride(1); a.x_sl = xr.stride(2);
  a.conv_w = conv_w.data_ptr<float>(); a.conv_b = conv_b.data_ptr<float>();
  auto scalar = [](const c10::optional<Tensor>& t) -> const float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->numel() == 1, "jacobi: mix weights are fp32 device scalars");
    return t->data_ptr<float>();
  };
  a.inj_lambda = scalar(inj_lambda); a.ro_lambda = scalar(ro_lambda);
  a.stream = cur_stream();
}

void jacobi_fwd(const Tensor& Bm, const Tensor& Cm, const Tensor& theta, const Tensor& xr, const Tensor& alpha, const Tensor& gamma,
                const Tensor& conv_w, const Tensor& conv_b, const c10::optional<Tensor>& inj_lambda, const c10::optional<Tensor>& ro_lambda,
                int64_t n_iters, Tensor gated, const c10::optional<Tensor>& Hs) {
  const c10::cuda::CUDAGuard guard(Bm.device());
  b200::JacobiArgs a;
  jacobi_fill(a, Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda, n_iters);
  const int64_t state = (int64_t)a.batch * a.R * a.L * a.N;
  TORCH_CHECK(gated.scalar_type() == at::kFloat && gated.is_contiguous() && gated.numel() == state, "jacobi_fwd: gated fp32 [batch, L, R * N]");
  a.gated = gated.data_ptr<float>();
  if (Hs.has_value()) {
    TORCH_CHECK(Hs->scalar_type() == at::kFloat && Hs->is_contiguous() && Hs->numel() == state * n_iters, "jacobi_fwd: states fp32 [n_iters, batch, R, L, N]");
    a.Hs = Hs->data_ptr<float>();
  }
  b200::jacobi_fwd(a);
}

void jacobi_bwd(const Tensor& dgated, const Tensor& Hs, const Tensor& Bm, const Tensor& Cm, const Tensor& theta, const Tensor& xr,
                const Tensor& alpha, const Tensor& gamma, const Tensor& conv_w, const Tensor& conv_b, const c10::optional<Tensor>& inj_lambda,
                const c10::optional<Tensor>& ro_lambda, int64_t n_iters, Tensor dBm, Tensor dCm, Tensor dtheta, Tensor dxr, Tensor dalpha,
                Tensor dgamma, Tensor dconv_w, Tensor dconv_b, Tensor dlam) {
  const c10::cuda::CUDAGuard guard(Bm.device());
  b200::JacobiArgs a;
  jacobi_fill(a, Bm, Cm, theta, xr, alpha, gamma, conv_w, conv_b, inj_lambda, ro_lambda, n_iters);
  const int64_t state = (int64_t)a.batch * a.R * a.L * a.N, rows = (int64_t)a.batch * a.L;
  auto out = [](Tensor& t, int64_t n, const char* what) -> float* {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == n, "jacobi_bwd: ", what);
    return t.data_ptr<float>();
  };
  TORCH_CHECK(dgated.scalar_type() == at::kFloat && dgated.is_contiguous() && dgated.numel() == state, "jacobi_bwd: dgated fp32 [batch, L, R * N]");
  TORCH_CHECK(Hs.scalar_type() == at::kFloat && Hs.is_contiguous() && Hs.numel() == state * n_iters, "jacobi_bwd: states fp32 [n_iters, batch, R, L, N]");
  a.dgated = dgated.data_ptr<float>(); a.Hs = const_cast<float*>(Hs.data_ptr<float>());
  a.dBm = out(dBm, state, "dB [batch, R, L, N]"); a.dCm = out(dCm, state, "dC [batch, R, L, N]");
  a.dtheta = out(dtheta, rows * (a.N / 2), "dtheta"); a.dxr = out(dxr, rows * a.R, "dx_r [batch, R, L]");
  a.dalpha = out(dalpha, rows * a.N, "dalpha"); a.dgamma = out(dgamma, rows, "dgamma");
  a.dconv_w = out(dconv_w, 3 * a.N, "dtaps"); a.dconv_b = out(dconv_b, a.N, "dbias"); a.dlam = out(dlam, 2, "dlam [2]");
  b200::jacobi_bwd(a);
}

bool ssd_fwd_supported(int64_t L, int64_t H, int64_t Hb, int64_t N, int64_t P) {
  return b200::ssd_fwd_supported((int)L, (int)H, (int)Hb, (int)N, (int)P);
}

void ssd_fwd(const Tensor& x, const Tensor& Bm, const Tensor& Cm, const Tensor& log_a, const Tensor& g_off, const Tensor& g_diag,
             Tensor y, const c10::optional<Tensor>& init_state, const c10::optional<Tensor>& final_state, Tensor status,
             const c10::optional<Tensor>& chunk_states) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 4 && Bm.dim() == 4 && Cm.dim() == 4, "ssd_fwd: x [b, L, H, P], B / C [b, L, Hb, N]");
  for (const Tensor* t : {&x, &Bm, &Cm, (const Tensor*)&y}) TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->is_contiguous(), "ssd_fwd: bf16 contiguous x, B, C, y");
  for (const Tensor* t : {&log_a, &g_off, &g_diag})
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == x.size(0) * x.size(1) * x.size(2), "ssd_fwd: fp32 [b, L, H] decay / weights");
  TORCH_CHECK(Bm.sizes() == Cm.sizes() && Bm.size(0) == x.size(0) && Bm.size(1) == x.size(1) && y.sizes() == x.sizes(), "ssd_fwd: shapes");
  b200::SsdArgs a;
  a.batch = (int)x.size(0); a.L = (int)x.size(1); a.H = (int)x.size(2); a.P = (int)x.size(3);
  a.Hb = (int)Bm.size(2); a.N = (int)Bm.size(3);
  const int64_t ns = (int64_t)a.batch * a.H * a.N * a.P;
  auto st = [&](const c10::optional<Tensor>& t) -> float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == ns, "ssd_fwd: state fp32 [b, H, N, P]");
    return t->data_ptr<float>();
  };
  a.x = x.data_ptr(); a.B = Bm.data_ptr(); a.C = Cm.data_ptr(); a.y = y.data_ptr();
  a.log_a = log_a.data_ptr<float>(); a.g_off = g_off.data_ptr<float>(); a.g_diag = g_diag.data_ptr<float>();
  a.init_state = st(init_state); a.final_state = st(final_state);
  if (chunk_states.has_value()) {
    TORCH_CHECK(chunk_states->scalar_type() == at::kFloat && chunk_states->is_contiguous() && chunk_states->numel() == ns * (a.L / 128),
                "ssd_fwd: chunk states fp32 [b, H, L / 128, N, P]");
    a.chunk_states = chunk_states->data_ptr<float>();
  }
  a.status = status.data_ptr<int>(); a.stream = cur_stream();
  b200::ssd_fwd_sm100(a);
}

Tensor ssd_flip_time(const Tensor& src) {
  const c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.dim() >= 3 && (reinterpret_cast<uintptr_t>(src.data_ptr()) & 15) == 0 && src.numel() > 0,
              "ssd_flip_time: contiguous, 16-byte aligned [batch, L, ...]");
  Tensor dst = at::empty_like(src);
  const int64_t row_bytes = src.numel() / (src.size(0) * src.size(1)) * src.element_size();
  b200::ssd_flip_time(src.data_ptr(), dst.data_ptr(), (int)src.size(0), (int)src.size(1), row_bytes, cur_stream());
  return dst;
}

void ssd_bwd_post(const Tensor& x, const Tensor& dy, const Tensor& y, const Tensor& dx_rev, const Tensor& dB_rev, const Tensor& dC_heads,
                  const Tensor& Bm, const Tensor& Cm, const Tensor& g_off, const Tensor& g_diag, Tensor dx, Tensor dB, Tensor dC,
                  Tensor d_goff, Tensor d_gdiag, Tensor inner) {
  const c10::cuda::CUDAGuard guard(x.device());
  b200::SsdPostArgs a;
  a.batch = (int)x.size(0); a.L = (int)x.size(1); a.H = (int)x.size(2); a.P = (int)x.size(3);
  a.Hb = (int)Bm.size(2); a.N = (int)Bm.size(3);
  const int64_t np = x.numel(), nn = (int64_t)a.batch * a.L * a.H * a.N, ng = Bm.numel(), ns = (int64_t)a.batch * a.L * a.H;
  auto b16 = [](const Tensor& t, int64_t n, const char* what) -> void* {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.numel() == n, "ssd_bwd_post: bf16 contiguous ", what);
    return t.data_ptr();
  };
  auto f32 = [](const Tensor& t, int64_t n, const char* what) -> float* {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == n, "ssd_bwd_post: fp32 contiguous ", what);
    return t.data_ptr<float>();
  };
  a.x = b16(x, np, "x"); a.dy = b16(dy, np, "dy"); a.y = b16(y, np, "y"); a.dx_rev = b16(dx_rev, np, "dx_rev");
  a.dB_rev = b16(dB_rev, nn, "dB_rev"); a.dC_heads = b16(dC_heads, nn, "dC_heads");
  a.B = b16(Bm, ng, "B"); a.C = b16(Cm, ng, "C");
  a.g_off = f32(g_off, ns, "g_off"); a.g_diag = f32(g_diag, ns, "g_diag");
  a.dx = b16(dx, np, "dx"); a.dB = b16(dB, ng, "dB"); a.dC = b16(dC, ng, "dC");
  a.d_goff = f32(d_goff, ns, "d_goff"); a.d_gdiag = f32(d_gdiag, ns, "d_gdiag"); a.inner = f32(inner, ns, "inner");
  a.stream = cur_stream();
  b200::ssd_bwd_post(a);
}

void s6_scan_fwd(const Tensor& u, const Tensor& delta, const c10::optional<Tensor>& delta_bias, bool softplus, const Tensor& A,
                 const Tensor& Bm, const Tensor& Cm, const c10::optional<Tensor>& Dv, const c10::optional<Tensor>& z,
                 const c10::optional<Tensor>& y_pre, Tensor out, const c10::optional<Tensor>& state) {
  const c10::cuda::CUDAGuard guard(u.device());
  chk_bf16c(u, "u"); chk_bf16c(out, "out");
  TORCH_CHECK(u.dim() == 3 && (delta.scalar_type() == at::kFloat || delta.scalar_type() == at::kBFloat16) && delta.is_contiguous() && delta.sizes() == u.sizes(), "delta: fp32 or bf16 [B, L, Din]");
  const int B = (int)u.size(0), L = (int)u.size(1), Din = (int)u.size(2), N = (int)A.size(1);
  TORCH_CHECK(A.scalar_type() == at::kFloat && A.is_contiguous() && A.size(0) == Din, "A: fp32 [Din, N]");
  TORCH_CHECK(Bm.scalar_type() == at::kFloat && Bm.is_contiguous() && Bm.size(0) == B && Bm.size(1) == L && Bm.size(2) == N, "B: fp32 [B, L, N]");
  TORCH_CHECK(Cm.scalar_type() == at::kFloat && Cm.is_contiguous() && Cm.sizes() == Bm.sizes(), "C: fp32 [B, L, N]");
  if (z.has_value()) chk_bf16c(*z, "z");
  if (y_pre.has_value()) chk_bf16c(*y_pre, "y_pre");
  if (state.has_value())
    TORCH_CHECK(state->scalar_type() == at::kFloat && state->is_contiguous() &&
                state->numel() == (int64_t)B * b200::s6_num_chunks(L) * Din * N, "state: fp32 [B, tiles, 4, Din, 4] with tiles = s6_num_chunks(L)");
  b200::s6_scan_fwd(u.data_ptr(), delta.data_ptr(), delta.scalar_type() == at::kBFloat16, optf(delta_bias), softplus, A.data_ptr<float>(), Bm.data_ptr<float>(),
                    Cm.data_ptr<float>(), optf(Dv), optp(z), y_pre.has_value() ? y_pre->data_ptr() : nullptr, out.data_ptr(),
                    state.has_value() ? state->data_ptr<float>() : nullptr, B, L, Din, N, cur_stream());
}

void s6_scan_bwd(const Tensor& u, const Tensor& delta, const c10::optional<Tensor>& delta_bias, bool softplus, const Tensor& A,
                 const Tensor& Bm, const Tensor& Cm, const c10::optional<Tensor>& Dv, const c10::optional<Tensor>& z,
                 const c10::optional<Tensor>& y_pre, const Tensor& dout, const Tensor& state, Tensor du, Tensor ddelta, Tensor dA,
                 Tensor dB_part, Tensor dC_part, const c10::optional<Tensor>& dD, const c10::optional<Tensor>& dz,
                 const c10::optional<Tensor>& ddelta_bias) {
  const c10::cuda::CUDAGuard guard(u.device());
  chk_bf16c(u, "u"); chk_bf16c(dout, "dout"); chk_bf16c(du, "du");
  if (z.has_value()) { chk_bf16c(*z, "z"); TORCH_CHECK(y_pre.has_value(), "s6_scan_bwd: z needs y_pre"); chk_bf16c(*y_pre, "y_pre"); }
  if (dz.has_value()) chk_bf16c(*dz, "dz");
  const int B = (int)u.size(0), L = (int)u.size(1), Din = (int)u.size(2), N = (int)A.size(1);
  TORCH_CHECK(ddelta.scalar_type() == delta.scalar_type() && ddelta.is_contiguous() && delta.is_contiguous() && ddelta.sizes() == u.sizes() && dA.scalar_type() == at::kFloat &&
              dB_part.scalar_type() == at::kFloat && dC_part.scalar_type() == at::kFloat, "s6_scan_bwd: fp32 gradient buffers");
  TORCH_CHECK(dB_part.numel() == (int64_t)B * b200::s6_channel_blocks(Din) * L * N && dC_part.numel() == dB_part.numel(), "partial buffers: [B, ceil(Din/32), L, N]");
  TORCH_CHECK(state.scalar_type() == at::kFloat && state.numel() == (int64_t)B * b200::s6_num_chunks(L) * Din * N, "state: fp32 [B, tiles, 4, Din, 4] with tiles = s6_num_chunks(L)");
  b200::s6_scan_bwd(u.data_ptr(), delta.data_ptr(), delta.scalar_type() == at::kBFloat16, optf(delta_bias), softplus, A.data_ptr<float>(), Bm.data_ptr<float>(),
                    Cm.data_ptr<float>(), optf(Dv), optp(z), optp(y_pre), dout.data_ptr(), state.data_ptr<float>(), du.data_ptr(),
                    ddelta.data_ptr(), dA.data_ptr<float>(), dB_part.data_ptr<float>(), dC_part.data_ptr<float>(),
                    dD.has_value() ? dD->data_ptr<float>() : nullptr, dz.has_value() ? dz->data_ptr() : nullptr,
                    ddelta_bias.has_value() ? ddelta_bias->data_ptr<float>() : nullptr, B, L, Din, N, cur_stream());
}


void causal_conv1d_silu_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, Tensor y) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 3 && x.scalar_type() == at::kBFloat16 && x.stride(2) == 1 && x.stride(0) == x.size(1) * x.stride(1), "x: bf16 [B, L, C] (channel slice allowed)");
  chk_bf16c(y, "y");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2);
  TORCH_CHECK(w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == (int64_t)C * 4, "w: fp32 [C, 4]");
  b200::causal_conv1d_silu_fwd(x.data_ptr(), x.stride(1), w.data_ptr<float>(), optf(bias), y.data_ptr(), B, L, C, cur_stream());
}

void causal_conv1d_silu_bwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, const Tensor& dy, Tensor dx,
                            Tensor dw, const c10::optional<Tensor>& dbias) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(dy, "dy");
  TORCH_CHECK(dx.scalar_type() == at::kBFloat16 && dx.stride(2) == 1 && dx.stride(0) == dx.size(1) * dx.stride(1), "dx: bf16 [B, L, C]");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2);
  b200::causal_conv1d_silu_bwd(x.data_ptr(), x.stride(1), w.data_ptr<float>(), optf(bias), dy.data_ptr(), dx.data_ptr(),
                               dx.stride(1), dw.data_ptr<float>(), dbias.has_value() ? dbias->data_ptr<float>() : nullptr, B, L, C,
                               cur_stream());
}


// ---------------------------------------------------------------------------------------------- gather convolution
void gather_conv_fwd(const Tensor& x, const Tensor& pos, const Tensor& wgt, Tensor out, int64_t H, double pos_max) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x"); chk_bf16c(out, "out");
  TORCH_CHECK(x.dim() == 3 && pos.scalar_type() == at::kFloat && wgt.scalar_type() == at::kFloat && pos.is_contiguous() &&
              wgt.is_contiguous() && pos.sizes() == wgt.sizes() && pos.dim() == 4, "gather_conv: x [B,L,C] bf16, pos/wgt [B,L,H,S] fp32");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2), S = (int)pos.size(3);
  const int Lq = (int)pos.size(1);
  TORCH_CHECK(pos.size(0) == B && pos.size(2) == H && C % H == 0 && out.numel() == (int64_t)B * Lq * C, "gather_conv: shape mismatch");
  b200::gather_conv_fwd(x.data_ptr(), pos.data_ptr<float>(), wgt.data_ptr<float>(), out.data_ptr(), B, L, Lq, (int)H, C / (int)H, S, (float)pos_max, cur_stream());
}

void gather_conv_bwd(const Tensor& x, const Tensor& pos, const Tensor& wgt, const Tensor& dout, Tensor dx, Tensor dpos,
                     Tensor dwgt, int64_t H, double pos_max) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x"); chk_bf16c(dout, "dout");
  TORCH_CHECK(dx.scalar_type() == at::kFloat && dx.is_contiguous() && dx.numel() == x.numel(), "dx: fp32, zeroed, x's shape");
  TORCH_CHECK(dpos.scalar_type() == at::kFloat && dwgt.scalar_type() == at::kFloat && dpos.is_contiguous() && dwgt.is_contiguous(), "dpos/dwgt: fp32");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2), S = (int)pos.size(3);
  b200::gather_conv_bwd(x.data_ptr(), pos.data_ptr<float>(), wgt.data_ptr<float>(), dout.data_ptr(), dx.data_ptr<float>(),
                        dpos.data_ptr<float>(), dwgt.data_ptr<float>(), B, L, (int)pos.size(1), (int)H, C / (int)H, S, (float)pos_max, cur_stream());
}


// ---------------------------------------------------------------------------------------------- RWKV time mixing
bool wkv_io(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && (t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16), n, ": contiguous fp32 or bf16 CUDA tensor");
  return t.scalar_type() == at::kBFloat16;
}
void chk_f32c(const Tensor& t, const char* n) { TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kFloat, n, ": contiguous fp32 CUDA tensor"); }

void wkv4_fwd(const Tensor& k, const Tensor& v, const Tensor& w, const Tensor& u, Tensor y) {
  const c10::cuda::CUDAGuard guard(k.device());
  const bool bf = wkv_io(k, "k");
  TORCH_CHECK(k.dim() == 3 && v.sizes() == k.sizes() && y.sizes() == k.sizes() && wkv_io(v, "v") == bf && wkv_io(y, "y") == bf, "wkv4: k, v, y [B, T, C] of one dtype");
  chk_f32c(w, "w"); chk_f32c(u, "u");
  TORCH_CHECK(w.numel() == k.size(2) && u.numel() == k.size(2), "wkv4: w, u [C]");
  b200::wkv4_fwd(k.data_ptr(), v.data_ptr(), w.data_ptr<float>(), u.data_ptr<float>(), y.data_ptr(), bf, (int)k.size(0), (int)k.size(1), (int)k.size(2), cur_stream());
}

void wkv4_bwd(const Tensor& k, const Tensor& v, const Tensor& w, const Tensor& u, const Tensor& gy, Tensor gk, Tensor gv, Tensor gw, Tensor gu, Tensor scratch) {
  const c10::cuda::CUDAGuard guard(k.device());
  const bool bf = wkv_io(k, "k");
  TORCH_CHECK(wkv_io(v, "v") == bf && wkv_io(gy, "gy") == bf && wkv_io(gk, "gk") == bf && wkv_io(gv, "gv") == bf, "wkv4_bwd: one I/O dtype");
  TORCH_CHECK(v.sizes() == k.sizes() && gy.sizes() == k.sizes() && gk.sizes() == k.sizes() && gv.sizes() == k.sizes(), "wkv4_bwd: [B, T, C] tensors");
  chk_f32c(w, "w"); chk_f32c(u, "u"); chk_f32c(gw, "gw"); chk_f32c(gu, "gu"); chk_f32c(scratch, "scratch");
  const int64_t B = k.size(0), T = k.size(1), C = k.size(2);
  TORCH_CHECK(gw.numel() == B * C && gu.numel() == B * C && scratch.numel() == 3 * B * T * C, "wkv4_bwd: gw, gu [B, C]; scratch [3, B, T, C]");
  b200::wkv4_bwd(k.data_ptr(), v.data_ptr(), w.data_ptr<float>(), u.data_ptr<float>(), gy.data_ptr(), gk.data_ptr(), gv.data_ptr(),
                 gw.data_ptr<float>(), gu.data_ptr<float>(), scratch.data_ptr<float>(), bf, (int)B, (int)T, (int)C, cur_stream());
}

void wkv5_fwd(const Tensor& r, const Tensor& k, const Tensor& v, const Tensor& w, const Tensor& u, Tensor y) {
  const c10::cuda::CUDAGuard guard(r.device());
  const bool bf = wkv_io(r, "r");
  TORCH_CHECK(r.dim() == 3 && k.sizes() == r.sizes() && v.sizes() == r.sizes() && y.sizes() == r.sizes(), "wkv5: r, k, v, y [B, T, C]");
  TORCH_CHECK(wkv_io(k, "k") == bf && wkv_io(v, "v") == bf && wkv_io(y, "y") == bf, "wkv5: one I/O dtype");
  chk_f32c(w, "w"); chk_f32c(u, "u");
  TORCH_CHECK(w.dim() == 2 && u.sizes() == w.sizes() && w.numel() == r.size(2), "wkv5: w, u [H, N] with H * N == C");
  b200::wkv5_fwd(r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr<float>(), u.data_ptr<float>(), y.data_ptr(), bf, (int)r.size(0),
                 (int)r.size(1), (int)w.size(0), (int)w.size(1), cur_stream());
}

void wkv5_bwd(const Tensor& r, const Tensor& k, const Tensor& v, const Tensor& w, const Tensor& u, const Tensor& gy, Tensor gr, Tensor gk,
              Tensor gv, Tensor gw, Tensor gu) {
  const c10::cuda::CUDAGuard guard(r.device());
  const bool bf = wkv_io(r, "r");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&k, &v, &gy, &gr, &gk, &gv})
    TORCH_CHECK(wkv_io(*t, "wkv5_bwd tensor") == bf && t->sizes() == r.sizes(), "wkv5_bwd: [B, T, C] tensors of one dtype");
  chk_f32c(w, "w"); chk_f32c(u, "u"); chk_f32c(gw, "gw"); chk_f32c(gu, "gu");
  TORCH_CHECK(w.dim() == 2 && w.numel() == r.size(2) && gw.numel() == r.size(0) * r.size(2) && gu.numel() == gw.numel(), "wkv5_bwd: w [H, N]; gw, gu [B, C]");
  b200::wkv5_bwd(r.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr<float>(), u.data_ptr<float>(), gy.data_ptr(), gr.data_ptr(),
                 gk.data_ptr(), gv.data_ptr(), gw.data_ptr<float>(), gu.data_ptr<float>(), bf, (int)r.size(0), (int)r.size(1),
                 (int)w.size(0), (int)w.size(1), cur_stream());
}

// ---------------------------------------------------------------------------------------------- local window attention
void window_attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& bias, Tensor out, Tensor P, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  chk_bf16c(q, "q"); chk_bf16c(k, "k"); chk_bf16c(v, "v"); chk_bf16c(out, "out"); chk_f32c(bias, "bias"); chk_f32c(P, "P");
  TORCH_CHECK(q.dim() == 4 && k.sizes() == q.sizes() && v.sizes() == q.sizes() && out.sizes() == q.sizes(), "window_attn: q, k, v, out [B, L, H, D]");
  TORCH_CHECK(bias.dim() == 4 && bias.size(0) == q.size(0) && bias.size(1) == q.size(1) && bias.size(2) == q.size(2) && P.sizes() == bias.sizes(), "window_attn: bias, P [B, L, H, K]");
  b200::window_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), bias.data_ptr<float>(), out.data_ptr(), P.data_ptr<float>(), (float)scale,
                        (int)q.size(0), (int)q.size(1), (int)q.size(2), (int)q.size(3), (int)bias.size(3), cur_stream());
}

void window_attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& P, const Tensor& dout, Tensor dq, Tensor dk, Tensor dv,
                     Tensor dbias, double scale) {
  const c10::cuda::CUDAGuard guard(q.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&q, &k, &v, &dout, &dq, &dk, &dv}) {
    chk_bf16c(*t, "window_attn_bwd tensor");
    TORCH_CHECK(t->sizes() == q.sizes(), "window_attn_bwd: [B, L, H, D] tensors");
  }
  chk_f32c(P, "P"); chk_f32c(dbias, "dbias");
  TORCH_CHECK(P.dim() == 4 && dbias.sizes() == P.sizes(), "window_attn_bwd: P, dbias [B, L, H, K]");
  b200::window_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), P.data_ptr<float>(), dout.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                        dv.data_ptr(), dbias.data_ptr<float>(), (float)scale, (int)q.size(0), (int)q.size(1), (int)q.size(2), (int)q.size(3),
                        (int)P.size(3), cur_stream());
}

// ---------------------------------------------------------------------------------------------- MRA block-sparse ops
void chk_i32c(const Tensor& t, const char* n) { TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kInt, n, ": contiguous int32 CUDA tensor"); }

void mra_sddmm(const Tensor& Q, const Tensor& K, const Tensor& indices, Tensor S) {
  const c10::cuda::CUDAGuard guard(Q.device());
  chk_f32c(Q, "Q"); chk_f32c(K, "K"); chk_f32c(S, "S"); chk_i32c(indices, "indices");
  TORCH_CHECK(Q.dim() == 3 && K.dim() == 3 && Q.size(0) == K.size(0) && Q.size(2) == K.size(2) && Q.size(1) % 32 == 0 && K.size(1) % 32 == 0, "mra_sddmm: Q [B, Lq, D], K [B, Lk, D], lengths multiples of 32");
  TORCH_CHECK(indices.dim() == 2 && indices.size(0) == Q.size(0) && S.numel() == indices.numel() * 1024, "mra_sddmm: indices [B, n], S [B, n, 32, 32]");
  b200::mra_sddmm(Q.data_ptr<float>(), K.data_ptr<float>(), indices.data_ptr<int>(), S.data_ptr<float>(), (int)Q.size(0), (int)Q.size(1),
                  (int)K.size(1), (int)Q.size(2), (int)indices.size(1), cur_stream());
}

void mra_spmm(const Tensor& P, const Tensor& indices, const Tensor& V, Tensor out, int64_t Lq, int64_t Lk, bool transposed) {
  const c10::cuda::CUDAGuard guard(P.device());
  chk_f32c(P, "P"); chk_f32c(V, "V"); chk_f32c(out, "out"); chk_i32c(indices, "indices");
  TORCH_CHECK(V.dim() == 3 && out.dim() == 3 && V.size(1) == (transposed ? Lq : Lk) && out.size(1) == (transposed ? Lk : Lq) && V.size(2) == out.size(2), "mra_spmm: operand lengths do not match the block grid");
  TORCH_CHECK(P.numel() == indices.numel() * 1024 && Lq % 32 == 0 && Lk % 32 == 0, "mra_spmm: P [B, n, 32, 32]");
  b200::mra_spmm(P.data_ptr<float>(), indices.data_ptr<int>(), V.data_ptr<float>(), out.data_ptr<float>(), (int)V.size(0), (int)Lq, (int)Lk,
                 (int)V.size(2), (int)indices.size(1), transposed, cur_stream());
}

void mra_rowmax(const Tensor& S, const Tensor& indices, Tensor m, int64_t Lk) {
  const c10::cuda::CUDAGuard guard(S.device());
  chk_f32c(S, "S"); chk_f32c(m, "m"); chk_i32c(indices, "indices");
  TORCH_CHECK(m.dim() == 2 && S.numel() == indices.numel() * 1024 && m.size(0) == indices.size(0), "mra_rowmax: S [B, n, 32, 32], m [B, Lq]");
  b200::mra_rowmax(S.data_ptr<float>(), indices.data_ptr<int>(), m.data_ptr<float>(), (int)m.size(0), (int)m.size(1), (int)Lk, (int)indices.size(1), cur_stream());
}
// ---------------------------------------------------------------------------------------------- fused tap kernels
void chk_rows_f32(const Tensor& t, int64_t n, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == n, name, ": contiguous fp32 CUDA tensor of ", n, " elements");
}

void tele_fused_fwd(const Tensor& x, const Tensor& freq, const Tensor& phase, const Tensor& kern, const Tensor& expo, Tensor out,
                    int64_t H, int64_t half, double max_rec) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x"); chk_bf16c(out, "out");
  TORCH_CHECK(x.dim() == 3 && out.sizes() == x.sizes() && kern.dim() == 4, "tele_fused: x/out [B,L,C], kern [B,L,H,K]");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2), K = (int)kern.size(3);
  const int64_t rows = (int64_t)B * L * H;
  chk_rows_f32(freq, rows, "freq"); chk_rows_f32(phase, rows, "phase"); chk_rows_f32(kern, rows * K, "kern"); chk_rows_f32(expo, (int64_t)B * L, "expo");
  b200::tele_fused_fwd(x.data_ptr(), freq.data_ptr<float>(), phase.data_ptr<float>(), kern.data_ptr<float>(), expo.data_ptr<float>(),
                       out.data_ptr(), B, L, (int)H, C / (int)H, K, (int)half, (float)max_rec, cur_stream());
}

void tele_fused_bwd(const Tensor& x, const Tensor& freq, const Tensor& phase, const Tensor& kern, const Tensor& expo, const Tensor& dout,
                    Tensor dx, Tensor dfreq, Tensor dphase, Tensor dkern, Tensor dexpo_h, int64_t H, int64_t half, double max_rec) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x"); chk_bf16c(dout, "dout");
  TORCH_CHECK(x.dim() == 3 && dout.sizes() == x.sizes() && kern.dim() == 4, "tele_fused: x/dout [B,L,C], kern [B,L,H,K]");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2), K = (int)kern.size(3);
  const int64_t rows = (int64_t)B * L * H;
  chk_rows_f32(freq, rows, "freq"); chk_rows_f32(phase, rows, "phase"); chk_rows_f32(kern, rows * K, "kern"); chk_rows_f32(expo, (int64_t)B * L, "expo");
  chk_rows_f32(dx, x.numel(), "dx"); chk_rows_f32(dfreq, rows, "dfreq"); chk_rows_f32(dphase, rows, "dphase");
  chk_rows_f32(dkern, rows * K, "dkern"); chk_rows_f32(dexpo_h, rows, "dexpo_h");
  b200::tele_fused_bwd(x.data_ptr(), freq.data_ptr<float>(), phase.data_ptr<float>(), kern.data_ptr<float>(), expo.data_ptr<float>(),
                       dout.data_ptr(), dx.data_ptr<float>(), dfreq.data_ptr<float>(), dphase.data_ptr<float>(), dkern.data_ptr<float>(),
                       dexpo_h.data_ptr<float>(), B, L, (int)H, C / (int)H, K, (int)half, (float)max_rec, cur_stream());
}

void alc_fused_fwd(const Tensor& x, const Tensor& half_w, const Tensor& center, const Tensor& kern, Tensor out, int64_t H, int64_t half) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x"); chk_bf16c(out, "out");
  TORCH_CHECK(x.dim() == 3 && out.sizes() == x.sizes() && kern.dim() == 4, "alc_fused: x/out [B,L,C], kern [B,L,H,K]");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2), K = (int)kern.size(3);
  const int64_t rows = (int64_t)B * L * H;
  chk_rows_f32(half_w, rows, "half_w"); chk_rows_f32(center, rows, "center"); chk_rows_f32(kern, rows * K, "kern");
  b200::alc_fused_fwd(x.data_ptr(), half_w.data_ptr<float>(), center.data_ptr<float>(), kern.data_ptr<float>(), out.data_ptr(), B, L,
                      (int)H, C / (int)H, K, (int)half, cur_stream());
}

void alc_fused_bwd(const Tensor& x, const Tensor& half_w, const Tensor& center, const Tensor& kern, const Tensor& dout, Tensor dx,
                   Tensor dhalf_w, Tensor dcenter, Tensor dkern, int64_t H, int64_t half) {
  const c10::cuda::CUDAGuard guard(x.device());
  chk_bf16c(x, "x"); chk_bf16c(dout, "dout");
  TORCH_CHECK(x.dim() == 3 && dout.sizes() == x.sizes() && kern.dim() == 4, "alc_fused: x/dout [B,L,C], kern [B,L,H,K]");
  const int B = (int)x.size(0), L = (int)x.size(1), C = (int)x.size(2), K = (int)kern.size(3);
  const int64_t rows = (int64_t)B * L * H;
  chk_rows_f32(half_w, rows, "half_w"); chk_rows_f32(center, rows, "center"); chk_rows_f32(kern, rows * K, "kern");
  chk_rows_f32(dx, x.numel(), "dx"); chk_rows_f32(dhalf_w, rows, "dhalf_w"); chk_rows_f32(dcenter, rows, "dcenter"); chk_rows_f32(dkern, rows * K, "dkern");
  b200::alc_fused_bwd(x.data_ptr(), half_w.data_ptr<float>(), center.data_ptr<float>(), kern.data_ptr<float>(), dout.data_ptr(),
                      dx.data_ptr<float>(), dhalf_w.data_ptr<float>(), dcenter.data_ptr<float>(), dkern.data_ptr<float>(), B, L, (int)H,
                      C / (int)H, K, (int)half, cur_stream());
}

// ---------------------------------------------------------------------------------------------- RMSNorm + activation
bool norm_io_bf16(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && (t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat), n, ": contiguous bf16 or fp32 CUDA tensor");
  return t.scalar_type() == at::kBFloat16;
}

// The row kernels move 4 bf16 (8 bytes) per lane: the base address and every stride a row offset is built from must be
// multiples of 8 bytes, or the access faults on the device. Views with odd offsets are refused here, on the host.
static bool aligned8(const Tensor& t) { return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 7) == 0; }
static bool strides_mult4(const Tensor& t) {
  for (int i = 0; i + 1 < t.dim(); ++i)
    if (t.size(i) > 1 && t.stride(i) % 4 != 0) return false;
  return true;
}

static void norm_rope_args(const Tensor& x, const Tensor& f1, const Tensor& f2, int64_t& rows, int& H, int& T, int& D, int& W) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.scalar_type() == at::kBFloat16 && x.stride(3) == 1, "norm_rope: x bf16 [batch, T, H, D], unit stride over D");
  TORCH_CHECK(x.size(0) == 1 || x.stride(0) == x.size(1) * x.stride(1), "norm_rope: batch entries must follow each other token-wise");
  TORCH_CHECK(aligned8(x) && strides_mult4(x) && aligned8(f1) && aligned8(f2), "norm_rope: x and the tables must be 8-byte aligned, x's strides multiples of 4 elements");
  T = (int)x.size(1); H = (int)x.size(2); D = (int)x.size(3);
  rows = x.size(0) * x.size(1) * x.size(2);
  TORCH_CHECK(f1.scalar_type() == at::kBFloat16 && f2.scalar_type() == at::kBFloat16 && f1.is_contiguous() && f2.is_contiguous() &&
              f1.dim() == 2 && f1.sizes() == f2.sizes() && f1.size(0) >= T && (f1.size(1) == D || f1.size(1) == 2 * D),
              "norm_rope: tables bf16 [>= T, D or 2 D]");
  W = (int)f1.size(1);
  TORCH_CHECK(W == D || H % 2 == 0, "norm_rope: the paired table needs an even number of heads");
}

void norm_rope_fwd(const Tensor& x, const Tensor& f1, const Tensor& f2, Tensor y, Tensor rstd, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  int64_t rows; int H, T, D, W;
  norm_rope_args(x, f1, f2, rows, H, T, D, W);
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.is_contiguous() && y.numel() == rows * D && rstd.scalar_type() == at::kFloat && rstd.numel() == rows &&
              aligned8(y), "norm_rope_fwd: outputs");
  b200::norm_rope_fwd(x.data_ptr(), x.stride(1), x.stride(2), f1.data_ptr(), f2.data_ptr(), W, y.data_ptr(), rstd.data_ptr<float>(), rows, H, T, D,
                      (float)eps, cur_stream());
}

void norm_rope_bwd(const Tensor& x, const Tensor& f1, const Tensor& f2, const Tensor& rstd, const Tensor& dy, Tensor dx) {
  const c10::cuda::CUDAGuard guard(x.device());
  int64_t rows; int H, T, D, W;
  norm_rope_args(x, f1, f2, rows, H, T, D, W);
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.numel() == rows * D && dx.scalar_type() == at::kBFloat16 && dx.is_contiguous() &&
              dx.numel() == rows * D && rstd.numel() == rows && aligned8(dy) && aligned8(dx), "norm_rope_bwd: dy / dx bf16 contiguous, 8-byte aligned");
  b200::norm_rope_bwd(x.data_ptr(), x.stride(1), x.stride(2), f1.data_ptr(), f2.data_ptr(), W, rstd.data_ptr<float>(), dy.data_ptr(), dx.data_ptr(), rows,
                      H, T, D, cur_stream());
}

void rowscale_add_fwd(const c10::optional<Tensor>& a, const Tensor& g, const Tensor& b, Tensor out) {
  const c10::cuda::CUDAGuard guard(b.device());
  TORCH_CHECK(b.is_cuda() && b.dim() == 4 && b.scalar_type() == at::kBFloat16 && b.is_contiguous(), "rowscale_add: b bf16 contiguous [batch, T, H, D]");
  const int H = (int)b.size(2), D = (int)b.size(3);
  const int64_t rows = b.numel() / D;
  TORCH_CHECK(g.scalar_type() == at::kBFloat16 && g.is_contiguous() && g.numel() == rows, "rowscale_add: g bf16 [batch * T * H]");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() == b.numel(), "rowscale_add: out");
  TORCH_CHECK(aligned8(b) && aligned8(out), "rowscale_add: b and out must be 8-byte aligned");
  const void* ap = nullptr;
  int64_t st = 0, sh = 0;
  if (a.has_value()) {
    TORCH_CHECK(a->scalar_type() == at::kBFloat16 && a->sizes() == b.sizes() && a->stride(3) == 1 &&
                (a->size(0) == 1 || a->stride(0) == a->size(1) * a->stride(1)), "rowscale_add: a bf16 [batch, T, H, D], unit stride over D");
    TORCH_CHECK(aligned8(*a) && strides_mult4(*a), "rowscale_add: a must be 8-byte aligned with strides that are multiples of 4 elements");
    ap = a->data_ptr(); st = a->stride(1); sh = a->stride(2);
  }
  b200::rowscale_add_fwd(ap, st, sh, g.data_ptr(), b.data_ptr(), out.data_ptr(), rows, H, D, cur_stream());
}

void rowscale_add_bwd(const Tensor& g, const Tensor& b, const Tensor& dout, Tensor db, Tensor dg) {
  const c10::cuda::CUDAGuard guard(b.device());
  const int D = (int)b.size(-1);
  const int64_t rows = b.numel() / D;
  for (const Tensor* t : {&b, &dout, (const Tensor*)&db})
    TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->is_contiguous() && t->numel() == rows * D && aligned8(*t), "rowscale_add_bwd: bf16 contiguous [rows, D], 8-byte aligned");
  TORCH_CHECK(g.numel() == rows && dg.numel() == rows && dg.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kBFloat16 && g.is_contiguous() && dg.is_contiguous(), "rowscale_add_bwd: g, dg bf16 [rows]");
  b200::rowscale_add_bwd(g.data_ptr(), b.data_ptr(), dout.data_ptr(), db.data_ptr(), dg.data_ptr(), rows, D, cur_stream());
}

static void lincomb_check(const Tensor& t, int64_t n, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.numel() == n && aligned8(t), "lincomb3: bf16 contiguous, 8-byte aligned ", what);
}

void lincomb3_fwd(const Tensor& x, const Tensor& y, const c10::optional<Tensor>& z, const Tensor& c, Tensor out) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t n = x.numel();
  lincomb_check(x, n, "x"); lincomb_check(y, n, "y"); lincomb_check(out, n, "out");
  if (z.has_value()) lincomb_check(*z, n, "z");
  TORCH_CHECK(c.is_cuda() && c.scalar_type() == at::kFloat && c.is_contiguous() && c.numel() >= (z.has_value() ? 3 : 2), "lincomb3: c fp32 on the device");
  b200::lincomb3_fwd(x.data_ptr(), y.data_ptr(), z.has_value() ? z->data_ptr() : nullptr, c.data_ptr<float>(), out.data_ptr(), n, cur_stream());
}

void lincomb3_bwd(const Tensor& x, const Tensor& y, const c10::optional<Tensor>& z, const Tensor& c, const Tensor& dout, Tensor dx, Tensor dy,
                  const c10::optional<Tensor>& dz, Tensor dc) {
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t n = x.numel();
  lincomb_check(x, n, "x"); lincomb_check(y, n, "y"); lincomb_check(dout, n, "dout"); lincomb_check(dx, n, "dx"); lincomb_check(dy, n, "dy");
  TORCH_CHECK(z.has_value() == dz.has_value(), "lincomb3_bwd: z and dz go together");
  if (z.has_value()) { lincomb_check(*z, n, "z"); lincomb_check(*dz, n, "dz"); }
  TORCH_CHECK(dc.scalar_type() == at::kFloat && dc.is_contiguous() && dc.numel() >= 3, "lincomb3_bwd: dc fp32 [3], zeroed");
  b200::lincomb3_bwd(x.data_ptr(), y.data_ptr(), z.has_value() ? z->data_ptr() : nullptr, c.data_ptr<float>(), dout.data_ptr(), dx.data_ptr(),
                     dy.data_ptr(), dz.has_value() ? dz->data_ptr() : nullptr, dc.data_ptr<float>(), n, cur_stream());
}

void rms_act_fwd(const Tensor& x, const Tensor& w, Tensor y, Tensor rstd, double eps, int64_t act) {
  const c10::cuda::CUDAGuard guard(x.device());
  const bool xb = norm_io_bf16(x, "x"), yb = norm_io_bf16(y, "y");
  const int C = (int)x.size(-1);
  const int64_t R = x.numel() / C;
  TORCH_CHECK(y.numel() == x.numel(), "y: x's shape");
  chk_rows_f32(w, C, "weight"); chk_rows_f32(rstd, R, "rstd");
  b200::rms_act_fwd(x.data_ptr(), xb, w.data_ptr<float>(), y.data_ptr(), yb, rstd.data_ptr<float>(), R, C, (float)eps, (int)act, cur_stream());
}

void rms_act_bwd(const Tensor& x, const Tensor& w, const Tensor& rstd, const Tensor& dy, const c10::optional<Tensor>& dres,
                 const c10::optional<Tensor>& dlead, Tensor dx, Tensor dw, int64_t act) {
  const c10::cuda::CUDAGuard guard(x.device());
  const bool xb = norm_io_bf16(x, "x"), gb = norm_io_bf16(dy, "dy");
  TORCH_CHECK(norm_io_bf16(dx, "dx") == xb && dx.numel() == x.numel() && dy.numel() == x.numel(), "dx: x's dtype and shape; dy: x's shape");
  const int C = (int)x.size(-1);
  const int64_t R = x.numel() / C;
  chk_rows_f32(w, C, "weight"); chk_rows_f32(rstd, R, "rstd"); chk_rows_f32(dw, C, "dw");
  const void* res = nullptr;
  if (dres.has_value()) {
    TORCH_CHECK(dres->is_cuda() && dres->is_contiguous() && dres->scalar_type() == x.scalar_type() && dres->numel() == x.numel(),
                "dres: a dense tensor of x's dtype and shape");
    res = dres->data_ptr();
  }
  const void* lead_p = nullptr;
  int lead = 0;
  if (dlead.has_value()) {
    TORCH_CHECK(dlead->is_cuda() && dlead->is_contiguous() && dlead->scalar_type() == dy.scalar_type() && dlead->dim() >= 1 &&
                dlead->size(-1) <= C && dlead->numel() == R * dlead->size(-1), "dlead: dense [rows, lead <= C] of dy's dtype");
    lead_p = dlead->data_ptr();
    lead = (int)dlead->size(-1);
  }
  b200::rms_act_bwd(x.data_ptr(), xb, w.data_ptr<float>(), rstd.data_ptr<float>(), dy.data_ptr(), gb, res, lead_p, lead, dx.data_ptr(),
                    dw.data_ptr<float>(), R, C, (int)act, cur_stream());
}

}  // namespace

TORCH_LIBRARY(b200, m) {
  m.def(
      "gemm(Tensor a, Tensor b, Tensor(a!) c, Tensor? aux, bool a_mn, bool b_mn, int epilogue, float alpha, "
      "float beta, int split_k, bool accumulate, Tensor status) -> ()");
  m.def("attn_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) o, Tensor(b!) lse, Tensor doc_start, Tensor doc_end, float scale, int window_blocks, Tensor status) -> ()");
  m.def("attn_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor d_o, Tensor lse, Tensor(a!) delta, Tensor(b!) dq_acc, Tensor(c!) dk, Tensor(d!) dv, Tensor doc_start, Tensor doc_end, float scale, int window_blocks, Tensor status) -> ()");
  m.def("mix_norm_fwd(Tensor x, Tensor? x0, Tensor? skip, Tensor? lam, Tensor? skip_w, Tensor(a!)? x_mix, Tensor(b!)? xn, float eps) -> ()");
  m.def("norm_bwd_add(Tensor dy, Tensor x, Tensor? dres, Tensor(a!) out, float eps) -> ()");
  m.def("mix_bwd(Tensor dmix, Tensor x, Tensor x0, Tensor? skip, Tensor lam, Tensor? skip_w, Tensor(a!) dx, Tensor(b!)? dskip, Tensor(c!) dx0_acc, Tensor(d!) dlam, Tensor(e!)? dskip_w, Tensor? dx_add=None) -> ()");
  m.def("qkv_post_fwd(Tensor qkv, Tensor? ve, Tensor lam, Tensor cos, Tensor sin, Tensor(a!) out, int H, int D, float eps) -> ()");
  m.def("qkv_post_bwd(Tensor dq, Tensor dk, Tensor dv, Tensor qkv, Tensor? ve, Tensor lam, Tensor cos, Tensor sin, Tensor(a!) dqkv, Tensor(b!)? dve, Tensor(c!) dlam, int H, int D, float eps) -> ()");
  m.def("embed_gather(Tensor idx, Tensor table, Tensor(a!) out, bool normalize, float eps) -> ()");
  m.def("embed_scatter_add(Tensor idx, Tensor src, Tensor(a!) grad_table, Tensor? src2=None) -> ()");
  m.def("softcap_ce_set_cache(bool on, Tensor like) -> ()");
  m.def("doc_bounds(Tensor tokens, int bos, Tensor(a!) doc_start, Tensor(b!) doc_end) -> ()");
  m.def("cast_fp8(Tensor x, Tensor(a!) out, float scale) -> ()");
  m.def("softcap_ce(Tensor logits, Tensor targets, Tensor(a!) loss_rows, Tensor(b!)? grad, float cap, float div, float loss_scale, float grad_scale, float shift=0.0, Tensor? mtp_w=None) -> ()");
  m.def("adam_step(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, float lr, float beta1, float beta2, float eps, float wd, float bias1, float bias2, float grad_scale, Tensor(d!)? shadow=None, float shadow_scale=1.0) -> ()");
  m.def("adam_cautious(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, float b1, float b2, float eps, float step_size, float wd_lr) -> ()");
  m.def("normuon_scales(Tensor v, Tensor(a!) stat, Tensor(b!) second, bool red_cols, float beta2) -> ()");
  m.def("normuon_update(Tensor(a!) p, Tensor(b!)? mant, Tensor v, Tensor? scale, bool scale_per_row, float lr, float wd_lr, Tensor? lr_mat=None, Tensor? wd_mat=None) -> ()");
  m.def("muon_momentum(Tensor g, Tensor(a!) buf, Tensor(b!) out, Tensor(c!) sumsq, float mu, bool nesterov, float grad_scale) -> ()");
  m.def("scale_by_inv_norm(Tensor(a!) x, Tensor sumsq, float eps) -> ()");
  m.def("axpy_bf16_to_f32(Tensor(a!) p, Tensor u, Tensor(b!)? p_bf16, float alpha) -> ()");
  m.def("comm_signal(int[] peer_flags, int rank, int channel, int epoch, Tensor like) -> ()");
  m.def("adam_shard(int[] grad_ptrs, int[] param_ptrs, int rank, int lo, int hi, int dtype, Tensor(a!) m, Tensor(b!) v, float lr, float beta1, float beta2, float eps, float wd, float bias1, float bias2, Tensor flags, int[] peer_flags, int channel, int epoch, Tensor(c!) status, int max_blocks=0) -> ()");
  m.def("comm_wait(Tensor flags, int world, int channel, int epoch, Tensor(a!) status) -> ()");
  m.def("muon_rs_momentum(int[] grad_ptrs, int elem_off, int nmat, int mat_elems, Tensor(a!) mom, Tensor(b!) u_out, Tensor(c!) sumsq, float mu, bool nesterov, Tensor flags, int channel, int epoch, Tensor(d!) status) -> ()");
  m.def("stack_scale_by_inv_norm(Tensor(a!) x, Tensor sumsq, int nmat, int mat_elems, float eps) -> ()");
  m.def("ag_push(Tensor src, int[] u_full_ptrs, int rank, int dst_off, int[] peer_flags, int channel, int epoch, int slot=0) -> ()");
  m.def("ag_wait_apply(Tensor(a!) p, Tensor u, Tensor(b!)? p_bf16, float alpha, int world, Tensor flags, int channel, int epoch, Tensor(c!) status) -> ()");
  m.def("allreduce_mean_multimem(int mc_ptr, int world, int rank, int n, int dtype, Tensor flags, int[] peer_flags, int channel, int epoch, Tensor(a!) status) -> ()");
  m.def("allreduce_mean(int[] buf_ptrs, int rank, int n, int dtype, Tensor flags, int[] peer_flags, int channel, int epoch, Tensor(a!) status) -> ()");
  m.def("s6_set_states_per_thread(int fwd_qs, int bwd_qs, Tensor like) -> ()");
  m.def("jacobi_fwd(Tensor Bm, Tensor Cm, Tensor theta, Tensor xr, Tensor alpha, Tensor gamma, Tensor conv_w, Tensor conv_b, Tensor? inj_lambda, Tensor? ro_lambda, int n_iters, Tensor(a!) gated, Tensor(b!)? Hs) -> ()");
  m.def("jacobi_bwd(Tensor dgated, Tensor Hs, Tensor Bm, Tensor Cm, Tensor theta, Tensor xr, Tensor alpha, Tensor gamma, Tensor conv_w, Tensor conv_b, Tensor? inj_lambda, Tensor? ro_lambda, int n_iters, Tensor(a!) dBm, Tensor(b!) dCm, Tensor(c!) dtheta, Tensor(d!) dxr, Tensor(e!) dalpha, Tensor(f!) dgamma, Tensor(g!) dconv_w, Tensor(h!) dconv_b, Tensor(i!) dlam) -> ()");
  m.def("ssd_flip_time(Tensor src) -> Tensor");
  m.def("ssd_bwd_post(Tensor x, Tensor dy, Tensor y, Tensor dx_rev, Tensor dB_rev, Tensor dC_heads, Tensor B, Tensor C, Tensor g_off, Tensor g_diag, Tensor(a!) dx, Tensor(b!) dB, Tensor(c!) dC, Tensor(d!) d_goff, Tensor(e!) d_gdiag, Tensor(f!) inner) -> ()");
  m.def("ssd_fwd(Tensor x, Tensor B, Tensor C, Tensor log_a, Tensor g_off, Tensor g_diag, Tensor(a!) y, Tensor? init_state, Tensor(b!)? final_state, Tensor(c!) status, Tensor(d!)? chunk_states=None) -> ()");
  m.def("s6_scan_fwd(Tensor u, Tensor delta, Tensor? delta_bias, bool softplus, Tensor A, Tensor Bm, Tensor Cm, Tensor? Dv, Tensor? z, Tensor(a!)? y_pre, Tensor(b!) out, Tensor(c!)? state) -> ()");
  m.def("s6_scan_bwd(Tensor u, Tensor delta, Tensor? delta_bias, bool softplus, Tensor A, Tensor Bm, Tensor Cm, Tensor? Dv, Tensor? z, Tensor? y_pre, Tensor dout, Tensor state, Tensor(a!) du, Tensor(b!) ddelta, Tensor(c!) dA, Tensor(d!) dB_part, Tensor(e!) dC_part, Tensor(f!)? dD, Tensor(g!)? dz, Tensor(h!)? ddelta_bias) -> ()");
  m.def("causal_conv1d_silu_fwd(Tensor x, Tensor w, Tensor? bias, Tensor(a!) y) -> ()");
  m.def("causal_conv1d_silu_bwd(Tensor x, Tensor w, Tensor? bias, Tensor dy, Tensor(a!) dx, Tensor(b!) dw, Tensor(c!)? dbias) -> ()");
  m.def("norm_rope_fwd(Tensor x, Tensor f1, Tensor f2, Tensor(a!) y, Tensor(b!) rstd, float eps) -> ()");
  m.def("norm_rope_bwd(Tensor x, Tensor f1, Tensor f2, Tensor rstd, Tensor dy, Tensor(a!) dx) -> ()");
  m.def("rowscale_add_fwd(Tensor? a, Tensor g, Tensor b, Tensor(a!) out) -> ()");
  m.def("rowscale_add_bwd(Tensor g, Tensor b, Tensor dout, Tensor(a!) db, Tensor(b!) dg) -> ()");
  m.def("lincomb3_fwd(Tensor x, Tensor y, Tensor? z, Tensor c, Tensor(a!) out) -> ()");
  m.def("lincomb3_bwd(Tensor x, Tensor y, Tensor? z, Tensor c, Tensor dout, Tensor(a!) dx, Tensor(b!) dy, Tensor(c!)? dz, Tensor(d!) dc) -> ()");
  m.def("rms_act_fwd(Tensor x, Tensor w, Tensor(a!) y, Tensor(b!) rstd, float eps, int act) -> ()");
  m.def("rms_act_bwd(Tensor x, Tensor w, Tensor rstd, Tensor dy, Tensor? dres, Tensor? dlead, Tensor(a!) dx, Tensor(b!) dw, int act) -> ()");
  m.def("tele_fused_fwd(Tensor x, Tensor freq, Tensor phase, Tensor kern, Tensor expo, Tensor(a!) out, int H, int half, float max_rec) -> ()");
  m.def("tele_fused_bwd(Tensor x, Tensor freq, Tensor phase, Tensor kern, Tensor expo, Tensor dout, Tensor(a!) dx, Tensor(b!) dfreq, Tensor(c!) dphase, Tensor(d!) dkern, Tensor(e!) dexpo_h, int H, int half, float max_rec) -> ()");
  m.def("alc_fused_fwd(Tensor x, Tensor half_w, Tensor center, Tensor kern, Tensor(a!) out, int H, int half) -> ()");
  m.def("alc_fused_bwd(Tensor x, Tensor half_w, Tensor center, Tensor kern, Tensor dout, Tensor(a!) dx, Tensor(b!) dhalf_w, Tensor(c!) dcenter, Tensor(d!) dkern, int H, int half) -> ()");
  m.def("gather_conv_fwd(Tensor x, Tensor pos, Tensor wgt, Tensor(a!) out, int H, float pos_max) -> ()");
  m.def("gather_conv_bwd(Tensor x, Tensor pos, Tensor wgt, Tensor dout, Tensor(a!) dx, Tensor(b!) dpos, Tensor(c!) dwgt, int H, float pos_max) -> ()");
  m.def("wkv4_fwd(Tensor k, Tensor v, Tensor w, Tensor u, Tensor(a!) y) -> ()");
  m.def("wkv4_bwd(Tensor k, Tensor v, Tensor w, Tensor u, Tensor gy, Tensor(a!) gk, Tensor(b!) gv, Tensor(c!) gw, Tensor(d!) gu, Tensor(e!) scratch) -> ()");
  m.def("wkv5_fwd(Tensor r, Tensor k, Tensor v, Tensor w, Tensor u, Tensor(a!) y) -> ()");
  m.def("wkv5_bwd(Tensor r, Tensor k, Tensor v, Tensor w, Tensor u, Tensor gy, Tensor(a!) gr, Tensor(b!) gk, Tensor(c!) gv, Tensor(d!) gw, Tensor(e!) gu) -> ()");
  m.def("window_attn_fwd(Tensor q, Tensor k, Tensor v, Tensor bias, Tensor(a!) out, Tensor(b!) P, float scale) -> ()");
  m.def("window_attn_bwd(Tensor q, Tensor k, Tensor v, Tensor P, Tensor dout, Tensor(a!) dq, Tensor(b!) dk, Tensor(c!) dv, Tensor(d!) dbias, float scale) -> ()");
  m.def("mra_sddmm(Tensor Q, Tensor K, Tensor indices, Tensor(a!) S) -> ()");
  m.def("mra_spmm(Tensor P, Tensor indices, Tensor V, Tensor(a!) out, int Lq, int Lk, bool transposed) -> ()");
  m.def("mra_rowmax(Tensor S, Tensor indices, Tensor(a!) m, int Lk) -> ()");
  // <<DEFS>>
}

TORCH_LIBRARY_IMPL(b200, CUDA, m) {
  m.impl("gemm", &gemm);
  m.impl("attn_fwd", &attn_fwd);
  m.impl("attn_bwd", &attn_bwd);
  m.impl("mix_norm_fwd", &mix_norm_fwd);
  m.impl("norm_bwd_add", &norm_bwd_add);
  m.impl("mix_bwd", &mix_bwd);
  m.impl("qkv_post_fwd", &qkv_post_fwd);
  m.impl("qkv_post_bwd", &qkv_post_bwd);
  m.impl("embed_gather", &embed_gather);
  m.impl("embed_scatter_add", &embed_scatter_add);
  m.impl("softcap_ce_set_cache", &softcap_ce_set_cache);
  m.impl("doc_bounds", &doc_bounds);
  m.impl("cast_fp8", &cast_fp8);
  m.impl("softcap_ce", &softcap_ce);
  m.impl("adam_step", &adam_step);
  m.impl("adam_cautious", &adam_cautious);
  m.impl("normuon_scales", &normuon_scales);
  m.impl("normuon_update", &normuon_update);
  m.impl("muon_momentum", &muon_momentum);
  m.impl("scale_by_inv_norm", &scale_by_inv_norm);
  m.impl("axpy_bf16_to_f32", &axpy_bf16_to_f32);
  m.impl("comm_signal", &comm_signal);
  m.impl("adam_shard", &adam_shard);
  m.impl("comm_wait", &comm_wait);
  m.impl("muon_rs_momentum", &muon_rs_momentum);
  m.impl("stack_scale_by_inv_norm", &stack_scale_by_inv_norm);
  m.impl("ag_push", &ag_push);
  m.impl("ag_wait_apply", &ag_wait_apply);
  m.impl("allreduce_mean_multimem", &allreduce_mean_multimem);
  m.impl("allreduce_mean", &allreduce_mean);
  m.impl("s6_set_states_per_thread", &s6_set_states_per_thread);
  m.impl("ssd_fwd", &ssd_fwd);
  m.impl("ssd_flip_time", &ssd_flip_time);
  m.impl("ssd_bwd_post", &ssd_bwd_post);
  m.impl("jacobi_fwd", &jacobi_fwd);
  m.impl("jacobi_bwd", &jacobi_bwd);
  m.impl("s6_scan_fwd", &s6_scan_fwd);
  m.impl("s6_scan_bwd", &s6_scan_bwd);
  m.impl("causal_conv1d_silu_fwd", &causal_conv1d_silu_fwd);
  m.impl("causal_conv1d_silu_bwd", &causal_conv1d_silu_bwd);
  m.impl("norm_rope_fwd", &norm_rope_fwd);
  m.impl("norm_rope_bwd", &norm_rope_bwd);
  m.impl("rowscale_add_fwd", &rowscale_add_fwd);
  m.impl("rowscale_add_bwd", &rowscale_add_bwd);
  m.impl("lincomb3_fwd", &lincomb3_fwd);
  m.impl("lincomb3_bwd", &lincomb3_bwd);
  m.impl("rms_act_fwd", &rms_act_fwd);
  m.impl("rms_act_bwd", &rms_act_bwd);
  m.impl("tele_fused_fwd", &tele_fused_fwd);
  m.impl("tele_fused_bwd", &tele_fused_bwd);
  m.impl("alc_fused_fwd", &alc_fused_fwd);
  m.impl("alc_fused_bwd", &alc_fused_bwd);
  m.impl("gather_conv_fwd", &gather_conv_fwd);
  m.impl("gather_conv_bwd", &gather_conv_bwd);
  m.impl("wkv4_fwd", &wkv4_fwd);
  m.impl("wkv4_bwd", &wkv4_bwd);
  m.impl("wkv5_fwd", &wkv5_fwd);
  m.impl("wkv5_bwd", &wkv5_bwd);
  m.impl("window_attn_fwd", &window_attn_fwd);
  m.impl("window_attn_bwd", &window_attn_bwd);
  m.impl("mra_sddmm", &mra_sddmm);
  m.impl("mra_spmm", &mra_spmm);
  m.impl("mra_rowmax", &mra_rowmax);
  // <<IMPLS>>
}
