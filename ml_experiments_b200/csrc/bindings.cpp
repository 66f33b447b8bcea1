// torch op registrations (namespace b200). The .cu files are torch-free; this file adapts
// at::Tensor arguments to their plain C++ launch structs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include "gemm/gemm.h"

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

}  // namespace

TORCH_LIBRARY(b200, m) {
  m.def(
      "gemm(Tensor a, Tensor b, Tensor(a!) c, Tensor? aux, bool a_mn, bool b_mn, int epilogue, float alpha, "
      "float beta, int split_k, bool accumulate, Tensor status) -> ()");
  // <<DEFS>>
}

TORCH_LIBRARY_IMPL(b200, CUDA, m) {
  m.impl("gemm", &gemm);
  // <<IMPLS>>
}
