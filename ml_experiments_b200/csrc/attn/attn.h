// Causal, document-masked, block-sliding-window flash attention on tcgen05/TMEM (torch-free interface).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {

// q, k, v, o, do, dk, dv : bf16, element (t, h, d) at  base + t * ld + h * D + d   (ld in elements)
// dq_acc                 : fp32, same addressing, must be zero on entry (accumulated with TMA reduce-add)
// lse                    : fp32 [H][T], log2-domain log-sum-exp of the scaled scores
// delta                  : fp32 [H][T], rowsum(O * dO)
// doc_start / doc_end    : int32 [T], first token / one-past-last token of the document holding token t
// window_blocks          : a query in 128-token block qb sees key blocks (qb - window_blocks, qb]; <= 0: no window
struct AttnArgs {
  const void* q = nullptr; const void* k = nullptr; const void* v = nullptr;
  void* o = nullptr;
  const void* d_o = nullptr;
  void* dq_acc = nullptr; void* dk = nullptr; void* dv = nullptr;
  float* lse = nullptr; float* delta = nullptr;
  const int* doc_start = nullptr; const int* doc_end = nullptr;
  int T = 0, H = 0, D = 128;
  long long ld_q = 0, ld_k = 0, ld_v = 0, ld_o = 0, ld_do = 0, ld_dq = 0, ld_dk = 0, ld_dv = 0;
  float scale = 1.f;
  int window_blocks = 0;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
};

void attn_fwd_sm100(const AttnArgs& a);        // writes o, lse
void attn_delta_sm100(const AttnArgs& a);      // writes delta from o, d_o
void attn_bwd_sm100(const AttnArgs& a);        // needs lse, delta; writes dk, dv, accumulates dq_acc

}  // namespace b200
