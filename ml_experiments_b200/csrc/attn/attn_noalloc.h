// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference code base; it exists for hosts of this library that run
// inside someone else's memory budget: an inference / training runtime that has already handed all device memory
// to its own pool, a plug-in called from a latency-critical loop where cudaMalloc would synchronise the device, or
// code running where the CUDA allocator is off limits. Such callers can supply their inputs and outputs but cannot
// ask this library to create the temporary "delta" buffer (rowsum(O * dO), one float per head and token) that the
// regular backward allocates per call.
//
// Here that temporary lives in a fixed array inside the library image: B200_ATTN_NOALLOC_MAX_HT floats (4 MiB) per
// GPU that loads the library, held until the process exits. Consequences for the caller:
//   * H * T must not exceed B200_ATTN_NOALLOC_MAX_HT; larger problems are refused with an error code.
//   * The first call on each device (with that device current) looks up the array's device address
//     (cudaGetSymbolAddress) and opts the kernels into their shared-memory size on that device; make that first
//     call outside of any stream capture. Both pieces of set-up are remembered per device ordinal, so one process
//     may drive several GPUs. `stream` must belong to the device that is current at the call.
//   * The per-device set-up is not locked: two host threads that make the first call on the same device at the same
//     time both perform it (same address, same attribute value), which is harmless.
//   * All calls on one device share the array. It is fully rewritten at the start of every call, so nothing needs
//     clearing, but two calls whose kernels may overlap on the GPU (different streams) race on it: serialise them.
//   * The function itself never calls cudaMalloc / cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define B200_ATTN_NOALLOC_MAX_HT (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Tensors: bf16, element (t, h, d) at base + t * ld + h * D + d (ld in elements), D = 64 or 128.
//   q, k, v, o, d_o : inputs;  lse : fp32 [H][T] from the forward;  doc_start / doc_end : int32 [T]
//   dq_acc          : fp32 [T][H][D] with row pitch ld_dq, must be zero on entry, receives dQ
//   dk, dv          : bf16 outputs
//   status          : device int32 that stays 0 unless a bounded in-kernel wait expired (may be NULL)
// Returns 0 on success; -1 invalid argument, -2 H*T exceeds the built-in scratch, -3 CUDA error.
// b200_attn_bwd_noalloc_error() gives the message of the last failure on the calling thread.
int b200_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const float* lse, float* dq_acc, void* dk, void* dv, const int* doc_start,
                          const int* doc_end, int T, int H, int D, long long ld_q, long long ld_k, long long ld_v,
                          long long ld_o, long long ld_do, long long ld_dq, long long ld_dk, long long ld_dv,
                          float scale, int window_blocks, int* status, cudaStream_t stream);

const char* b200_attn_bwd_noalloc_error(void);

#ifdef __cplusplus
}
#endif
