// Fused compute + collective kernels over peer memory (NVLink / NVSwitch), torch-free interface.
//
// Every rank owns one buffer of each kind at the same offset of a symmetric allocation; `peers[r]` is rank r's
// copy as seen from this GPU (peers[rank] is the local one). Cross-rank ordering uses epoch flags:
// `flags` is this rank's int32 flag array [channels][world]; `peer_flags[r]` is rank r's copy. A rank announces
// "my data for epoch e is complete" by storing e into slot [channel][rank] of every peer with release semantics;
// a consumer spins (bounded) on its local slots with acquire loads. Epochs only grow, so flags never need clearing.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {

constexpr int kMaxWorld = 16;

struct PeerPtrs {
  void* p[kMaxWorld];
};

// Writes `epoch` into slot [channel][rank] of every peer's flag array (after a system-scope fence).
void comm_signal(const PeerPtrs& peer_flags, int world, int rank, int channel, int epoch, cudaStream_t s);

// Reduce-scatter fused with the Muon momentum update, for one stack of `nmat` owned matrices of `mat_elems`
// elements each, starting at element `elem_off` of every rank's fp32 gradient stack:
//   g   = mean_r grads_r[elem_off + i]                     (peer loads)
//   buf = mu * buf + (1 - mu) * g ;  u = nesterov ? (1 - mu) * g + mu * buf : buf
//   u_out[i] = bf16(u) ;  sumsq[m] += sum(u_bf16^2) over matrix m
// Waits (bounded) until flags[channel][r] >= epoch for every r before touching peer memory.
void muon_rs_momentum(const PeerPtrs& grads, int world, long long elem_off, int nmat, long long mat_elems, float* mom,
                      void* u_out_bf16, float* sumsq, float mu, int nesterov, const int* flags, int channel, int epoch,
                      int* status, cudaStream_t s);

// x[m] *= 1 / (sqrt(sumsq[m]) + eps) for a stack of nmat bf16 matrices.
void stack_scale_by_inv_norm(void* x_bf16, const float* sumsq, int nmat, long long mat_elems, float eps,
                             cudaStream_t s);

// All-gather by peer stores: copies this rank's `n` bf16 elements to element offset `dst_off` of every rank's
// `u_full` buffer (16-byte vector stores), then signals flags[channel][rank] = epoch on every peer.
// `slot` (0..15) selects the completion counter: launches that can overlap on the device must use different slots.
void ag_push(const void* src_bf16, const PeerPtrs& u_full, int world, int rank, long long dst_off, long long n,
             const PeerPtrs& peer_flags, int channel, int epoch, int slot, cudaStream_t s);

// Waits for every rank's ag_push of `epoch`, then applies p += alpha * u (fp32 master) and refreshes the bf16 copy.
void ag_wait_apply(float* p, const void* u_bf16, void* p_bf16, long long n, float alpha, int world, const int* flags,
                   int channel, int epoch, int* status, cudaStream_t s);

// In-place all-reduce (mean) of `n` elements of a symmetric buffer, two-shot over peer memory:
// every rank reduces its 1/world slice from all peers, scales by 1/world and stores the result into every peer.
// dtype: 0 = fp32, 1 = bf16 (fp32 accumulation). Waits on `channel` (inputs ready) and signals `channel + 1`
// (slice written everywhere); consumers wait for channel + 1 with comm_wait before reading the buffer.
void allreduce_mean(const PeerPtrs& bufs, int world, int rank, long long n, int dtype, const int* flags,
                    const PeerPtrs& peer_flags, int channel, int epoch, int* status, cudaStream_t s);

// The same all-reduce through NVSwitch multicast (NVLS): `mc` is the multicast address of the symmetric buffer; the sum
// is formed inside the switch by multimem.ld_reduce and written to every rank by multimem.st. Same flag protocol.
void allreduce_mean_multimem(void* mc, int world, int rank, long long n, int dtype, const int* flags,
                             const PeerPtrs& peer_flags, int channel, int epoch, int* status, cudaStream_t s);

// Sharded Adam fused with its collectives. `grads` / `params` are symmetric buffers (same layout on every rank, dtype 0 =
// fp32, 1 = bf16, both of the same type); this rank owns elements [lo, hi) (multiples of the 16-byte vector) and keeps
// the fp32 moments m, v of that slice only (indexed from lo). The kernel waits for `channel` (every rank's gradients are
// in place), averages the slice over the ranks by peer loads, applies Adam (decoupled weight decay wd * lr) and stores
// the new parameters into every rank's buffer, then signals `channel + 1`. Two launches that use the same channel
// pair must be enqueued in the same order on every rank. `max_blocks` > 0 caps the grid (a small grid leaves SMs to a
// concurrent compute stream; the copy is link-bound long before it needs the whole machine).
void adam_shard(const PeerPtrs& grads, const PeerPtrs& params, int world, int rank, long long lo, long long hi, int dtype,
                float* m, float* v, float lr, float beta1, float beta2, float eps, float wd, float bias1, float bias2,
                const int* flags, const PeerPtrs& peer_flags, int channel, int epoch, int* status, int max_blocks,
                cudaStream_t s);

// Blocks the stream (bounded) until flags[channel][r] >= epoch for every r.
void comm_wait(const int* flags, int world, int channel, int epoch, int* status, cudaStream_t s);

}  // namespace b200
