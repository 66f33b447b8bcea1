// Fused compute + collective kernels over peer memory: plain peer loads / stores through NVLink (no TMA, no
// multicast), epoch flags with release / acquire at system scope, every spin bounded by a wall-clock limit.
#include "comm.h"

#include <cuda_bf16.h>

#include <atomic>
#include <stdexcept>
#include <string>

#include "../common/ptx.cuh"

namespace b200 {
namespace {

using bf16 = __nv_bfloat16;

// A peer rank can lag by a whole step (data loading, host jitter): allow far more than an on-chip wait.
// The default can be overridden at run time: word 1 of the status buffer holds the limit in microseconds (0 = default),
// so a host can shorten it (failure-detection tests let a wait on a flag that nobody sets expire after a millisecond).
constexpr unsigned long long kPeerWaitNs = 5000000000ull;

__device__ __forceinline__ unsigned long long peer_wait_limit_ns(const int* status) {
  if (status == nullptr) return kPeerWaitNs;
  const int us = *reinterpret_cast<const volatile int*>(status + 1);
  return us > 0 ? (unsigned long long)us * 1000ull : kPeerWaitNs;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All threads of the block return once every rank's flag of `channel` has reached `epoch` (or the wait expired,
// which is recorded in *status and reported through the return value).
__device__ bool block_wait_flags(const int* flags, int world, int channel, int epoch, int* status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* f = flags + channel * kMaxWorld + threadIdx.x;
    if (ld_acquire_sys(f) < epoch) {
      const uint64_t t0 = globaltimer_ns();
      const unsigned long long limit = peer_wait_limit_ns(status);
      for (;;) {
        if (ld_acquire_sys(f) >= epoch) break;
        if (status_poisoned(status)) { s_fail = 1; break; }
        if (globaltimer_ns() - t0 > limit) {
          if (status) atomicCAS(status, 0, ERR_WAIT_PEER_FLAG);
          s_fail = 1;
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  return s_fail == 0;
}

__global__ void signal_kernel(PeerPtrs peer_flags, int world, int rank, int channel, int epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(peer_flags.p[threadIdx.x]) + channel * kMaxWorld + rank, epoch);
  }
}

__global__ void wait_kernel(const int* flags, int world, int channel, int epoch, int* status) {
  block_wait_flags(flags, world, channel, epoch, status);
}

// The last block to finish (device-scope counter after a system-scope fence) announces completion to every peer.
__device__ void block_done_then_signal(int* counter, const PeerPtrs& peer_flags, int world, int rank, int channel,
                                       int epoch) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(counter, 1) + 1;
    s_last = (done == (int)(gridDim.x * gridDim.y));
    if (s_last) *counter = 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(peer_flags.p[threadIdx.x]) + channel * kMaxWorld + rank, epoch);
  }
}

// grid (blocks per matrix, nmat)
__global__ void __launch_bounds__(256)
rs_momentum_kernel(PeerPtrs grads, int world, int rank, long long elem_off, long long mat_elems, float* __restrict__ mom,
                   bf16* __restrict__ u_out, float* __restrict__ sumsq, float mu, int nesterov, const int* flags,
                   int channel, int epoch, int* status) {
  __shared__ float red[8];
  if (status_poisoned(status)) return;
  if (!block_wait_flags(flags, world, channel, epoch, status)) return;
  const int m = blockIdx.y;
  const long long base = (long long)m * mat_elems;
  const float inv_w = 1.f / world;
  float acc = 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < mat_elems;
       i += (long long)gridDim.x * blockDim.x * 4) {
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {   // starting after the own rank, so that the ranks pull from different peers at a time
      const float4 v = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[(rank + 1 + r) % world]) + elem_off + base + i));
      g.x += v.x; g.y += v.y; g.z += v.z; g.w += v.w;
    }
    float4 b = *reinterpret_cast<float4*>(mom + base + i);
    float gi[4] = {g.x * inv_w, g.y * inv_w, g.z * inv_w, g.w * inv_w};
    float bi[4] = {b.x, b.y, b.z, b.w};
    float u[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      bi[k] = mu * bi[k] + (1.f - mu) * gi[k];
      u[k] = nesterov ? (1.f - mu) * gi[k] + mu * bi[k] : bi[k];
    }
    *reinterpret_cast<float4*>(mom + base + i) = make_float4(bi[0], bi[1], bi[2], bi[3]);
    __nv_bfloat162 lo = __floats2bfloat162_rn(u[0], u[1]), hi = __floats2bfloat162_rn(u[2], u[3]);
    uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(u_out + base + i) = packed;
    const float2 l2 = __bfloat1622float2(lo), h2 = __bfloat1622float2(hi);
    acc += l2.x * l2.x + l2.y * l2.y + h2.x * h2.x + h2.y * h2.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    atomicAdd(&sumsq[m], t);
  }
}

__global__ void stack_scale_kernel(bf16* __restrict__ x, const float* __restrict__ sumsq, long long mat_elems,
                                   float eps) {
  const int m = blockIdx.y;
  const float s = 1.f / (sqrtf(sumsq[m]) + eps);
  bf16* xm = x + (long long)m * mat_elems;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < mat_elems;
       i += (long long)gridDim.x * blockDim.x * 2) {
    float2 v = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(xm + i));
    *reinterpret_cast<__nv_bfloat162*>(xm + i) = __floats2bfloat162_rn(v.x * s, v.y * s);
  }
}

__global__ void __launch_bounds__(256)
ag_push_kernel(const bf16* __restrict__ src, PeerPtrs u_full, int world, int rank, long long dst_off, long long n,
               PeerPtrs peer_flags, int channel, int epoch, int* counter) {
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n;
       i += (long long)gridDim.x * blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + i);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(u_full.p[r]) + dst_off + i) = v;
  }
  block_done_then_signal(counter, peer_flags, world, rank, channel, epoch);
}

__global__ void __launch_bounds__(256)
ag_wait_apply_kernel(float* __restrict__ p, const bf16* __restrict__ u, bf16* __restrict__ p_bf16, long long n,
                     float alpha, int world, const int* flags, int channel, int epoch, int* status) {
  if (status_poisoned(status)) return;
  if (!block_wait_flags(flags, world, channel, epoch, status)) return;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(u + i));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float4 v = *reinterpret_cast<float4*>(p + i);
    v.x = fmaf(alpha, a.x, v.x); v.y = fmaf(alpha, a.y, v.y); v.z = fmaf(alpha, b.x, v.z); v.w = fmaf(alpha, b.y, v.w);
    *reinterpret_cast<float4*>(p + i) = v;
    if (p_bf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      *reinterpret_cast<uint2*>(p_bf16 + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

template <int DT>  // 0: fp32 (4 per thread-iteration), 1: bf16 (8 per thread-iteration)
__global__ void __launch_bounds__(256)
allreduce_kernel(PeerPtrs bufs, int world, int rank, long long lo, long long hi, const int* flags, PeerPtrs peer_flags,
                 int channel, int epoch, int* status, int* counter) {
  if (status_poisoned(status)) return;
  const bool ok = block_wait_flags(flags, world, channel, epoch, status);
  constexpr int VEC = DT == 0 ? 4 : 8;
  const float inv_w = 1.f / world;
  if (ok) {
    // UNR vectors per thread and pass: all peer loads of a pass are issued before the first sum, which is what keeps
    // enough 16-byte loads in flight over NVLink (one vector per pass reached 300 of the 770 GB/s a plain copy gets at two ranks)
    constexpr int UNR = 2, GRP = 4;
    const long long stride = (long long)gridDim.x * blockDim.x * VEC;
    for (long long i0 = lo + ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i0 < hi; i0 += stride * UNR) {
      uint4 raw[UNR][GRP];
      float a[UNR][8];
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) a[u][k] = 0.f;
      for (int r0 = 0; r0 < world; r0 += GRP) {  // peers in groups of GRP
        const int nr = min(GRP, world - r0);
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long i = i0 + u * stride;
#pragma unroll
          for (int r = 0; r < GRP; ++r)
            if (r < nr && i < hi) {
              // peers are walked starting after the own rank: at any moment the ranks pull from different GPUs instead
              // of all from the same one (whose outbound links would be the bottleneck while the others idle)
              const int src = (rank + 1 + r0 + r) % world;
              raw[u][r] = DT == 0 ? __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(bufs.p[src]) + i))
                                  : __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(bufs.p[src]) + i));
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          if (i0 + u * stride >= hi) continue;
#pragma unroll
          for (int r = 0; r < GRP; ++r) {
            if (r >= nr) continue;
            if (DT == 0) {
              const float4 v = *reinterpret_cast<const float4*>(&raw[u][r]);
              a[u][0] += v.x; a[u][1] += v.y; a[u][2] += v.z; a[u][3] += v.w;
            } else {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][r]);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 x = __bfloat1622float2(h[k]);
                a[u][2 * k] += x.x;
                a[u][2 * k + 1] += x.y;
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * stride;
        if (i >= hi) continue;
        if (DT == 0) {
          const float4 o = make_float4(a[u][0] * inv_w, a[u][1] * inv_w, a[u][2] * inv_w, a[u][3] * inv_w);
          for (int r = 0; r < world; ++r) *reinterpret_cast<float4*>(reinterpret_cast<float*>(bufs.p[(rank + r) % world]) + i) = o;
        } else {
          uint4 o;
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int k = 0; k < 4; ++k) oh[k] = __floats2bfloat162_rn(a[u][2 * k] * inv_w, a[u][2 * k + 1] * inv_w);
          for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(bufs.p[(rank + r) % world]) + i) = o;
        }
      }
    }
  }
  block_done_then_signal(counter, peer_flags, world, rank, channel + 1, epoch);
}

// In-switch variant: `mc` is the NVLink multicast address of the same symmetric buffer. One multimem.ld_reduce returns
// the sum over all ranks of 16 bytes (reduced inside NVSwitch), one multimem.st writes the scaled result to every rank;
// each rank handles its 1/world slice, so every byte crosses this GPU's links once in each direction.
template <int DT>
__global__ void __launch_bounds__(256)
allreduce_multimem_kernel(void* mc, int world, int rank, long long lo, long long hi, const int* flags, PeerPtrs peer_flags,
                          int channel, int epoch, int* status, int* counter) {
  if (status_poisoned(status)) return;
  const bool ok = block_wait_flags(flags, world, channel, epoch, status);
  constexpr int VEC = DT == 0 ? 4 : 8;
  const float inv_w = 1.f / world;
  if (ok) {
    for (long long i = lo + ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < hi;
         i += (long long)gridDim.x * blockDim.x * VEC) {
      if (DT == 0) {
        float* addr = reinterpret_cast<float*>(mc) + i;
        float4 a;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "l"(addr) : "memory");
        a.x *= inv_w; a.y *= inv_w; a.z *= inv_w; a.w *= inv_w;
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                     :: "l"(addr), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w) : "memory");
      } else {
        bf16* addr = reinterpret_cast<bf16*>(mc) + i;
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = __bfloat1622float2(h[k]);
          h[k] = __floats2bfloat162_rn(x.x * inv_w, x.y * inv_w);
        }
        asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                     :: "l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
      }
    }
  }
  block_done_then_signal(counter, peer_flags, world, rank, channel + 1, epoch);
}


// ---------------------------------------------------------------------------------------------- sharded Adam
// Reduce-scatter + Adam + all-gather in one kernel. Gradients and parameters live in symmetric buffers of the same
// layout on every rank; this rank owns elements [lo, hi): it sums the peers' gradients for its slice by peer loads,
// runs Adam on its fp32 moments (held only here), and stores the updated parameter into every rank's parameter buffer.
// Afterwards it raises flag [channel + 1][rank] on every peer; a rank's parameters are complete when all `world`
// flags of channel + 1 have reached `epoch`.
template <typename T>
struct Vec16 {};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(&r);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    const float4 v = make_float4(f[0], f[1], f[2], f[3]);
    return *reinterpret_cast<const uint4*>(&v);
  }
};
template <>
struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __bfloat1622float2(h[k]);
      f[2 * k] = x.x; f[2 * k + 1] = x.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    return o;
  }
};

struct AdamHyper {
  float lr, b1, b2, eps, wd, bias1, inv_sqrt_bias2;
};

template <typename T>
__global__ void __launch_bounds__(256)
adam_shard_kernel(PeerPtrs grads, PeerPtrs params, int world, int rank, long long lo, long long hi,
                  float* __restrict__ m, float* __restrict__ v, AdamHyper h, const int* flags, PeerPtrs peer_flags,
                  int channel, int epoch, int* status, int* counter) {
  if (status_poisoned(status)) return;
  const bool ok = block_wait_flags(flags, world, channel, epoch, status);
  constexpr int VEC = Vec16<T>::N;
  const float inv_w = 1.f / world;
  if (ok) {
    constexpr int UNR = 2;
    const long long stride = (long long)gridDim.x * blockDim.x * VEC;
    for (long long i0 = lo + ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i0 < hi; i0 += stride * UNR) {
      float g[UNR][VEC];
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int k = 0; k < VEC; ++k) g[u][k] = 0.f;
      // the peers are walked starting after this rank, so that at any moment the ranks read from different peers
      for (int r0 = 0; r0 < world; r0 += 4) {
        uint4 raw[UNR][4];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long i = i0 + u * stride;
#pragma unroll
          for (int r = 0; r < 4; ++r)
            if (r0 + r < world && i < hi) {
              const int src = (rank + 1 + r0 + r) % world;
              raw[u][r] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(grads.p[src]) + i));
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          if (i0 + u * stride >= hi) continue;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            if (r0 + r >= world) continue;
            float f[VEC];
            Vec16<T>::unpack(raw[u][r], f);
#pragma unroll
            for (int k = 0; k < VEC; ++k) g[u][k] += f[k];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * stride;
        if (i >= hi) continue;
        float pf[VEC];
        const uint4 praw = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(params.p[rank]) + i);
        Vec16<T>::unpack(praw, pf);
        float* mp = m + (i - lo);
        float* vp = v + (i - lo);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          float4 mm = *reinterpret_cast<float4*>(mp + 4 * q), vv = *reinterpret_cast<float4*>(vp + 4 * q);
          float mf[4] = {mm.x, mm.y, mm.z, mm.w}, vf[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float gi = g[u][4 * q + k] * inv_w;
            mf[k] = h.b1 * mf[k] + (1.f - h.b1) * gi;
            vf[k] = h.b2 * vf[k] + (1.f - h.b2) * gi * gi;
            float pi = pf[4 * q + k];
            pi -= h.lr * h.wd * pi;
            pi -= (h.lr / h.bias1) * mf[k] / (sqrtf(vf[k]) * h.inv_sqrt_bias2 + h.eps);
            pf[4 * q + k] = pi;
          }
          *reinterpret_cast<float4*>(mp + 4 * q) = make_float4(mf[0], mf[1], mf[2], mf[3]);
          *reinterpret_cast<float4*>(vp + 4 * q) = make_float4(vf[0], vf[1], vf[2], vf[3]);
        }
        const uint4 out = Vec16<T>::pack(pf);
        for (int r = 0; r < world; ++r) {
          const int dst = (rank + r) % world;
          *reinterpret_cast<uint4*>(reinterpret_cast<T*>(params.p[dst]) + i) = out;
        }
      }
    }
  }
  block_done_then_signal(counter, peer_flags, world, rank, channel + 1, epoch);
}

void check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

int* device_counter() {
  // One zero-initialised array of completion counters per device, shared by the kernels of this file (each kernel kind
  // and each concurrent slot has its own entry). The zeroing must be COMPLETE before the first kernel that counts in it
  // runs on whatever stream: a plain cudaMemset is queued on the legacy default stream, which a kernel on a non-blocking
  // side stream does not wait for (it would count from uninitialised memory and never, or too early, announce
  // completion). So the first call on a device zeroes the array and waits for the device once.
  static std::atomic<int*> ctr[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  int* p = ctr[dev].load(std::memory_order_acquire);
  if (!p) {
    if (cudaMalloc(&p, 64 * sizeof(int)) != cudaSuccess) throw std::runtime_error("comm: cannot allocate the completion counters");
    cudaMemset(p, 0, 64 * sizeof(int));
    cudaDeviceSynchronize();
    int* expected = nullptr;
    if (!ctr[dev].compare_exchange_strong(expected, p, std::memory_order_acq_rel)) {
      cudaFree(p);          // another host thread initialised this device first
      p = expected;
    }
  }
  return p;
}

}  // namespace

void comm_signal(const PeerPtrs& peer_flags, int world, int rank, int channel, int epoch, cudaStream_t s) {
  signal_kernel<<<1, 32, 0, s>>>(peer_flags, world, rank, channel, epoch);
  check("comm_signal");
}

void comm_wait(const int* flags, int world, int channel, int epoch, int* status, cudaStream_t s) {
  wait_kernel<<<1, 32, 0, s>>>(flags, world, channel, epoch, status);
  check("comm_wait");
}

void muon_rs_momentum(const PeerPtrs& grads, int world, long long elem_off, int nmat, long long mat_elems, float* mom,
                      void* u_out_bf16, float* sumsq, float mu, int nesterov, const int* flags, int channel, int epoch,
                      int* status, cudaStream_t s) {
  if (mat_elems % 4 != 0 || elem_off % 4 != 0) throw std::runtime_error("muon_rs_momentum: sizes must be multiples of 4");
  if (nmat <= 0) return;
  int bx = (int)((mat_elems / 4 + 255) / 256);
  const int cap = (148 * 8 + nmat - 1) / nmat;
  if (bx > cap) bx = cap;
  if (bx < 1) bx = 1;
  // the owned slice starts at elem_off = rank * nmat * mat_elems: the rank only sets the order in which peers are read
  const int rank = (int)((elem_off / ((long long)nmat * mat_elems)) % world);
  rs_momentum_kernel<<<dim3(bx, nmat), 256, 0, s>>>(grads, world, rank, elem_off, mat_elems, mom, (bf16*)u_out_bf16, sumsq, mu,
                                                     nesterov, flags, channel, epoch, status);
  check("muon_rs_momentum");
}

void stack_scale_by_inv_norm(void* x_bf16, const float* sumsq, int nmat, long long mat_elems, float eps,
                             cudaStream_t s) {
  if (nmat <= 0) return;
  int bx = (int)((mat_elems / 2 + 255) / 256);
  const int cap = (148 * 8 + nmat - 1) / nmat;
  if (bx > cap) bx = cap;
  stack_scale_kernel<<<dim3(bx, nmat), 256, 0, s>>>((bf16*)x_bf16, sumsq, mat_elems, eps);
  check("stack_scale_by_inv_norm");
}

void ag_push(const void* src_bf16, const PeerPtrs& u_full, int world, int rank, long long dst_off, long long n,
             const PeerPtrs& peer_flags, int channel, int epoch, int slot, cudaStream_t s) {
  if (slot < 0 || slot >= 16) throw std::runtime_error("ag_push: slot must be in 0..15");
  if (n % 8 != 0 || dst_off % 8 != 0) throw std::runtime_error("ag_push: sizes must be multiples of 8");
  int blocks = (int)((n / 8 + 255) / 256);
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  // pushes that may run at the same time (different streams) count their finished blocks in different slots
  ag_push_kernel<<<blocks, 256, 0, s>>>((const bf16*)src_bf16, u_full, world, rank, dst_off, n, peer_flags, channel, epoch,
                                        slot == 0 ? device_counter() : device_counter() + 16 + slot);
  check("ag_push");
}

void ag_wait_apply(float* p, const void* u_bf16, void* p_bf16, long long n, float alpha, int world, const int* flags,
                   int channel, int epoch, int* status, cudaStream_t s) {
  if (n % 4 != 0) throw std::runtime_error("ag_wait_apply: size must be a multiple of 4");
  int blocks = (int)((n / 4 + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  ag_wait_apply_kernel<<<blocks, 256, 0, s>>>(p, (const bf16*)u_bf16, (bf16*)p_bf16, n, alpha, world, flags, channel, epoch,
                                              status);
  check("ag_wait_apply");
}

void allreduce_mean(const PeerPtrs& bufs, int world, int rank, long long n, int dtype, const int* flags,
                    const PeerPtrs& peer_flags, int channel, int epoch, int* status, cudaStream_t s) {
  const int vec = dtype == 0 ? 4 : 8;
  if (n % vec != 0) throw std::runtime_error("allreduce_mean: element count must be a multiple of the 16-byte vector");
  const long long chunks = n / vec;
  const long long lo = (chunks * rank / world) * vec, hi = (chunks * (rank + 1) / world) * vec;
  int blocks = (int)(((hi - lo) / vec + 255) / 256);
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  int* ctr = device_counter() + 1;
  if (dtype == 0)
    allreduce_kernel<0><<<blocks, 256, 0, s>>>(bufs, world, rank, lo, hi, flags, peer_flags, channel, epoch, status, ctr);
  else
    allreduce_kernel<1><<<blocks, 256, 0, s>>>(bufs, world, rank, lo, hi, flags, peer_flags, channel, epoch, status, ctr);
  check("allreduce_mean");
}

void allreduce_mean_multimem(void* mc, int world, int rank, long long n, int dtype, const int* flags, const PeerPtrs& peer_flags,
                             int channel, int epoch, int* status, cudaStream_t s) {
  const int vec = dtype == 0 ? 4 : 8;
  if (n % vec != 0) throw std::runtime_error("allreduce_mean_multimem: element count must be a multiple of the 16-byte vector");
  if (!mc) throw std::runtime_error("allreduce_mean_multimem: no multicast address (NVLS not available for this buffer)");
  const long long chunks = n / vec;
  const long long lo = (chunks * rank / world) * vec, hi = (chunks * (rank + 1) / world) * vec;
  int blocks = (int)(((hi - lo) / vec + 255) / 256);
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  int* ctr = device_counter() + 2;
  if (dtype == 0)
    allreduce_multimem_kernel<0><<<blocks, 256, 0, s>>>(mc, world, rank, lo, hi, flags, peer_flags, channel, epoch, status, ctr);
  else
    allreduce_multimem_kernel<1><<<blocks, 256, 0, s>>>(mc, world, rank, lo, hi, flags, peer_flags, channel, epoch, status, ctr);
  check("allreduce_mean_multimem");
}

void adam_shard(const PeerPtrs& grads, const PeerPtrs& params, int world, int rank, long long lo, long long hi, int dtype,
                float* m, float* v, float lr, float beta1, float beta2, float eps, float wd, float bias1, float bias2,
                const int* flags, const PeerPtrs& peer_flags, int channel, int epoch, int* status, int max_blocks,
                cudaStream_t s) {
  const int vec = dtype == 0 ? 4 : 8;
  if (lo % vec != 0 || hi % vec != 0 || hi < lo) throw std::runtime_error("adam_shard: the owned range must be aligned to 16-byte vectors");
  int blocks = (int)(((hi - lo) / vec + 511) / 512);
  const int cap = max_blocks > 0 ? max_blocks : 148 * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  AdamHyper h{lr, beta1, beta2, eps, wd, bias1, 1.f / sqrtf(bias2)};
  int* ctr = device_counter() + 3;
  if (dtype == 0)
    adam_shard_kernel<float><<<blocks, 256, 0, s>>>(grads, params, world, rank, lo, hi, m, v, h, flags, peer_flags, channel,
                                                    epoch, status, ctr);
  else
    adam_shard_kernel<bf16><<<blocks, 256, 0, s>>>(grads, params, world, rank, lo, hi, m, v, h, flags, peer_flags, channel,
                                                   epoch, status, ctr);
  check("adam_shard");
}

}  // namespace b200
