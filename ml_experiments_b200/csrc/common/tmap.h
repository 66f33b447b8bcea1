// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled), resolved at run time
// through cudaGetDriverEntryPoint so the extension has no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace b200 {

enum class TmapDtype { BF16, F32, U8, F16 };

inline size_t tmap_elt_size(TmapDtype t) {
  switch (t) {
    case TmapDtype::BF16: return 2;
    case TmapDtype::F16: return 2;
    case TmapDtype::F32: return 4;
    case TmapDtype::U8: return 1;
  }
  return 0;
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || p == nullptr) throw std::runtime_error("cuTensorMapEncodeTiled entry point not found");
    fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// A training step issues the same few hundred (pointer, shape, box) combinations every iteration (the caching
// allocator hands the same activation buffers back), so encoded maps are kept per host thread and looked up by value.
struct TmapKey {
  uint64_t v[10];
  bool operator==(const TmapKey& o) const { return std::memcmp(v, o.v, sizeof v) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) { h ^= x; h *= 1099511628211ull; h ^= h >> 29; }
    return (size_t)h;
  }
};

inline CUtensorMap encode_tmap_3d(const void* base, TmapDtype dt, uint64_t d0, uint64_t d1, uint64_t d2,
                                  uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                                  bool swizzle128);

// rank-3 row-major tensor map: dims (fastest first) {d0, d1, d2}, strides in BYTES for d1, d2,
// box {b0, b1, 1}. swizzle128 selects CU_TENSOR_MAP_SWIZZLE_128B (b0 * elt must be 128 bytes then).
inline CUtensorMap make_tmap_3d(const void* base, TmapDtype dt, uint64_t d0, uint64_t d1, uint64_t d2,
                                uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                                bool swizzle128) {
  thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const TmapKey key{{(uint64_t)reinterpret_cast<uintptr_t>(base), (uint64_t)dt, d0, d1, d2, stride1_bytes, stride2_bytes, b0, b1,
                     (uint64_t)swizzle128}};
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 8192) cache.clear();
  const CUtensorMap m = encode_tmap_3d(base, dt, d0, d1, d2, stride1_bytes, stride2_bytes, b0, b1, swizzle128);
  cache.emplace(key, m);
  return m;
}

inline CUtensorMap encode_tmap_3d(const void* base, TmapDtype dt, uint64_t d0, uint64_t d1, uint64_t d2,
                                  uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                                  bool swizzle128) {
  CUtensorMap m;
  CUtensorMapDataType cdt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  switch (dt) {
    case TmapDtype::BF16: cdt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case TmapDtype::F16: cdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case TmapDtype::F32: cdt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    case TmapDtype::U8: cdt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
  }
  cuuint64_t dims[3] = {d0, d1, d2 ? d2 : 1};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes ? stride2_bytes : stride1_bytes * d1};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base address must be 16-byte aligned");
  if ((strides[0] & 15) != 0 || (strides[1] & 15) != 0)
    throw std::runtime_error("TMA strides must be multiples of 16 bytes (row length * element size)");
  CUresult r = get_encode_fn()(&m, cdt, 3, const_cast<void*>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE,
                               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof buf,
             "cuTensorMapEncodeTiled failed (%d): dims=(%llu,%llu,%llu) strides=(%llu,%llu) box=(%u,%u)", (int)r,
             (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
             (unsigned long long)strides[0], (unsigned long long)strides[1], b0, b1);
    throw std::runtime_error(buf);
  }
  return m;
}

}  // namespace b200
