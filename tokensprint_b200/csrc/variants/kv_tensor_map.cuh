// Tensor maps (TMA descriptors) of the paged key/value pools, shared by the attention kernels
// that fetch pages with the copy engine.  Encoding a map costs a driver call, so maps are kept
// by (pointer, shape); the cache is per library (every variant is a library of its own).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <functional>
#include <mutex>
#include <unordered_map>

typedef CUresult (*TsEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline TsEncodeTiledFn ts_encode_tiled() {
  static TsEncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TsEncodeTiledFn)ptr;
  }
  return fn;
}

struct TsMapKey {
  const void* ptr;
  long long a, b, c;
  bool operator==(const TsMapKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c; }
};
struct TsMapKeyHash {
  size_t operator()(const TsMapKey& k) const {
    return std::hash<const void*>()(k.ptr) * 1000003u ^ std::hash<long long>()(k.a * 131 + k.b * 31 + k.c);
  }
};
static inline std::mutex& ts_map_mutex() {
  static std::mutex m;
  return m;
}
static inline std::unordered_map<TsMapKey, CUtensorMap, TsMapKeyHash>& ts_map_cache() {
  static std::unordered_map<TsMapKey, CUtensorMap, TsMapKeyHash> cache;
  return cache;
}

// K or V pool [slots, nkv, head_dim] (bfloat16) as a 3-d tensor {head_dim, nkv, slots}; boxes of
// {64, 1, box_rows} with the 128-byte swizzle: `box_rows` consecutive slots of one head, half a
// 128-wide head (64 elements = 128 bytes) per box.  0, or TS_ERR_* (common.cuh).
static inline int ts_kv_cache_map(const void* ptr, long long slots, int nkv, int head_dim, int box_rows, CUtensorMap* out) {
  TsMapKey key{ptr, slots, (long long)nkv * 1024 + head_dim, box_rows};
  std::lock_guard<std::mutex> lock(ts_map_mutex());
  auto& cache = ts_map_cache();
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  TsEncodeTiledFn fn = ts_encode_tiled();
  if (!fn) return -2;
  cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)nkv, (cuuint64_t)slots};
  cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)nkv * head_dim * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -1;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}
