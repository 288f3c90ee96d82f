// Host side of the tensor copies (TMA): the driver's encoder, found through the runtime (no link
// against libcuda), and a cache of encoded maps per (base address, geometry): a model asks for
// the same few maps again every step. bfloat16 tensors, 128-byte swizzle.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <functional>
#include <mutex>
#include <unordered_map>

namespace r2 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// A bfloat16 tensor of `rank` dimensions (innermost first; strides in bytes for all but the
// innermost), copied in boxes of `box` elements.
inline bool encode_bf16_map(CUtensorMap* out, const void* base, cuuint32_t rank, const cuuint64_t* dims, const cuuint64_t* strides,
                            const cuuint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapKey {
  const void* base;
  long long a, b;
  int c, d, e, f;
  bool operator==(const MapKey& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d && e == o.e && f == o.f; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    h = h * 1315423911u + std::hash<long long>()(k.a);
    h = h * 1315423911u + std::hash<long long>()(k.b);
    return h * 1315423911u + size_t(k.c) * 131u + size_t(k.d) * 31u + size_t(k.e) * 7u + size_t(k.f);
  }
};

// The map for `key`, encoded at its first use. The key must say everything that dims, strides
// and box depend on.
inline bool cached_bf16_map(CUtensorMap* out, const MapKey& key, cuuint32_t rank, const cuuint64_t* dims, const cuuint64_t* strides,
                            const cuuint32_t* box) {
  static std::mutex lock;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  std::lock_guard<std::mutex> guard(lock);
  auto it = maps.find(key);
  if (it != maps.end()) {
    *out = it->second;
    return true;
  }
  CUtensorMap map;
  if (!encode_bf16_map(&map, key.base, rank, dims, strides, box)) return false;
  if (maps.size() > 4096) maps.clear();  // pools and activations that came and went
  maps.emplace(key, map);
  *out = map;
  return true;
}

// One layer's keys (or values) in the page pool as [page][kv head][offset][dim] (head size
// `head_dim`, page stride in elements), boxes of `box_rows` offsets of one head of one page.
inline bool page_map(CUtensorMap* out, const void* base, long long page_stride, int page_size, int n_kv_heads, int n_pages, int box_rows,
                     int head_dim) {
  cuuint64_t dims[4] = {cuuint64_t(head_dim), cuuint64_t(page_size), cuuint64_t(n_kv_heads), cuuint64_t(n_pages)};
  cuuint64_t strides[3] = {cuuint64_t(head_dim) * 2, cuuint64_t(page_size) * head_dim * 2, cuuint64_t(page_stride) * 2};
  cuuint32_t box[4] = {cuuint32_t(head_dim), cuuint32_t(box_rows), 1, 1};
  return cached_bf16_map(out, MapKey{base, page_stride, head_dim, page_size, n_kv_heads, n_pages, box_rows}, 4, dims, strides, box);
}

}  // namespace r2
