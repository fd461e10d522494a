// Host side of TMA: building (and caching) 2-D tensor maps for bf16 row-major matrices whose
// tiles are fetched as boxes of `box_rows` rows x 64 elements with the 128-byte swizzle.
// The driver's cuTensorMapEncodeTiled is looked up at run time, so nothing links libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

namespace tma_host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

struct Key {
  const void* ptr; long long rows, cols, ld; int box_rows;
  bool operator==(const Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    return h * 1000003u ^ (size_t)k.box_rows;
  }
};

// bf16 [rows, cols], row stride ld elements (ld % 8 == 0, ptr 16-byte aligned); boxes of
// box_rows x 64 elements; out-of-range parts of a box read as zero.
inline bool tensor_map_2d(const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                          CUtensorMap* out) {
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  static std::mutex mu;
  Key key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

// The same matrix (cols a multiple of 64) seen as [cols / 64] k-blocks of [rows, 64]: boxes of
// `box_kblocks` k-blocks x box_rows rows x 64 elements, laid out in shared memory k-block after
// k-block, each a 128-byte-swizzled tile of box_rows rows.  One copy brings several k-blocks.
inline bool tensor_map_kblocks(const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                               int box_kblocks, CUtensorMap* out) {
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  static std::mutex mu;
  if (cols % 64) return false;
  Key key{ptr, rows, cols, ld, box_rows * 1024 + box_kblocks};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_kblocks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

}  // namespace tma_host
