// Host side of the TMA descriptors: cuTensorMapEncodeTiled reached through the runtime's
// driver entry point (nothing links against the driver library), and a small cache so that a
// step does not encode the same map again.
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace tma_host {

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  });
  return fn;
}

struct Key {
  const void* ptr;
  long long rows, cols;
  int box_rows, box_cols;
  bool operator==(const Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols;
  }
};
struct Hash {
  size_t operator()(const Key& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^
           (std::hash<long long>()(k.cols) * 131) ^ ((size_t)k.box_rows << 8) ^ (size_t)k.box_cols;
  }
};

// A [rows, cols] row-major bfloat16 matrix as a tiled map with boxes of box_rows x box_cols
// (box_cols * 2 bytes = 128: one swizzle span) and 128-byte swizzle.  0 on success.
inline int bf16_map(const void* ptr, long long rows, long long cols, int box_rows, int box_cols, CUtensorMap* out) {
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{ptr, rows, cols, box_rows, box_cols};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiled enc = encoder();
  if (!enc) return MF_ERR_BAD_ARG;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 20000 + (int)r;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// The same matrix seen as [cols/64 chunks][rows][64 elements]: a box of box_chunks x box_rows
// spans of 128 bytes brings box_rows rows of 64 * box_chunks consecutive columns with ONE
// copy, laid out in shared memory chunk by chunk ([chunk][row][128 bytes], 128-byte swizzle).
// cols must be a multiple of 64.  0 on success.
inline int bf16_map_chunked(const void* ptr, long long rows, long long cols, int box_rows, int box_chunks,
                            CUtensorMap* out) {
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  if (cols % 64) return MF_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(mu);
  const Key key{ptr, rows, cols, box_rows, box_chunks};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  EncodeTiled enc = encoder();
  if (!enc) return MF_ERR_BAD_ARG;
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_chunks};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 20000 + (int)r;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace tma_host
