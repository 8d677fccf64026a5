// Tensor maps for TMA: the driver's encoder looked up through the runtime (no link against
// libcuda), a 2-D bfloat16 map with 128-byte swizzle, and the tiled load itself.
#pragma once
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

typedef CUresult (*VostiEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline VostiEncodeTiledFn tensor_map_encoder() {
  static VostiEncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<VostiEncodeTiledFn>(p);
  });
  return fn;
}

// Map of a row-major [rows, cols] bfloat16 matrix (cols * 2 a multiple of 16 bytes, base
// 16-byte aligned), box [box_rows, box_cols] with box_cols * 2 <= 128, 128-byte swizzle; what
// lies outside the matrix reads as zero.
inline bool encode_tensor_map_2d(CUtensorMap* map, const void* base, int64_t rows, int cols, int box_rows,
                                 int box_cols) {
  VostiEncodeTiledFn fn = tensor_map_encoder();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map of the same kind of matrix with cols a multiple of 64, seen as [cols / 64, rows, 64]: one
// box [cols / 64, box_rows, 64] brings box_rows whole rows and lays them out as cols / 64
// column blocks of [box_rows, 128 bytes] each, every block swizzled like a 2-D box.
inline bool encode_tensor_map_rows(CUtensorMap* map, const void* base, int64_t rows, int cols, int box_rows) {
  VostiEncodeTiledFn fn = tensor_map_encoder();
  if (!fn || cols % 64 != 0) return false;
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)(cols / 64)};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// General form: `rank` dimensions (innermost first), byte strides of dimensions 1.. (multiples
// of 16), box extents; bfloat16, 128-byte swizzle (the innermost box extent at most 64).
inline bool encode_tensor_map_nd(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims,
                                 const cuuint64_t* strides, const cuuint32_t* box) {
  VostiEncodeTiledFn fn = tensor_map_encoder();
  if (!fn) return false;
  const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor maps of long-lived matrices (weights, caches) are kept by address and shape.
// box_rows < 0 asks for the whole-row map of -box_rows rows.
struct TensorMapKey {
  const void* p;
  int64_t rows;
  int cols, box_rows;
  bool operator==(const TensorMapKey& o) const { return p == o.p && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct TensorMapKeyHash {
  size_t operator()(const TensorMapKey& key) const {
    return std::hash<const void*>()(key.p) ^ ((size_t)key.rows * 1000003u) ^ ((size_t)key.cols << 20) ^ (size_t)key.box_rows;
  }
};
inline bool cached_tensor_map(const void* base, int64_t rows, int cols, int box_rows, CUtensorMap* out) {
  static std::unordered_map<TensorMapKey, CUtensorMap, TensorMapKeyHash> maps;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  TensorMapKey key{base, rows, cols, box_rows};
  auto it = maps.find(key);
  if (it != maps.end()) {
    *out = it->second;
    return true;
  }
  if (maps.size() > 8192) maps.clear();
  if (box_rows < 0 ? !encode_tensor_map_rows(out, base, rows, cols, -box_rows)
                   : !encode_tensor_map_2d(out, base, rows, cols, box_rows, 64))
    return false;
  maps.emplace(key, *out);
  return true;
}

// Tiled load of one box at (c0 = column, c1 = row); c0 * 2 must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
