// Host-side TMA descriptor helpers.  The driver entry point is resolved at run time through the
// CUDA runtime, so the library carries no link-time dependency on libcuda and loads on a machine
// without a GPU (where only the CPU paths are used).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

namespace cafd {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Row-major 2D tensor [rows, cols] of `elem_bytes` elements (row pitch `pitch_bytes`), box
// [box_rows, box_cols], 128-byte swizzle (box_cols * elem_bytes must be 128) or none.
// Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                        uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_bytes;
  return r == CUDA_SUCCESS ? 0 : -3 - static_cast<int>(r);
}

// General N-D (up to 4) tiled map; dims/box innermost first, strides in bytes for dims 1..n-1.
inline int make_tmap_nd(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5];
  cuuint32_t e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i > 0) s[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, dt, rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3 - static_cast<int>(r);
}

// Small cache keyed by the arguments: descriptors for long-lived buffers (weights, KV pages,
// preallocated activation slabs) are encoded once.
struct TmapKey {
  const void* base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, box_cols;
  int dt;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows &&
           box_cols == o.box_cols && dt == o.dt;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.rows); mix(k.cols); mix(k.pitch); mix(k.box_rows); mix(k.box_cols); mix(static_cast<uint64_t>(k.dt));
    return h;
  }
};

inline int cached_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                          uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{base, rows, cols, pitch_bytes, box_rows, box_cols, static_cast<int>(dt)};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap m;
    int rc = make_tmap_2d(&m, base, dt, elem_bytes, rows, cols, pitch_bytes, box_rows, box_cols, true);
    if (rc) return rc;
    if (cache.size() > 65536) cache.clear();
    it = cache.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

}  // namespace cafd
