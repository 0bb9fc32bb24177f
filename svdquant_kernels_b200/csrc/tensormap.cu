// Host-side TMA descriptor construction.  The driver entry point is looked up
// through the runtime so the library links against libcudart only.
#include <mutex>

#include "svdq_internal.h"

namespace svdq {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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

// Encoded descriptors are kept in a small direct-mapped table keyed by everything that goes into one
// (a descriptor holds an address and extents, never data, so an entry cannot go stale): a serving
// loop that calls with the same buffers again encodes nothing.  Guarded by a mutex; a collision
// just re-encodes.
namespace {
struct TmapKey {
  const void* base;
  uint64_t rows, cols, stride;
  uint32_t box_rows, box_cols;
  int elem_bytes, swz;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows &&
           box_cols == o.box_cols && elem_bytes == o.elem_bytes && swz == o.swz;
  }
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kTmapCacheSlots = 512;
TmapEntry g_tmap_cache[kTmapCacheSlots];
std::mutex g_tmap_mutex;

inline uint32_t tmap_slot(const TmapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
  h ^= (k.rows * 0xC2B2AE3D27D4EB4Full) ^ (k.cols << 17) ^ (k.stride << 3) ^ (static_cast<uint64_t>(k.box_rows) << 40) ^
       (static_cast<uint64_t>(k.box_cols) << 52) ^ static_cast<uint64_t>(k.elem_bytes * 4 + k.swz);
  h ^= h >> 29;
  return static_cast<uint32_t>(h % kTmapCacheSlots);
}
}  // namespace

static int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                          uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, TmapSwizzle swz);

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, TmapSwizzle swz) {
  const TmapKey key{base, rows, cols, row_stride_bytes, box_rows, box_cols, elem_bytes, static_cast<int>(swz)};
  const uint32_t slot = tmap_slot(key);
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    const TmapEntry& e = g_tmap_cache[slot];
    if (e.valid && e.key == key) { *out = e.map; return SVDQ_OK; }
  }
  const int rc = encode_tmap_2d(out, base, elem_bytes, rows, cols, row_stride_bytes, box_rows, box_cols, swz);
  if (rc != SVDQ_OK) return rc;
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  TmapEntry& e = g_tmap_cache[slot];
  e.key = key; e.map = *out; e.valid = true;
  return SVDQ_OK;
}

static int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                          uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, TmapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return SVDQ_ERR_LAUNCH;
  CUtensorMapDataType dt;
  switch (elem_bytes) {
    case 1: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case 2: dt = CU_TENSOR_MAP_DATA_TYPE_UINT16; break;
    case 4: dt = CU_TENSOR_MAP_DATA_TYPE_UINT32; break;
    default: return SVDQ_ERR_DTYPE;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swz == kTmapSwizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SVDQ_OK : SVDQ_ERR_LAUNCH;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace svdq
