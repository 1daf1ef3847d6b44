#include "tmap.h"

#include <mutex>
#include <unordered_map>
#include <stdarg.h>
#include <string.h>

namespace blr {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_last_error; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// Encoding a descriptor costs about a microsecond of host time and a call needs up to 18 of them, while
// the same weights come back call after call: keep the encoded descriptors, keyed by everything
// that went into them.
struct TmapKey {
  uint64_t v[10];
  bool operator==(const TmapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 10; ++i) {
      h ^= k.v[i];
      h *= 1099511628211ull;
    }
    return (size_t)h;
  }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
static std::mutex g_tmap_mu;

int encode_tmap_3d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, const uint64_t dims[3],
                   const uint64_t strides[2], const uint32_t box[3], Swz swz) {
  int dev = 0;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  TmapKey key = {{(uint64_t)reinterpret_cast<uintptr_t>(base), dims[0], dims[1], dims[2], strides[0], strides[1],
                  ((uint64_t)box[0] << 32) | box[1], ((uint64_t)box[2] << 32) | (uint64_t)dt, (uint64_t)swz,
                  (uint64_t)dev}};
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *map = it->second;
      return BLR_OK;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  BLR_REQUIRE(fn != nullptr, BLR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  BLR_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, BLR_ERR_ALIGN, "tensor base %p is not 16-byte aligned", base);
  BLR_REQUIRE((strides[0] & 15) == 0 && (strides[1] & 15) == 0, BLR_ERR_ALIGN,
              "tensor strides (%llu, %llu bytes) must be multiples of 16", (unsigned long long)strides[0],
              (unsigned long long)strides[1]);
  cuuint64_t gdims[3] = {dims[0], dims[1], dims[2]};
  cuuint64_t gstr[2] = {strides[0], strides[1]};
  cuuint32_t bx[3] = {box[0], box[1], box[2]};
  cuuint32_t es[3] = {1, 1, 1};
  CUtensorMapSwizzle s = swz == Swz::B128 ? CU_TENSOR_MAP_SWIZZLE_128B
                         : swz == Swz::B64 ? CU_TENSOR_MAP_SWIZZLE_64B
                         : swz == Swz::B32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                           : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), gdims, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, s,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BLR_REQUIRE(r == CUDA_SUCCESS, BLR_ERR_CUDA,
              "cuTensorMapEncodeTiled failed (%d): dims=(%llu,%llu,%llu) strides=(%llu,%llu) box=(%u,%u,%u)", (int)r,
              (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
              (unsigned long long)strides[0], (unsigned long long)strides[1], box[0], box[1], box[2]);
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    if (g_tmap_cache.size() > 16384) g_tmap_cache.clear();
    g_tmap_cache.emplace(key, *map);
  }
  return BLR_OK;
}

int device_info(DeviceInfo* out) {
  static DeviceInfo cache[64];
  static bool have[64] = {};
  static std::mutex mu;
  int dev = 0;
  BLR_CUDA_OK(cudaGetDevice(&dev));
  BLR_REQUIRE(dev >= 0 && dev < 64, BLR_ERR_ARG, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (!have[dev]) {
    DeviceInfo d;
    BLR_CUDA_OK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    BLR_CUDA_OK(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    BLR_CUDA_OK(cudaDeviceGetAttribute(&d.coop, cudaDevAttrCooperativeLaunch, dev));
    cache[dev] = d;
    have[dev] = true;
  }
  *out = cache[dev];
  return BLR_OK;
}

}  // namespace blr
