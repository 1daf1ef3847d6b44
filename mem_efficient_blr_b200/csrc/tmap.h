// Host-side helpers: CUDA error plumbing, the driver entry point for TMA descriptors, and a
// 3-D tiled tensor-map encoder.  No dependency on libcuda at link time: the encoder is looked up
// through the runtime (cudaGetDriverEntryPoint).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/blr_b200.h"  // BLR_OK / BLR_ERR_* codes returned by every entry point

namespace blr {

void set_last_error(const char* fmt, ...);

#define BLR_CUDA_OK(expr)                                                                  \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      ::blr::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return BLR_ERR_CUDA;                                                          \
    }                                                                                      \
  } while (0)

#define BLR_REQUIRE(cond, code, ...)          \
  do {                                        \
    if (!(cond)) {                            \
      ::blr::set_last_error(__VA_ARGS__);     \
      return (code);                          \
    }                                         \
  } while (0)

enum class Swz { B32, B64, B128, None };

// Encodes a rank-3 tiled tensor map.  dims are in elements (innermost first); strides[0..1] are the
// byte strides of dims 1 and 2 (multiples of 16); box is in elements.  Out-of-range elements read 0.
int encode_tmap_3d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, const uint64_t dims[3],
                   const uint64_t strides[2], const uint32_t box[3], Swz swz);

struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
  int coop;
};
int device_info(DeviceInfo* out);  // for the current device, cached per device

}  // namespace blr
