// Host-side helpers shared by the translation units of libfp4b200: error reporting for the
// C ABI, CUDA error checking, device properties, tensor-map encoding, the device status word.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

namespace fp4b200 {

// Records a printf-style message retrievable through fp4b200_last_error(); returns -1.
int set_error(const char* fmt, ...);

#define FP4_CUDA_CHECK(expr)                                                                    \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess)                                                                      \
      return ::fp4b200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

int device_sm_count();

// Device address of the per-device status word array (4 ints); nullptr + error on failure.
int* device_status_ptr();

// Encodes a 2-D tiled tensor map: inner extent dim0 (elements), outer extent dim1, row pitch
// in bytes, box (box0 x box1) elements.  Returns 0 or -1 (message set).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                 uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle);

// 3-D variant (dim2 outermost with its own byte stride).
int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                 uint64_t dim1, uint64_t dim2, uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t box0,
                 uint32_t box1, uint32_t box2, CUtensorMapSwizzle swizzle);

}  // namespace fp4b200
