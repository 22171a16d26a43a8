// Host-side plumbing of libfp4b200 (no kernels besides the status word).
#include "host_util.h"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

namespace fp4b200 {

static thread_local char g_err[512] = "";

int set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return -1;
}

int device_sm_count() {
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

__device__ int g_device_status[4];

int* device_status_ptr() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("device_status_ptr: cudaGetDevice failed");
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_device_status);
    if (e != cudaSuccess) {
      set_error("cudaGetSymbolAddress(g_device_status) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

float* stream_scratch(cudaStream_t st) {
  static std::mutex mu;
  static std::map<std::pair<int, uintptr_t>, float*> table;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_error("stream_scratch: cudaGetDevice failed");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_pair(dev, reinterpret_cast<uintptr_t>(st));
  auto it = table.find(key);
  if (it != table.end()) return it->second;
  void* p = nullptr;
  const cudaError_t e = cudaMalloc(&p, kScratchFloats * sizeof(float));
  if (e != cudaSuccess || p == nullptr) {
    (void)cudaGetLastError();
    set_error("stream_scratch: cudaMalloc of %zu bytes failed: %s (the first call on a stream must not be inside a "
              "stream capture)", kScratchFloats * sizeof(float), cudaGetErrorString(e));
    return nullptr;
  }
  table.emplace(key, static_cast<float*>(p));
  return static_cast<float*>(p);
}

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

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                 uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle) {
  (void)elem_bytes;
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error("cuTensorMapEncodeTiled(2d) failed with CUresult %d (dims %llu x %llu, pitch %llu, box %u x %u)",
                     (int)r, (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)pitch_bytes,
                     box0, box1);
  return 0;
}

}  // namespace fp4b200

using namespace fp4b200;

extern "C" {

const char* fp4b200_last_error(void) { return g_err; }

int fp4b200_abi_version(void) { return 1; }

// Synchronises the device, reads and clears the status word; returns it (0 = no kernel gave up
// a bounded wait), or -1 on a CUDA error.
int fp4b200_device_status(void) {
  int* p = device_status_ptr();
  if (p == nullptr) return -1;
  int v = 0;
  FP4_CUDA_CHECK(cudaDeviceSynchronize());
  FP4_CUDA_CHECK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    int zero = 0;
    FP4_CUDA_CHECK(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  return v;
}

}  // extern "C"
