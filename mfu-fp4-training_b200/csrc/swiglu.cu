// SwiGLU producers between the FFN GEMMs (sm_100a).
//   forward : h = bf16(silu(h1) * h3), tensor amax of h, then the NVFP4 row+column quantiser on h
//             (tk_silu_quantize_split_for_gemm, fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:8985-9123;
//              element kernel silu_split_bf16.cuh:62-140)
//   backward: dh1 = bf16(dh*h3*silu'(h1)), dh3 = bf16(dh*silu(h1)), their amaxes, then each quantised
//             (tk_silu_deriv_quantize_split_for_gemm, tk_quantize.cu:10063-10255; silu_split_bf16.cuh:181-300)
// silu(x) = x / (1 + __expf(-x)); sigma = 1 / (1 + __expf(-x)); silu' = sigma * (1 + x - x*sigma); products are
// evaluated left to right in fp32 and rounded to bf16 once, as in the reference kernels.
#include "fp4_common.cuh"
#include "host_util.h"
#include "swiglu_math.cuh"

namespace fp4b200 {

__device__ __forceinline__ void block_amax_commit(float v, float* amax) {
  v = warp_max(v);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < 8 ? part[threadIdx.x] : 0.0f;
    v = warp_max(v);
    if (threadIdx.x == 0 && v > 0.0f) atomic_max_nonneg(amax, v);
  }
}

__global__ void __launch_bounds__(256) silu_mul_kernel(const uint4* __restrict__ h1, const uint4* __restrict__ h3,
                                                       uint4* __restrict__ out, size_t n_vec,
                                                       float* __restrict__ amax) {
  constexpr int kU = 4;   // vectors per stream and thread in flight (see silu_deriv_kernel)
  uint32_t mx = 0;
  const size_t tile = (size_t)blockDim.x * kU;
  for (size_t base = (size_t)blockIdx.x * tile; base < n_vec; base += (size_t)gridDim.x * tile) {
    uint4 a[kU], b[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const size_t i = base + (size_t)u * blockDim.x + threadIdx.x;
      if (i < n_vec) { a[u] = __ldg(h1 + i); b[u] = __ldg(h3 + i); }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const size_t i = base + (size_t)u * blockDim.x + threadIdx.x;
      if (i >= n_vec) continue;
      const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
      uint32_t o[4];
      silu_mul_bf16x8(aw, bw, o);
#pragma unroll
      for (int q = 0; q < 4; ++q) mx = bf16x2_absmax(mx, o[q]);
      out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  block_amax_commit(bf16x2_hmax_to_f32(mx), amax);
}

// Four vectors per stream and thread in flight (a block works on tiles of 1024 vectors = 16 KB per stream): five
// streams at once leave each one short runs between DRAM page switches otherwise (0.45 -> 0.38 ms at 16384 x 14336).
__global__ void __launch_bounds__(256)
silu_deriv_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ h3, const uint4* __restrict__ h1,
                  uint4* __restrict__ dh1, uint4* __restrict__ dh3, size_t n_vec, float* __restrict__ amax1,
                  float* __restrict__ amax3) {
  constexpr int kU = 4;
  uint32_t mx1 = 0, mx3 = 0;
  const size_t tile = (size_t)blockDim.x * kU;
  for (size_t base = (size_t)blockIdx.x * tile; base < n_vec; base += (size_t)gridDim.x * tile) {
    uint4 d[kU], a[kU], b[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const size_t i = base + (size_t)u * blockDim.x + threadIdx.x;
      if (i < n_vec) { d[u] = __ldg(dh + i); a[u] = __ldg(h3 + i); b[u] = __ldg(h1 + i); }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const size_t i = base + (size_t)u * blockDim.x + threadIdx.x;
      if (i >= n_vec) continue;
      const uint32_t dw[4] = {d[u].x, d[u].y, d[u].z, d[u].w}, aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w},
                     bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
      uint32_t o1[4], o3[4];
      silu_deriv_bf16x8(dw, aw, bw, o1, o3);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        mx1 = bf16x2_absmax(mx1, o1[q]);
        mx3 = bf16x2_absmax(mx3, o3[q]);
      }
      dh1[i] = make_uint4(o1[0], o1[1], o1[2], o1[3]);
      dh3[i] = make_uint4(o3[0], o3[1], o3[2], o3[3]);
    }
  }
  block_amax_commit(bf16x2_hmax_to_f32(mx1), amax1);
  __syncthreads();
  block_amax_commit(bf16x2_hmax_to_f32(mx3), amax3);
}

// Every bf16 pattern x with |x| < 64: the short division sequence against the general division, for x / d and 1 / d
// with d = 1 + __expf(-x).  out[0], out[1]: patterns that differ (must both be 0).
__global__ void __launch_bounds__(256) silu_division_selftest_kernel(unsigned int* __restrict__ out) {
  const uint32_t pattern = blockIdx.x * blockDim.x + threadIdx.x;
  const float x = __uint_as_float(pattern << 16);
  if (!(fabsf(x) < 64.0f)) return;
  const float d = 1.0f + __expf(-x);
  const float r1 = rcp_refined(d);
  if (__float_as_uint(quotient_given_rcp(x, d, r1)) != __float_as_uint(x / d)) atomicAdd(out, 1u);
  if (__float_as_uint(sigmoid_given_rcp(d, r1)) != __float_as_uint(1.0f / d)) atomicAdd(out + 1, 1u);
}

__global__ void finalize_sg2_kernel(float* a, float* b) {
  a[1] = a[0] / 2688.0f;
  if (b) b[1] = b[0] / 2688.0f;
}

}  // namespace fp4b200

using namespace fp4b200;

static int check_mh(const void* p, int64_t M, int64_t H, const char* who) {
  if (!p) return set_error("%s: null input", who);
  if (M <= 0 || H <= 0 || (M % 128) || (H % 128))
    return set_error("%s: M and H must be positive multiples of 128 (got %lld x %lld)", who, (long long)M, (long long)H);
  if (reinterpret_cast<uintptr_t>(p) & 15) return set_error("%s: inputs must be 16-byte aligned", who);
  return 0;
}

extern "C" {

int fp4b200_selftest_silu_division(uint32_t* mismatches_dev, void* stream) {
  if (!mismatches_dev || (reinterpret_cast<uintptr_t>(mismatches_dev) & 3))
    return set_error("selftest_silu_division: two 32-bit words of device memory are required");
  cudaStream_t st = (cudaStream_t)stream;
  FP4_CUDA_CHECK(cudaMemsetAsync(mismatches_dev, 0, 2 * sizeof(uint32_t), st));
  silu_division_selftest_kernel<<<256, 256, 0, st>>>(mismatches_dev);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_silu_mul_bf16(const void* h1, const void* h3, int64_t n_elems, void* h_out, float* amax_sg,
                          void* stream) {
  if (!h1 || !h3 || !h_out || !amax_sg) return set_error("silu_mul_bf16: null pointer");
  if (n_elems < 0 || (n_elems % 8)) return set_error("silu_mul_bf16: element count must be a multiple of 8");
  cudaStream_t st = (cudaStream_t)stream;
  FP4_CUDA_CHECK(cudaMemsetAsync(amax_sg, 0, 2 * sizeof(float), st));
  const size_t n_vec = (size_t)n_elems / 8;
  if (n_vec) {
    const int grid = (int)std::min<size_t>((n_vec + 1023) / 1024, (size_t)device_sm_count() * 8);
    silu_mul_kernel<<<grid, 256, 0, st>>>((const uint4*)h1, (const uint4*)h3, (uint4*)h_out, n_vec, amax_sg);
    FP4_CUDA_CHECK(cudaGetLastError());
  }
  finalize_sg2_kernel<<<1, 1, 0, st>>>(amax_sg, nullptr);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_nvfp4_silu_quantize(const void* h1, const void* h3, int64_t M, int64_t H, void* h_bf16,
                                int encode_centric, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                float* amax_sg, void* stream) {
  if (int rc = check_mh(h1, M, H, "nvfp4_silu_quantize")) return rc;
  if (int rc = check_mh(h3, M, H, "nvfp4_silu_quantize")) return rc;
  if (!h_bf16 || !row_fp4 || !row_sc || !amax_sg) return set_error("nvfp4_silu_quantize: null output");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("nvfp4_silu_quantize: col_fp4 and col_sc must both be given or both be null");
  if (int rc = fp4b200_silu_mul_bf16(h1, h3, M * H, h_bf16, amax_sg, stream)) return rc;
  return launch_quantize(h_bf16, M, H, amax_sg, amax_sg, encode_centric != 0, nullptr, nullptr, row_fp4, row_sc,
                         col_fp4, col_sc, nullptr, true, (cudaStream_t)stream);
}

int fp4b200_silu_deriv_bf16(const void* dh, const void* h3, const void* h1, int64_t n_elems, void* dh1_out,
                            void* dh3_out, float* amax_sg1, float* amax_sg3, void* stream) {
  if (!dh || !h3 || !h1 || !dh1_out || !dh3_out || !amax_sg1 || !amax_sg3)
    return set_error("silu_deriv_bf16: null pointer");
  if (n_elems < 0 || (n_elems % 8)) return set_error("silu_deriv_bf16: element count must be a multiple of 8");
  cudaStream_t st = (cudaStream_t)stream;
  FP4_CUDA_CHECK(cudaMemsetAsync(amax_sg1, 0, 2 * sizeof(float), st));
  FP4_CUDA_CHECK(cudaMemsetAsync(amax_sg3, 0, 2 * sizeof(float), st));
  const size_t n_vec = (size_t)n_elems / 8;
  if (n_vec) {
    const int grid = (int)std::min<size_t>((n_vec + 1023) / 1024, (size_t)device_sm_count() * 8);
    silu_deriv_kernel<<<grid, 256, 0, st>>>((const uint4*)dh, (const uint4*)h3, (const uint4*)h1, (uint4*)dh1_out,
                                            (uint4*)dh3_out, n_vec, amax_sg1, amax_sg3);
    FP4_CUDA_CHECK(cudaGetLastError());
  }
  finalize_sg2_kernel<<<1, 1, 0, st>>>(amax_sg1, amax_sg3);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
