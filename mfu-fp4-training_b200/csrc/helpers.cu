// Small entry points around the hot path: the reference GEMM module's test helpers (element-wise
// fp32 <-> packed E2M1, its stand-alone tile quantiser) and the reduction of GEMM-epilogue row
// partials into 1/rms.  None of them is performance critical; they exist so that callers and tests
// written against the reference's modules find the same functions.
//   fp32_to_fp4x2 / fp4x2_to_fp32   ThunderKittens/kernels/gemm/nvfp4_b200/nvfp4_quantize.cuh:293-308
//   nvfp4_quantize                  ThunderKittens/kernels/gemm/nvfp4_b200/nvfp4_quantize.cuh:57-255,
//                                   nvfp4_b200_gemm.cu:1443-1478
//   row_rms_reduce                  ThunderKittens/kernels/gemm/common/c1_rms_reduce.cuh:11-86
#include "fp4_common.cuh"
#include "host_util.h"

namespace fp4b200 {

// Two fp32 -> one byte: element 2i in the low nibble, RN-even, saturating to +-6.
__global__ void __launch_bounds__(256) fp32_to_fp4x2_kernel(const float2* __restrict__ in, size_t n_pairs,
                                                            uint8_t* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += (size_t)gridDim.x * blockDim.x) {
    const float2 v = in[i];
    out[i] = (uint8_t)f32x2_to_e2m1x2(v.x, v.y);
  }
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  // magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6 as halves: 0, 1, 2, 3, 4, 6, 8, 12
  const uint32_t halves = (0xC8643210u >> ((code & 7u) * 4)) & 15u;
  const float m = 0.5f * (float)halves;
  return (code & 8u) ? -m : m;
}

__global__ void __launch_bounds__(256) fp4x2_to_fp32_kernel(const uint8_t* __restrict__ in, size_t n_bytes,
                                                            float2* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t b = in[i];
    out[i] = make_float2(e2m1_to_f32(b & 15u), e2m1_to_f32(b >> 4));
  }
}

// One warp per row: lane l adds partial columns l, l+32, ... in order, then the shuffle-down tree
// 16, 8, 4, 2, 1; inv_rms = rsqrtf(sum / hidden + eps).  Same order of additions as the reference.
__global__ void __launch_bounds__(128) row_rms_reduce_kernel(const float* __restrict__ partial, float* __restrict__ inv_rms,
                                                             int64_t rows, int64_t partial_cols, int64_t hidden, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const float* p = partial + row * partial_cols;
  float sum = 0.0f;
  for (int64_t c = lane; c < partial_cols; c += 32) sum += p[c];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, off);
  if (lane == 0) inv_rms[row] = rsqrtf(sum / static_cast<float>(hidden) + eps);
}

// Stand-alone quantiser of the reference's GEMM module (its tests' operand producer): decode-scale
// convention sg = amax / (6 * 448); block scale e4m3((b / 6) * (1 / max(sg, 1e-12))); codes
// e2m1(x * (1 / max(float(scale) * sg, 1e-12))); optional 16x16 tiles sharing one scale.  One thread
// per 16-element block (with scale_2d it scans its tile's 16 rows): a test helper, not a hot kernel.
__global__ void __launch_bounds__(256) tk_amax_kernel(const uint4* __restrict__ x, size_t n_vec, float* __restrict__ sg) {
  uint32_t m = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = __ldg(x + i);
    m = bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(m, v.x), v.y), v.z), v.w);
  }
  float v = warp_max(bf16x2_hmax_to_f32(m));
  if ((threadIdx.x & 31) == 0 && v > 0.0f) atomic_max_nonneg(sg, v);
}

__global__ void tk_divide_kernel(float* __restrict__ sg) { sg[0] /= 6.0f * 448.0f; }

__global__ void __launch_bounds__(256) tk_quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int64_t N,
                                                          uint8_t* __restrict__ codes, uint8_t* __restrict__ sc,
                                                          const float* __restrict__ sg, int scale_2d) {
  const int64_t blocks_per_row = N / 16;
  const int64_t n_blocks = M * blocks_per_row;
  const float s_global_dec = *sg;
  const float s_global_enc = 1.0f / fmaxf(s_global_dec, 0.000000000001f);
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = b / blocks_per_row, kb = b - r * blocks_per_row;
    const uint4* src = reinterpret_cast<const uint4*>(x + r * N + kb * 16);
    const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t mx = 0;
    if (scale_2d) {
      const int64_t r0 = r & ~int64_t(15);
      for (int rr = 0; rr < 16; ++rr) {
        const uint4* s2 = reinterpret_cast<const uint4*>(x + (r0 + rr) * N + kb * 16);
        const uint4 a = __ldg(s2), c = __ldg(s2 + 1);
        mx = bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(mx, a.x), a.y), a.z), a.w);
        mx = bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(mx, c.x), c.y), c.z), c.w);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) mx = bf16x2_absmax(mx, w[q]);
    }
    const float amax = bf16x2_hmax_to_f32(mx);
    const uint8_t s8 = f32_to_e4m3(amax / 6.0f * s_global_enc);
    const float s_local_dec = e4m3_to_f32(s8);
    const float s_enc = 1.0f / fmaxf(s_local_dec * s_global_dec, 0.000000000001f);
    uint32_t out[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t* ww = w + 4 * h;
      out[h] = f32x8_to_e2m1x8(bf16lo_to_f32(ww[0]) * s_enc, bf16hi_to_f32(ww[0]) * s_enc, bf16lo_to_f32(ww[1]) * s_enc,
                               bf16hi_to_f32(ww[1]) * s_enc, bf16lo_to_f32(ww[2]) * s_enc, bf16hi_to_f32(ww[2]) * s_enc,
                               bf16lo_to_f32(ww[3]) * s_enc, bf16hi_to_f32(ww[3]) * s_enc);
    }
    *reinterpret_cast<uint2*>(codes + r * (N / 2) + kb * 8) = make_uint2(out[0], out[1]);
    // 512-byte tiles of 128 rows x 4 blocks, [M/128, N/64, 512]; the reference also rewrites E4M3 NaN
    // bytes to +-448, which a saturating cast never produces
    sc[((r >> 7) * (N >> 6) + (kb >> 2)) * 512 + scale_tile_offset((int)(r & 127), (int)(kb & 3))] = s8;
  }
}

static int grid_for(size_t n, int threads) {
  return (int)std::max<size_t>(1, std::min<size_t>((n + threads - 1) / threads, (size_t)device_sm_count() * 8));
}

}  // namespace fp4b200

using namespace fp4b200;

// Rotary embedding (or its inverse) of contiguous bf16 Q [rows, q_dim] and K [rows, k_dim] in one launch:
// pairs of neighbouring columns, (cos, sin) = cs[row mod seq_len, (pair index) mod (head_dim / 2)].
// forward: even' = fma(-y, sin, x*cos), odd' = fma(x, sin, y*cos); inverse: even' = fma(y, sin, x*cos),
// odd' = fma(-x, sin, y*cos)   (reference: nvfp4_b200_gemm.cu:1083-1131).  Thread = 8 elements (16 bytes).
template <bool INVERSE>
__global__ void __launch_bounds__(256)
rope_packed_qk_kernel(const uint4* __restrict__ q, const uint4* __restrict__ k, uint4* __restrict__ q_out,
                      uint4* __restrict__ k_out, const float2* __restrict__ cs, size_t q_vecs, size_t k_vecs, int q_vec_row,
                      int k_vec_row, int pair_dim, int seq_mask) {
  const int pair_mask = pair_dim - 1;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < q_vecs + k_vecs; i += (size_t)gridDim.x * blockDim.x) {
    const bool is_q = i < q_vecs;
    const size_t v = is_q ? i : i - q_vecs;
    const int vec_row = is_q ? q_vec_row : k_vec_row;
    const size_t row = v / (size_t)vec_row;
    const int pair0 = (int)(v - row * (size_t)vec_row) * 4;        // first of this vector's four pairs inside the row
    const float2* cs_row = cs + (size_t)((int)row & seq_mask) * pair_dim;
    const uint4 in = __ldcs((is_q ? q : k) + v);
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
    uint32_t o[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float x = bf16lo_to_f32(w[p]), y = bf16hi_to_f32(w[p]);
      const float2 c = __ldg(cs_row + ((pair0 + p) & pair_mask));
      const float e = INVERSE ? __fmaf_rn(y, c.y, __fmul_rn(x, c.x)) : __fmaf_rn(-y, c.y, __fmul_rn(x, c.x));
      const float d = INVERSE ? __fmaf_rn(-x, c.y, __fmul_rn(y, c.x)) : __fmaf_rn(x, c.y, __fmul_rn(y, c.x));
      o[p] = f32x2_to_bf16x2(e, d);
    }
    st_cs_u4((is_q ? q_out : k_out) + v, make_uint4(o[0], o[1], o[2], o[3]));
  }
}

extern "C" {

int fp4b200_fp32_to_fp4x2(const float* in_f32, int64_t n_pairs, void* out_fp4x2, void* stream) {
  if (n_pairs < 0 || (n_pairs > 0 && (in_f32 == nullptr || out_fp4x2 == nullptr)))
    return set_error("fp32_to_fp4x2: null pointer or negative size");
  if ((reinterpret_cast<uintptr_t>(in_f32) & 7) != 0) return set_error("fp32_to_fp4x2: input must be 8-byte aligned");
  if (n_pairs == 0) return 0;
  fp32_to_fp4x2_kernel<<<grid_for((size_t)n_pairs, 256), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const float2*>(in_f32), (size_t)n_pairs, static_cast<uint8_t*>(out_fp4x2));
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_fp4x2_to_fp32(const void* in_fp4x2, int64_t n_bytes, float* out_f32, void* stream) {
  if (n_bytes < 0 || (n_bytes > 0 && (in_fp4x2 == nullptr || out_f32 == nullptr)))
    return set_error("fp4x2_to_fp32: null pointer or negative size");
  if ((reinterpret_cast<uintptr_t>(out_f32) & 7) != 0) return set_error("fp4x2_to_fp32: output must be 8-byte aligned");
  if (n_bytes == 0) return 0;
  fp4x2_to_fp32_kernel<<<grid_for((size_t)n_bytes, 256), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const uint8_t*>(in_fp4x2), (size_t)n_bytes, reinterpret_cast<float2*>(out_f32));
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_row_rms_reduce(const float* row_rms_partial, int64_t M, int64_t partial_cols, int64_t hidden_size, float eps,
                           float* inv_rms, void* stream) {
  if (row_rms_partial == nullptr || inv_rms == nullptr) return set_error("row_rms_reduce: null pointer");
  if (M < 0) return set_error("row_rms_reduce: negative row count");
  if (hidden_size <= 0 || (hidden_size % 32) != 0) return set_error("row_rms_reduce: hidden_size must be a positive multiple of 32");
  if (partial_cols <= 0 || partial_cols > hidden_size / 32 || (hidden_size % partial_cols) != 0)
    return set_error("row_rms_reduce: partial columns must evenly partition hidden_size (at most hidden_size/32)");
  if (partial_cols > 128) return set_error("row_rms_reduce: at most 128 partial columns");
  if (!(eps >= 0.0f) || !(eps <= 3.0e38f)) return set_error("row_rms_reduce: eps must be finite and non-negative");
  if (M == 0) return 0;
  row_rms_reduce_kernel<<<(unsigned)((M + 3) / 4), 128, 0, (cudaStream_t)stream>>>(row_rms_partial, inv_rms, M, partial_cols,
                                                                                    hidden_size, eps);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_rope_packed_qk(const void* q, const void* k, const float* rope_cs, int64_t rope_seq_len, int64_t rope_head_dim,
                           void* q_out, void* k_out, int64_t rows, int64_t q_dim, int64_t k_dim, int inverse, void* stream) {
  const char* fn = "rope_packed_qk";
  if (!q || !k || !rope_cs || !q_out || !k_out) return set_error("%s: null pointer", fn);
  if (rope_seq_len <= 0 || (rope_seq_len & (rope_seq_len - 1)))
    return set_error("%s: rope_seq_len must be a positive power of two", fn);
  if (rope_head_dim < 8 || (rope_head_dim & (rope_head_dim - 1)))
    return set_error("%s: rope_head_dim must be a power of two, at least 8 (got %lld)", fn, (long long)rope_head_dim);
  if (rows <= 0 || (rows % rope_seq_len)) return set_error("%s: rows must be a positive multiple of rope_seq_len", fn);
  if (q_dim <= 0 || k_dim <= 0 || (q_dim % rope_head_dim) || (k_dim % rope_head_dim))
    return set_error("%s: Q/K columns must be positive multiples of rope_head_dim", fn);
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(q_out) |
       reinterpret_cast<uintptr_t>(k_out)) & 15)
    return set_error("%s: Q/K inputs and outputs must be 16-byte aligned", fn);
  if (reinterpret_cast<uintptr_t>(rope_cs) & 7) return set_error("%s: rope_cs must be 8-byte aligned", fn);
  const size_t qv = (size_t)rows * (size_t)q_dim / 8, kv = (size_t)rows * (size_t)k_dim / 8;
  const unsigned grid = grid_for(qv + kv, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (inverse)
    rope_packed_qk_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint4*>(q), static_cast<const uint4*>(k),
                                                      static_cast<uint4*>(q_out), static_cast<uint4*>(k_out),
                                                      reinterpret_cast<const float2*>(rope_cs), qv, kv, (int)(q_dim / 8),
                                                      (int)(k_dim / 8), (int)(rope_head_dim / 2), (int)(rope_seq_len - 1));
  else
    rope_packed_qk_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint4*>(q), static_cast<const uint4*>(k),
                                                       static_cast<uint4*>(q_out), static_cast<uint4*>(k_out),
                                                       reinterpret_cast<const float2*>(rope_cs), qv, kv, (int)(q_dim / 8),
                                                       (int)(k_dim / 8), (int)(rope_head_dim / 2), (int)(rope_seq_len - 1));
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_tk_nvfp4_quantize(const void* A_bf16, int64_t M, int64_t N, void* A_fp4x2, void* A_sc, float* A_sc_global,
                              int scale_2d, void* stream) {
  if (!A_bf16 || !A_fp4x2 || !A_sc || !A_sc_global) return set_error("tk_nvfp4_quantize: null pointer");
  if (M <= 0 || N <= 0 || (M % 128) != 0 || (N % 128) != 0)
    return set_error("tk_nvfp4_quantize: M and N must be positive multiples of 128 (got %lld x %lld)", (long long)M, (long long)N);
  if ((reinterpret_cast<uintptr_t>(A_bf16) & 15) != 0 || (reinterpret_cast<uintptr_t>(A_fp4x2) & 7) != 0)
    return set_error("tk_nvfp4_quantize: input must be 16-byte and codes 8-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  FP4_CUDA_CHECK(cudaMemsetAsync(A_sc_global, 0, sizeof(float), st));
  const size_t n_vec = (size_t)M * (size_t)N / 8;
  tk_amax_kernel<<<grid_for(n_vec, 256), 256, 0, st>>>(static_cast<const uint4*>(A_bf16), n_vec, A_sc_global);
  FP4_CUDA_CHECK(cudaGetLastError());
  tk_divide_kernel<<<1, 1, 0, st>>>(A_sc_global);
  FP4_CUDA_CHECK(cudaGetLastError());
  tk_quantize_kernel<<<grid_for((size_t)M * (size_t)N / 16, 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(A_bf16), M, N, static_cast<uint8_t*>(A_fp4x2), static_cast<uint8_t*>(A_sc), A_sc_global,
      scale_2d != 0);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // extern "C"
