// NVFP4 producers for sm_100a: tensor amax, RMSNorm statistics, and the row+column
// quantiser (16-element blocks, E4M3 block scales in 512-byte tcgen05 scale tiles, packed
// E2M1 codes), with optional fused RMSNorm.  All kernels are HBM-bound; the quantiser is a
// persistent kernel fed by a 3-stage TMA pipeline and transposes through shared memory.
//
// Arithmetic follows the reference kernels so that codes and scale bytes are identical:
//   scale rules        fp4_runtime/TK_quantisation/nvfp4_v5/core.cuh:36-113
//   row / column math  fp4_runtime/TK_quantisation/nvfp4_v5/fused_amax_quantize.cuh:216-381
//   scale tile layout  fp4_runtime/TK_quantisation/nvfp4_v5/persistent_quantize.cuh:33-36
//   RMSNorm pass       fp4_runtime/TK_quantisation/nvfp4_v5/tk_quantize.cu:1025-1111
#include "fp4_common.cuh"
#include "host_util.h"

namespace fp4b200 {

// ---------------------------------------------------------------------------------------
// Tensor amax of a bf16 buffer (pass 1 of the plain quantiser)
// ---------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint4* __restrict__ x, size_t n_vec,
                                                        float* __restrict__ amax) {
  uint32_t m0 = 0, m1 = 0, m2 = 0, m3 = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // four independent 16-byte loads in flight per thread
  for (; i + 3 * stride < n_vec; i += 4 * stride) {
    const uint4 a = __ldg(x + i), b = __ldg(x + i + stride), c = __ldg(x + i + 2 * stride),
                d = __ldg(x + i + 3 * stride);
    m0 = bf16x2_absmax(bf16x2_absmax(m0, a.x), b.x); m1 = bf16x2_absmax(bf16x2_absmax(m1, a.y), b.y);
    m2 = bf16x2_absmax(bf16x2_absmax(m2, a.z), b.z); m3 = bf16x2_absmax(bf16x2_absmax(m3, a.w), b.w);
    m0 = bf16x2_absmax(bf16x2_absmax(m0, c.x), d.x); m1 = bf16x2_absmax(bf16x2_absmax(m1, c.y), d.y);
    m2 = bf16x2_absmax(bf16x2_absmax(m2, c.z), d.z); m3 = bf16x2_absmax(bf16x2_absmax(m3, c.w), d.w);
  }
  for (; i < n_vec; i += stride) {
    const uint4 a = __ldg(x + i);
    m0 = bf16x2_absmax(m0, a.x); m1 = bf16x2_absmax(m1, a.y);
    m2 = bf16x2_absmax(m2, a.z); m3 = bf16x2_absmax(m3, a.w);
  }
  m0 = bf16x2_absmax(bf16x2_absmax(m0, m1), bf16x2_absmax(m2, m3));
  float v = warp_max(bf16x2_hmax_to_f32(m0));
  __shared__ float warp_part[8];
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < 8 ? warp_part[threadIdx.x] : 0.0f;
    v = warp_max(v);
    if (threadIdx.x == 0 && v > 0.0f) atomic_max_nonneg(amax, v);
  }
}

// amax_sg[1] = amax_sg[0] / 2688 (GEMM-side tensor scale)
__global__ void finalize_sg_kernel(float* __restrict__ amax_sg) { amax_sg[1] = amax_sg[0] / 2688.0f; }

// ---------------------------------------------------------------------------------------
// RMSNorm statistics: inv_rms per row, and amax of bf16(x * inv_rms * gamma)
// ---------------------------------------------------------------------------------------
//
// One warp per row.  The sum of squares reproduces the summation tree of the reference's
// 256-thread kernel bit for bit: "virtual lane" t accumulates columns 2t, 2t+1, 2t+512, ...
// sequentially with fmaf; partials are combined by xor butterflies over masks 16,8,4,2,1
// inside each virtual warp and 4,2,1 across the eight virtual warps.  Here lane L holds
// virtual lanes 4L+128i+q (i = 0,1; q = 0..3) in acc[i][q], so the butterfly levels map to
// shuffles over lane masks 4,2,1, register adds over q, a register add over i, and
// shuffles over lane masks 16,8.
template <int NV /* 16-byte vectors held per lane; K <= NV*256 */, bool COMPUTE_INV_RMS>
__global__ void __launch_bounds__(256)
rmsnorm_stats_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                     float* __restrict__ inv_rms, float* __restrict__ amax, float eps, int M, int K) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  const int nvec_row = K >> 3;  // 16-byte vectors per row
  float run_max = 0.0f;

  for (int row = warp_global; row < M; row += n_warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * K);
    uint4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int q = lane + 32 * j;
      v[j] = (q < nvec_row) ? __ldg(xr + q) : make_uint4(0, 0, 0, 0);
    }
    float inv;
    if constexpr (COMPUTE_INV_RMS) {
      float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = j & 1;  // vector index within a 512-column block = lane + 32*i
        const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float lo = bf16lo_to_f32(w[q]), hi = bf16hi_to_f32(w[q]);
          acc[i][q] = fmaf(lo, lo, acc[i][q]);
          acc[i][q] = fmaf(hi, hi, acc[i][q]);
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[i][q] += __shfl_xor_sync(0xffffffffu, acc[i][q], 4);
          acc[i][q] += __shfl_xor_sync(0xffffffffu, acc[i][q], 2);
          acc[i][q] += __shfl_xor_sync(0xffffffffu, acc[i][q], 1);
        }
      }
      float part[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float a = acc[i][0] + acc[i][2];
        const float b = acc[i][1] + acc[i][3];
        part[i] = a + b;
      }
      float s = part[0] + part[1];
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      inv = rsqrtf(s / static_cast<float>(K) + eps);
      if (lane == 0) inv_rms[row] = inv;
    } else {
      inv = __ldg(inv_rms + row);
    }

    uint32_t mx = 0;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int q = lane + 32 * j;
      if (q < nvec_row) {
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + q);
        const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = bf16lo_to_f32(w[e]) * inv * bf16lo_to_f32(gw[e]);
          const float hi = bf16hi_to_f32(w[e]) * inv * bf16hi_to_f32(gw[e]);
          mx = bf16x2_absmax(mx, f32x2_to_bf16x2(lo, hi));
        }
      }
    }
    run_max = fmaxf(run_max, bf16x2_hmax_to_f32(mx));
  }
  run_max = warp_max(run_max);
  if (lane == 0 && run_max > 0.0f) atomic_max_nonneg(amax, run_max);
}

// Any-K variant: the row is read twice (second read hits L1/L2).
template <bool COMPUTE_INV_RMS>
__global__ void __launch_bounds__(256)
rmsnorm_stats_generic_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                             float* __restrict__ inv_rms, float* __restrict__ amax, float eps, int M, int K) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  const int nvec_row = K >> 3;
  float run_max = 0.0f;
  for (int row = warp_global; row < M; row += n_warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * K);
    float inv;
    if constexpr (COMPUTE_INV_RMS) {
      float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
      for (int q0 = 0; q0 < nvec_row; q0 += 64) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int q = q0 + lane + 32 * i;
          if (q < nvec_row) {
            const uint4 vv = __ldg(xr + q);
            const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = bf16lo_to_f32(w[e]), hi = bf16hi_to_f32(w[e]);
              acc[i][e] = fmaf(lo, lo, acc[i][e]);
              acc[i][e] = fmaf(hi, hi, acc[i][e]);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[i][q] += __shfl_xor_sync(0xffffffffu, acc[i][q], 4);
          acc[i][q] += __shfl_xor_sync(0xffffffffu, acc[i][q], 2);
          acc[i][q] += __shfl_xor_sync(0xffffffffu, acc[i][q], 1);
        }
      }
      const float p0 = (acc[0][0] + acc[0][2]) + (acc[0][1] + acc[0][3]);
      const float p1 = (acc[1][0] + acc[1][2]) + (acc[1][1] + acc[1][3]);
      float s = p0 + p1;
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      inv = rsqrtf(s / static_cast<float>(K) + eps);
      if (lane == 0) inv_rms[row] = inv;
    } else {
      inv = __ldg(inv_rms + row);
    }
    uint32_t mx = 0;
    for (int q = lane; q < nvec_row; q += 32) {
      const uint4 vv = __ldg(xr + q);
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + q);
      const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = bf16lo_to_f32(w[e]) * inv * bf16lo_to_f32(gw[e]);
        const float hi = bf16hi_to_f32(w[e]) * inv * bf16hi_to_f32(gw[e]);
        mx = bf16x2_absmax(mx, f32x2_to_bf16x2(lo, hi));
      }
    }
    run_max = fmaxf(run_max, bf16x2_hmax_to_f32(mx));
  }
  run_max = warp_max(run_max);
  if (lane == 0 && run_max > 0.0f) atomic_max_nonneg(amax, run_max);
}

// ---------------------------------------------------------------------------------------
// Row + column quantiser
// ---------------------------------------------------------------------------------------

constexpr int kChunk = 128;            // chunk edge in elements
constexpr int kQThreads = 256;
constexpr int kQStages = 3;
constexpr int kTileBytes = kChunk * kChunk * 2;  // 32 KiB of bf16
constexpr int kColPitch = 72;          // bytes per column of staged column codes (64 + pad)

struct QuantSmem {
  alignas(128) uint8_t in[kQStages][kTileBytes];
  alignas(16) uint8_t col_codes[kChunk * kColPitch];
  alignas(16) uint8_t row_sc[2][1024];
  alignas(16) uint8_t col_sc[1024];
  alignas(16) float inv_rms[2][kChunk];
  alignas(16) float gamma[2][kChunk];
  alignas(8) uint64_t full[kQStages];
};

struct QuantArgs {
  const float* amax_row;   // device scalar: tensor amax of the row-wise operand
  const float* amax_col;   // device scalar for the column-wise operand (may equal amax_row)
  const float* inv_rms;    // [M]   (NORM only)
  const __nv_bfloat16* gamma;  // [K] (NORM only)
  uint8_t* row_fp4;        // [M, K/2]
  uint8_t* row_sc;         // [M/128, K/64, 512]
  uint8_t* col_fp4;        // [K, M/2]      (may be null: row-wise only)
  uint8_t* col_sc;         // [K/128, M/64, 512]
  float* sg_out;           // optional: sg_out[0] = amax_row / 2688
  int* status;
  int M, K;
  int chunks_m, chunks_k;
  int reverse;             // walk chunks from the last row block to the first
};

template <bool ENCODE_CENTRIC, bool NORM>
__global__ void __launch_bounds__(kQThreads, 2)
nvfp4_quantize_kernel(const __grid_constant__ CUtensorMap tmap_x, const QuantArgs a) {
  extern __shared__ uint8_t smem_raw[];
  QuantSmem& sm = *reinterpret_cast<QuantSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int n_chunks = a.chunks_m * a.chunks_k;
  const int first = blockIdx.x;
  const int step = gridDim.x;
  const int my_count = first < n_chunks ? (n_chunks - first + step - 1) / step : 0;

  auto chunk_coords = [&](int it, int& cm, int& ck) {
    int c = first + it * step;
    if (a.reverse) c = n_chunks - 1 - c;
    cm = c / a.chunks_k;
    ck = c - cm * a.chunks_k;
  };

  if (tid == 0) {
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < kQStages; ++s) mbar_init(&sm.full[s], 1);
    fence_mbar_init();
    if (blockIdx.x == 0 && a.sg_out != nullptr) a.sg_out[0] = *a.amax_row / 2688.0f;
  }
  __syncthreads();
  if (tid == 0) {
    for (int s = 0; s < kQStages && s < my_count; ++s) {
      int cm, ck;
      chunk_coords(s, cm, ck);
      mbar_expect_tx(&sm.full[s], kTileBytes);
      tma_load_2d(sm.in[s], &tmap_x, ck * kChunk, cm * kChunk, &sm.full[s]);
    }
  }

  const float s_enc_row = nvfp4_global_encode_scale(*a.amax_row);
  const float s_enc_col = nvfp4_global_encode_scale(*a.amax_col);
  const bool want_col = a.col_fp4 != nullptr;

  for (int it = 0; it < my_count; ++it) {
    const int s = it % kQStages;
    const uint32_t parity = (it / kQStages) & 1;
    int cm, ck;
    chunk_coords(it, cm, ck);
    const int m0 = cm * kChunk, k0 = ck * kChunk;
    const int pp = it & 1;

    if constexpr (NORM) {
      // stage this chunk's 128 inv_rms values and 128 gammas (as fp32)
      if (tid < kChunk) sm.inv_rms[pp][tid] = __ldg(a.inv_rms + m0 + tid);
      else sm.gamma[pp][tid - kChunk] = __bfloat162float(a.gamma[k0 + tid - kChunk]);
      __syncthreads();
    }

    if (!mbar_wait_bounded(&sm.full[s], parity)) {
      if (tid == 0) atomicExch(a.status, kStatusQuantTmaTimeout);
      return;
    }

    uint8_t* tile = sm.in[s];

    // ---- row pass: each thread owns 16 contiguous elements of one row, 4 times -------
#pragma unroll
    for (int rep = 0; rep < 4; ++rep) {
      const int b = rep * kQThreads + tid;
      const int r = b >> 3, kb = b & 7;
      uint4* p = reinterpret_cast<uint4*>(tile + r * (kChunk * 2) + kb * 32);
      uint4 v0 = p[0], v1 = p[1];
      uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      if constexpr (NORM) {
        const float inv = sm.inv_rms[pp][r];
        const float4* g4 = reinterpret_cast<const float4*>(&sm.gamma[pp][kb * 16]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 g = g4[q];
          w[2 * q] = f32x2_to_bf16x2(bf16lo_to_f32(w[2 * q]) * inv * g.x, bf16hi_to_f32(w[2 * q]) * inv * g.y);
          w[2 * q + 1] =
              f32x2_to_bf16x2(bf16lo_to_f32(w[2 * q + 1]) * inv * g.z, bf16hi_to_f32(w[2 * q + 1]) * inv * g.w);
        }
        if (want_col) {  // the column pass reads the normalised values
          p[0] = make_uint4(w[0], w[1], w[2], w[3]);
          p[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      uint32_t mx = 0;
#pragma unroll
      for (int q = 0; q < 8; ++q) mx = bf16x2_absmax(mx, w[q]);
      const float bmax = bf16x2_hmax_to_f32(mx);
      uint8_t stored;
      float coeff;
      nvfp4_block_scale<ENCODE_CENTRIC>(bmax, s_enc_row, stored, coeff);
      uint2 codes;
      codes.x = f32x8_to_e2m1x8(bf16lo_to_f32(w[0]) * coeff, bf16hi_to_f32(w[0]) * coeff,
                                bf16lo_to_f32(w[1]) * coeff, bf16hi_to_f32(w[1]) * coeff,
                                bf16lo_to_f32(w[2]) * coeff, bf16hi_to_f32(w[2]) * coeff,
                                bf16lo_to_f32(w[3]) * coeff, bf16hi_to_f32(w[3]) * coeff);
      codes.y = f32x8_to_e2m1x8(bf16lo_to_f32(w[4]) * coeff, bf16hi_to_f32(w[4]) * coeff,
                                bf16lo_to_f32(w[5]) * coeff, bf16hi_to_f32(w[5]) * coeff,
                                bf16lo_to_f32(w[6]) * coeff, bf16hi_to_f32(w[6]) * coeff,
                                bf16lo_to_f32(w[7]) * coeff, bf16hi_to_f32(w[7]) * coeff);
      st_cs_u2(a.row_fp4 + (size_t)(m0 + r) * (a.K >> 1) + ((k0 + kb * 16) >> 1), codes);
      sm.row_sc[pp][(kb >> 2) * 512 + scale_tile_offset(r, kb & 3)] = stored;
    }
    __syncthreads();

    // ---- column pass: warp w owns rows 16w..16w+15, lane owns two adjacent columns ---
    if (want_col) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = 2 * lane + 64 * h;  // first of the two columns
        uint32_t w[16];
        uint32_t mx = 0;
        const uint32_t* col = reinterpret_cast<const uint32_t*>(tile + (warp * 16) * (kChunk * 2) + c * 2);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          w[i] = col[i * (kChunk / 2)];
          mx = bf16x2_absmax(mx, w[i]);
        }
        uint8_t st0, st1;
        float c0, c1;
        nvfp4_block_scale<ENCODE_CENTRIC>(bf16lo_to_f32(mx), s_enc_col, st0, c0);
        nvfp4_block_scale<ENCODE_CENTRIC>(bf16hi_to_f32(mx), s_enc_col, st1, c1);
        uint2 q0, q1;
        q0.x = f32x8_to_e2m1x8(bf16lo_to_f32(w[0]) * c0, bf16lo_to_f32(w[1]) * c0, bf16lo_to_f32(w[2]) * c0,
                               bf16lo_to_f32(w[3]) * c0, bf16lo_to_f32(w[4]) * c0, bf16lo_to_f32(w[5]) * c0,
                               bf16lo_to_f32(w[6]) * c0, bf16lo_to_f32(w[7]) * c0);
        q0.y = f32x8_to_e2m1x8(bf16lo_to_f32(w[8]) * c0, bf16lo_to_f32(w[9]) * c0, bf16lo_to_f32(w[10]) * c0,
                               bf16lo_to_f32(w[11]) * c0, bf16lo_to_f32(w[12]) * c0, bf16lo_to_f32(w[13]) * c0,
                               bf16lo_to_f32(w[14]) * c0, bf16lo_to_f32(w[15]) * c0);
        q1.x = f32x8_to_e2m1x8(bf16hi_to_f32(w[0]) * c1, bf16hi_to_f32(w[1]) * c1, bf16hi_to_f32(w[2]) * c1,
                               bf16hi_to_f32(w[3]) * c1, bf16hi_to_f32(w[4]) * c1, bf16hi_to_f32(w[5]) * c1,
                               bf16hi_to_f32(w[6]) * c1, bf16hi_to_f32(w[7]) * c1);
        q1.y = f32x8_to_e2m1x8(bf16hi_to_f32(w[8]) * c1, bf16hi_to_f32(w[9]) * c1, bf16hi_to_f32(w[10]) * c1,
                               bf16hi_to_f32(w[11]) * c1, bf16hi_to_f32(w[12]) * c1, bf16hi_to_f32(w[13]) * c1,
                               bf16hi_to_f32(w[14]) * c1, bf16hi_to_f32(w[15]) * c1);
        *reinterpret_cast<uint2*>(&sm.col_codes[c * kColPitch + warp * 8]) = q0;
        *reinterpret_cast<uint2*>(&sm.col_codes[(c + 1) * kColPitch + warp * 8]) = q1;
        sm.col_sc[(warp >> 2) * 512 + scale_tile_offset(c, warp & 3)] = st0;
        sm.col_sc[(warp >> 2) * 512 + scale_tile_offset(c + 1, warp & 3)] = st1;
      }
    }
    __syncthreads();

    // stage s is free again: refill it with the chunk kQStages ahead
    if (tid == 0 && it + kQStages < my_count) {
      int ncm, nck;
      chunk_coords(it + kQStages, ncm, nck);
      fence_proxy_async_smem();
      mbar_expect_tx(&sm.full[s], kTileBytes);
      tma_load_2d(sm.in[s], &tmap_x, nck * kChunk, ncm * kChunk, &sm.full[s]);
    }

    // ---- write-out: scales (two 512-byte tiles per orientation) and column codes -----
    {
      uint8_t* dst = a.row_sc + ((size_t)cm * (a.K >> 6) + (size_t)ck * 2) * 512;
      st_cs_u32(dst + tid * 4, *reinterpret_cast<const uint32_t*>(&sm.row_sc[pp][tid * 4]));
    }
    if (want_col) {
      uint8_t* dst = a.col_sc + ((size_t)ck * (a.M >> 6) + (size_t)cm * 2) * 512;
      st_cs_u32(dst + tid * 4, *reinterpret_cast<const uint32_t*>(&sm.col_sc[tid * 4]));
#pragma unroll
      for (int rep = 0; rep < 4; ++rep) {
        const int idx = rep * kQThreads + tid;  // 1024 pieces of 8 bytes
        const int c = idx >> 3, part = idx & 7;
        const uint2 v = *reinterpret_cast<const uint2*>(&sm.col_codes[c * kColPitch + part * 8]);
        st_cs_u2(a.col_fp4 + (size_t)(k0 + c) * (a.M >> 1) + (m0 >> 1) + part * 8, v);
      }
      // no barrier needed here: col_codes / col_sc are next written after the barrier that
      // follows the next chunk's row pass, which every thread reaches only after this loop
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------

static int launch_amax(const void* x, int64_t n_elems, float* amax_sg, cudaStream_t st) {
  FP4_CUDA_CHECK(cudaMemsetAsync(amax_sg, 0, 2 * sizeof(float), st));
  const size_t n_vec = (size_t)n_elems / 8;
  if (n_vec > 0) {
    int grid = (int)std::min<size_t>((n_vec + 255) / 256, (size_t)device_sm_count() * 8);
    amax_bf16_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(x), n_vec, amax_sg);
    FP4_CUDA_CHECK(cudaGetLastError());
  }
  finalize_sg_kernel<<<1, 1, 0, st>>>(amax_sg);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

template <bool EC, bool NORM>
static int launch_quantize_t(const CUtensorMap& tmap, const QuantArgs& args, cudaStream_t st) {
  auto kern = nvfp4_quantize_kernel<EC, NORM>;
  const int smem = (int)sizeof(QuantSmem) + 128;
  FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int n_chunks = args.chunks_m * args.chunks_k;
  const int grid = std::min(n_chunks, 2 * device_sm_count());
  if (grid == 0) return 0;
  kern<<<grid, kQThreads, smem, st>>>(tmap, args);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

static int launch_quantize(const void* x, int64_t M, int64_t K, const float* amax_row, const float* amax_col,
                           bool encode_centric, const float* inv_rms, const void* gamma, void* row_fp4,
                           void* row_sc, void* col_fp4, void* col_sc, float* sg_out, bool reverse,
                           cudaStream_t st) {
  CUtensorMap tmap;
  if (int rc = make_tmap_2d(&tmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                            (uint64_t)K * 2, kChunk, kChunk, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  QuantArgs a{};
  a.amax_row = amax_row;
  a.amax_col = amax_col ? amax_col : amax_row;
  a.inv_rms = inv_rms;
  a.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  a.row_fp4 = (uint8_t*)row_fp4; a.row_sc = (uint8_t*)row_sc;
  a.col_fp4 = (uint8_t*)col_fp4; a.col_sc = (uint8_t*)col_sc;
  a.sg_out = sg_out;
  a.status = device_status_ptr();
  if (a.status == nullptr) return -1;
  a.M = (int)M; a.K = (int)K;
  a.chunks_m = (int)(M / kChunk); a.chunks_k = (int)(K / kChunk);
  a.reverse = reverse ? 1 : 0;
  const bool norm = inv_rms != nullptr;
  if (encode_centric) return norm ? launch_quantize_t<true, true>(tmap, a, st) : launch_quantize_t<true, false>(tmap, a, st);
  return norm ? launch_quantize_t<false, true>(tmap, a, st) : launch_quantize_t<false, false>(tmap, a, st);
}

static int launch_rmsnorm_stats(const void* x, const void* gamma, float* inv_rms, float* amax_sg, float eps,
                                int64_t M, int64_t K, bool compute_inv, cudaStream_t st) {
  FP4_CUDA_CHECK(cudaMemsetAsync(amax_sg, 0, 2 * sizeof(float), st));
  const int warps_per_block = 8;
  int grid = (int)std::min<int64_t>((M + warps_per_block - 1) / warps_per_block, (int64_t)device_sm_count() * 8);
  if (grid > 0) {
    auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
    auto gb = reinterpret_cast<const __nv_bfloat16*>(gamma);
    if (K <= 2048) {
      if (compute_inv) rmsnorm_stats_kernel<8, true><<<grid, 256, 0, st>>>(xb, gb, inv_rms, amax_sg, eps, (int)M, (int)K);
      else rmsnorm_stats_kernel<8, false><<<grid, 256, 0, st>>>(xb, gb, inv_rms, amax_sg, eps, (int)M, (int)K);
    } else if (K <= 4096) {
      if (compute_inv) rmsnorm_stats_kernel<16, true><<<grid, 256, 0, st>>>(xb, gb, inv_rms, amax_sg, eps, (int)M, (int)K);
      else rmsnorm_stats_kernel<16, false><<<grid, 256, 0, st>>>(xb, gb, inv_rms, amax_sg, eps, (int)M, (int)K);
    } else {
      if (compute_inv) rmsnorm_stats_generic_kernel<true><<<grid, 256, 0, st>>>(xb, gb, inv_rms, amax_sg, eps, (int)M, (int)K);
      else rmsnorm_stats_generic_kernel<false><<<grid, 256, 0, st>>>(xb, gb, inv_rms, amax_sg, eps, (int)M, (int)K);
    }
    FP4_CUDA_CHECK(cudaGetLastError());
  }
  finalize_sg_kernel<<<1, 1, 0, st>>>(amax_sg);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace fp4b200

using namespace fp4b200;

static int check_quant_shapes(const void* x, int64_t M, int64_t K, const char* who) {
  if (x == nullptr) return set_error("%s: input pointer is null", who);
  if (M <= 0 || K <= 0 || (M % 128) != 0 || (K % 128) != 0)
    return set_error("%s: M and K must be positive multiples of 128 (got M=%lld K=%lld)", who, (long long)M,
                     (long long)K);
  if (M > (1 << 30) || K > (1 << 30)) return set_error("%s: dimension too large", who);
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return set_error("%s: input must be 16-byte aligned", who);
  return 0;
}

extern "C" {

int fp4b200_nvfp4_amax(const void* x_bf16, int64_t n_elems, float* amax_sg, void* stream) {
  if (x_bf16 == nullptr || amax_sg == nullptr) return set_error("nvfp4_amax: null pointer");
  if (n_elems < 0 || (n_elems % 8) != 0) return set_error("nvfp4_amax: element count must be a multiple of 8");
  return launch_amax(x_bf16, n_elems, amax_sg, (cudaStream_t)stream);
}

int fp4b200_nvfp4_quantize(const void* x_bf16, int64_t M, int64_t K, const float* amax_row,
                           const float* amax_col, int encode_centric, void* row_fp4, void* row_sc,
                           void* col_fp4, void* col_sc, float* sg_out, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_quantize")) return rc;
  if (amax_row == nullptr || row_fp4 == nullptr || row_sc == nullptr)
    return set_error("nvfp4_quantize: amax_row, row_fp4 and row_sc are required");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("nvfp4_quantize: col_fp4 and col_sc must both be given or both be null");
  return launch_quantize(x_bf16, M, K, amax_row, amax_col, encode_centric != 0, nullptr, nullptr, row_fp4,
                         row_sc, col_fp4, col_sc, sg_out, false, (cudaStream_t)stream);
}

int fp4b200_nvfp4_quantize_for_gemm(const void* x_bf16, int64_t M, int64_t K, int return_transpose,
                                    int encode_centric, void* row_fp4, void* row_sc, void* col_fp4,
                                    void* col_sc, float* amax_sg, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_quantize_for_gemm")) return rc;
  if (row_fp4 == nullptr || row_sc == nullptr || amax_sg == nullptr)
    return set_error("nvfp4_quantize_for_gemm: row_fp4, row_sc and amax_sg are required");
  if (return_transpose && (col_fp4 == nullptr || col_sc == nullptr))
    return set_error("nvfp4_quantize_for_gemm: return_transpose needs col_fp4 and col_sc");
  if (int rc = launch_amax(x_bf16, M * K, amax_sg, (cudaStream_t)stream)) return rc;
  return launch_quantize(x_bf16, M, K, amax_sg, amax_sg, encode_centric != 0, nullptr, nullptr, row_fp4, row_sc,
                         return_transpose ? col_fp4 : nullptr, return_transpose ? col_sc : nullptr, nullptr,
                         true, (cudaStream_t)stream);
}

int fp4b200_nvfp4_rmsnorm_stats(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                float* inv_rms, int compute_inv_rms, float* amax_sg, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_rmsnorm_stats")) return rc;
  if (gamma_bf16 == nullptr || inv_rms == nullptr || amax_sg == nullptr)
    return set_error("nvfp4_rmsnorm_stats: gamma, inv_rms and amax_sg are required");
  return launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, amax_sg, eps, M, K, compute_inv_rms != 0,
                              (cudaStream_t)stream);
}

int fp4b200_nvfp4_fused_norm_quantize(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M,
                                      int64_t K, float* inv_rms, int compute_inv_rms, int encode_centric,
                                      void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                      float* amax_sg, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_fused_norm_quantize")) return rc;
  if (gamma_bf16 == nullptr || inv_rms == nullptr || amax_sg == nullptr || row_fp4 == nullptr ||
      row_sc == nullptr)
    return set_error("nvfp4_fused_norm_quantize: gamma, inv_rms, amax_sg, row_fp4 and row_sc are required");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("nvfp4_fused_norm_quantize: col_fp4 and col_sc must both be given or both be null");
  if ((reinterpret_cast<uintptr_t>(gamma_bf16) & 15) != 0)
    return set_error("nvfp4_fused_norm_quantize: gamma must be 16-byte aligned");
  if (int rc = launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, amax_sg, eps, M, K, compute_inv_rms != 0,
                                    (cudaStream_t)stream))
    return rc;
  return launch_quantize(x_bf16, M, K, amax_sg, amax_sg, encode_centric != 0, inv_rms, gamma_bf16, row_fp4,
                         row_sc, col_fp4, col_sc, nullptr, true, (cudaStream_t)stream);
}


int fp4b200_nvfp4_quantize_normed(const void* x_bf16, const void* gamma_bf16, const float* inv_rms,
                                  const float* amax, int64_t M, int64_t K, int encode_centric, void* row_fp4,
                                  void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_quantize_normed")) return rc;
  if (gamma_bf16 == nullptr || inv_rms == nullptr || amax == nullptr || row_fp4 == nullptr || row_sc == nullptr)
    return set_error("nvfp4_quantize_normed: gamma, inv_rms, amax, row_fp4 and row_sc are required");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("nvfp4_quantize_normed: col_fp4 and col_sc must both be given or both be null");
  return launch_quantize(x_bf16, M, K, amax, amax, encode_centric != 0, inv_rms, gamma_bf16, row_fp4, row_sc,
                         col_fp4, col_sc, nullptr, true, (cudaStream_t)stream);
}

}  // extern "C"
