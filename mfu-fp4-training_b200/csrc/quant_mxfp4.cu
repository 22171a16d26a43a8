// MXFP4 producers for sm_100a: row + column quantisation in 32-element blocks with E8M0 scales
// (no tensor-level scale, so a single pass over the input), optional fused RMSNorm.
//
// Arithmetic follows the reference (fp4_runtime/TK_quantisation/mxfp4_v4/mxfp4_v3_quantize.cuh):
//   E8M0 of the block amax, modes RTE / ceil / floor            :1295-1342
//   coefficient 6 * 2^(127-e), codes = e2m1_rn(x * coefficient) :1601-1603 (exp2f_rcp util/ptx.cuh:330-338)
//   scale bytes in 512-byte tiles of 128 rows x 4 blocks        :5059-5086
//   weights: one scale per 32x32 tile for both orientations, ceil exponent lowered by one when the
//   tile amax sits in the lower part of its binade ("4 over 6")  :1797-1960
// Pipeline and shared-memory geometry are those of the NVFP4 quantiser (quant_nvfp4.cu): persistent
// CTAs, 128x128 chunks as two 128-byte-swizzled TMA boxes, three stages.
#include "fp4_common.cuh"
#include "host_util.h"
#include "swiglu_math.cuh"

namespace fp4b200 {

constexpr int kMxChunk = 128;
constexpr int kMxThreads = 256;
constexpr int kMxStages = 3;
constexpr int kMxHalfBytes = kMxChunk * 128;
constexpr int kMxTileBytes = 2 * kMxHalfBytes;

struct MxSmem {
  alignas(1024) uint8_t in[kMxStages][kMxTileBytes];
  alignas(16) uint4 col_codes[4][kMxChunk];   // [32-row group][column] -> 16 bytes of codes
  alignas(16) uint8_t row_sc[2][512];
  alignas(16) uint8_t col_sc[512];
  alignas(16) float inv_rms[2][kMxChunk];
  alignas(16) float gamma[2][kMxChunk];
  alignas(8) uint64_t full[kMxStages];
  uint8_t tile_e8[4][4];                      // W2D: scale byte of each 32x32 tile of the chunk
};

struct MxArgs {
  const float* inv_rms;        // [M] (NORM only)
  const __nv_bfloat16* gamma;  // [K] (NORM only)
  uint8_t* row_fp4;            // [M, K/2]
  uint8_t* row_sc;             // [M/128, K/128, 512]
  uint8_t* col_fp4;            // [K, M/2]   (may be null)
  uint8_t* col_sc;             // [K/128, M/128, 512]
  int* status;
  int M, K, chunks_m, chunks_k;
  int mode;                    // 0 RTE, 1 ceil ("encode"), 2 floor ("decode")
  // the matrix may be the column concatenation of up to three inputs that are never concatenated in memory: column
  // chunks [0, split_chunk[0]) come from the first tensor map, [split_chunk[0], split_chunk[1]) from the second, the
  // rest from the third (one input: both = chunks_k)
  int split_chunk[2];
  // > 0: the input is [B, heads, seq, dim] (dim a multiple of 64, seq of 128) and the matrix [B*seq, heads*dim] with
  // element (b*seq + s, h*dim + d) = input[b, h, s, d]; tmap_x then describes [B*heads*seq, dim]
  int nhsd_heads, nhsd_seq, nhsd_dim;
  const float2* rope_cs;       // ROPE: [seq_len, 32] (cos, sin) per token position and column pair of a 64-wide head
  int rope_seq_mask;
};

__device__ __forceinline__ uint32_t mx_e8m0(float b, int mode) {
  if (b <= 1e-38f) return 0;
  const uint32_t u = __float_as_uint(b);
  uint32_t e = (u >> 23) & 0xFF;
  const uint32_t m = u & 0x7FFFFF;
  bool up;
  if (mode == 1) up = m != 0;
  else if (mode == 0) up = (m > 0x400000u) || (m == 0x400000u && (e & 1));
  else up = false;
  if (up && e < 0xFE) ++e;
  return e;
}

// 6 * 2^(127-e); e = 254 needs the denormal 2^-127, e = 0 gives 2^127 (product overflows to inf)
__device__ __forceinline__ float mx_coeff(uint32_t e) {
  const float rcp = (e == 254) ? __uint_as_float(0x00400000u) : __uint_as_float((254u - e) << 23);
  return 6.0f * rcp;
}

// Scale byte of a 32x32 weight tile: the ceil exponent of the tile amax, lowered by one (values up to
// 2x the top code then saturate) when amax * 2^-(e-127) < 0.87, i.e. when most of the finer grid
// would otherwise go unused (reference mx_weight_2d_quantize, mxfp4_v3_quantize.cuh:1864-1878).
__device__ __forceinline__ uint32_t mx_weight_tile_e8m0(float tile_amax) {
  const uint32_t safe = mx_e8m0(tile_amax, 1);
  const float rcp = (safe == 254) ? __uint_as_float(0x00400000u) : __uint_as_float((254u - safe) << 23);
  const float phase = tile_amax * rcp;
  return (safe > 0 && phase < 0.87f) ? safe - 1 : safe;
}

// ROPE: the inverse rotary embedding (heads of 64, neighbouring columns paired) of the first two split inputs on the
// way in: the row pass rotates the tile in place, as it normalises it with NORM.
template <bool NORM, bool W2D, bool ROPE = false>
__global__ void __launch_bounds__(kMxThreads, 2)
mxfp4_quantize_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_x1,
                      const __grid_constant__ CUtensorMap tmap_x2, const MxArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  MxSmem& sm = *reinterpret_cast<MxSmem*>(smem_align_1024(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_chunks = a.chunks_m * a.chunks_k;
  const int first = blockIdx.x, step = gridDim.x;
  const int my_count = first < n_chunks ? (n_chunks - first + step - 1) / step : 0;
  auto chunk_coords = [&](int it, int& cm, int& ck) {
    const int c = first + it * step;
    cm = c / a.chunks_k;
    ck = c - cm * a.chunks_k;
  };
  auto issue_load = [&](int it, int s) {
    int cm, ck;
    chunk_coords(it, cm, ck);
    mbar_expect_tx(&sm.full[s], kMxTileBytes);
    const CUtensorMap* src = &tmap_x;
    if (ck >= a.split_chunk[1]) { src = &tmap_x2; ck -= a.split_chunk[1]; }
    else if (ck >= a.split_chunk[0]) { src = &tmap_x1; ck -= a.split_chunk[0]; }
    if (a.nhsd_seq > 0) {
      // a half tile (128 tokens of one sequence x 64 columns of one head) is a contiguous block of rows of [B*heads*seq, dim]
      const int b = (cm * kMxChunk) / a.nhsd_seq, s0 = cm * kMxChunk - b * a.nhsd_seq;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int col = ck * kMxChunk + h2 * 64, head = col / a.nhsd_dim;
        tma_load_2d(sm.in[s] + h2 * kMxHalfBytes, src, col - head * a.nhsd_dim, (b * a.nhsd_heads + head) * a.nhsd_seq + s0,
                    &sm.full[s]);
      }
      return;
    }
    tma_load_2d(sm.in[s], src, ck * kMxChunk, cm * kMxChunk, &sm.full[s]);
    tma_load_2d(sm.in[s] + kMxHalfBytes, src, ck * kMxChunk + 64, cm * kMxChunk, &sm.full[s]);
  };
  if (tid == 0) {
    tma_prefetch_desc(&tmap_x);
    if (a.split_chunk[0] < a.chunks_k) tma_prefetch_desc(&tmap_x1);
    if (a.split_chunk[1] < a.chunks_k) tma_prefetch_desc(&tmap_x2);
    for (int s = 0; s < kMxStages; ++s) mbar_init(&sm.full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0)
    for (int s = 0; s < kMxStages && s < my_count; ++s) issue_load(s, s);
  const bool want_col = a.col_fp4 != nullptr;
  if constexpr (NORM) {
    if (my_count > 0) {
      int cm, ck;
      chunk_coords(0, cm, ck);
      if (tid < kMxChunk) sm.inv_rms[0][tid] = __ldg(a.inv_rms + cm * kMxChunk + tid);
      else sm.gamma[0][tid - kMxChunk] = __bfloat162float(a.gamma[ck * kMxChunk + tid - kMxChunk]);
    }
    __syncthreads();
  }
  // row pass: lane = (row & 7, 32-column unit = one MX block); column pass: warp = (32-row group, half)
  const int unit = lane >> 3, r_lo = lane & 7;
  const int half_off = (unit >> 1) * kMxHalfBytes, cb = (unit & 1) * 4;
  int row_off[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) row_off[j] = ((cb + j) ^ r_lo) << 4;
  int col_off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) col_off[j] = (((lane >> 2) ^ j) << 4) + (lane & 3) * 4;
  const int grp = warp >> 1, chalf = warp & 1;

  for (int it = 0; it < my_count; ++it) {
    const int s = it % kMxStages;
    const uint32_t parity = (it / kMxStages) & 1;
    int cm, ck;
    chunk_coords(it, cm, ck);
    const int m0 = cm * kMxChunk, k0 = ck * kMxChunk, pp = it & 1;
    float pre = 0.0f;
    if constexpr (NORM) {
      if (it + 1 < my_count) {
        int ncm, nck;
        chunk_coords(it + 1, ncm, nck);
        pre = (tid < kMxChunk) ? __ldg(a.inv_rms + ncm * kMxChunk + tid)
                               : __bfloat162float(a.gamma[nck * kMxChunk + tid - kMxChunk]);
      }
    }
    if (!mbar_wait_bounded(&sm.full[s], parity)) {
      if (tid == 0) atomicExch(a.status, kStatusQuantTmaTimeout);
      return;
    }
    uint8_t* tile = sm.in[s];
    if constexpr (W2D) {
      // tile amaxes in the column-pass geometry: this warp holds rows grp*32.., columns chalf*64..;
      // 16 lanes (32 columns) make one tile
      const uint8_t* base = tile + chalf * kMxHalfBytes + (grp * 32) * 128;
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = absmax_xs(mx, *reinterpret_cast<const uint32_t*>(base + i * 128 + col_off[i & 7]));
      float b = fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx)));
      b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 1));
      b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 2));
      b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 4));
      b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 8));
      if ((lane & 15) == 0) sm.tile_e8[grp][chalf * 2 + (lane >> 4)] = (uint8_t)mx_weight_tile_e8m0(b);
      __syncthreads();
    }
    // the row pass also normalises the tile in place for the column pass (NORM); without row outputs it is skipped otherwise
    const bool rope_here = ROPE && ck < a.split_chunk[1];
    const bool row_pass = NORM || rope_here || a.row_fp4 != nullptr;
#pragma unroll
    for (int rep = 0; rep < 2 && row_pass; ++rep) {
      const int r = warp * 16 + rep * 8 + r_lo;
      uint8_t* rowp = tile + half_off + r * 128;
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(rowp + row_off[j]);
        w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
      }
      if constexpr (NORM) {
        const float inv = sm.inv_rms[pp][r];
        const float2 inv2 = make_float2(inv, inv);
        const float2* g2 = reinterpret_cast<const float2*>(&sm.gamma[pp][unit * 32]);
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          float2 t = mul2(make_float2(bf16lo_to_f32(w[q]), bf16hi_to_f32(w[q])), inv2);
          t = mul2(t, g2[q]);
          w[q] = f32x2_to_bf16x2(t.x, t.y);
        }
        if (want_col) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(rowp + row_off[j]) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        }
      }
      if constexpr (ROPE) {
        if (rope_here) {
          // even' = x cos + y sin, odd' = y cos - x sin, each as one product and one fused multiply-add, rounded to bf16
          // (reference apply_inverse_rope_tile_inplace_live64, mxfp4_v3_quantize.cuh:251-285)
          const float4* cs4 = reinterpret_cast<const float4*>(a.rope_cs + (size_t)((m0 + r) & a.rope_seq_mask) * 32 + (unit & 1) * 16);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 cs = __ldg(cs4 + q);
            const float x0 = bf16lo_to_f32(w[2 * q]), y0 = bf16hi_to_f32(w[2 * q]);
            const float x1 = bf16lo_to_f32(w[2 * q + 1]), y1 = bf16hi_to_f32(w[2 * q + 1]);
            w[2 * q] = f32x2_to_bf16x2(__fmaf_rn(y0, cs.y, __fmul_rn(x0, cs.x)), __fmaf_rn(-x0, cs.y, __fmul_rn(y0, cs.x)));
            w[2 * q + 1] = f32x2_to_bf16x2(__fmaf_rn(y1, cs.w, __fmul_rn(x1, cs.z)), __fmaf_rn(-x1, cs.w, __fmul_rn(y1, cs.z)));
          }
          if (want_col) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(rowp + row_off[j]) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
        }
      }
      uint32_t mx = 0;
#pragma unroll
      for (int q = 0; q < 16; ++q) mx = absmax_xs(mx, w[q]);
      const float b = fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx)));
      uint32_t e = mx_e8m0(b, a.mode);
      if constexpr (W2D) e = sm.tile_e8[r >> 5][unit];
      const float coeff = mx_coeff(e);
      uint4 codes;
      codes.x = quant8(w, coeff); codes.y = quant8(w + 4, coeff);
      codes.z = quant8(w + 8, coeff); codes.w = quant8(w + 12, coeff);
      if (a.row_fp4 != nullptr) st_cs_u4(a.row_fp4 + (size_t)(m0 + r) * (a.K >> 1) + ((k0 + unit * 32) >> 1), codes);
      sm.row_sc[pp][scale_tile_offset(r, unit)] = (uint8_t)e;
    }
    __syncthreads();
    if (want_col) {
      const uint8_t* base = tile + chalf * kMxHalfBytes + (grp * 32) * 128;
      uint32_t w[32];
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        w[i] = *reinterpret_cast<const uint32_t*>(base + i * 128 + col_off[i & 7]);
        mx = absmax_xs(mx, w[i]);
      }
      uint32_t e0 = mx_e8m0(fabsf(bf16lo_to_f32(mx)), a.mode), e1 = mx_e8m0(fabsf(bf16hi_to_f32(mx)), a.mode);
      if constexpr (W2D) e0 = e1 = sm.tile_e8[grp][chalf * 2 + (lane >> 4)];
      const float2 cc = make_float2(mx_coeff(e0), mx_coeff(e1));
      uint32_t q0[4], q1[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        float2 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          v[i] = mul2(make_float2(bf16lo_to_f32(w[8 * p + i]), bf16hi_to_f32(w[8 * p + i])), cc);
        q0[p] = f32x8_to_e2m1x8(v[0].x, v[1].x, v[2].x, v[3].x, v[4].x, v[5].x, v[6].x, v[7].x);
        q1[p] = f32x8_to_e2m1x8(v[0].y, v[1].y, v[2].y, v[3].y, v[4].y, v[5].y, v[6].y, v[7].y);
      }
      const int c = 2 * lane + 64 * chalf;
      sm.col_codes[grp][c] = make_uint4(q0[0], q0[1], q0[2], q0[3]);
      sm.col_codes[grp][c + 1] = make_uint4(q1[0], q1[1], q1[2], q1[3]);
      sm.col_sc[scale_tile_offset(c, grp)] = (uint8_t)e0;
      sm.col_sc[scale_tile_offset(c + 1, grp)] = (uint8_t)e1;
    }
    if constexpr (NORM) {
      if (tid < kMxChunk) sm.inv_rms[pp ^ 1][tid] = pre;
      else sm.gamma[pp ^ 1][tid - kMxChunk] = pre;
    }
    __syncthreads();
    if (tid == 0 && it + kMxStages < my_count) {
      fence_proxy_async_smem();
      issue_load(it + kMxStages, s);
    }
    if (tid < 128) {
      if (a.row_fp4 != nullptr) {
        uint8_t* dst = a.row_sc + ((size_t)cm * a.chunks_k + ck) * 512;
        st_cs_u32(dst + tid * 4, *reinterpret_cast<const uint32_t*>(&sm.row_sc[pp][tid * 4]));
      }
    } else if (want_col) {
      uint8_t* dst = a.col_sc + ((size_t)ck * a.chunks_m + cm) * 512;
      const int t = tid - 128;
      st_cs_u32(dst + t * 4, *reinterpret_cast<const uint32_t*>(&sm.col_sc[t * 4]));
    }
    if (want_col) {
#pragma unroll
      for (int rep = 0; rep < 2; ++rep) {
        const int idx = rep * kMxThreads + tid;   // 512 pieces of 16 bytes: column = idx/4, 32-row group = idx%4
        const int c = idx >> 2, g = idx & 3;
        st_cs_u4(a.col_fp4 + (size_t)(k0 + c) * (a.M >> 1) + (m0 >> 1) + g * 16, sm.col_codes[g][c]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// One-pass SwiGLU producers: the activation is computed on the chunk in shared memory
// ---------------------------------------------------------------------------------------
//
// MXFP4 has no tensor-level scale, so bf16(silu(h1) * h3) (ACT 1) or the pair dh1 = bf16(dh * h3 * silu'(h1)),
// dh3 = bf16(dh * silu(h1)) (ACT 2) never has to exist in HBM: the inputs' chunks arrive by TMA, the row pass
// computes the product(s) on its way through the chunk (the thread that quantises a 32-element row block computes
// it, and writes the bf16 values back IN PLACE for the column pass), and only codes and scales are written:
// 5.06 instead of 9.06 bytes per element (ACT 1), 8.1 instead of 16.1 (ACT 2).  As the reference's fused producers
// (mxfp4_v4/tk_quantize.cu:3231-3310, 4513-4700), which keep the product in shared memory too.  Geometry of the
// passes as in mxfp4_quantize_kernel; three chunk buffers per CTA, two CTAs per SM:
//   ACT 1: h1 of chunk i alternates between buffers 0 / 1 and becomes h; h3 always sits in buffer 2, which is free
//          again after the row pass (h3 of chunk i+1 is then requested) while h1 of chunk i+1 was requested a chunk
//          earlier;
//   ACT 2: dh -> buffer 0 (becomes dh1), h3 -> buffer 1 (becomes dh3), h1 -> buffer 2; each buffer is refilled for the
//          next chunk as soon as its last reader is past it (the other CTA of the SM covers the rest of the latency).
struct MxActSmem {
  alignas(1024) uint8_t buf[3][kMxTileBytes];
  alignas(16) uint4 col_codes[4][kMxChunk];
  alignas(16) uint8_t row_sc[2][2][512];   // [output][parity of the chunk]
  alignas(16) uint8_t col_sc[512];
  alignas(8) uint64_t full[3];
};

struct MxActArgs {
  uint8_t* row_fp4[2];   // [M, H/2] per output (ACT 1: one output)
  uint8_t* row_sc[2];    // [M/128, H/128, 512]
  uint8_t* col_fp4[2];   // [H, M/2]
  uint8_t* col_sc[2];    // [H/128, M/128, 512]
  int* status;
  int M, K, chunks_m, chunks_k;
  int mode;
  int row_pitch_bytes;   // pitch of the row-wise code matrices (K/2, or the width of the matrix they are column slices of)
  int row_sc_row_tiles;  // 512-byte scale tiles from one 128-row block of row_sc to the next (K/128, or the wider tensor's)
};

// one 32-element row block held as sixteen bf16x2 words: scale byte and 16 bytes of codes
__device__ __forceinline__ uint4 mx_row_block(const uint32_t (&w)[16], int mode, uint32_t& e) {
  uint32_t mx = 0;
#pragma unroll
  for (int q = 0; q < 16; ++q) mx = absmax_xs(mx, w[q]);
  const float b = fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx)));
  e = mx_e8m0(b, mode);
  const float coeff = mx_coeff(e);
  uint4 codes;
  codes.x = quant8(w, coeff); codes.y = quant8(w + 4, coeff);
  codes.z = quant8(w + 8, coeff); codes.w = quant8(w + 12, coeff);
  return codes;
}

// column pass of one warp over its 32 rows x 64 columns of a chunk (lane = two adjacent columns)
__device__ __forceinline__ void mx_col_pass(const uint8_t* tile, int grp, int chalf, int lane, const int (&col_off)[8],
                                            int mode, uint4 (*col_codes)[kMxChunk], uint8_t* col_sc) {
  const uint8_t* base = tile + chalf * kMxHalfBytes + (grp * 32) * 128;
  uint32_t w[32];
  uint32_t mx = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    w[i] = *reinterpret_cast<const uint32_t*>(base + i * 128 + col_off[i & 7]);
    mx = absmax_xs(mx, w[i]);
  }
  const uint32_t e0 = mx_e8m0(fabsf(bf16lo_to_f32(mx)), mode), e1 = mx_e8m0(fabsf(bf16hi_to_f32(mx)), mode);
  const float2 cc = make_float2(mx_coeff(e0), mx_coeff(e1));
  uint32_t q0[4], q1[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    float2 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = mul2(make_float2(bf16lo_to_f32(w[8 * p + i]), bf16hi_to_f32(w[8 * p + i])), cc);
    q0[p] = f32x8_to_e2m1x8(v[0].x, v[1].x, v[2].x, v[3].x, v[4].x, v[5].x, v[6].x, v[7].x);
    q1[p] = f32x8_to_e2m1x8(v[0].y, v[1].y, v[2].y, v[3].y, v[4].y, v[5].y, v[6].y, v[7].y);
  }
  const int c = 2 * lane + 64 * chalf;
  col_codes[grp][c] = make_uint4(q0[0], q0[1], q0[2], q0[3]);
  col_codes[grp][c + 1] = make_uint4(q1[0], q1[1], q1[2], q1[3]);
  col_sc[scale_tile_offset(c, grp)] = (uint8_t)e0;
  col_sc[scale_tile_offset(c + 1, grp)] = (uint8_t)e1;
}

template <int ACT>
__global__ void __launch_bounds__(kMxThreads, 2)
mxfp4_act_quantize_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_c, const MxActArgs a) {
  static_assert(ACT == 1 || ACT == 2, "ACT 1: silu(h1) * h3 from (a = h1, b = h3); ACT 2: dh1, dh3 from (a = dh, b = h3, c = h1)");
  constexpr int kOut = ACT;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  MxActSmem& sm = *reinterpret_cast<MxActSmem*>(smem_align_1024(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_chunks = a.chunks_m * a.chunks_k;
  const int first = blockIdx.x, step = gridDim.x;
  const int my_count = first < n_chunks ? (n_chunks - first + step - 1) / step : 0;
  auto chunk_coords = [&](int it, int& cm, int& ck) {
    const int c = first + it * step;
    cm = c / a.chunks_k;
    ck = c - cm * a.chunks_k;
  };
  auto issue_load = [&](int it, int b, const CUtensorMap* map) {
    int cm, ck;
    chunk_coords(it, cm, ck);
    mbar_expect_tx(&sm.full[b], kMxTileBytes);
    tma_load_2d(sm.buf[b], map, ck * kMxChunk, cm * kMxChunk, &sm.full[b]);
    tma_load_2d(sm.buf[b] + kMxHalfBytes, map, ck * kMxChunk + 64, cm * kMxChunk, &sm.full[b]);
  };
  if (tid == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (ACT == 2) tma_prefetch_desc(&tmap_c);
    for (int b = 0; b < 3; ++b) mbar_init(&sm.full[b], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0 && my_count > 0) {
    if (ACT == 1) {
      issue_load(0, 0, &tmap_a);
      issue_load(0, 2, &tmap_b);
      if (my_count > 1) issue_load(1, 1, &tmap_a);
    } else {
      issue_load(0, 0, &tmap_a);
      issue_load(0, 1, &tmap_b);
      issue_load(0, 2, &tmap_c);
    }
  }
  const int unit = lane >> 3, r_lo = lane & 7;
  const int half_off = (unit >> 1) * kMxHalfBytes, cb = (unit & 1) * 4;
  int row_off[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) row_off[j] = ((cb + j) ^ r_lo) << 4;
  int col_off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) col_off[j] = (((lane >> 2) ^ j) << 4) + (lane & 3) * 4;
  const int grp = warp >> 1, chalf = warp & 1;
  uint32_t phase[3] = {0, 0, 0};

  // scale tiles and column codes of one output, from shared memory to their places
  auto store_col = [&](int o, int cm, int ck, int m0, int k0) {
    if (tid >= 128) {
      uint8_t* dst = a.col_sc[o] + ((size_t)ck * a.chunks_m + cm) * 512;
      const int t = tid - 128;
      st_cs_u32(dst + t * 4, *reinterpret_cast<const uint32_t*>(&sm.col_sc[t * 4]));
    }
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int idx = rep * kMxThreads + tid;
      const int c = idx >> 2, g = idx & 3;
      st_cs_u4(a.col_fp4[o] + (size_t)(k0 + c) * (a.M >> 1) + (m0 >> 1) + g * 16, sm.col_codes[g][c]);
    }
  };

  for (int it = 0; it < my_count; ++it) {
    int cm, ck;
    chunk_coords(it, cm, ck);
    const int m0 = cm * kMxChunk, k0 = ck * kMxChunk, pp = it & 1;
    const int bx = ACT == 1 ? (it & 1) : 0;       // buffer whose contents become the (first) output
    const int by = ACT == 1 ? 2 : 1;              // h3; ACT 2: becomes the second output
    bool ok = mbar_wait_bounded(&sm.full[bx], phase[bx]) && mbar_wait_bounded(&sm.full[by], phase[by]);
    if (ACT == 2) ok = ok && mbar_wait_bounded(&sm.full[2], phase[2]);
    if (!ok) {
      if (tid == 0) atomicExch(a.status, kStatusQuantTmaTimeout);
      return;
    }
    phase[bx] ^= 1; phase[by] ^= 1;
    if (ACT == 2) phase[2] ^= 1;
    uint8_t* tx = sm.buf[bx];
    uint8_t* ty = sm.buf[by];
    // ---- activation + row pass
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int r = warp * 16 + rep * 8 + r_lo;
      const int ro = half_off + r * 128;
      uint32_t w0[16], w1[kOut == 2 ? 16 : 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 va = *reinterpret_cast<const uint4*>(tx + ro + row_off[j]);
        const uint4 vb = *reinterpret_cast<const uint4*>(ty + ro + row_off[j]);
        const uint32_t aw[4] = {va.x, va.y, va.z, va.w}, bw[4] = {vb.x, vb.y, vb.z, vb.w};
        if constexpr (ACT == 1) {
          uint32_t o[4];
          silu_mul_bf16x8(aw, bw, o);
#pragma unroll
          for (int q = 0; q < 4; ++q) w0[4 * j + q] = o[q];
        } else {
          const uint4 vc = *reinterpret_cast<const uint4*>(sm.buf[2] + ro + row_off[j]);
          const uint32_t cw[4] = {vc.x, vc.y, vc.z, vc.w};
          uint32_t o1[4], o3[4];
          silu_deriv_bf16x8(aw, bw, cw, o1, o3);
#pragma unroll
          for (int q = 0; q < 4; ++q) { w0[4 * j + q] = o1[q]; w1[4 * j + q] = o3[q]; }
          *reinterpret_cast<uint4*>(ty + ro + row_off[j]) = make_uint4(w1[4 * j], w1[4 * j + 1], w1[4 * j + 2], w1[4 * j + 3]);
        }
        *reinterpret_cast<uint4*>(tx + ro + row_off[j]) = make_uint4(w0[4 * j], w0[4 * j + 1], w0[4 * j + 2], w0[4 * j + 3]);
      }
      uint32_t e;
      const size_t at = (size_t)(m0 + r) * a.row_pitch_bytes + ((k0 + unit * 32) >> 1);
      st_cs_u4(a.row_fp4[0] + at, mx_row_block(w0, a.mode, e));
      sm.row_sc[0][pp][scale_tile_offset(r, unit)] = (uint8_t)e;
      if constexpr (ACT == 2) {
        st_cs_u4(a.row_fp4[1] + at, mx_row_block(w1, a.mode, e));
        sm.row_sc[1][pp][scale_tile_offset(r, unit)] = (uint8_t)e;
      }
    }
    __syncthreads();
    if (tid == 0 && it + 1 < my_count) {
      fence_proxy_async_smem();
      if (ACT == 1) issue_load(it + 1, 2, &tmap_b);    // h3 is consumed
      else issue_load(it + 1, 2, &tmap_c);             // h1 is consumed
    }
    if (tid < 128) {
#pragma unroll
      for (int o = 0; o < kOut; ++o)
        st_cs_u32(a.row_sc[o] + ((size_t)cm * a.row_sc_row_tiles + ck) * 512 + tid * 4,
                  *reinterpret_cast<const uint32_t*>(&sm.row_sc[o][pp][tid * 4]));
    }
    // ---- column pass(es)
    mx_col_pass(tx, grp, chalf, lane, col_off, a.mode, sm.col_codes, sm.col_sc);
    __syncthreads();
    if (tid == 0) {
      fence_proxy_async_smem();
      if (ACT == 1) { if (it + 2 < my_count) issue_load(it + 2, bx, &tmap_a); }
      else if (it + 1 < my_count) issue_load(it + 1, 0, &tmap_a);
    }
    store_col(0, cm, ck, m0, k0);
    if constexpr (ACT == 2) {
      __syncthreads();   // the first output's column codes have left shared memory
      mx_col_pass(ty, grp, chalf, lane, col_off, a.mode, sm.col_codes, sm.col_sc);
      __syncthreads();
      if (tid == 0 && it + 1 < my_count) {
        fence_proxy_async_smem();
        issue_load(it + 1, 1, &tmap_b);
      }
      store_col(1, cm, ck, m0, k0);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Row quantiser with stochastic rounding (of the codes and / or of the E8M0 scale byte)
// ---------------------------------------------------------------------------------------
//
// One thread per 16 contiguous elements, two adjacent threads per 32-block.  The random words follow the
// reference kernel (mxfp4_v3_quantize.cuh:1618-1790, launched by tk_quantize.cu:1796-1846): its 128 threads
// walk a 128x128 chunk as four 64x64 tiles, a thread (tid_Y = row % 32, tid_X = 16-column segment) owning the
// rows tid_Y and tid_Y + 32 of a tile; its Philox stream (subsequence base + ((chunk * 4 + tile) * 128 + thread),
// offset 0) yields, per row, one word for the scale byte (scale SR) and then four words for the codes (data
// SR), the two 8-element halves taken in swapped order by the upper half-warp.  Every thread rounds the scale
// of its block with its OWN word: the byte stored is the even segment's, while the odd segment's codes use the
// odd thread's byte, as in the reference.
struct MxSrArgs {
  const __nv_bfloat16* x;
  uint8_t* row_fp4;   // [M, K/2]
  uint8_t* row_sc;    // [M/128, K/128, 512]
  int64_t M, K;
  int mode, data_sr, scale_sr;
  unsigned long long seed, subseq;
  int correlated;     // row + column launch: the codes round with the position's shared 16-bit integer (below)
  int rht_block;      // 0, or 16 / 32: Hadamard transform of that many consecutive elements along the quantised axis
  int rht_sign;       // the reference's fixed sign diagonal (bit i of 0x2817 set: +1) in front of the transform
  int row_rht, col_rht;
  uint8_t* col_fp4;   // [K, M/2]            (column kernel)
  uint8_t* col_sc;    // [K/128, M/128, 512]
};

// Rounding words of 16 consecutive elements of a row (ROW_VECTOR) or column such that both views of element
// (i, j) add the same 16-bit integer (reference: mxfp4_correlated_sr_rbits16, mxfp4_v3_quantize.cuh:1375-1432).
// A hash of (base, i >> 4, j >> 4) gives two GF(2^16) elements (a, b) per 16x16 tile; the 2x2 cell (i >> 1, j >> 1)
// rounds with the field b + a * p, p the polynomial with bits (j >> 1) | (i >> 1) << 3.  A word carries two fields in
// the byte order cvt.rs.satfinite.e2m1x4.f32 reads them: elements 0 and 2 of its group of four add fields 2k and
// 2k+1, elements 1 and 3 the same fields bit-reversed.
__device__ __forceinline__ uint32_t gf16_times_x(uint32_t v) { return ((v << 1) & 0xFFFFu) ^ ((0u - (v >> 15)) & 0x100Bu); }

template <bool ROW_VECTOR>
__device__ __forceinline__ uint4 mx_correlated_words(unsigned long long base, uint32_t row, uint32_t col) {
  uint32_t t = (uint32_t)base ^ (uint32_t)(base >> 32);
  t ^= (row >> 4) * 0x9E3779B9u;
  t ^= (col >> 4) * 0x85EBCA6Bu;
  t ^= t >> 16; t *= 0x7FEB352Du;
  t ^= t >> 15; t *= 0x846CA68Bu;
  t ^= t >> 16;
  uint32_t ap[6];
  ap[0] = t & 0xFFFFu;
#pragma unroll
  for (int i = 1; i < 6; ++i) ap[i] = gf16_times_x(ap[i - 1]);
  const uint32_t grp = ((ROW_VECTOR ? row : col) & 14u) >> 1;
  constexpr int fixed = ROW_VECTOR ? 3 : 0, step = ROW_VECTOR ? 0 : 3;
  uint32_t f0 = t >> 16;
#pragma unroll
  for (int b = 0; b < 3; ++b) f0 ^= ap[fixed + b] & (0u - ((grp >> b) & 1u));
  uint32_t f[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) f[m] = f0 ^ ((m & 1) ? ap[step] : 0u) ^ ((m & 2) ? ap[step + 1] : 0u) ^ ((m & 4) ? ap[step + 2] : 0u);
  auto pack = [](uint32_t ef, uint32_t ab) { return ((ab & 0xFF00u) << 16) | ((ef & 0xFF00u) << 8) | ((ab & 0xFFu) << 8) | (ef & 0xFFu); };
  return make_uint4(pack(f[0], f[1]), pack(f[2], f[3]), pack(f[4], f[5]), pack(f[6], f[7]));
}

// 16 bf16 values (eight packed words) times coeff -> 8 bytes of codes, stochastic rounding with one word per group
// of four; swap: neighbours exchanged before the conversion and their codes exchanged back after it
__device__ __forceinline__ uint2 mx_quant16_sr(const uint32_t (&w)[8], float coeff, const uint32_t (&wsel)[4], bool swap) {
  uint32_t h[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const float v0 = bf16lo_to_f32(w[2 * g]) * coeff, v1 = bf16hi_to_f32(w[2 * g]) * coeff;
    const float v2 = bf16lo_to_f32(w[2 * g + 1]) * coeff, v3 = bf16hi_to_f32(w[2 * g + 1]) * coeff;
    const uint32_t c = swap ? f32x4_to_e2m1x4_sr(v1, v0, v3, v2, wsel[g]) : f32x4_to_e2m1x4_sr(v0, v1, v2, v3, wsel[g]);
    h[g] = swap ? (((c & 0xF0F0u) >> 4) | ((c & 0x0F0Fu) << 4)) : c;
  }
  return make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
}

constexpr unsigned long long kMxCorrelatedSalt = 0xA0761D6478BD642Full;
constexpr uint32_t kMxRhtSignBits = 0x00002817u;   // make_rht_sign_bits, mxfp4_v3_quantize.cuh:1461-1476

// Signs and the 16-point butterflies (steps 1, 2, 4, 8; sum to the low index, difference to the high one), not yet
// normalised (reference: apply_block_rht_registers / fwht16_unnormalized, mxfp4_v3_quantize.cuh:1478-1530).
__device__ __forceinline__ void mx_fwht16(float (&v)[16], bool sign) {
  if (sign) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= ((kMxRhtSignBits >> i) & 1u) ? 1.0f : -1.0f;
  }
#pragma unroll
  for (int step = 1; step < 16; step <<= 1) {
#pragma unroll
    for (int base = 0; base < 16; base += 2 * step) {
#pragma unroll
      for (int j = 0; j < step; ++j) {
        const float p = v[base + j], q = v[base + j + step];
        v[base + j] = p + q;
        v[base + j + step] = p - q;
      }
    }
  }
}

// Last stage of the 32-point transform (first half: own + peer, second half: peer - own) and the normalisation
__device__ __forceinline__ void mx_rht_finish(float (&v)[16], const float (&peer)[16], int block, int rank) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (block == 32) v[i] = ((rank == 0) ? (v[i] + peer[i]) : (peer[i] - v[i])) * 0.1767766952966369f;
    else v[i] *= 0.25f;
  }
}

__device__ __forceinline__ float mx_amax16(const float (&v)[16]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

__device__ __forceinline__ uint32_t mx_e8m0_sr(float b, uint32_t rbits) {
  if (b <= 1e-38f) return 0;
  const uint32_t u = __float_as_uint(b);
  const uint32_t e = (u >> 23) & 0xFF, m = u & 0x7FFFFF;
  if (m == 0 || e >= 0xFE) return e;
  return ((unsigned long long)rbits < ((unsigned long long)m << 9)) ? e + 1 : e;
}

__global__ void __launch_bounds__(256) mxfp4_quantize_row_sr_kernel(const MxSrArgs a) {
  const int64_t segs_per_row = a.K >> 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // segment index; whole warps are in range
  if (idx >= a.M * segs_per_row) return;
  const int64_t r = idx / segs_per_row;
  const int c = (int)(idx - r * segs_per_row) << 4;
  const uint4* src = reinterpret_cast<const uint4*>(a.x + r * a.K + c);
  const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
  uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  float bm;
  if (a.row_rht) {
    float t[16], peer[16];
#pragma unroll
    for (int q = 0; q < 8; ++q) { t[2 * q] = bf16lo_to_f32(w[q]); t[2 * q + 1] = bf16hi_to_f32(w[q]); }
    mx_fwht16(t, a.rht_sign != 0);
#pragma unroll
    for (int i = 0; i < 16; ++i) peer[i] = __shfl_xor_sync(0xffffffffu, t[i], 1);
    mx_rht_finish(t, peer, a.rht_block, (c >> 4) & 1);
    bm = mx_amax16(t);   // of the transform's fp32 output; the codes come from its bf16 rounding
#pragma unroll
    for (int q = 0; q < 8; ++q) w[q] = f32x2_to_bf16x2(t[2 * q], t[2 * q + 1]);
  } else {
    uint32_t mx = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) mx = absmax_xs(mx, w[q]);
    bm = fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx)));
  }
  bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));

  // the reference thread that owns this segment, and where this row sits in its draw order
  const int rr = (int)(r & 127), cc = c & 127;
  const int tile = (rr >> 6) * 2 + (cc >> 6);
  const int it = (rr & 63) >> 5;
  const int tid_ref = (rr & 31) * 4 + ((cc & 63) >> 4);
  const int bank_group = (tid_ref & 31) >> 4;
  const unsigned long long chunk = (unsigned long long)(r >> 7) * (unsigned long long)(a.K >> 7) + (unsigned long long)(c >> 7);
  const unsigned long long seq = a.subseq + (chunk * 4ull + (unsigned long long)tile) * 128ull + (unsigned long long)tid_ref;
  const int q = (a.scale_sr ? 1 : 0) + ((a.data_sr && !a.correlated) ? 4 : 0);
  uint32_t dr[5];
  philox_draws(a.seed, seq, 0ull, it * q, q, dr);

  const uint32_t e = a.scale_sr ? mx_e8m0_sr(bm, dr[0]) : mx_e8m0(bm, a.mode);
  const float coeff = mx_coeff(e);   // 6 * 2^(127-e): exact in bf16, as the reference rounds it
  uint32_t lo, hi;
  if (a.data_sr) {
    uint32_t wsel[4];
    if (a.correlated) {
      const uint4 cw = mx_correlated_words<true>((a.subseq + chunk * 512ull) ^ a.seed ^ kMxCorrelatedSalt, (uint32_t)r, (uint32_t)c);
      wsel[0] = cw.x; wsel[1] = cw.y; wsel[2] = cw.z; wsel[3] = cw.w;
    } else {
      const int d0 = a.scale_sr ? 1 : 0;
#pragma unroll
      for (int g = 0; g < 4; ++g) wsel[g] = (((g >> 1) - bank_group) & 1) ? dr[d0 + 2 + (g & 1)] : dr[d0 + (g & 1)];
    }
    const uint2 cd = mx_quant16_sr(w, coeff, wsel, a.correlated && (r & 1));
    lo = cd.x;
    hi = cd.y;
  } else {
    lo = quant8(w, coeff);
    hi = quant8(w + 4, coeff);
  }
  *reinterpret_cast<uint2*>(a.row_fp4 + r * (a.K >> 1) + (c >> 1)) = make_uint2(lo, hi);
  if (((c >> 4) & 1) == 0)
    a.row_sc[((size_t)(r >> 7) * (size_t)(a.K >> 7) + (size_t)(c >> 7)) * 512 + scale_tile_offset(rr, cc >> 5)] = (uint8_t)e;
}

// Column view of the row + column launch (reference: mx_colwise_quantize_direct_opt, mxfp4_v3_quantize.cuh:4031-4230,
// called by quantize_chunk_rowcol_pipelined_opt, 3321-3430).  One thread per (16 rows, two adjacent columns), as the
// reference thread; it reads the partner's 16 rows as well for the 32-row block maximum.  Scale SR: draws 0 and 1 of
// the thread's stream (subsequence base + ((column-view chunk * 4 + tile) * 128 + thread)) for its two columns.
__global__ void __launch_bounds__(256) mxfp4_quantize_col_sr_kernel(const MxSrArgs a) {
  const int64_t pairs = a.K >> 1;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (a.M >> 4) * pairs) return;
  const int64_t g16 = idx / pairs;
  const int j = (int)(idx - g16 * pairs) << 1;   // first of the two columns
  const int64_t i0 = g16 << 4;
  const uint32_t* own = reinterpret_cast<const uint32_t*>(a.x + i0 * a.K + j);
  const uint32_t* other = reinterpret_cast<const uint32_t*>(a.x + (i0 ^ 16) * a.K + j);
  const int64_t ld = a.K >> 1;   // row pitch in 32-bit words
  uint32_t v[16];
  float bm0, bm1;
  if (a.col_rht) {
    // both halves of the 32-row block are transformed here: the partner's output is needed for the block maximum
    // (and, for 32-point blocks, its butterflies for this half's last stage)
    const int rank = (int)(i0 >> 4) & 1;
    float bm[2];
#pragma unroll
    for (int cpar = 0; cpar < 2; ++cpar) {
      float t[16], u[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t wo = __ldg(own + i * ld), wp = __ldg(other + i * ld);
        t[i] = cpar ? bf16hi_to_f32(wo) : bf16lo_to_f32(wo);
        u[i] = cpar ? bf16hi_to_f32(wp) : bf16lo_to_f32(wp);
      }
      mx_fwht16(t, a.rht_sign != 0);
      mx_fwht16(u, a.rht_sign != 0);
      float tt[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) tt[i] = t[i];
      mx_rht_finish(t, u, a.rht_block, rank);
      mx_rht_finish(u, tt, a.rht_block, rank ^ 1);
      bm[cpar] = fmaxf(mx_amax16(t), mx_amax16(u));
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t h = f32x2_to_bf16x2(t[i], 0.0f) & 0xFFFFu;
        v[i] = cpar ? (v[i] | (h << 16)) : h;
      }
    }
    bm0 = bm[0];
    bm1 = bm[1];
  } else {
    uint32_t mx = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] = __ldg(own + i * ld);
      mx = absmax_xs(mx, v[i]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) mx = absmax_xs(mx, __ldg(other + i * ld));
    bm0 = fabsf(bf16lo_to_f32(mx));
    bm1 = fabsf(bf16hi_to_f32(mx));
  }

  const int jj = j & 127, ii = (int)(i0 & 127);
  const int tile = (jj >> 6) * 2 + (ii >> 6);
  const int tx = (jj & 63) >> 1, ty = (ii & 63) >> 4;
  const int tid_ref = ((tx >> 4) * 2 + (ty >> 1)) * 32 + (ty & 1) * 16 + (tx & 15);
  const unsigned long long chunk_col = (unsigned long long)(j >> 7) * (unsigned long long)(a.M >> 7) + (unsigned long long)(i0 >> 7);
  const unsigned long long chunk_in = (unsigned long long)(i0 >> 7) * (unsigned long long)(a.K >> 7) + (unsigned long long)(j >> 7);
  uint32_t e0, e1;
  const unsigned long long seq = a.subseq + (chunk_col * 4ull + (unsigned long long)tile) * 128ull + (unsigned long long)tid_ref;
  if (a.scale_sr) {
    const uint4 rw = philox4x32_10(a.seed, seq, 0ull);
    e0 = mx_e8m0_sr(bm0, rw.x);
    e1 = mx_e8m0_sr(bm1, rw.y);
  } else {
    e0 = mx_e8m0(bm0, a.mode);
    e1 = mx_e8m0(bm1, a.mode);
  }
  // the two columns as packed pairs of consecutive rows
  uint32_t c0[8], c1[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    c0[q] = __byte_perm(v[2 * q], v[2 * q + 1], 0x5410);
    c1[q] = __byte_perm(v[2 * q], v[2 * q + 1], 0x7632);
  }
  uint2 o0, o1;
  if (a.data_sr && a.correlated) {
    const unsigned long long base = (a.subseq + chunk_in * 512ull) ^ a.seed ^ kMxCorrelatedSalt;
    const uint4 w0 = mx_correlated_words<false>(base, (uint32_t)i0, (uint32_t)j);
    const uint4 w1 = mx_correlated_words<false>(base, (uint32_t)i0, (uint32_t)j + 1u);
    const uint32_t ws0[4] = {w0.x, w0.y, w0.z, w0.w}, ws1[4] = {w1.x, w1.y, w1.z, w1.w};
    o0 = mx_quant16_sr(c0, mx_coeff(e0), ws0, false);   // j is even
    o1 = mx_quant16_sr(c1, mx_coeff(e1), ws1, true);
  } else if (a.data_sr) {
    // the thread's own stream: after the two scale words (scale SR), four words for each of its two columns
    const int d0 = a.scale_sr ? 2 : 0;
    uint32_t da[5], db[5];
    philox_draws(a.seed, seq, 0ull, d0, 4, da);
    philox_draws(a.seed, seq, 0ull, d0 + 4, 4, db);
    const uint32_t ws0[4] = {da[0], da[1], da[2], da[3]}, ws1[4] = {db[0], db[1], db[2], db[3]};
    o0 = mx_quant16_sr(c0, mx_coeff(e0), ws0, false);
    o1 = mx_quant16_sr(c1, mx_coeff(e1), ws1, false);
  } else {
    o0 = make_uint2(quant8(c0, mx_coeff(e0)), quant8(c0 + 4, mx_coeff(e0)));
    o1 = make_uint2(quant8(c1, mx_coeff(e1)), quant8(c1 + 4, mx_coeff(e1)));
  }
  uint8_t* dst = a.col_fp4 + (size_t)j * (size_t)(a.M >> 1) + (size_t)(i0 >> 1);
  *reinterpret_cast<uint2*>(dst) = o0;
  *reinterpret_cast<uint2*>(dst + (a.M >> 1)) = o1;
  if ((i0 & 16) == 0) {
    uint8_t* sdst = a.col_sc + ((size_t)(j >> 7) * (size_t)(a.M >> 7) + (size_t)(i0 >> 7)) * 512;
    sdst[scale_tile_offset(jj, ii >> 5)] = (uint8_t)e0;
    sdst[scale_tile_offset(jj + 1, ii >> 5)] = (uint8_t)e1;
  }
}

static int launch_mx_col_sr(const MxSrArgs& a, cudaStream_t st) {
  const int64_t n = (a.M >> 4) * (a.K >> 1);
  const int64_t blocks = (n + 255) / 256;
  if (blocks == 0) return 0;
  mxfp4_quantize_col_sr_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

static int launch_mx_row_sr(const MxSrArgs& a, cudaStream_t st) {
  const int64_t segs = a.M * (a.K >> 4);
  const int64_t blocks = (segs + 255) / 256;
  if (blocks == 0) return 0;
  mxfp4_quantize_row_sr_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// x1 / x2 with their widths k1 / k2 (elements): further inputs whose columns follow x's (K is the total width).
static int launch_mx(const void* x, int64_t M, int64_t K, int mode, const float* inv_rms, const void* gamma,
                     void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, cudaStream_t st, bool weight_2d = false,
                     const void* x1 = nullptr, int64_t k1 = 0, const void* x2 = nullptr, int64_t k2 = 0,
                     int nhsd_heads = 0, int nhsd_seq = 0, int nhsd_dim = 0, const float* rope_cs = nullptr,
                     int64_t rope_seq_len = 0) {
  const int64_t k0 = K - k1 - k2;
  CUtensorMap tmap, tmap1, tmap2;
  if (int rc = nhsd_seq > 0
                   ? make_tmap_2d(&tmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)nhsd_dim, (uint64_t)M * nhsd_heads,
                                  (uint64_t)nhsd_dim * 2, 64, kMxChunk, CU_TENSOR_MAP_SWIZZLE_128B)
                   : make_tmap_2d(&tmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k0, (uint64_t)M, (uint64_t)k0 * 2,
                                  64, kMxChunk, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  tmap1 = tmap2 = tmap;
  if (x1 != nullptr)
    if (int rc = make_tmap_2d(&tmap1, x1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k1, (uint64_t)M, (uint64_t)k1 * 2,
                              64, kMxChunk, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  if (x2 != nullptr)
    if (int rc = make_tmap_2d(&tmap2, x2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k2, (uint64_t)M, (uint64_t)k2 * 2,
                              64, kMxChunk, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  MxArgs a{};
  a.inv_rms = inv_rms; a.gamma = (const __nv_bfloat16*)gamma;
  a.row_fp4 = (uint8_t*)row_fp4; a.row_sc = (uint8_t*)row_sc; a.col_fp4 = (uint8_t*)col_fp4; a.col_sc = (uint8_t*)col_sc;
  a.status = device_status_ptr();
  if (!a.status) return -1;
  a.M = (int)M; a.K = (int)K; a.chunks_m = (int)(M / kMxChunk); a.chunks_k = (int)(K / kMxChunk); a.mode = mode;
  a.split_chunk[0] = (int)(k0 / kMxChunk);
  a.split_chunk[1] = (int)((k0 + k1) / kMxChunk);
  a.nhsd_heads = nhsd_heads; a.nhsd_seq = nhsd_seq; a.nhsd_dim = nhsd_dim;
  a.rope_cs = reinterpret_cast<const float2*>(rope_cs); a.rope_seq_mask = (int)(rope_seq_len - 1);
  const int smem = (int)sizeof(MxSmem) + 1024;
  const int grid = std::min(a.chunks_m * a.chunks_k, 2 * device_sm_count());
  if (grid == 0) return 0;
  if (rope_cs != nullptr) {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_quantize_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    mxfp4_quantize_kernel<false, false, true><<<grid, kMxThreads, smem, st>>>(tmap, tmap1, tmap2, a);
  } else if (weight_2d) {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_quantize_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    mxfp4_quantize_kernel<false, true><<<grid, kMxThreads, smem, st>>>(tmap, tmap1, tmap2, a);
  } else if (inv_rms) {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_quantize_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    mxfp4_quantize_kernel<true, false><<<grid, kMxThreads, smem, st>>>(tmap, tmap1, tmap2, a);
  } else {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_quantize_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    mxfp4_quantize_kernel<false, false><<<grid, kMxThreads, smem, st>>>(tmap, tmap1, tmap2, a);
  }
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// pitch_*: row pitch of each input in elements (0: K).  combined (ACT 2): the two row-wise code matrices are the left and
// right halves of one [M, K] byte matrix and their scale tiles the left and right halves of one [M/128, 2K/128, 512]
// tensor; else the second output is stacked behind the first in every array.  col_fp4_1 / col_sc_1: the second
// output's column operand, when it is not stacked behind the first's.
static int launch_mx_act(int act, const void* in_a, const void* in_b, const void* in_c, int64_t M, int64_t K, int mode,
                         uint8_t* row_fp4, uint8_t* row_sc, uint8_t* col_fp4, uint8_t* col_sc, cudaStream_t st,
                         int64_t pitch_a = 0, int64_t pitch_b = 0, int64_t pitch_c = 0, bool combined = false,
                         uint8_t* col_fp4_1 = nullptr, uint8_t* col_sc_1 = nullptr) {
  CUtensorMap tm[3];
  const void* src[3] = {in_a, in_b, act == 2 ? in_c : in_a};
  const int64_t pitch[3] = {pitch_a ? pitch_a : K, pitch_b ? pitch_b : K, act == 2 ? (pitch_c ? pitch_c : K) : (pitch_a ? pitch_a : K)};
  for (int i = 0; i < 3; ++i)
    if (int rc = make_tmap_2d(&tm[i], src[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                              (uint64_t)pitch[i] * 2, 64, kMxChunk, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  MxActArgs a{};
  const size_t codes = (size_t)M * K / 2, scales = (size_t)(M / 128) * (K / 128) * 512;
  for (int o = 0; o < 2; ++o) {
    a.row_fp4[o] = row_fp4 + o * (combined ? (size_t)K / 2 : codes);
    a.row_sc[o] = row_sc + o * (combined ? (size_t)(K / 128) * 512 : scales);
    a.col_fp4[o] = col_fp4 + o * codes; a.col_sc[o] = col_sc + o * scales;
  }
  if (col_fp4_1 != nullptr) { a.col_fp4[1] = col_fp4_1; a.col_sc[1] = col_sc_1; }   // column operands in tensors of their own
  a.status = device_status_ptr();
  if (!a.status) return -1;
  a.M = (int)M; a.K = (int)K; a.chunks_m = (int)(M / kMxChunk); a.chunks_k = (int)(K / kMxChunk); a.mode = mode;
  a.row_pitch_bytes = (int)(combined ? K : K / 2);
  a.row_sc_row_tiles = (int)(combined ? 2 * (K / 128) : K / 128);
  const int smem = (int)sizeof(MxActSmem) + 1024;
  const int grid = std::min(a.chunks_m * a.chunks_k, 2 * device_sm_count());
  if (grid == 0) return 0;
  if (act == 1) {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_act_quantize_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    mxfp4_act_quantize_kernel<1><<<grid, kMxThreads, smem, st>>>(tm[0], tm[1], tm[2], a);
  } else {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(mxfp4_act_quantize_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    mxfp4_act_quantize_kernel<2><<<grid, kMxThreads, smem, st>>>(tm[0], tm[1], tm[2], a);
  }
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace fp4b200

using namespace fp4b200;

static int check_mx(const void* x, int64_t M, int64_t K, int mode, const char* who) {
  if (!x) return set_error("%s: input pointer is null", who);
  if (M <= 0 || K <= 0 || (M % 128) || (K % 128))
    return set_error("%s: M and K must be positive multiples of 128 (got %lld x %lld)", who, (long long)M, (long long)K);
  if (mode < 0 || mode > 2) return set_error("%s: mode must be 0 (RTE), 1 (ceil) or 2 (floor)", who);
  if (reinterpret_cast<uintptr_t>(x) & 15) return set_error("%s: input must be 16-byte aligned", who);
  return 0;
}

extern "C" {

int fp4b200_mxfp4_quantize(const void* x_bf16, int64_t M, int64_t K, int mode, void* row_fp4, void* row_sc,
                           void* col_fp4, void* col_sc, void* stream) {
  if (int rc = check_mx(x_bf16, M, K, mode, "mxfp4_quantize")) return rc;
  if ((row_fp4 == nullptr) != (row_sc == nullptr))
    return set_error("mxfp4_quantize: row_fp4 and row_sc must both be given or both be null");
  if (!row_fp4 && !col_fp4) return set_error("mxfp4_quantize: no output was given");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("mxfp4_quantize: col_fp4 and col_sc must both be given or both be null");
  return launch_mx(x_bf16, M, K, mode, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc, (cudaStream_t)stream);
}

int fp4b200_mxfp4_quantize_normed(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M,
                                  int64_t K, int mode, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                  void* stream) {
  if (int rc = check_mx(x_bf16, M, K, mode, "mxfp4_quantize_normed")) return rc;
  if (!gamma_bf16 || !inv_rms || !row_fp4 || !row_sc)
    return set_error("mxfp4_quantize_normed: gamma, inv_rms, row_fp4 and row_sc are required");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("mxfp4_quantize_normed: col_fp4 and col_sc must both be given or both be null");
  return launch_mx(x_bf16, M, K, mode, inv_rms, gamma_bf16, row_fp4, row_sc, col_fp4, col_sc, (cudaStream_t)stream);
}

int fp4b200_mxfp4_quantize_weight_2d(const void* w_bf16, int64_t N, int64_t K, void* row_fp4, void* row_sc,
                                     void* col_fp4, void* col_sc, void* stream) {
  if (int rc = check_mx(w_bf16, N, K, 1, "mxfp4_quantize_weight_2d")) return rc;
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("mxfp4_quantize_weight_2d: all outputs are required");
  return launch_mx(w_bf16, N, K, 1, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc, (cudaStream_t)stream, true);
}

int fp4b200_mxfp4_silu_mul_quantize(const void* h1_raw, const void* h3, int64_t M, int64_t H, int mode, void* row_fp4,
                                    void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  if (int rc = check_mx(h1_raw, M, H, mode, "mxfp4_silu_mul_quantize")) return rc;
  if (int rc = check_mx(h3, M, H, mode, "mxfp4_silu_mul_quantize")) return rc;
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("mxfp4_silu_mul_quantize: all outputs are required");
  return launch_mx_act(1, h1_raw, h3, nullptr, M, H, mode, (uint8_t*)row_fp4, (uint8_t*)row_sc, (uint8_t*)col_fp4,
                       (uint8_t*)col_sc, (cudaStream_t)stream);
}

int fp4b200_mxfp4_quantize_nhsd_wo(const void* x_bf16, int64_t B, int64_t H, int64_t S, int64_t D, int mode, void* row_fp4,
                                   void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  const char* fn = "mxfp4_quantize_nhsd_wo";
  if (B <= 0 || H <= 0 || S <= 0 || D <= 0) return set_error("%s: B, H, S and D must be positive", fn);
  if (D % 64) return set_error("%s: head_dim must be a multiple of 64 (got %lld)", fn, (long long)D);
  if (S % 128) return set_error("%s: the sequence length must be a multiple of 128 (got %lld)", fn, (long long)S);
  if (B * S > INT32_MAX || H * D > INT32_MAX || B * H * S > INT32_MAX) return set_error("%s: dimension too large", fn);
  if (int rc = check_mx(x_bf16, B * S, H * D, mode, fn)) return rc;
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("%s: all four outputs are required", fn);
  return launch_mx(x_bf16, B * S, H * D, mode, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc, (cudaStream_t)stream, false,
                   nullptr, 0, nullptr, 0, (int)H, (int)S, (int)D);
}

int fp4b200_mxfp4_quantize_split(const void* const* xs, const int64_t* widths, int n, int64_t M, int mode, void* row_fp4,
                                 void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  const char* fn = "mxfp4_quantize_split";
  if (!xs || !widths || n < 2 || n > 3) return set_error("%s: two or three inputs are supported", fn);
  int64_t K = 0;
  for (int i = 0; i < n; ++i) {
    if (int rc = check_mx(xs[i], M, widths[i], mode, fn)) return rc;
    K += widths[i];
  }
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("%s: all four outputs are required", fn);
  return launch_mx(xs[0], M, K, mode, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc, (cudaStream_t)stream, false,
                   xs[1], widths[1], n == 3 ? xs[2] : nullptr, n == 3 ? widths[2] : 0);
}

int fp4b200_mxfp4_quantize_split3_inverse_rope(const void* dq, const void* dk, const void* dv, int64_t M, int64_t kq,
                                               int64_t kk, int64_t kv, const float* rope_cs, int64_t rope_seq_len, int mode,
                                               void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  const char* fn = "mxfp4_quantize_split3_inverse_rope";
  if (int rc = check_mx(dq, M, kq, mode, fn)) return rc;
  if (int rc = check_mx(dk, M, kk, mode, fn)) return rc;
  if (int rc = check_mx(dv, M, kv, mode, fn)) return rc;
  if (!rope_cs || (reinterpret_cast<uintptr_t>(rope_cs) & 15)) return set_error("%s: rope_cs must be a 16-byte aligned table", fn);
  if (rope_seq_len <= 0 || (rope_seq_len & (rope_seq_len - 1)))
    return set_error("%s: rope_seq_len must be a positive power of two (got %lld)", fn, (long long)rope_seq_len);
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("%s: all four outputs are required", fn);
  return launch_mx(dq, M, kq + kk + kv, mode, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc, (cudaStream_t)stream, false,
                   dk, kk, dv, kv, 0, 0, 0, rope_cs, rope_seq_len);
}

int fp4b200_mxfp4_silu_mul_quantize_strided(const void* h13, int64_t h13_stride, int64_t h3_offset, int64_t M, int64_t H,
                                            int mode, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  const char* fn = "mxfp4_silu_mul_quantize_strided";
  if (int rc = check_mx(h13, M, H, mode, fn)) return rc;
  if (h3_offset < H || h3_offset + H > h13_stride || (h3_offset % 8) || (h13_stride % 8))
    return set_error("%s: h13 must hold h1 in columns [0, H) and h3 in [h3_offset, h3_offset + H), both 16-byte aligned", fn);
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("%s: all outputs are required", fn);
  const auto* h3 = reinterpret_cast<const uint8_t*>(h13) + (size_t)h3_offset * 2;
  return launch_mx_act(1, h13, h3, nullptr, M, H, mode, (uint8_t*)row_fp4, (uint8_t*)row_sc, (uint8_t*)col_fp4,
                       (uint8_t*)col_sc, (cudaStream_t)stream, h13_stride, h13_stride);
}

int fp4b200_mxfp4_silu_deriv_quantize_split2(const void* dh, const void* h3, const void* h1_raw, int64_t M, int64_t H,
                                             int mode, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                             void* stream) {
  if (int rc = check_mx(dh, M, H, mode, "mxfp4_silu_deriv_quantize_split2")) return rc;
  if (int rc = check_mx(h3, M, H, mode, "mxfp4_silu_deriv_quantize_split2")) return rc;
  if (int rc = check_mx(h1_raw, M, H, mode, "mxfp4_silu_deriv_quantize_split2")) return rc;
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc)
    return set_error("mxfp4_silu_deriv_quantize_split2: all outputs are required");
  return launch_mx_act(2, dh, h3, h1_raw, M, H, mode, (uint8_t*)row_fp4, (uint8_t*)row_sc, (uint8_t*)col_fp4,
                       (uint8_t*)col_sc, (cudaStream_t)stream);
}

int fp4b200_mxfp4_silu_deriv_quantize_split2_combined(const void* dh, int64_t dh_stride, const void* h13, int64_t h13_stride,
                                                      int64_t h3_offset, int64_t M, int64_t H, int mode, void* row_fp4,
                                                      void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  const char* fn = "mxfp4_silu_deriv_quantize_split2_combined";
  if (int rc = check_mx(dh, M, H, mode, fn)) return rc;
  if (int rc = check_mx(h13, M, H, mode, fn)) return rc;
  if (dh_stride < H || (dh_stride % 8)) return set_error("%s: the row stride of dh must cover H and be a multiple of 8", fn);
  if (h3_offset < H || h3_offset + H > h13_stride || (h3_offset % 8) || (h13_stride % 8))
    return set_error("%s: h13 must hold h1 in columns [0, H) and h3 in [h3_offset, h3_offset + H), both 16-byte aligned", fn);
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("%s: all outputs are required", fn);
  const auto* h3 = reinterpret_cast<const uint8_t*>(h13) + (size_t)h3_offset * 2;
  return launch_mx_act(2, dh, h3, h13, M, H, mode, (uint8_t*)row_fp4, (uint8_t*)row_sc, (uint8_t*)col_fp4, (uint8_t*)col_sc,
                       (cudaStream_t)stream, dh_stride, h13_stride, h13_stride, true);
}

int fp4b200_mxfp4_silu_deriv_quantize_split2_splitcols(const void* dh, const void* h3, const void* h1_raw, int64_t M,
                                                       int64_t H, int mode, void* row_fp4, void* row_sc, void* col0_fp4,
                                                       void* col0_sc, void* col1_fp4, void* col1_sc, void* stream) {
  const char* fn = "mxfp4_silu_deriv_quantize_split2_splitcols";
  if (int rc = check_mx(dh, M, H, mode, fn)) return rc;
  if (int rc = check_mx(h3, M, H, mode, fn)) return rc;
  if (int rc = check_mx(h1_raw, M, H, mode, fn)) return rc;
  if (!row_fp4 || !row_sc || !col0_fp4 || !col0_sc || !col1_fp4 || !col1_sc) return set_error("%s: all outputs are required", fn);
  return launch_mx_act(2, dh, h3, h1_raw, M, H, mode, (uint8_t*)row_fp4, (uint8_t*)row_sc, (uint8_t*)col0_fp4,
                       (uint8_t*)col0_sc, (cudaStream_t)stream, 0, 0, 0, true, (uint8_t*)col1_fp4, (uint8_t*)col1_sc);
}

static int check_mx_rht(int rht_block, const char* who) {
  if (rht_block != 0 && rht_block != 16 && rht_block != 32) return set_error("%s: RHT block size must be 16 or 32 (0: no transform)", who);
  return 0;
}

int fp4b200_mxfp4_quantize_row_sr(const void* x_bf16, int64_t M, int64_t K, int mode, int data_sr, int scale_sr,
                                  int rht_block, int rht_sign, uint64_t rng_seed, uint64_t rng_subsequence, void* row_fp4,
                                  void* row_sc, void* stream) {
  if (int rc = check_mx(x_bf16, M, K, mode, "mxfp4_quantize_row_sr")) return rc;
  if (int rc = check_mx_rht(rht_block, "mxfp4_quantize_row_sr")) return rc;
  if (!row_fp4 || !row_sc) return set_error("mxfp4_quantize_row_sr: row_fp4 and row_sc are required");
  if (reinterpret_cast<uintptr_t>(row_fp4) & 7) return set_error("mxfp4_quantize_row_sr: row_fp4 must be 8-byte aligned");
  if (M * (K >> 4) > (int64_t)0x7fffffff * 256) return set_error("mxfp4_quantize_row_sr: tensor too large");
  MxSrArgs a{};
  a.x = reinterpret_cast<const __nv_bfloat16*>(x_bf16); a.row_fp4 = (uint8_t*)row_fp4; a.row_sc = (uint8_t*)row_sc;
  a.M = M; a.K = K; a.mode = mode; a.data_sr = data_sr != 0; a.scale_sr = scale_sr != 0;
  a.seed = rng_seed; a.subseq = rng_subsequence;
  a.rht_block = rht_block; a.rht_sign = rht_sign != 0; a.row_rht = rht_block != 0;
  return launch_mx_row_sr(a, (cudaStream_t)stream);
}

int fp4b200_mxfp4_quantize_row_and_col_sr(const void* x_bf16, int64_t M, int64_t K, int mode, int data_sr, int scale_sr,
                                          int rht_block, int rht_sign, int row_rht, int col_rht, uint64_t rng_seed,
                                          uint64_t rng_subsequence, void* row_fp4, void* row_sc, void* col_fp4,
                                          void* col_sc, void* stream) {
  if (int rc = check_mx(x_bf16, M, K, mode, "mxfp4_quantize_row_and_col_sr")) return rc;
  if (int rc = check_mx_rht(rht_block, "mxfp4_quantize_row_and_col_sr")) return rc;
  if ((rht_block == 0) != (!row_rht && !col_rht))
    return set_error("mxfp4_quantize_row_and_col_sr: a transform needs a block size and at least one axis");
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc) return set_error("mxfp4_quantize_row_and_col_sr: all four outputs are required");
  if ((reinterpret_cast<uintptr_t>(row_fp4) | reinterpret_cast<uintptr_t>(col_fp4)) & 7)
    return set_error("mxfp4_quantize_row_and_col_sr: code outputs must be 8-byte aligned");
  if (M * (K >> 4) > (int64_t)0x7fffffff * 128) return set_error("mxfp4_quantize_row_and_col_sr: tensor too large");
  MxSrArgs a{};
  a.x = reinterpret_cast<const __nv_bfloat16*>(x_bf16); a.row_fp4 = (uint8_t*)row_fp4; a.row_sc = (uint8_t*)row_sc;
  a.col_fp4 = (uint8_t*)col_fp4; a.col_sc = (uint8_t*)col_sc;
  a.M = M; a.K = K; a.mode = mode; a.data_sr = data_sr != 0; a.scale_sr = scale_sr != 0;
  a.rht_block = rht_block; a.rht_sign = rht_sign != 0; a.row_rht = row_rht != 0; a.col_rht = col_rht != 0;
  a.correlated = a.data_sr && !a.row_rht && !a.col_rht;   // with a transform both views draw from their Philox streams
  a.seed = rng_seed; a.subseq = rng_subsequence;
  if (int rc = launch_mx_row_sr(a, (cudaStream_t)stream)) return rc;
  return launch_mx_col_sr(a, (cudaStream_t)stream);
}

}  // extern "C"
