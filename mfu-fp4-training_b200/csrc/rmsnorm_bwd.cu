// RMSNorm backward right behind the dgrad GEMMs: dx (optionally of the sum of three gradient streams,
// optionally plus the residual stream's gradient) and the norm weight's gradient through fixed row
// tiles, so that the result does not depend on scheduling.
//   sum3_rmsnorm_bwd_out        ThunderKittens/kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:196-252 (dx, any K),
//                               :254-323 (dx, K = 4096), :382-430 (dgamma tiles + reduction), :432-562 (entry)
//   rmsnorm_bwd_residual_out    nvfp4_b200_gemm.cu:325-380 (kernel), :564-646 (entry)
// Arithmetic restated from those kernels (compiled there with fused multiply-add contraction on):
//   dy      = bf16(bf16(d0 + d1) + d2)                      (sum3)   |  d_normed            (residual)
//   s(t)    = fma(dy, (x*inv)*gamma, s(t)) over the columns t, t+B, t+2B, ... of "thread" t in turn,
//             B = 512 (sum3) | 256 (residual)
//   S       = block sum of s(t): inside every 32 threads the balanced tree of a shuffle-down reduction,
//             then the warp sums added one after another in warp order (cub::BlockReduce, warp reductions)
//   mean    = S / K
//   dx      = bf16(inv * fma(dy, gamma, -((x*inv)*mean)))   [residual: bf16(dx + residual)]
//   tile[c] = fma(dy*x, inv, tile[c]) over the tile's 256 rows in turn;  dgamma[c] = tiles added in turn
// The residual form of the reference adds dgamma with atomics (order not fixed); here it goes through
// the same row tiles, which is one of the orders the atomics may take.
#include "fp4_common.cuh"
#include "host_util.h"

#include <cuda_bf16.h>

#include <cstdlib>

namespace fp4b200 {

constexpr int kBwdRowTile = 256;      // rows per dgamma tile (fixed by the layout of dgamma_partials)
constexpr int kBwdMaxVec = 32;        // 16-byte vectors per lane and row: K <= 8192 (kernels are built for 16 and 32)

__device__ __forceinline__ uint32_t bf16x2_add(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// One CTA per SM with a ring of row slots in shared memory; a slot holds one row of every input
// stream (sum3: d0 | d1 | d2 | x; residual: dy | x | residual), brought in by one bulk copy per stream.
// A warp claims the band's next row, computes dy in place, the row sum in the summation order of the
// reference's B-thread block, then dx in place over a stream it has consumed, and sends the finished
// rows back with bulk copies before it refills the slot.  Lane L holds columns 8L + 256j + e
// (j = vector index, e = 0..7), i.e. "threads" t = (8L + e) mod B: for B = 512 the vectors of even j
// belong to t < 256 and those of odd j to t >= 256, and ascending j walks a thread's columns in order.
//
// FUSE_DGAMMA: the CTA's rows are interleaved over the grid (row = CTA + i * CTAs) so that all CTAs sweep
// the matrix together, every finished row is counted on its 256-row tile, and kDgammaWarps extra warps per
// CTA turn finished tiles into dgamma partials inside the same launch, filling the bandwidth the dx warps
// leave (no second launch, no tail of its own).  The second pass over dy and x still mostly reaches HBM:
// at this streaming rate a line stays in L2 for some ten microseconds, less than a 256-row column chain of
// dependent round trips takes.  Those warps wait (bounded) on other CTAs' progress, so the grid must be
// co-resident: the kernel is then launched cooperatively with at most one CTA per SM.  The dx warps never
// wait on anything but their own copies.
constexpr int kDgammaWarps = 4;
constexpr int kDgammaRows = 16;     // rows requested ahead per column chain

__device__ __forceinline__ uint2 ld_cg_u2(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.cg.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One dgamma chain segment: rows [row, row + n) of 4 columns, in turn.
__device__ __forceinline__ void dgamma_rows(const uint2* dp, const uint2* xp, size_t pitch, const float* __restrict__ inv_rms,
                                            int row, int n, float (&p)[4]) {
  int i = 0;
#pragma unroll 1
  for (; i + kDgammaRows <= n; i += kDgammaRows) {
    uint2 dv[kDgammaRows], xv[kDgammaRows];
#pragma unroll
    for (int u = 0; u < kDgammaRows; ++u) {
      dv[u] = ld_cg_u2(dp + (size_t)(i + u) * pitch);
      xv[u] = ld_cg_u2(xp + (size_t)(i + u) * pitch);
    }
#pragma unroll
    for (int u = 0; u < kDgammaRows; ++u) {
      const float iv = __ldg(inv_rms + row + i + u);
      p[0] = fmaf(bf16lo_to_f32(dv[u].x) * bf16lo_to_f32(xv[u].x), iv, p[0]);
      p[1] = fmaf(bf16hi_to_f32(dv[u].x) * bf16hi_to_f32(xv[u].x), iv, p[1]);
      p[2] = fmaf(bf16lo_to_f32(dv[u].y) * bf16lo_to_f32(xv[u].y), iv, p[2]);
      p[3] = fmaf(bf16hi_to_f32(dv[u].y) * bf16hi_to_f32(xv[u].y), iv, p[3]);
    }
  }
  for (; i < n; ++i) {
    const uint2 d = ld_cg_u2(dp + (size_t)i * pitch), xx = ld_cg_u2(xp + (size_t)i * pitch);
    const float iv = __ldg(inv_rms + row + i);
    p[0] = fmaf(bf16lo_to_f32(d.x) * bf16lo_to_f32(xx.x), iv, p[0]);
    p[1] = fmaf(bf16hi_to_f32(d.x) * bf16hi_to_f32(xx.x), iv, p[1]);
    p[2] = fmaf(bf16lo_to_f32(d.y) * bf16lo_to_f32(xx.y), iv, p[2]);
    p[3] = fmaf(bf16hi_to_f32(d.y) * bf16hi_to_f32(xx.y), iv, p[3]);
  }
}

template <bool SUM3, bool FUSE_DGAMMA, int MAXV /* vectors per lane the row loops are unrolled for */>
__global__ void __launch_bounds__((8 + kDgammaWarps) * 32, 1)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ in0, const __nv_bfloat16* __restrict__ in1,
                      const __nv_bfloat16* __restrict__ in2, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ inv_rms,
                      const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ d_sum,
                      __nv_bfloat16* __restrict__ dx_out, int M, int K, int n_slots, int n_dx_warps,
                      int* __restrict__ tile_done, float* __restrict__ dgamma_partials, int* __restrict__ status) {
  constexpr int NT = SUM3 ? 4 : 3;      // streams per slot
  constexpr int H = SUM3 ? 2 : 1;       // halves of the virtual block held per lane
  extern __shared__ __align__(128) uint8_t bwd_smem[];
  __shared__ int next_row;
  const uint32_t row_bytes = (uint32_t)K * 2u;
  const uint32_t slot_bytes = row_bytes * NT;
  float4* gamma_lo = reinterpret_cast<float4*>(bwd_smem);   // [K/8] gamma of elements 0-3 of each vector
  float4* gamma_hi = gamma_lo + (K >> 3);                   // [K/8] gamma of elements 4-7
  uint8_t* slots = bwd_smem + (size_t)K * 4;
  uint64_t* bars = reinterpret_cast<uint64_t*>(slots + (size_t)n_slots * slot_bytes);
  // uses[s]: copies issued into slot s so far (a barrier's one phase bit cannot tell two uses apart)
  volatile int* uses = reinterpret_cast<volatile int*>(bars + n_slots);
  const int lane = threadIdx.x & 31;
  // rows of this CTA: a contiguous band, or (FUSE_DGAMMA) every gridDim.x-th row
  const int band = (M + gridDim.x - 1) / gridDim.x;
  const int n_band = FUSE_DGAMMA ? (M - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x
                                 : min(band, M - (int)blockIdx.x * band);
  auto global_row = [&](int r) { return FUSE_DGAMMA ? (int)blockIdx.x + r * (int)gridDim.x : (int)blockIdx.x * band + r; };
  const uint64_t once = l2_policy_evict_first();
  auto issue = [&](int r) {
    const int s = r % n_slots;
    uint8_t* dst = slots + (size_t)s * slot_bytes;
    const size_t off = (size_t)global_row(r) * K;
    mbar_expect_tx(&bars[s], slot_bytes);
    // streams nobody reads again leave L2 first, so that the rows the dgamma warps come back for stay
    if constexpr (SUM3) {
      bulk_load_1d_hint(dst, in0 + off, row_bytes, &bars[s], once);
      bulk_load_1d_hint(dst + row_bytes, in1 + off, row_bytes, &bars[s], once);
      bulk_load_1d_hint(dst + 2 * row_bytes, in2 + off, row_bytes, &bars[s], once);
      bulk_load_1d(dst + 3 * row_bytes, x + off, row_bytes, &bars[s]);
    } else {
      bulk_load_1d(dst, in0 + off, row_bytes, &bars[s]);
      bulk_load_1d(dst + row_bytes, x + off, row_bytes, &bars[s]);
      bulk_load_1d_hint(dst + 2 * row_bytes, residual + off, row_bytes, &bars[s], once);
    }
    __threadfence_block();
    uses[s] = r / n_slots + 1;
  };
  if (threadIdx.x == 0) next_row = 0;
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    mbar_init(&bars[s], 1);
    uses[s] = 0;
    fence_mbar_init();
    if (s < n_band) issue(s);
  }
  for (int q = threadIdx.x; q < (K >> 3); q += blockDim.x) {
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + q);
    gamma_lo[q] = make_float4(bf16lo_to_f32(g.x), bf16hi_to_f32(g.x), bf16lo_to_f32(g.y), bf16hi_to_f32(g.y));
    gamma_hi[q] = make_float4(bf16lo_to_f32(g.z), bf16hi_to_f32(g.z), bf16lo_to_f32(g.w), bf16hi_to_f32(g.w));
  }
  __syncthreads();

  if constexpr (FUSE_DGAMMA) {
    const int warp = threadIdx.x >> 5;
    if (warp >= n_dx_warps) {
      // ---- dgamma warps: items = (tile, slice of 128 columns), tile-major, dealt round-robin over all such warps
      const int slices = K >> 7;
      const int n_tiles = (M + kBwdRowTile - 1) / kBwdRowTile;
      const int n_items = n_tiles * slices;
      const int n_workers = kDgammaWarps * (int)gridDim.x;
      const size_t pitch = (size_t)K >> 2;
      const __nv_bfloat16* dy_src = SUM3 ? d_sum : in0;
      for (int item = (warp - n_dx_warps) * (int)gridDim.x + (int)blockIdx.x; item < n_items; item += n_workers) {
        const int t = item / slices, c4 = (item - t * slices) * 32 + lane;
        const int row0 = t * kBwdRowTile, rows = min(kBwdRowTile, M - row0);
        bool ok = true;
        if (lane == 0) {
          uint32_t spins = 0;
          while (ld_acquire_gpu(tile_done + t) < rows && ++spins < kSpinLimit) __nanosleep(256);
          ok = ld_acquire_gpu(tile_done + t) >= rows;
        }
        if (__shfl_sync(0xffffffffu, (int)ok, 0) == 0) {
          if (lane == 0) atomicExch(status, kStatusQuantTmaTimeout);
          return;
        }
        float p[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        dgamma_rows(reinterpret_cast<const uint2*>(dy_src) + (size_t)row0 * pitch + c4,
                    reinterpret_cast<const uint2*>(x) + (size_t)row0 * pitch + c4, pitch, inv_rms, row0, rows, p);
        reinterpret_cast<float4*>(dgamma_partials + (size_t)t * K)[c4] = make_float4(p[0], p[1], p[2], p[3]);
      }
      return;
    }
  }

  const int nvec_row = K >> 3;
  const int nv = (nvec_row + 31) >> 5;     // vectors per lane (K is a multiple of 256: the same for all lanes)
  const float k_f = static_cast<float>(K);
  int pending_row = -1;                    // lane 0: row whose stores are in flight and not yet counted on its tile
  auto count_pending = [&]() {
    if (pending_row >= 0) {
      bulk_wait_group0();                  // the row's stores are complete ...
      __threadfence();                     // ... and ordered before the count that publishes them
      atomicAdd(tile_done + pending_row / kBwdRowTile, 1);
      pending_row = -1;
    }
  };
  while (true) {
    int r = 0;
    if (lane == 0) r = atomicAdd(&next_row, 1);
    r = __shfl_sync(0xffffffffu, r, 0);
    if (r >= n_band) break;
    const int s = r % n_slots;
    const int use = r / n_slots;
    bool ok = true;
    if (lane == 0) {
      uint32_t spins = 0;
      while (uses[s] <= use && ++spins < kSpinLimit) {}
      ok = uses[s] > use;
    }
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    if (!ok || !mbar_wait_bounded(&bars[s], (uint32_t)use & 1u)) {
      if (lane == 0) atomicExch(status, kStatusQuantTmaTimeout);
      break;
    }
    const int row = global_row(r);
    uint8_t* slot = slots + (size_t)s * slot_bytes;
    uint4* s_dy = reinterpret_cast<uint4*>(slot);                                   // d0 -> dy (sum3) | dy
    uint4* s_x = reinterpret_cast<uint4*>(slot + (SUM3 ? 3 : 1) * row_bytes);
    uint4* s_out = reinterpret_cast<uint4*>(slot + (SUM3 ? 1 : 2) * row_bytes);     // d1 -> dx | residual -> dx + residual
    const float inv = __ldg(inv_rms + row);
    const float2 inv2 = make_float2(inv, inv);

    // ---- row sum in the block's order
    float2 acc[H][4];
#pragma unroll
    for (int h = 0; h < H; ++h)
#pragma unroll
      for (int p = 0; p < 4; ++p) acc[h][p] = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      if (j < nv) {
        const int q = lane + 32 * j;
        uint4 dy = s_dy[q];
        if constexpr (SUM3) {
          const uint4 b = reinterpret_cast<const uint4*>(slot + row_bytes)[q];
          const uint4 c = reinterpret_cast<const uint4*>(slot + 2 * row_bytes)[q];
          dy.x = bf16x2_add(bf16x2_add(dy.x, b.x), c.x);
          dy.y = bf16x2_add(bf16x2_add(dy.y, b.y), c.y);
          dy.z = bf16x2_add(bf16x2_add(dy.z, b.z), c.z);
          dy.w = bf16x2_add(bf16x2_add(dy.w, b.w), c.w);
          s_dy[q] = dy;
        }
        const uint4 xv = s_x[q];
        const float4 g01 = gamma_lo[q], g23 = gamma_hi[q];
        const uint32_t dw[4] = {dy.x, dy.y, dy.z, dy.w};
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
        const float2 gw[4] = {make_float2(g01.x, g01.y), make_float2(g01.z, g01.w), make_float2(g23.x, g23.y),
                              make_float2(g23.z, g23.w)};
        const int h = SUM3 ? (j & 1) : 0;   // a constant once the loop is unrolled
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 dyf = make_float2(bf16lo_to_f32(dw[p]), bf16hi_to_f32(dw[p]));
          const float2 xf = make_float2(bf16lo_to_f32(xw[p]), bf16hi_to_f32(xw[p]));
          const float2 normed = mul2(mul2(xf, inv2), gw[p]);
          acc[h][p] = fma2(dyf, normed, acc[h][p]);
        }
      }
    }
    // 32 consecutive "threads" = the 8 elements of 4 neighbouring lanes: balanced tree
    float wsum[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const float a = (acc[h][0].x + acc[h][0].y) + (acc[h][1].x + acc[h][1].y);
      const float b = (acc[h][2].x + acc[h][2].y) + (acc[h][3].x + acc[h][3].y);
      float w = a + b;
      w += __shfl_xor_sync(0xffffffffu, w, 1);
      w += __shfl_xor_sync(0xffffffffu, w, 2);
      wsum[h] = w;
    }
    // warp sums one after another: warps 0-7 are lane groups 0-7 of half 0, warps 8-15 those of half 1
    float total = __shfl_sync(0xffffffffu, wsum[0], 0);
#pragma unroll
    for (int w = 1; w < 8; ++w) total += __shfl_sync(0xffffffffu, wsum[0], 4 * w);
    if constexpr (SUM3) {
#pragma unroll
      for (int w = 0; w < 8; ++w) total += __shfl_sync(0xffffffffu, wsum[H - 1], 4 * w);
    }
    const float mean = __fdiv_rn(total, k_f);
    const float2 neg_mean2 = make_float2(-mean, -mean);   // (x*inv)*(-mean) = -((x*inv)*mean) exactly

    // ---- dx, written over a stream this lane has already consumed
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      if (j < nv) {
        const int q = lane + 32 * j;
        const uint4 dy = s_dy[q];
        const uint4 xv = s_x[q];
        const float4 g01 = gamma_lo[q], g23 = gamma_hi[q];
        const uint32_t dw[4] = {dy.x, dy.y, dy.z, dy.w};
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
        const float2 gw[4] = {make_float2(g01.x, g01.y), make_float2(g01.z, g01.w), make_float2(g23.x, g23.y),
                              make_float2(g23.z, g23.w)};
        uint32_t ow[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 dyf = make_float2(bf16lo_to_f32(dw[p]), bf16hi_to_f32(dw[p]));
          const float2 xf = make_float2(bf16lo_to_f32(xw[p]), bf16hi_to_f32(xw[p]));
          const float2 v = fma2(dyf, gw[p], mul2(mul2(xf, inv2), neg_mean2));
          const float2 d = mul2(inv2, v);
          ow[p] = f32x2_to_bf16x2(d.x, d.y);
        }
        if constexpr (!SUM3) {
          const uint4 res = s_out[q];
          ow[0] = bf16x2_add(ow[0], res.x);
          ow[1] = bf16x2_add(ow[1], res.y);
          ow[2] = bf16x2_add(ow[2], res.z);
          ow[3] = bf16x2_add(ow[3], res.w);
        }
        s_out[q] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      const size_t off = (size_t)row * K;
      if constexpr (FUSE_DGAMMA) {
        count_pending();                   // stores committed a whole row ago: no wait in practice
        pending_row = row;
      }
      if constexpr (SUM3) bulk_store_1d(d_sum + off, s_dy, row_bytes);
      bulk_store_1d_hint(dx_out + off, s_out, row_bytes, once);
      bulk_commit_group();
      if (r + n_slots < n_band) {
        bulk_wait_group_read0();   // the stores have read the slot: it may be overwritten
        issue(r + n_slots);
      }
    }
  }
  if (lane == 0) {
    if constexpr (FUSE_DGAMMA) count_pending();
    bulk_wait_group0();
  }
}

// dgamma tiles as a kernel of its own (grids that cannot be co-resident, A/B runs): thread = 4 columns, rows
// of the tile in turn, sixteen rows of both streams requested before the first is used.
__global__ void __launch_bounds__(128)
rmsnorm_bwd_dgamma_tile_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                               const float* __restrict__ inv_rms, float* __restrict__ partials, int M, int K) {
  const int c4 = blockIdx.x * blockDim.x + threadIdx.x;   // group of 4 columns
  if (c4 * 4 >= K) return;
  const int row0 = blockIdx.y * kBwdRowTile;
  const int rows = min(kBwdRowTile, M - row0);
  const size_t pitch = (size_t)K >> 2;                    // uint2 per row
  float p[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  dgamma_rows(reinterpret_cast<const uint2*>(dy) + (size_t)row0 * pitch + c4,
              reinterpret_cast<const uint2*>(x) + (size_t)row0 * pitch + c4, pitch, inv_rms, row0, rows, p);
  const float p0 = p[0], p1 = p[1], p2 = p[2], p3 = p[3];
  reinterpret_cast<float4*>(partials + (size_t)blockIdx.y * K)[c4] = make_float4(p0, p1, p2, p3);
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(64)
rmsnorm_bwd_dgamma_reduce_kernel(const float* __restrict__ partials, void* __restrict__ dgamma, int row_tiles, int K) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= K) return;
  float sum = 0.0f;
  int t = 0;
  for (; t + 16 <= row_tiles; t += 16) {   // sixteen independent loads, then the adds in tile order
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) v[u] = __ldg(partials + (size_t)(t + u) * K + col);
#pragma unroll
    for (int u = 0; u < 16; ++u) sum += v[u];
  }
  for (; t < row_tiles; ++t) sum += __ldg(partials + (size_t)t * K + col);
  if constexpr (OUT_BF16) static_cast<__nv_bfloat16*>(dgamma)[col] = __float2bfloat16_rn(sum);
  else static_cast<float*>(dgamma)[col] = sum;
}

namespace {

struct Range {
  const void* p;
  size_t bytes;
  const char* name;
};

bool overlaps(const Range& a, const Range& b) {
  const uintptr_t a0 = reinterpret_cast<uintptr_t>(a.p), b0 = reinterpret_cast<uintptr_t>(b.p);
  return a0 < b0 + b.bytes && b0 < a0 + a.bytes;
}

int check_no_overlap(const char* fn, const Range* outs, int n_out, const Range* ins, int n_in) {
  for (int i = 0; i < n_out; ++i) {
    for (int j = 0; j < n_in; ++j)
      if (overlaps(outs[i], ins[j])) return set_error("%s: output %s overlaps input %s", fn, outs[i].name, ins[j].name);
    for (int j = i + 1; j < n_out; ++j)
      if (overlaps(outs[i], outs[j])) return set_error("%s: outputs %s and %s overlap", fn, outs[i].name, outs[j].name);
  }
  return 0;
}

int bwd_slots_for(int64_t K, int streams) {
  const int64_t budget = 227 * 1024 - K * 4 - 1024;
  return (int)std::min<int64_t>(16, budget / (K * 2 * streams));
}

bool fused_dgamma_enabled() {
  static const bool on = [] {
    const char* e = getenv("FP4B200_BWD_FUSED_DGAMMA");   // "0": dgamma tiles as a kernel of their own (A/B runs)
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

bool cooperative_launch_supported() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) return false;
  return v != 0;
}

int launch_dgamma_reduce(const float* partials, void* dgamma, bool out_bf16, int row_tiles, int64_t K, cudaStream_t st) {
  const unsigned rgrid = (unsigned)((K + 63) / 64);
  if (out_bf16) rmsnorm_bwd_dgamma_reduce_kernel<true><<<rgrid, 64, 0, st>>>(partials, dgamma, row_tiles, (int)K);
  else rmsnorm_bwd_dgamma_reduce_kernel<false><<<rgrid, 64, 0, st>>>(partials, dgamma, row_tiles, (int)K);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// dx (+ d_sum), the dgamma tiles and their reduction.  dy_for_dgamma: the stream dgamma is taken from (d_sum, which
// the dx kernel writes, or the caller's d_normed).
template <bool SUM3>
int launch_rmsnorm_bwd(const void* in0, const void* in1, const void* in2, const void* x, const void* gamma,
                       const float* inv_rms, const void* residual, void* d_sum, void* dx, float* partials, void* dgamma,
                       bool dgamma_bf16, int64_t M, int64_t K, cudaStream_t st) {
  int* status = device_status_ptr();
  if (status == nullptr) return -1;
  const int sms = device_sm_count();
  if (sms <= 0) return -1;
  const int slots = bwd_slots_for(K, SUM3 ? 4 : 3);
  int warps = std::min(8, slots);
  const size_t smem = (size_t)K * 4 + (size_t)slots * K * 2 * (SUM3 ? 4 : 3) + (size_t)slots * 12 + 16;
  const int grid = (int)std::min<int64_t>(sms, M);
  const int row_tiles = (int)((M + kBwdRowTile - 1) / kBwdRowTile);
  const __nv_bfloat16* p_in0 = static_cast<const __nv_bfloat16*>(in0);
  const __nv_bfloat16* p_in1 = static_cast<const __nv_bfloat16*>(in1);
  const __nv_bfloat16* p_in2 = static_cast<const __nv_bfloat16*>(in2);
  const __nv_bfloat16* p_x = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* p_gamma = static_cast<const __nv_bfloat16*>(gamma);
  const __nv_bfloat16* p_res = static_cast<const __nv_bfloat16*>(residual);
  __nv_bfloat16* p_dsum = static_cast<__nv_bfloat16*>(d_sum);
  __nv_bfloat16* p_dx = static_cast<__nv_bfloat16*>(dx);
  int m_i = (int)M, k_i = (int)K, slots_i = slots;

  bool fused = fused_dgamma_enabled() && row_tiles <= kScratchFloats && cooperative_launch_supported();
  if (fused) {
    auto kern = K <= 4096 ? rmsnorm_bwd_dx_kernel<SUM3, true, 16> : rmsnorm_bwd_dx_kernel<SUM3, true, 32>;
    FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int block = (warps + kDgammaWarps) * 32;
    int per_sm = 0;
    FP4_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, block, smem));
    if (per_sm < 1) fused = false;
    if (fused) {
      float* scratch = stream_scratch(st);
      if (scratch == nullptr) return -1;
      int* tile_done = reinterpret_cast<int*>(scratch);
      FP4_CUDA_CHECK(cudaMemsetAsync(tile_done, 0, (size_t)row_tiles * sizeof(int), st));
      void* args[] = {&p_in0, &p_in1, &p_in2, &p_x, &p_gamma, &inv_rms, &p_res, &p_dsum, &p_dx, &m_i, &k_i,
                      &slots_i, &warps, &tile_done, &partials, &status};
      FP4_CUDA_CHECK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), dim3(grid), dim3(block), args, smem, st));
      return launch_dgamma_reduce(partials, dgamma, dgamma_bf16, row_tiles, K, st);
    }
  }
  auto kern = K <= 4096 ? rmsnorm_bwd_dx_kernel<SUM3, false, 16> : rmsnorm_bwd_dx_kernel<SUM3, false, 32>;
  FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<grid, warps * 32, smem, st>>>(p_in0, p_in1, p_in2, p_x, p_gamma, inv_rms, p_res, p_dsum, p_dx, m_i, k_i, slots_i,
                                       warps, nullptr, nullptr, status);
  FP4_CUDA_CHECK(cudaGetLastError());
  const dim3 tgrid((unsigned)((K / 4 + 127) / 128), (unsigned)row_tiles);
  rmsnorm_bwd_dgamma_tile_kernel<<<tgrid, 128, 0, st>>>(SUM3 ? p_dsum : p_in0, p_x, inv_rms, partials, m_i, k_i);
  FP4_CUDA_CHECK(cudaGetLastError());
  return launch_dgamma_reduce(partials, dgamma, dgamma_bf16, row_tiles, K, st);
}

int check_shape(const char* fn, int64_t M, int64_t K) {
  if (M <= 0 || K <= 0) return set_error("%s: M and K must be positive (got %lld x %lld)", fn, (long long)M, (long long)K);
  if (M > INT32_MAX / K) return set_error("%s: M*K must be int32-indexable (got %lld x %lld)", fn, (long long)M, (long long)K);
  if ((K % 256) != 0 || K > 256 * kBwdMaxVec)
    return set_error("%s: K must be a multiple of 256, at most %d (got %lld)", fn, 256 * kBwdMaxVec, (long long)K);
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace fp4b200

using namespace fp4b200;

extern "C" {

int fp4b200_sum3_rmsnorm_bwd(const void* d0, const void* d1, const void* d2, const void* input, const void* norm_weight,
                             const float* inv_rms, void* d_sum, void* grad_input, float* dgamma_partials, void* dgamma,
                             int dgamma_is_bf16, int64_t M, int64_t K, void* stream) {
  const char* fn = "sum3_rmsnorm_bwd";
  if (!d0 || !d1 || !d2 || !input || !norm_weight || !inv_rms || !d_sum || !grad_input || !dgamma_partials || !dgamma)
    return set_error("%s: null pointer", fn);
  if (check_shape(fn, M, K) != 0) return -1;
  if (!aligned16(d0) || !aligned16(d1) || !aligned16(d2) || !aligned16(input) || !aligned16(norm_weight) || !aligned16(d_sum) ||
      !aligned16(grad_input) || !aligned16(dgamma_partials))
    return set_error("%s: matrices, norm_weight and dgamma_partials must be 16-byte aligned", fn);
  const size_t mat = (size_t)M * (size_t)K * 2;
  const size_t tiles = (size_t)((M + kBwdRowTile - 1) / kBwdRowTile);
  const Range outs[] = {{d_sum, mat, "d_sum"},
                        {grad_input, mat, "grad_input"},
                        {dgamma_partials, tiles * (size_t)K * 4, "dgamma_partials"},
                        {dgamma, (size_t)K * (dgamma_is_bf16 ? 2 : 4), "dgamma"}};
  const Range ins[] = {{d0, mat, "d0"}, {d1, mat, "d1"}, {d2, mat, "d2"}, {input, mat, "input"},
                       {norm_weight, (size_t)K * 2, "norm_weight"}, {inv_rms, (size_t)M * 4, "inv_rms"}};
  if (check_no_overlap(fn, outs, 4, ins, 6) != 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  return launch_rmsnorm_bwd<true>(d0, d1, d2, input, norm_weight, inv_rms, nullptr, d_sum, grad_input, dgamma_partials, dgamma,
                                  dgamma_is_bf16 != 0, M, K, st);
}

int fp4b200_rmsnorm_bwd_residual(const void* d_normed, const void* input, const void* norm_weight, const float* inv_rms,
                                 const void* residual_grad, void* grad_input, float* dgamma_partials, float* dgamma, int64_t M,
                                 int64_t K, void* stream) {
  const char* fn = "rmsnorm_bwd_residual";
  if (!d_normed || !input || !norm_weight || !inv_rms || !residual_grad || !grad_input || !dgamma_partials || !dgamma)
    return set_error("%s: null pointer", fn);
  if (check_shape(fn, M, K) != 0) return -1;
  if (K != 4096) return set_error("%s: requires [M,4096] (got K = %lld)", fn, (long long)K);
  if (!aligned16(d_normed) || !aligned16(input) || !aligned16(norm_weight) || !aligned16(residual_grad) ||
      !aligned16(grad_input) || !aligned16(dgamma_partials))
    return set_error("%s: matrices, norm_weight and dgamma_partials must be 16-byte aligned", fn);
  const size_t mat = (size_t)M * (size_t)K * 2;
  const size_t tiles = (size_t)((M + kBwdRowTile - 1) / kBwdRowTile);
  const Range outs[] = {{grad_input, mat, "grad_input"},
                        {dgamma_partials, tiles * (size_t)K * 4, "dgamma_partials"},
                        {dgamma, (size_t)K * 4, "dgamma"}};
  const Range ins[] = {{d_normed, mat, "d_normed"}, {input, mat, "input"}, {norm_weight, (size_t)K * 2, "norm_weight"},
                       {inv_rms, (size_t)M * 4, "inv_rms"}, {residual_grad, mat, "residual_grad"}};
  if (check_no_overlap(fn, outs, 3, ins, 5) != 0) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  return launch_rmsnorm_bwd<false>(d_normed, nullptr, nullptr, input, norm_weight, inv_rms, residual_grad, nullptr, grad_input,
                                   dgamma_partials, dgamma, false, M, K, st);
}

}  // extern "C"
