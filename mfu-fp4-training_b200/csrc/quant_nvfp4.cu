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
#include <atomic>

#include "fp4_common.cuh"
#include "host_util.h"

namespace fp4b200 {

// ---------------------------------------------------------------------------------------
// Tensor amax of a bf16 buffer (pass 1 of the plain quantiser)
// ---------------------------------------------------------------------------------------

// Maximum |x| over the share CTA `cta` of `n_ctas` takes of n_vec 16-byte vectors; the result is in thread 0 (the
// first warp holds it), and ends with a CTA barrier.
__device__ __forceinline__ float cta_share_absmax(const uint4* __restrict__ x, size_t n_vec, int cta, int n_ctas) {
  uint32_t m0 = 0, m1 = 0, m2 = 0, m3 = 0;
  const size_t stride = (size_t)n_ctas * blockDim.x;
  size_t i = (size_t)cta * blockDim.x + threadIdx.x;
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
  }
  return v;
}

// partials[blockIdx.x] = max|x| over this CTA's share (every CTA writes, so nothing needs clearing)
// early_reads: the caller has promised that x was not written by the kernel launched just before this one (see
// fp4b200_set_pdl_early_reads), so x may be read while that kernel still runs; otherwise nothing is read before
// that kernel's writes are visible.
__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint4* __restrict__ x, size_t n_vec,
                                                        float* __restrict__ partials, int early_reads) {
  pdl_launch_dependents();   // a quantiser launched behind this kernel may set up and prefetch meanwhile
  if (!early_reads) pdl_wait();
  const float v = cta_share_absmax(x, n_vec, (int)blockIdx.x, (int)gridDim.x);
  if (threadIdx.x < 32) {
    // Launched behind a quantiser that lets its dependents start early, this kernel may have only read x so far;
    // that quantiser may still be reading the partial maxima of ITS input from the same scratch, so the write waits.
    pdl_wait();
    if (threadIdx.x == 0) partials[blockIdx.x] = v;
  }
}

// The same over three tensors in one launch: CTAs [0, cta_end[0]) take the first, [cta_end[0], cta_end[1]) the second,
// the rest the third; partials[b] is CTA b's maximum, so each tensor's partial maxima are contiguous.
struct AmaxGroup3 {
  const uint4* x[3];
  size_t n_vec[3];
  int cta_end[2];
};

__global__ void __launch_bounds__(256) amax3_bf16_kernel(const AmaxGroup3 g, float* __restrict__ partials, int early_reads) {
  pdl_launch_dependents();
  if (!early_reads) pdl_wait();
  const int b = (int)blockIdx.x;
  float v;
  if (b < g.cta_end[0]) v = cta_share_absmax(g.x[0], g.n_vec[0], b, g.cta_end[0]);
  else if (b < g.cta_end[1]) v = cta_share_absmax(g.x[1], g.n_vec[1], b - g.cta_end[0], g.cta_end[1] - g.cta_end[0]);
  else v = cta_share_absmax(g.x[2], g.n_vec[2], b - g.cta_end[1], (int)gridDim.x - g.cta_end[1]);
  if (threadIdx.x < 32) {
    pdl_wait();   // as in amax_bf16_kernel: the scratch may still be read by the kernel before
    if (threadIdx.x == 0) partials[b] = v;
  }
}

// amax_sg[0] = max of the partial maxima, amax_sg[1] = amax / 2688 (GEMM-side tensor scale); one CTA.
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partials, int n,
                                                              float* __restrict__ amax_sg) {
  pdl_wait();
  float v = 0.0f;
  for (int i = threadIdx.x; i < n; i += 256) v = fmaxf(v, partials[i]);
  v = warp_max(v);
  __shared__ float warp_part[8];
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) v = fmaxf(v, warp_part[w]);
    amax_sg[0] = v;
    amax_sg[1] = v / 2688.0f;
  }
}

// amax_sg[1] = amax_sg[0] / 2688
__global__ void finalize_sg_kernel(float* __restrict__ amax_sg) { amax_sg[1] = amax_sg[0] / 2688.0f; }

// Tensor amax of a quantiser launch behind a pass-1 kernel: maximum of that kernel's per-CTA partial
// maxima, computed by every CTA for itself (n <= 2048 floats that sit in L2).  Contains a CTA barrier.
__device__ __forceinline__ float amax_from_partials(const float* partials, int n, float* slot) {
  if (threadIdx.x < 32) {
    float v = 0.0f;
    for (int i = threadIdx.x; i < n; i += 32) v = fmaxf(v, partials[i]);
    v = warp_max(v);
    if (threadIdx.x == 0) *slot = v;
  }
  __syncthreads();
  return *slot;
}

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
constexpr int kStatsMaxWarps = 16;   // warps per CTA, one CTA per SM

// Sum of squares of the row held in v -> 1/rms, identical on all lanes.
template <int NV>
__device__ __forceinline__ float stats_inv_rms(const uint4 (&v)[NV], int K, float eps) {
  // acc[i][q]: virtual lane 4*lane + 128*i + q accumulates elements 2q, 2q+1 of vectors j = i, i+2, ...
  float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = j & 1;
    acc[i][0] = fma_sq_bf16x2(v[j].x, acc[i][0]);
    acc[i][1] = fma_sq_bf16x2(v[j].y, acc[i][1]);
    acc[i][2] = fma_sq_bf16x2(v[j].z, acc[i][2]);
    acc[i][3] = fma_sq_bf16x2(v[j].w, acc[i][3]);
  }
  float part[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float a4[4] = {acc[i][0], acc[i][1], acc[i][2], acc[i][3]};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      a4[q] += __shfl_xor_sync(0xffffffffu, a4[q], 4);
      a4[q] += __shfl_xor_sync(0xffffffffu, a4[q], 2);
      a4[q] += __shfl_xor_sync(0xffffffffu, a4[q], 1);
    }
    const float a = a4[0] + a4[2];
    const float b = a4[1] + a4[3];
    part[i] = a + b;
  }
  float s = part[0] + part[1];
  s += __shfl_xor_sync(0xffffffffu, s, 16);
  s += __shfl_xor_sync(0xffffffffu, s, 8);
  return rsqrtf(s / static_cast<float>(K) + eps);
}

// The same for the summation tree of the reference's MXFP4 producer (mxfp4_v4/mxfp4_v3_quantize.cuh:109-172,
// compute_inv_rms_kernel): thread t of its 256 accumulates the eight elements of vector t, then of vector t + 256,
// ... in sequence; xor butterflies over 16,8,4,2,1 inside each of its eight warps, then over the eight warp sums
// (the same butterfly on a warp whose lanes 8-31 hold zeros).  Lane L here holds that kernel's threads
// 32*w + L (w = 0..7) in acc[w].
template <int NV>
__device__ __forceinline__ float stats_inv_rms_mx(const uint4 (&v)[NV], int K, float eps) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    float a = acc[j & 7];
    a = fma_sq_bf16x2(v[j].x, a);
    a = fma_sq_bf16x2(v[j].y, a);
    a = fma_sq_bf16x2(v[j].z, a);
    a = fma_sq_bf16x2(v[j].w, a);
    acc[j & 7] = a;
  }
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    if (w < NV) {
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) acc[w] += __shfl_xor_sync(0xffffffffu, acc[w], m);
    }
  }
  const float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
  return rsqrtf(s / static_cast<float>(K) + eps);
}

// And for the tree of the inverse-RMS kernel in front of the reference's optional-mode fused producer
// (nvfp4_v5/fused_norm_quantize.cuh:391-434, inv_rms_kernel_ns::compute_inv_rms_kernel<256>): thread t accumulates the
// single elements t, t + 256, ...; xor butterflies over 16,8,4,2,1 inside a warp, then 4,2,1 over the eight warp sums.
// Element e of lane L's vector j is element 256 j + 8 L + e of the row: that kernel's thread 8 L + e, i.e. warp L / 4,
// lane 8 (L % 4) + e — so its masks 16 and 8 are shuffles over this warp's lane masks 2 and 1, its masks 4,2,1 register
// adds over e, and the warp sums meet by shuffles over lane masks 16, 8, 4.
template <int NV>
__device__ __forceinline__ float stats_inv_rms_strided(const uint4 (&v)[NV], int K, float eps) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float lo = bf16lo_to_f32(w[q]), hi = bf16hi_to_f32(w[q]);
      acc[2 * q] = fmaf(lo, lo, acc[2 * q]);
      acc[2 * q + 1] = fmaf(hi, hi, acc[2 * q + 1]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
  }
  float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
  s += __shfl_xor_sync(0xffffffffu, s, 16);
  s += __shfl_xor_sync(0xffffffffu, s, 8);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  return rsqrtf(s / static_cast<float>(K) + eps);
}

// Running maximum of |(x * inv) * gamma| in fp32 over the row held in v.  Rounding to bf16 is
// monotonic, so the tensor amax of the bf16 values is the bf16 rounding of this maximum: no
// per-element conversion.  gamma is read as fp32 from two shared-memory tables (elements 0-3 and
// 4-7 of every vector), each a conflict-free 16-byte read per lane.
template <int NV>
__device__ __forceinline__ float stats_row_amax(const uint4 (&v)[NV], const float4* gamma_lo, const float4* gamma_hi,
                                                float inv, int K, int lane, float mx) {
  const float2 inv2 = make_float2(inv, inv);
  const int nvec_row = K >> 3;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int q = lane + 32 * j;
    if (q < nvec_row) {
      const float4 g01 = gamma_lo[q];
      const float4 g23 = gamma_hi[q];
      const float2 t0 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].x), bf16hi_to_f32(v[j].x)), inv2), make_float2(g01.x, g01.y));
      const float2 t1 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].y), bf16hi_to_f32(v[j].y)), inv2), make_float2(g01.z, g01.w));
      const float2 t2 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].z), bf16hi_to_f32(v[j].z)), inv2), make_float2(g23.x, g23.y));
      const float2 t3 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].w), bf16hi_to_f32(v[j].w)), inv2), make_float2(g23.z, g23.w));
      mx = absmax3(mx, t0.x, t0.y);
      mx = absmax3(mx, t1.x, t1.y);
      mx = absmax3(mx, t2.x, t2.y);
      mx = absmax3(mx, t3.x, t3.y);
    }
  }
  return mx;
}

// One CTA per SM.  The CTA owns a contiguous band of rows and a ring of row slots in shared memory
// (as many as fit: 24 of 8 KB at K = 4096); row r of the band lives in slot r % slots and arrives by
// one bulk copy (a row is contiguous).  A warp claims the band's next row from a shared counter, waits
// for that slot's barrier, lifts the row into registers and, as soon as the row's sum of squares has
// been reduced (the reduction needs every lane's values, so all reads of the slot are complete by
// then), refills the slot with the row `slots` further on.  Bytes in flight per SM are set by the ring,
// not by registers or by the number of warps, which is what a streaming reduction at HBM speed needs;
// rows are handed out one at a time, so the warps of a CTA finish within one row of each other.
template <int NV /* 16-byte vectors held per lane; K <= NV*256 */, bool COMPUTE_INV_RMS, int TREE = 0 /* 1: the MXFP4 producer's summation tree, 2: the optional-mode NVFP4 producer's */>
__global__ void __launch_bounds__(NV <= 16 ? kStatsMaxWarps * 32 : 192, 1)
rmsnorm_stats_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                     float* __restrict__ inv_rms, float* __restrict__ partials, float eps, int M, int K,
                     int n_slots, int* __restrict__ status, int early_reads, int want_amax) {
  extern __shared__ __align__(128) uint8_t stats_smem[];
  __shared__ int next_row;   // next unclaimed row of the band (band-relative)
  __shared__ float warp_max_s[kStatsMaxWarps];
  pdl_launch_dependents();   // the quantiser launched behind this kernel may set up and prefetch meanwhile
  const int warps = blockDim.x >> 5;
  const uint32_t row_bytes = (uint32_t)K * 2u;
  float4* gamma_lo = reinterpret_cast<float4*>(stats_smem);                 // [K/8] gamma of elements 0-3 of each vector
  float4* gamma_hi = gamma_lo + (K >> 3);                                   // [K/8] gamma of elements 4-7
  uint8_t* slots = stats_smem + (size_t)K * 4;                              // [n_slots][row_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(slots + (size_t)n_slots * row_bytes);
  // uses[s] = number of copies issued into slot s so far.  A barrier's parity alone cannot tell "the
  // copy of my row has landed" from "the copy two uses earlier has landed", so a warp first makes sure
  // that its row's copy has been issued (which implies that the use before it was fully consumed).
  volatile int* uses = reinterpret_cast<volatile int*>(bars + n_slots);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Rows are dealt round-robin: CTA b takes rows b, b + grid, b + 2*grid, ...  All CTAs so sweep x from its first
  // row to its last together, and what the L2 still holds when the kernel ends is the END of x — which the
  // quantiser launched next walks first (it goes through the row blocks backwards).  The copies carry an
  // evict-last hint for the same reason: the quantiser's own output must not push x out.
  const int n_band = (int)blockIdx.x < M ? (M - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;   // rows of this CTA
  const uint64_t keep = l2_policy_evict_last();
  auto row_of = [&](int r) { return (size_t)r * gridDim.x + blockIdx.x; };
  auto issue = [&](int r) {                   // r: this CTA's r-th row -> slot r % n_slots
    const int s = r % n_slots;
    mbar_expect_tx(&bars[s], row_bytes);
    bulk_load_1d_hint(slots + (size_t)s * row_bytes, x + row_of(r) * K, row_bytes, &bars[s], keep);
    __threadfence_block();
    uses[s] = r / n_slots + 1;
  };
  // thread s owns slot s at start-up: barrier, first copy (the ring fills while gamma is staged)
  if (threadIdx.x == 0) next_row = 0;
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    mbar_init(&bars[s], 1);
    uses[s] = 0;
    fence_mbar_init();
  }
  // Launched as a programmatic dependent, this kernel may have started while the kernel before it still runs.  By
  // default it reads nothing of the caller's before that kernel's writes are visible: x is usually what that kernel
  // just produced.  With early_reads (the caller's promise that x and gamma were written earlier than that) the
  // ring fills and gamma is staged meanwhile, and only the writes below wait.
  if (!early_reads) pdl_wait();
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x)
    if (s < n_band) issue(s);
  for (int q = threadIdx.x; q < (K >> 3); q += blockDim.x) {
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + q);
    gamma_lo[q] = make_float4(bf16lo_to_f32(g.x), bf16hi_to_f32(g.x), bf16lo_to_f32(g.y), bf16hi_to_f32(g.y));
    gamma_hi[q] = make_float4(bf16lo_to_f32(g.z), bf16hi_to_f32(g.z), bf16lo_to_f32(g.w), bf16hi_to_f32(g.w));
  }
  __syncthreads();
  // inv_rms and the partial maxima may still be read by the strip quantiser of the previous call, so nothing is
  // written (and a caller's inv_rms not read) before that kernel has ended.
  pdl_wait();

  float mx = 0.0f;
  const int nvec_row = K >> 3;
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
    const uint4* src = reinterpret_cast<const uint4*>(slots + (size_t)s * row_bytes);
    uint4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int q = lane + 32 * j;
      v[j] = (q < nvec_row) ? src[q] : make_uint4(0, 0, 0, 0);
    }
    const size_t row = row_of(r);
    float inv;
    if constexpr (COMPUTE_INV_RMS) {
      if constexpr (TREE == 1) inv = stats_inv_rms_mx<NV>(v, K, eps);
      else if constexpr (TREE == 2) inv = stats_inv_rms_strided<NV>(v, K, eps);
      else inv = stats_inv_rms<NV>(v, K, eps);
      if (lane == 0) {
        inv_rms[row] = inv;
        if (r + n_slots < n_band) issue(r + n_slots);
      }
      // want_amax == 0: the caller needs the inverse RMS only (a format without a tensor scale)
      if (want_amax) mx = stats_row_amax<NV>(v, gamma_lo, gamma_hi, inv, K, lane, mx);
    } else {
      inv = __ldg(inv_rms + row);
      mx = stats_row_amax<NV>(v, gamma_lo, gamma_hi, inv, K, lane, mx);
      // every lane's copy of the row has been consumed by the arithmetic above
      __syncwarp();
      if (lane == 0 && r + n_slots < n_band) issue(r + n_slots);
    }
  }
  float run_max = warp_max(mx);
  if (lane == 0) warp_max_s[warp] = run_max;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < warps; ++w) run_max = fmaxf(run_max, warp_max_s[w]);
    // the one rounding to bf16 that the element-wise maximum would have applied to its winner
    partials[blockIdx.x] = __bfloat162float(__float2bfloat16_rn(run_max));   // every CTA writes: nothing to clear
  }
}

// The same statistics with TWO warps per row: warp `half` of a pair takes the row's vectors of parity `half`, which is
// exactly the i = half accumulators of the summation tree above, so the pair's two partial sums are part[0] and
// part[1] of stats_inv_rms, exchanged through shared memory at a 64-thread named barrier and added in that order.
// A row then takes half as long and holds half the registers, so 24 warps (12 pairs) fit beside a ring of two row
// slots per pair: more warps to hide the reduction's latency, and a shorter tail when the CTA's rows run out.
// Rows are dealt to pairs round-robin (pair p: the CTA's rows p, p + pairs, ...) and a pair refills its own slots, so
// no counter and no cross-warp claim protocol is needed.
constexpr int kStatsPairSlots = 2;   // row slots per pair

template <int NVH /* 16-byte vectors per lane and warp: K <= NVH*512 */, bool COMPUTE_INV_RMS>
__global__ void __launch_bounds__(NVH <= 8 ? 768 : 384, 1)
rmsnorm_stats_pair_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                          float* __restrict__ inv_rms, float* __restrict__ partials, float eps, int M, int K,
                          int* __restrict__ status, int early_reads, int want_amax) {
  extern __shared__ __align__(128) uint8_t stats_smem[];
  __shared__ float warp_max_s[24];
  __shared__ volatile int pair_abort[12];   // set when a wait of the pair ran out
  if (threadIdx.x < 12) pair_abort[threadIdx.x] = 0;
  pdl_launch_dependents();   // the quantiser launched behind this kernel may set up and prefetch meanwhile
  const int warps = blockDim.x >> 5, pairs = warps >> 1;
  const uint32_t row_bytes = (uint32_t)K * 2u;
  float4* gamma_lo = reinterpret_cast<float4*>(stats_smem);                 // [K/8] gamma of elements 0-3 of each vector
  float4* gamma_hi = gamma_lo + (K >> 3);                                   // [K/8] gamma of elements 4-7
  uint8_t* slots = stats_smem + (size_t)K * 4;                              // [pairs][kStatsPairSlots][row_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(slots + (size_t)pairs * kStatsPairSlots * row_bytes);
  float* xchg = reinterpret_cast<float*>(bars + pairs * kStatsPairSlots);   // [2 buffers][pairs][2 halves][32 lanes]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = warp >> 1, half = warp & 1;
  // Rows r = blockIdx.x, blockIdx.x + grid, ... belong to this CTA (all CTAs sweep x front to back together, so that
  // the END of x is what L2 holds when the quantiser starts there); the CTA's k-th row goes to pair k % pairs.
  const int n_band = (int)blockIdx.x < M ? (M - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int my_rows = pair < n_band ? (n_band - pair + pairs - 1) / pairs : 0;
  const uint64_t keep = l2_policy_evict_last();
  uint8_t* my_slots = slots + (size_t)pair * kStatsPairSlots * row_bytes;
  uint64_t* my_bars = bars + pair * kStatsPairSlots;
  auto row_of = [&](int k) { return (size_t)(pair + k * pairs) * gridDim.x + blockIdx.x; };
  auto issue = [&](int k) {                   // the pair's k-th row -> its slot k % kStatsPairSlots
    const int sl = k % kStatsPairSlots;
    mbar_expect_tx(&my_bars[sl], row_bytes);
    bulk_load_1d_hint(my_slots + (size_t)sl * row_bytes, x + row_of(k) * K, row_bytes, &my_bars[sl], keep);
  };
  if (half == 0 && lane == 0) {
    for (int sl = 0; sl < kStatsPairSlots; ++sl) mbar_init(&my_bars[sl], 1);
    fence_mbar_init();
  }
  // By default nothing of the caller's is read before the previous kernel's writes are visible (x is usually what that
  // kernel just produced); with early_reads the ring fills and gamma is staged meanwhile.
  if (!early_reads) pdl_wait();
  if (half == 0 && lane == 0)
    for (int k = 0; k < kStatsPairSlots && k < my_rows; ++k) issue(k);
  if (want_amax) {
    for (int q = threadIdx.x; q < (K >> 3); q += blockDim.x) {
      const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + q);
      gamma_lo[q] = make_float4(bf16lo_to_f32(g.x), bf16hi_to_f32(g.x), bf16lo_to_f32(g.y), bf16hi_to_f32(g.y));
      gamma_hi[q] = make_float4(bf16lo_to_f32(g.z), bf16hi_to_f32(g.z), bf16lo_to_f32(g.w), bf16hi_to_f32(g.w));
    }
  }
  __syncthreads();
  // inv_rms and the partial maxima may still be read by the strip quantiser of the previous call
  pdl_wait();

  float mx = 0.0f;
  const int nvec_row = K >> 3;
  const float2 zero2 = make_float2(0.0f, 0.0f);
  (void)zero2;
  for (int k = 0; k < my_rows; ++k) {
    const int sl = k % kStatsPairSlots;
    // A wait that runs out is reported and both warps of the pair leave together AFTER the row's named barrier: a
    // warp must never wait there for a partner that has already left.
    if (!mbar_wait_bounded(&my_bars[sl], (uint32_t)(k / kStatsPairSlots) & 1u)) {
      if (lane == 0) {
        atomicExch(status, kStatusQuantTmaTimeout);
        pair_abort[pair] = 1;
      }
    }
    const uint4* src = reinterpret_cast<const uint4*>(my_slots + (size_t)sl * row_bytes);
    uint4 v[NVH];
#pragma unroll
    for (int j = 0; j < NVH; ++j) {
      const int q = lane + 32 * (2 * j + half);
      v[j] = (q < nvec_row) ? src[q] : make_uint4(0, 0, 0, 0);
    }
    const size_t row = row_of(k);
    float inv;
    if constexpr (COMPUTE_INV_RMS) {
      // acc[q]: virtual lane 4*lane + 128*half + q of the reference's 256-thread tree
      float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < NVH; ++j) {
        a4[0] = fma_sq_bf16x2(v[j].x, a4[0]);
        a4[1] = fma_sq_bf16x2(v[j].y, a4[1]);
        a4[2] = fma_sq_bf16x2(v[j].z, a4[2]);
        a4[3] = fma_sq_bf16x2(v[j].w, a4[3]);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        a4[q] += __shfl_xor_sync(0xffffffffu, a4[q], 4);
        a4[q] += __shfl_xor_sync(0xffffffffu, a4[q], 2);
        a4[q] += __shfl_xor_sync(0xffffffffu, a4[q], 1);
      }
      const float part = (a4[0] + a4[2]) + (a4[1] + a4[3]);
      float* xb = xchg + (size_t)(((k & 1) * pairs + pair) * 2) * 32;
      xb[half * 32 + lane] = part;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");   // both halves of the row are in registers, both sums written
      if (pair_abort[pair] != 0) break;
      const float other = xb[(half ^ 1) * 32 + lane];
      float s_ = half == 0 ? part + other : other + part;             // part[0] + part[1]
      s_ += __shfl_xor_sync(0xffffffffu, s_, 16);
      s_ += __shfl_xor_sync(0xffffffffu, s_, 8);
      inv = rsqrtf(s_ / static_cast<float>(K) + eps);
      if (half == 0 && lane == 0) {
        inv_rms[row] = inv;
        if (k + kStatsPairSlots < my_rows) issue(k + kStatsPairSlots);
      }
    } else {
      inv = __ldg(inv_rms + row);
      asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");   // both warps hold their halves: the slot may be refilled
      if (pair_abort[pair] != 0) break;
      if (half == 0 && lane == 0 && k + kStatsPairSlots < my_rows) issue(k + kStatsPairSlots);
    }
    if (want_amax) {
      const float2 inv2 = make_float2(inv, inv);
#pragma unroll
      for (int j = 0; j < NVH; ++j) {
        const int q = lane + 32 * (2 * j + half);
        if (q < nvec_row) {
          const float4 g01 = gamma_lo[q];
          const float4 g23 = gamma_hi[q];
          const float2 t0 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].x), bf16hi_to_f32(v[j].x)), inv2), make_float2(g01.x, g01.y));
          const float2 t1 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].y), bf16hi_to_f32(v[j].y)), inv2), make_float2(g01.z, g01.w));
          const float2 t2 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].z), bf16hi_to_f32(v[j].z)), inv2), make_float2(g23.x, g23.y));
          const float2 t3 = mul2(mul2(make_float2(bf16lo_to_f32(v[j].w), bf16hi_to_f32(v[j].w)), inv2), make_float2(g23.z, g23.w));
          mx = absmax3(mx, t0.x, t0.y);
          mx = absmax3(mx, t1.x, t1.y);
          mx = absmax3(mx, t2.x, t2.y);
          mx = absmax3(mx, t3.x, t3.y);
        }
      }
    }
  }
  float run_max = warp_max(mx);
  if (lane == 0) warp_max_s[warp] = run_max;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < warps; ++w) run_max = fmaxf(run_max, warp_max_s[w]);
    // the one rounding to bf16 that the element-wise maximum would have applied to its winner
    partials[blockIdx.x] = __bfloat162float(__float2bfloat16_rn(run_max));   // every CTA writes: nothing to clear
  }
}

// Any-K variant: the row is read twice (second read hits L1/L2).
template <bool COMPUTE_INV_RMS>
__global__ void __launch_bounds__(256)
rmsnorm_stats_generic_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                             float* __restrict__ inv_rms, float* __restrict__ partials, float eps, int M, int K,
                             int mx_tree) {
  __shared__ float warp_max_s[8];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int n_warps = gridDim.x * (blockDim.x >> 5);
  const int nvec_row = K >> 3;
  float run_max = 0.0f;
  for (int row = warp_global; row < M; row += n_warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * K);
    float inv;
    if (COMPUTE_INV_RMS && mx_tree == 2) {
      // the optional-mode NVFP4 producer's tree (see stats_inv_rms_strided); inverse RMS only
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = lane; q < nvec_row; q += 32) {
        const uint4 vv = __ldg(xr + q);
        const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = bf16lo_to_f32(w[e]), hi = bf16hi_to_f32(w[e]);
          acc[2 * e] = fmaf(lo, lo, acc[2 * e]);
          acc[2 * e + 1] = fmaf(hi, hi, acc[2 * e + 1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
        acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
      }
      float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (lane == 0) inv_rms[row] = rsqrtf(s / static_cast<float>(K) + eps);
      continue;
    }
    if (COMPUTE_INV_RMS && mx_tree == 1) {
      // the MXFP4 producer's tree (see stats_inv_rms_mx); inverse RMS only
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q0 = 0; q0 < nvec_row; q0 += 256) {
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          const int q = q0 + 32 * w + lane;
          if (q < nvec_row) {
            const uint4 vv = __ldg(xr + q);
            float a = acc[w];
            a = fma_sq_bf16x2(vv.x, a); a = fma_sq_bf16x2(vv.y, a);
            a = fma_sq_bf16x2(vv.z, a); a = fma_sq_bf16x2(vv.w, a);
            acc[w] = a;
          }
        }
      }
#pragma unroll
      for (int w = 0; w < 8; ++w) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc[w] += __shfl_xor_sync(0xffffffffu, acc[w], m);
      }
      const float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
      if (lane == 0) inv_rms[row] = rsqrtf(s / static_cast<float>(K) + eps);
      continue;
    }
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
  if (lane == 0) warp_max_s[threadIdx.x >> 5] = run_max;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) run_max = fmaxf(run_max, warp_max_s[w]);
    partials[blockIdx.x] = run_max;
  }
}

// ---------------------------------------------------------------------------------------
// Row + column quantiser
// ---------------------------------------------------------------------------------------
//
// Persistent CTAs (2 per SM, 256 threads) walk 128x128 chunks.  A chunk arrives as two TMA
// boxes of 128 rows x 64 columns in the 128-byte-swizzled layout, three chunks deep.
//   row pass   : lane = (row & 7, 32-column unit); four conflict-free 16-byte reads, optional
//                RMSNorm (normalised bf16 written back for the column pass), two 16-blocks
//                quantised, one 16-byte streaming store of codes per thread.
//   column pass: warp = 16-row group, lane = column pair; sixteen conflict-free 4-byte reads,
//                two blocks quantised, codes staged so that the write-out is 16-byte stores.
// The decode of a block's E4M3 multiplier into (coefficient, stored byte) is a 128-entry table
// built per CTA from S_enc, so a block costs one IEEE division and one cast.
// The instruction stream, not HBM, is what bounds this kernel (about 12 instructions per
// element are needed for two orientations), hence the packed mul.f32x2 and xorsign.abs forms.

constexpr int kChunk = 128;            // chunk edge in elements
constexpr int kQThreads = 256;
constexpr int kQStages = 3;
constexpr int kHalfBytes = kChunk * 128;         // one 128-row x 64-column swizzled box
constexpr int kTileBytes = 2 * kHalfBytes;       // 32 KiB of bf16

struct ScaleLut {
  float coeff;
  uint32_t stored;
};

struct QuantSmem {
  alignas(1024) uint8_t in[kQStages][kTileBytes];
  alignas(16) uint2 col_codes[8][kChunk];   // [16-row group][column] -> 8 bytes of codes
  alignas(16) uint8_t row_sc[2][1024];
  alignas(16) uint8_t col_sc[1024];
  alignas(16) float inv_rms[2][kChunk];
  alignas(16) float gamma[2][kChunk];
  alignas(16) float tile_amax[8][8];        // W2D: amax of each 16x16 tile of the chunk
  alignas(8) ScaleLut lut_row[128];
  alignas(8) ScaleLut lut_col[128];
  alignas(8) uint64_t full[kQStages];
  float amax_slot;
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
  const float* partials;   // n_partials > 0: the tensor amax (both orientations) is the maximum of these
  int n_partials;          //   per-CTA maxima of the pass-1 kernel launched before; amax_row/amax_col unused
  float* amax_out;         // with partials, optional: amax_out[0] = amax, amax_out[1] = amax / 2688
  float* amax_scalar_out;  // optional: amax_scalar_out[0] = amax_row (strip kernel only)
  int* status;
  int M, K;
  int chunks_m, chunks_k;
  int reverse;             // walk chunks from the last row block to the first
  int nhsd_heads, nhsd_seq; // > 0: x is [B, heads, seq, 64] and the matrix is [B*seq, heads*64] (strip kernel only)
  int row_pitch_bytes;     // > 0: pitch of the row-wise code matrix (it is a column slice of a wider one; strip kernel only)
  // ---- OPT instantiations only (stochastic rounding / 16-point Hadamard transform) ----
  int opt_sr_row, opt_sr_col;   // data stochastic rounding of the row pass / of the column pass
  int opt_scale_sr;             // stochastic rounding of the scale byte: every block draws one word before its data words
  int opt_row_per_stage;   // random words per 64x64 stage in the row pass's stream: 16 (launch with a column pass) or 8
  int opt_rht_row, opt_rht_col;   // per-16 Hadamard transform along K (row operand) / along M (column operand)
  int opt_sign;            // seeded sign flip before the transform
  int opt_return_row;      // 0: row-wise outputs are not written (their random words are still skipped)
  unsigned long long rng_seed, rng_offset, rng_offset_col;   // Philox key, counter offset of the row pass / column pass
  // non-null: device words {key, base} written by an earlier kernel on the stream (sr_prepare_state_kernel): the key
  // replaces rng_seed and base is added to both offsets, so a replayed CUDA graph draws from a new place every time
  const unsigned long long* rng_state;
  unsigned long long sign_seed, sign_subseq;   // sign-mask hash inputs
  // Encode-centric scale SR only: per (128x128 chunk, reference thread) the blocks that draw no scale word, bit p =
  // the block at position p of that thread's order in the row pass's stream / in the column pass's stream
  // (ec_zero_block_mask_kernel); null: every block is taken to draw one.
  const uint16_t* ec_zero_row_stream;
  const uint16_t* ec_zero_col_stream;
};

template <bool ENCODE_CENTRIC>
__device__ __forceinline__ ScaleLut lut_entry(int code, float s_enc) {
  ScaleLut e;
  const float f = e4m3_to_f32((uint8_t)code);
  if constexpr (ENCODE_CENTRIC) {
    e.coeff = f * s_enc;
    e.stored = f32_to_e4m3(1.0f / f);
  } else {
    const float s_dec = 1.0f / s_enc;
    e.coeff = fminf(1.0f / (f * s_dec), kFltMax);
    e.stored = (uint32_t)code;
  }
  return e;
}

// E4M3 code of the block's multiplier (encode-centric) or decode scale (decode-centric)
template <bool ENCODE_CENTRIC>
__device__ __forceinline__ uint32_t block_code(float b, float s_enc) {
  if constexpr (ENCODE_CENTRIC) {
    return (b <= 1.0e-9f) ? 0x7Eu : (uint32_t)f32_to_e4m3(fminf(6.0f / (b * s_enc), kFltMax));
  } else {
    return (uint32_t)f32_to_e4m3(fminf(b / 6.0f * s_enc, kFltMax));
  }
}

// The same value as block_code rounds, rounded stochastically by the block's first random word
// (reference: quantize_transpose_tuned.cuh:205-254).
template <bool ENCODE_CENTRIC>
__device__ __forceinline__ uint32_t block_code_sr(float b, float s_enc, uint32_t rbits) {
  if constexpr (ENCODE_CENTRIC) {
    return (b <= 1.0e-9f) ? 0x7Eu : (uint32_t)f32_to_e4m3_sr(fminf(6.0f / (b * s_enc), kFltMax), rbits);
  } else {
    return (uint32_t)f32_to_e4m3_sr(fminf(b / 6.0f * s_enc, kFltMax), rbits);
  }
}

// Table form of block_code for the large launches: a block maximum is a bf16 value, so for one S_enc the code is a
// function of 15 bits, and it is constant below and above a window of 24 binades (below: the multiplier saturates
// at 448 / the decode scale rounds to 0; above: the multiplier rounds to 0 / the decode scale saturates).  The window
// is placed by S_enc's exponent; entry i belongs to the bf16 value with bits base + i and is evaluated with the same
// instructions as the direct form, so the two agree bit for bit.  Encode-centric entries hold everything a block
// needs in one word — the multiplier f as bf16 (it has four significant bits) in the upper half, so that the
// coefficient f * S_enc is one multiplication away, and the stored byte in the lowest byte — because a second,
// dependent table read costs the shared-memory pipe more than the first; decode-centric entries hold the code
// (= the stored byte), whose coefficient 1 / (f * S_dec) comes from the 128-entry table.
constexpr int kCodeLutSize = 24 * 128;

template <bool ENCODE_CENTRIC>
__device__ __forceinline__ int code_lut_base_bits(float s_enc) {
  const int es = (int)((__float_as_uint(s_enc) >> 23) & 0xFFu) - 127;   // S_enc in [2^es, 2^(es+1))
  int e_hi = 13 - es;                                    // last binade of the window
  if (ENCODE_CENTRIC) e_hi = max(e_hi, -29);             // keeps the 1e-9 rule's values inside or below the window
  return (e_hi - 23 + 127) * 128;
}

template <bool ENCODE_CENTRIC>
__device__ __forceinline__ void code_lut_fill(uint32_t* lut, int base_bits, float s_enc, int tid, int n_threads) {
  for (int i = tid; i < kCodeLutSize; i += n_threads) {
    const int bits = base_bits + i;
    // bit patterns outside the finite non-negative bf16 values are never looked up
    const float b = (bits >= 0 && bits < 0x7F80) ? __uint_as_float((uint32_t)bits << 16) : 0.0f;
    const uint32_t code = block_code<ENCODE_CENTRIC>(b, s_enc);
    if constexpr (ENCODE_CENTRIC) {
      const float f = e4m3_to_f32((uint8_t)code);
      lut[i] = (__float_as_uint(f) & 0xFFFF0000u) | (uint32_t)f32_to_e4m3(1.0f / f);
    } else {
      lut[i] = code;
    }
  }
}

// (coefficient, stored byte) of the block whose maximum has these 15 bits
template <bool ENCODE_CENTRIC>
__device__ __forceinline__ ScaleLut code_lut_lookup(const uint32_t* lut, const ScaleLut* lut128, int base_bits, float s_enc,
                                                    uint32_t abs_bits) {
  const int idx = min(max((int)abs_bits - base_bits, 0), kCodeLutSize - 1);
  const uint32_t v = lut[idx];
  if constexpr (ENCODE_CENTRIC) {
    ScaleLut e;
    e.coeff = __uint_as_float(v & 0xFFFF0000u) * s_enc;
    e.stored = v & 0xFFu;
    return e;
  } else {
    return lut128[v];
  }
}

// ---- helpers of the OPT instantiations ------------------------------------------------------

// +1 / -1 per coordinate along the transformed axis (reference: tk_quantize.cu:483-488,620-627)
__device__ __forceinline__ float rht_sign(unsigned long long seed, unsigned long long subseq, unsigned long long coord) {
  unsigned long long x = seed ^ (subseq * 0xd1b54a32d192ed03ull) ^ (coord * 0x9e3779b97f4a7c15ull);
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  const uint32_t h = (uint32_t)((x ^ (x >> 31)) >> 32);
  return (h & 1u) ? 1.0f : -1.0f;
}
// 1 where the sign of that coordinate is -1
__device__ __forceinline__ uint32_t rht_sign_is_negative(unsigned long long seed, unsigned long long subseq,
                                                         unsigned long long coord) {
  return rht_sign(seed, subseq, coord) < 0.0f ? 1u : 0u;
}
// bit i = sign of coordinate coord0 + i is -1 (one thread, sixteen hashes: the slow form, for the kernels that are not
// on the fast path; the strip quantiser shares one hash per lane through a ballot instead)
__device__ __forceinline__ uint32_t rht_sign_mask16(unsigned long long seed, unsigned long long subseq,
                                                    unsigned long long coord0) {
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) m |= rht_sign_is_negative(seed, subseq, coord0 + (unsigned long long)i) << i;
  return m;
}

// unnormalised Sylvester butterflies (steps 1,2,4,8), then x0.25 (quantize_transpose_tuned.cuh:161-179)
__device__ __forceinline__ void fwht16(float (&v)[16]) {
#pragma unroll
  for (int step = 1; step < 16; step <<= 1) {
#pragma unroll
    for (int base = 0; base < 16; base += 2 * step) {
#pragma unroll
      for (int j = 0; j < step; ++j) {
        const float x = v[base + j], y = v[base + j + step];
        v[base + j] = x + y;
        v[base + j + step] = x - y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] *= 0.25f;
}

// the same transform of two independent 16-vectors at once (.x and .y), in packed fp32x2 arithmetic: the same IEEE
// additions in the same order, half the instructions
__device__ __forceinline__ void fwht16x2(float2 (&v)[16]) {
#pragma unroll
  for (int step = 1; step < 16; step <<= 1) {
#pragma unroll
    for (int base = 0; base < 16; base += 2 * step) {
#pragma unroll
      for (int j = 0; j < step; ++j) {
        const float2 x = v[base + j], y = v[base + j + step];
        v[base + j] = add2(x, y);
        v[base + j + step] = sub2(x, y);
      }
    }
  }
  const float2 q = make_float2(0.25f, 0.25f);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = mul2(v[i], q);
}

// 16 values times coeff -> 8 bytes of codes, stochastic rounding with words wsel[0..3] for the
// four groups of four elements
__device__ __forceinline__ uint2 quant16_sr(const float (&x)[16], float coeff, const uint32_t (&wsel)[4]) {
  uint32_t h[4];
#pragma unroll
  for (int g = 0; g < 4; ++g)
    h[g] = f32x4_to_e2m1x4_sr(x[4 * g] * coeff, x[4 * g + 1] * coeff, x[4 * g + 2] * coeff, x[4 * g + 3] * coeff, wsel[g]);
  return make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
}

__device__ __forceinline__ uint2 quant16_rn(const float (&x)[16], float coeff) {
  return make_uint2(f32x8_to_e2m1x8(x[0] * coeff, x[1] * coeff, x[2] * coeff, x[3] * coeff, x[4] * coeff, x[5] * coeff,
                                    x[6] * coeff, x[7] * coeff),
                    f32x8_to_e2m1x8(x[8] * coeff, x[9] * coeff, x[10] * coeff, x[11] * coeff, x[12] * coeff,
                                    x[13] * coeff, x[14] * coeff, x[15] * coeff));
}

// transform (optional sign flip, Hadamard, bf16 rounding), block scale, codes of one 16-element block
// neg_mask: bit i = element i is negated before the transform (the sign vector of the block's 16 coordinates; 0: none)
template <bool ENCODE_CENTRIC>
__device__ __forceinline__ uint2 opt_block(float (&x)[16], bool rht, uint32_t neg_mask, float s_enc,
                                           const ScaleLut* lut, bool sr, const uint32_t (&wsel)[4], uint32_t& stored,
                                           bool scale_sr = false, uint32_t scale_rbits = 0,
                                           const uint32_t* code_lut = nullptr, int code_base = 0) {
  if (rht) {
    if (neg_mask != 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] = ((neg_mask >> i) & 1u) ? -x[i] : x[i];
    }
    fwht16(x);
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = __bfloat162float(__float2bfloat16_rn(x[i]));
  }
  float bm = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(x[i]));
  // the block's values are bf16 values (inputs, or rounded after the transform), so its maximum's upper 16 bits index
  // the code table of the large launches
  const ScaleLut e = (code_lut != nullptr && !scale_sr)
                         ? code_lut_lookup<ENCODE_CENTRIC>(code_lut, lut, code_base, s_enc, __float_as_uint(bm) >> 16)
                         : lut[scale_sr ? block_code_sr<ENCODE_CENTRIC>(bm, s_enc, scale_rbits) : block_code<ENCODE_CENTRIC>(bm, s_enc)];
  stored = e.stored;
  return sr ? quant16_sr(x, e.coeff, wsel) : quant16_rn(x, e.coeff);
}

template <bool ENCODE_CENTRIC, bool NORM, bool W2D, bool OPT>
__global__ void __launch_bounds__(kQThreads, OPT ? 1 : 2)
nvfp4_quantize_kernel(const __grid_constant__ CUtensorMap tmap_x, const QuantArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  QuantSmem& sm = *reinterpret_cast<QuantSmem*>(smem_align_1024(smem_raw));

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
  auto issue_load = [&](int it, int s) {
    int cm, ck;
    chunk_coords(it, cm, ck);
    mbar_expect_tx(&sm.full[s], kTileBytes);
    tma_load_2d(sm.in[s], &tmap_x, ck * kChunk, cm * kChunk, &sm.full[s]);
    tma_load_2d(sm.in[s] + kHalfBytes, &tmap_x, ck * kChunk + 64, cm * kChunk, &sm.full[s]);
  };

  if (tid == 0) {
    tma_prefetch_desc(&tmap_x);
    for (int s = 0; s < kQStages; ++s) mbar_init(&sm.full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0) {
    for (int s = 0; s < kQStages && s < my_count; ++s) issue_load(s, s);
  }
  // The input is never written by the pass-1 kernel this one may have been launched behind, so the
  // first chunks are already on their way; amax / inv_rms are that kernel's results.
  pdl_wait();
  float amax_r, amax_c;
  if (a.n_partials > 0) {
    amax_r = amax_c = amax_from_partials(a.partials, a.n_partials, &sm.amax_slot);
    if (tid == 0 && blockIdx.x == 0 && a.amax_out != nullptr) {
      a.amax_out[0] = amax_r;
      a.amax_out[1] = amax_r / 2688.0f;
    }
  } else {
    amax_r = *a.amax_row;
    amax_c = *a.amax_col;
  }
  if (tid == 0 && blockIdx.x == 0 && a.sg_out != nullptr) a.sg_out[0] = amax_r / 2688.0f;

  const float s_enc_row = nvfp4_global_encode_scale(amax_r);
  const float s_enc_col = nvfp4_global_encode_scale(amax_c);
  const bool want_col = a.col_fp4 != nullptr;
  if (tid < 128) sm.lut_row[tid] = lut_entry<ENCODE_CENTRIC>(tid, s_enc_row);
  else sm.lut_col[tid - 128] = lut_entry<ENCODE_CENTRIC>(tid - 128, s_enc_col);
  // Philox key and the two counter offsets of this launch (OPT): from the arguments, or from the device words an
  // earlier kernel on the stream prepared (a.rng_state)
  __shared__ volatile unsigned long long rng_s[3];   // volatile: read where used, not held in registers across the loop
  if (OPT && tid == 0) {
    const unsigned long long base = a.rng_state != nullptr ? a.rng_state[1] : 0ull;
    rng_s[0] = a.rng_state != nullptr ? a.rng_state[0] : a.rng_seed;
    rng_s[1] = a.rng_offset + base;
    rng_s[2] = a.rng_offset_col + base;
  }
  if constexpr (NORM) {
    if (my_count > 0) {
      int cm, ck;
      chunk_coords(0, cm, ck);
      if (tid < kChunk) sm.inv_rms[0][tid] = __ldg(a.inv_rms + cm * kChunk + tid);
      else sm.gamma[0][tid - kChunk] = __bfloat162float(a.gamma[ck * kChunk + tid - kChunk]);
    }
  }
  __syncthreads();

  // row-pass geometry of this thread (loop invariant)
  const int unit = lane >> 3;                    // which 32 columns of the chunk
  const int r_lo = lane & 7;
  const int half_off = (unit >> 1) * kHalfBytes;
  const int cb = (unit & 1) * 4;                 // first 16-byte column group inside the half
  int row_off[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) row_off[j] = ((cb + j) ^ r_lo) << 4;
  // column-pass geometry
  int col_off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) col_off[j] = (((lane >> 2) ^ j) << 4) + (lane & 3) * 4;

  for (int it = 0; it < my_count; ++it) {
    const int s = it % kQStages;
    const uint32_t parity = (it / kQStages) & 1;
    int cm, ck;
    chunk_coords(it, cm, ck);
    const int m0 = cm * kChunk, k0 = ck * kChunk;
    const int pp = it & 1;

    // prefetch the next chunk's inv_rms / gamma into a register (stored after the column pass)
    // (raw bits: converting here would wait for the load before the chunk's work starts)
    uint32_t pre = 0;
    if constexpr (NORM) {
      if (it + 1 < my_count) {
        int ncm, nck;
        chunk_coords(it + 1, ncm, nck);
        pre = (tid < kChunk) ? __ldg(reinterpret_cast<const uint32_t*>(a.inv_rms) + ncm * kChunk + tid)
                             : (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(a.gamma) + nck * kChunk + tid - kChunk) << 16;
      }
    }

    if (!mbar_wait_bounded(&sm.full[s], parity)) {
      if (tid == 0) atomicExch(a.status, kStatusQuantTmaTimeout);
      return;
    }
    uint8_t* tile = sm.in[s];

    if constexpr (W2D) {
      // 16x16-tile amaxes (one scale shared by both orientations): column-pass geometry, then a
      // max over the 8 lanes that hold one 16-column block
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint8_t* base = tile + h * kHalfBytes + (warp * 16) * 128;
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          mx = absmax_xs(mx, *reinterpret_cast<const uint32_t*>(base + i * 128 + col_off[i & 7]));
        float b = fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx)));
        b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 1));
        b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 2));
        b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 4));
        if ((lane & 7) == 0) sm.tile_amax[warp][h * 4 + (lane >> 3)] = b;
      }
      __syncthreads();
    }

    // ---- row pass ---------------------------------------------------------------------
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
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
      if constexpr (OPT) {
        // The stochastic-rounding stream follows the reference kernel's thread/draw order, so that the
        // same (seed, offset) gives the same word to the same element: 128 threads per chunk, four
        // 64x64 stages, per stage a row pass (2 iterations x 4 words) then a column pass (2 x 4 words);
        // a 16-element block consumes exactly one Philox block (quantize_transpose_tuned.cuh:392-528).
        const int per_stage = a.opt_row_per_stage;
        uint32_t st_b[2];
        uint2 cd[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float x[16];
#pragma unroll
          for (int q = 0; q < 8; ++q) { x[2 * q] = bf16lo_to_f32(w[8 * b + q]); x[2 * q + 1] = bf16hi_to_f32(w[8 * b + q]); }
          const int lc0 = unit * 32 + b * 16;           // first column of the block inside the chunk
          uint32_t wsel[4] = {0, 0, 0, 0};
          if (a.opt_sr_row) {
            const int stage = (r >> 6) * 2 + (lc0 >> 6);
            const int lr = r & 63, it_ref = lr >> 5;
            const int tid_ref = (lr & 31) * 4 + ((lc0 & 63) >> 4);
            const unsigned long long seq = (unsigned long long)tid_ref + 128ull * (unsigned long long)ck +
                                           128ull * (unsigned long long)a.chunks_k * (unsigned long long)cm;
            const uint4 rw = philox4x32_10(rng_s[0], seq,
                                           rng_s[1] + (unsigned long long)((stage * per_stage + it_ref * 4) >> 2));
            const uint32_t words[4] = {rw.x, rw.y, rw.z, rw.w};
            const int bg = (tid_ref & 31) >> 4;
#pragma unroll
            for (int g = 0; g < 4; ++g) wsel[g] = words[2 * (((g >> 1) - bg) & 1) + (g & 1)];
          }
          const uint32_t neg = (a.opt_sign && a.opt_rht_row) ? rht_sign_mask16(a.sign_seed, a.sign_subseq, (unsigned long long)(k0 + lc0)) : 0u;
          cd[b] = opt_block<ENCODE_CENTRIC>(x, a.opt_rht_row != 0, neg, s_enc_row, sm.lut_row, a.opt_sr_row != 0, wsel, st_b[b]);
        }
        if (a.opt_return_row) {
          st_cs_u4(a.row_fp4 + (size_t)(m0 + r) * (a.K >> 1) + ((k0 + unit * 32) >> 1),
                   make_uint4(cd[0].x, cd[0].y, cd[1].x, cd[1].y));
          *reinterpret_cast<uint16_t*>(&sm.row_sc[pp][(unit >> 1) * 512 + scale_tile_offset(r, (unit & 1) * 2)]) =
              (uint16_t)(st_b[0] | (st_b[1] << 8));
        }
      } else {
        uint32_t mx0 = 0, mx1 = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) { mx0 = absmax_xs(mx0, w[q]); mx1 = absmax_xs(mx1, w[8 + q]); }
        float b0 = fmaxf(fabsf(bf16lo_to_f32(mx0)), fabsf(bf16hi_to_f32(mx0)));
        float b1 = fmaxf(fabsf(bf16lo_to_f32(mx1)), fabsf(bf16hi_to_f32(mx1)));
        if constexpr (W2D) {
          b0 = sm.tile_amax[r >> 4][unit * 2];
          b1 = sm.tile_amax[r >> 4][unit * 2 + 1];
        }
        const ScaleLut e0 = sm.lut_row[block_code<ENCODE_CENTRIC>(b0, s_enc_row)];
        const ScaleLut e1 = sm.lut_row[block_code<ENCODE_CENTRIC>(b1, s_enc_row)];
        uint4 codes;
        codes.x = quant8(w, e0.coeff);
        codes.y = quant8(w + 4, e0.coeff);
        codes.z = quant8(w + 8, e1.coeff);
        codes.w = quant8(w + 12, e1.coeff);
        st_cs_u4(a.row_fp4 + (size_t)(m0 + r) * (a.K >> 1) + ((k0 + unit * 32) >> 1), codes);
        // blocks kb = 2*unit, 2*unit+1 of tile kb>>2 = unit>>1: two adjacent bytes
        *reinterpret_cast<uint16_t*>(&sm.row_sc[pp][(unit >> 1) * 512 + scale_tile_offset(r, (unit & 1) * 2)]) =
            (uint16_t)(e0.stored | (e1.stored << 8));
      }
    }
    __syncthreads();

    // ---- column pass ------------------------------------------------------------------
    if (want_col) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint8_t* base = tile + h * kHalfBytes + (warp * 16) * 128;
        uint32_t w[16];
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          w[i] = *reinterpret_cast<const uint32_t*>(base + i * 128 + col_off[i & 7]);
          mx = absmax_xs(mx, w[i]);
        }
        uint4 q;
        uint32_t st0, st1;
        if constexpr (OPT) {
          uint2 cd[2];
          uint32_t st_c[2];
#pragma unroll
          for (int wq = 0; wq < 2; ++wq) {
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = wq ? bf16hi_to_f32(w[i]) : bf16lo_to_f32(w[i]);
            uint32_t wsel[4] = {0, 0, 0, 0};
            if (a.opt_sr_col) {
              const int stage = (warp >> 2) * 2 + h;
              const int tid_ref = (((warp & 3) - (lane & 3)) & 3) * 32 + lane;
              const unsigned long long seq = (unsigned long long)tid_ref + 128ull * (unsigned long long)ck +
                                             128ull * (unsigned long long)a.chunks_k * (unsigned long long)cm;
              const uint4 rw = philox4x32_10(rng_s[0], seq, rng_s[2] + (unsigned long long)((stage * 16 + 8 + wq * 4) >> 2));
              wsel[0] = rw.x; wsel[1] = rw.y; wsel[2] = rw.z; wsel[3] = rw.w;
            }
            const uint32_t neg = (a.opt_sign && a.opt_rht_col) ? rht_sign_mask16(a.sign_seed, a.sign_subseq, (unsigned long long)(m0 + warp * 16)) : 0u;
            cd[wq] = opt_block<ENCODE_CENTRIC>(x, a.opt_rht_col != 0, neg, s_enc_col, sm.lut_col, a.opt_sr_col != 0, wsel, st_c[wq]);
          }
          q = make_uint4(cd[0].x, cd[0].y, cd[1].x, cd[1].y);
          st0 = st_c[0]; st1 = st_c[1];
        }
        if constexpr (!OPT) {
          float b0 = fabsf(bf16lo_to_f32(mx)), b1 = fabsf(bf16hi_to_f32(mx));
          if constexpr (W2D) b0 = b1 = sm.tile_amax[warp][h * 4 + (lane >> 3)];
          const ScaleLut e0 = sm.lut_col[block_code<ENCODE_CENTRIC>(b0, s_enc_col)];
          const ScaleLut e1 = sm.lut_col[block_code<ENCODE_CENTRIC>(b1, s_enc_col)];
          const float2 cc = make_float2(e0.coeff, e1.coeff);
          float2 v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = mul2(make_float2(bf16lo_to_f32(w[i]), bf16hi_to_f32(w[i])), cc);
          q.x = f32x8_to_e2m1x8(v[0].x, v[1].x, v[2].x, v[3].x, v[4].x, v[5].x, v[6].x, v[7].x);
          q.y = f32x8_to_e2m1x8(v[8].x, v[9].x, v[10].x, v[11].x, v[12].x, v[13].x, v[14].x, v[15].x);
          q.z = f32x8_to_e2m1x8(v[0].y, v[1].y, v[2].y, v[3].y, v[4].y, v[5].y, v[6].y, v[7].y);
          q.w = f32x8_to_e2m1x8(v[8].y, v[9].y, v[10].y, v[11].y, v[12].y, v[13].y, v[14].y, v[15].y);
          st0 = e0.stored;
          st1 = e1.stored;
        }
        const int c = 2 * lane + 64 * h;
        *reinterpret_cast<uint4*>(&sm.col_codes[warp][c]) = q;   // columns c and c+1
        sm.col_sc[(warp >> 2) * 512 + scale_tile_offset(c, warp & 3)] = (uint8_t)st0;
        sm.col_sc[(warp >> 2) * 512 + scale_tile_offset(c + 1, warp & 3)] = (uint8_t)st1;
      }
    }
    if constexpr (NORM) {
      // the other inv_rms/gamma buffer was last read in the previous chunk's row pass
      if (tid < kChunk) sm.inv_rms[pp ^ 1][tid] = __uint_as_float(pre);
      else sm.gamma[pp ^ 1][tid - kChunk] = __uint_as_float(pre);
    }
    __syncthreads();

    // stage s is free again: refill it with the chunk kQStages ahead
    if (tid == 0 && it + kQStages < my_count) {
      fence_proxy_async_smem();
      issue_load(it + kQStages, s);
    }

    // ---- write-out: scales (two 512-byte tiles per orientation) and column codes -----
    if (!OPT || a.opt_return_row) {
      uint8_t* dst = a.row_sc + ((size_t)cm * (a.K >> 6) + (size_t)ck * 2) * 512;
      st_cs_u32(dst + tid * 4, *reinterpret_cast<const uint32_t*>(&sm.row_sc[pp][tid * 4]));
    }
    if (want_col) {
      uint8_t* dst = a.col_sc + ((size_t)ck * (a.M >> 6) + (size_t)cm * 2) * 512;
      st_cs_u32(dst + tid * 4, *reinterpret_cast<const uint32_t*>(&sm.col_sc[tid * 4]));
#pragma unroll
      for (int rep = 0; rep < 2; ++rep) {
        const int idx = rep * kQThreads + tid;   // 512 pieces of 16 bytes: column = idx/4, 32-row part = idx%4
        const int c = idx >> 2, part = idx & 3;
        const uint2 lo = sm.col_codes[2 * part][c];
        const uint2 hi = sm.col_codes[2 * part + 1][c];
        st_cs_u4(a.col_fp4 + (size_t)(k0 + c) * (a.M >> 1) + (m0 >> 1) + part * 16,
                 make_uint4(lo.x, lo.y, hi.x, hi.y));
      }
      // col_codes / col_sc are next written after the barrier that follows the next chunk's row
      // pass, which every thread reaches only after this loop: no barrier needed here
    }
  }
}


// ---------------------------------------------------------------------------------------
// Row + column quantiser, warp-autonomous form (round-to-nearest, 1-D blocks)
// ---------------------------------------------------------------------------------------
//
// One CTA of 16 warps per SM and no CTA-wide barrier after start-up.  A warp owns a strip of
// 32 rows x 64 columns (one TMA box, 4 KiB, 128-byte swizzle), two private strip slots with one
// mbarrier each, and 1 KiB of staging for its row codes; it quantises its strip in both orientations
// by itself:
//   row pass   : lane = row; eight conflict-free 16-byte reads, optional RMSNorm (normalised bf16
//                written back for the column pass), four 16-blocks -> 32 bytes of codes (staged)
//                and one 32-bit word of scales (stored straight to global memory);
//   column pass: lane = column pair; 32 conflict-free 4-byte reads, two 16-row blocks per column
//                -> 16 bytes of codes per column and two scale bytes, stored straight to global memory.
// The row codes leave as one TMA store per strip (32 rows x 32 B into [M, K/2]); the column codes
// (16 B per column) are stored per lane.  Two units set the pace besides instruction issue: the L1
// data path, which carries shared-memory traffic as well as global stores (a per-lane store touching
// 32 lines occupies it 32 cycles), and the TMA unit, whose cost is per box ROW (~3 cycles each,
// whatever the row's length); splitting the outputs this way loads both about equally.
// Eight warps (4 down x 2 across) cover the same 128 x 128 chunks, in the same order, as the
// CTA-synchronous kernel above, so neighbouring pieces of the outputs are written within a few
// microseconds of each other.  Warps drift freely: nothing waits at a barrier.

// Which 16-element blocks of x draw no scale word under encode-centric scale stochastic rounding: the reference
// stores the largest multiplier for a block whose maximum is <= 1e-9 before it would have drawn
// (quantize_transpose_tuned.cuh:244-254), and since a thread of its tuned kernel draws its words one after another,
// every later draw of that thread inside the 128x128 chunk moves up by one.  One CTA per chunk, one thread per
// reference thread t: its row blocks are rows 64*sy + (t >> 2) + 32*it, columns 16*(4*sx + (t & 3)) .. +15 of stage
// (sy, sx), its column blocks rows 64*sy + 16*g .. +15 of column 64*sx + 2*(t & 31) + wq with
// g = ((t >> 5) + (t & 3)) & 3.  Bit p of a mask = the block at position p of the thread's order in that stream:
// stage * sb + it for row blocks (sb = blocks per stage of the stream: 2 in a row-only launch, else 4) and
// stage * 4 + 2 + wq for column blocks.  The maxima are those of the raw input (exact for the plain quantiser; with a
// Hadamard transform or RMSNorm in front a block is taken to be zero when its input is).
__global__ void __launch_bounds__(128)
ec_zero_block_mask_kernel(const __nv_bfloat16* __restrict__ x, int K, int chunks_k, int sb_row_stream,
                          int rows_in_row_stream, int cols_in_row_stream, int rows_in_col_stream,
                          uint16_t* __restrict__ mask_row_stream, uint16_t* __restrict__ mask_col_stream) {
  const int chunk = blockIdx.x, t = threadIdx.x;
  const int cm = chunk / chunks_k, ck = chunk - cm * chunks_k;
  const __nv_bfloat16* base = x + (size_t)cm * 128 * K + (size_t)ck * 128;
  uint32_t zr = 0, zc = 0;   // bit stage*2 + it / stage*2 + wq
#pragma unroll
  for (int stage = 0; stage < 4; ++stage) {
    const int sy = stage >> 1, sx = stage & 1;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const uint4* p = reinterpret_cast<const uint4*>(base + (size_t)(64 * sy + (t >> 2) + 32 * it) * K + 16 * (4 * sx + (t & 3)));
      const uint4 a = __ldg(p), b = __ldg(p + 1);
      uint32_t m = bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(0u, a.x), a.y), bf16x2_absmax(bf16x2_absmax(0u, a.z), a.w));
      m = bf16x2_absmax(m, bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(0u, b.x), b.y), bf16x2_absmax(bf16x2_absmax(0u, b.z), b.w)));
      if (bf16x2_hmax_to_f32(m) <= 1.0e-9f) zr |= 1u << (stage * 2 + it);
    }
    const int g = ((t >> 5) + (t & 3)) & 3;
#pragma unroll
    for (int wq = 0; wq < 2; ++wq) {
      const __nv_bfloat16* p = base + (size_t)(64 * sy + 16 * g) * K + 64 * sx + 2 * (t & 31) + wq;
      float m = 0.0f;
#pragma unroll
      for (int r = 0; r < 16; ++r) m = fmaxf(m, fabsf(__bfloat162float(p[(size_t)r * K])));
      if (m <= 1.0e-9f) zc |= 1u << (stage * 2 + wq);
    }
  }
  uint32_t mr = 0, mc = 0;
#pragma unroll
  for (int stage = 0; stage < 4; ++stage) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t r = (zr >> (stage * 2 + i)) & 1u, c = (zc >> (stage * 2 + i)) & 1u;
      if (rows_in_row_stream) mr |= r << (stage * sb_row_stream + i);
      if (cols_in_row_stream) mr |= c << (stage * 4 + 2 + i);
      if (rows_in_col_stream) mc |= r << (stage * 4 + i);
      mc |= c << (stage * 4 + 2 + i);
    }
  }
  mask_row_stream[(size_t)chunk * 128 + t] = (uint16_t)mr;
  mask_col_stream[(size_t)chunk * 128 + t] = (uint16_t)mc;
}

constexpr int kStripRows = 32;
constexpr int kStripCols = 64;
constexpr int kStripBytes = kStripRows * kStripCols * 2;
constexpr int kStripWarps = 16;
constexpr int kStripDepth = 2;          // input slots per warp: one being processed, one in flight
constexpr int kStripStageBytes = 1024;  // per warp: row codes of one strip awaiting their TMA store

constexpr int kStripColStageBytes = 2048;   // per warp, paired form: column codes of two strips (64 columns x 32 B)

__host__ __device__ constexpr size_t strip_smem_bytes(int64_t k_norm, bool pair) {
  return (size_t)kStripWarps * (kStripDepth * kStripBytes + kStripStageBytes * (pair ? 2 : 1) + (pair ? kStripColStageBytes : 0)) +
         2 * 128 * sizeof(ScaleLut) + (size_t)kStripWarps * kStripDepth * sizeof(uint64_t) + 16 +
         (size_t)k_norm * sizeof(float) + (pair ? (k_norm > 0 ? 1 : 2) * kCodeLutSize * sizeof(uint32_t) : 0) + 1024;
}

// OPT: 0 = round to nearest, no transform; 1 = the optional modes (stochastic rounding of the codes, Hadamard
// transform, sign mask, row operand optional); 2 = those plus stochastic rounding of the scale bytes (a kernel
// of its own, so that the extra random-word bookkeeping costs the usual modes no registers).
// The work of CTA `cta` of the `n_ctas` that share one matrix (the whole grid, or one problem's range of a grouped
// launch); tmap_x, tmap_row and a name kernel parameters.
template <bool ENCODE_CENTRIC, bool NORM, int OPT, bool PAIR>
__device__ __forceinline__ void quantize_strip_cta(const CUtensorMap& tmap_x, const CUtensorMap& tmap_row, const QuantArgs& a,
                                                   const int cta, const int n_ctas) {
  constexpr int depth = kStripDepth;
  constexpr bool kScaleSr = OPT == 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = smem_align_1024(smem_raw);
  uint8_t* slots = base;                                                       // [warp][depth][4 KiB]
  uint8_t* staging = base + (size_t)kStripWarps * depth * kStripBytes;         // [warp][2 KiB]
  uint8_t* col_staging = staging + (size_t)kStripWarps * kStripStageBytes * (PAIR ? 2 : 1);   // [warp][2 KiB] (PAIR)
  ScaleLut* lut_row = reinterpret_cast<ScaleLut*>(col_staging + (PAIR ? (size_t)kStripWarps * kStripColStageBytes : 0));
  ScaleLut* lut_col = lut_row + 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(lut_col + 128);                 // [warp][depth]
  float* amax_slot = reinterpret_cast<float*>(bars + kStripWarps * depth);     // 16 bytes
  float* gamma_f = amax_slot + 4;                                              // [K] (NORM)
  // the large launches look block codes up (not with scale SR: its codes are drawn; not RMSNorm + modes: the two
  // operands' tensor scales differ there and the paired RMSNorm form keeps one table)
  constexpr bool kCodeLut = PAIR && (OPT == 0 || (OPT == 1 && !NORM));
  // [kCodeLutSize], and a second one for the column operand unless NORM (one tensor maximum for both operands)
  uint32_t* code_lut_row = reinterpret_cast<uint32_t*>(gamma_f + (NORM ? a.K : 0));
  uint32_t* code_lut_col = NORM ? code_lut_row : code_lut_row + kCodeLutSize;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // the same value, known to be uniform across the warp
  // Eight warps per chunk, one strip each (4 down x 2 across), or, paired, four warps per chunk with two
  // vertically adjacent strips each (2 x 2 down, 2 across): a paired warp collects the column codes of both
  // strips in shared memory and stores 32 contiguous bytes per column after the lower one.
  // A warp's unit of work is its share of one chunk: one strip, or, paired, the two strips (64 rows x 64 columns).
  constexpr int pair = PAIR ? 1 : 0;
  constexpr int halves = PAIR ? 2 : 1;
  const int wv_base = pair ? (warp & 1) * 2 : (warp & 3);   // first 32-row band of the chunk this warp works on
  const int wh = pair ? (warp >> 1) & 1 : (warp >> 2) & 1;  // which 64 columns of the chunk
  const int groups = pair ? 4 : 2;                           // chunks the CTA works on at a time
  const int n_chunks = a.chunks_m * a.chunks_k;
  const int first = cta * groups + (pair ? warp >> 2 : warp >> 3);
  const int step = n_ctas * groups;
  const int my_units = first < n_chunks ? (n_chunks - first + step - 1) / step : 0;
  uint8_t* my_slots = slots + (size_t)warp * depth * kStripBytes;
  uint64_t* my_bars = bars + warp * depth;
  uint8_t* my_stage = staging + (size_t)warp * (kStripStageBytes * halves);
  uint8_t* my_col_stage = col_staging + (size_t)warp * kStripColStageBytes;

  // The warp's chunks are first, first + step, ... (counted from the last chunk backwards when a.reverse): the
  // (row block, column block) pair of the next one follows from the current one by two additions and a wrap.
  const int step_m = step / a.chunks_k, step_k = step - step_m * a.chunks_k;
  auto advance = [&](int& m, int& k) {
    if (!a.reverse) {
      k += step_k; m += step_m;
      if (k >= a.chunks_k) { k -= a.chunks_k; ++m; }
    } else {
      k -= step_k; m -= step_m;
      if (k < 0) { k += a.chunks_k; --m; }
    }
  };
  int cm = 0, ck = 0;   // the unit being worked on
  if (my_units > 0) {
    const int c = a.reverse ? n_chunks - 1 - first : first;
    cm = c / a.chunks_k;
    ck = c - cm * a.chunks_k;
  }
  const uint64_t use_once = l2_policy_evict_first();   // the input's last use and the outputs: nothing to keep in L2
  auto issue_load = [&](int m, int k, int h, int s) {
    mbar_expect_tx(&my_bars[s], kStripBytes);
    int x = k * kChunk + wh * kStripCols, y = m * kChunk + (wv_base + h) * kStripRows;
    if (a.nhsd_seq > 0) {
      // head-major input: the strip (32 tokens of one sequence x one 64-wide head) is a contiguous block of the
      // [B * heads * seq, 64] matrix the tensor map describes (seq is a multiple of 128: no strip straddles two)
      const int b = y / a.nhsd_seq;
      y = (b * a.nhsd_heads + (x >> 6)) * a.nhsd_seq + (y - b * a.nhsd_seq);
      x = 0;
    }
    // read once here: the lines (kept in L2 by the statistics pass for this kernel) become the first to go
    tma_load_2d_hint(my_slots + (size_t)s * kStripBytes, &tmap_x, x, y, &my_bars[s], use_once);
  };

  if (tid == 0) {
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_row);
    for (int i = 0; i < kStripWarps * depth; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  __syncthreads();
  // A statistics kernel launched behind this one (the next call of the fused producer) may set up and fill its ring
  // as SMs free up; it writes nothing before this kernel has ended.
  pdl_launch_dependents();
  // Both slots are filled before the loop: paired, with the two strips of the first unit (slot = half, and a slot
  // is refilled with the same half of the next unit); else with the first two units (slot = unit & 1).
  int lm = cm, lk = ck, l_idx = 0;   // the next unit to request
  if (my_units > 0) {
    if (lane == 0) issue_load(lm, lk, 0, 0);
    if constexpr (PAIR) {
      if (lane == 0) issue_load(lm, lk, 1, 1);
    }
    advance(lm, lk);
    l_idx = 1;
    if constexpr (!PAIR) {
      if (my_units > 1) {
        if (lane == 0) issue_load(lm, lk, 0, 1);
        advance(lm, lk);
        l_idx = 2;
      }
    }
  }
  // The input is never written by the pass-1 kernel this one may have been launched behind, so the
  // first strips are already on their way; amax / inv_rms are that kernel's results.
  pdl_wait();
  float amax_r, amax_c;
  if (a.n_partials > 0) {
    amax_r = amax_c = amax_from_partials(a.partials, a.n_partials, amax_slot);
    if (tid == 0 && cta == 0 && a.amax_out != nullptr) {
      a.amax_out[0] = amax_r;
      a.amax_out[1] = amax_r / 2688.0f;
    }
  } else {
    amax_r = *a.amax_row;
    amax_c = *a.amax_col;
  }
  if (tid == 0 && cta == 0 && a.sg_out != nullptr) a.sg_out[0] = amax_r / 2688.0f;
  if (tid == 0 && cta == 0 && a.amax_scalar_out != nullptr) a.amax_scalar_out[0] = amax_r;
  const float s_enc_row = nvfp4_global_encode_scale(amax_r);
  const float s_enc_col = nvfp4_global_encode_scale(amax_c);
  const bool want_col = a.col_fp4 != nullptr;
  if (tid < 128) lut_row[tid] = lut_entry<ENCODE_CENTRIC>(tid, s_enc_row);
  else if (tid < 256) lut_col[tid - 128] = lut_entry<ENCODE_CENTRIC>(tid - 128, s_enc_col);
  // Philox key and the two counter offsets of this launch (OPT): from the arguments, or from the device words an
  // earlier kernel on the stream prepared (a.rng_state)
  __shared__ volatile unsigned long long rng_s[3];   // volatile: read where used, not held in registers across the loop
  if (OPT != 0 && tid == 0) {
    const unsigned long long base = a.rng_state != nullptr ? a.rng_state[1] : 0ull;
    rng_s[0] = a.rng_state != nullptr ? a.rng_state[0] : a.rng_seed;
    rng_s[1] = a.rng_offset + base;
    rng_s[2] = a.rng_offset_col + base;
  }
  int code_base_row = 0, code_base_col = 0;
  if constexpr (kCodeLut) {
    code_base_row = code_lut_base_bits<ENCODE_CENTRIC>(s_enc_row);
    code_base_col = code_lut_base_bits<ENCODE_CENTRIC>(s_enc_col);
    code_lut_fill<ENCODE_CENTRIC>(code_lut_row, code_base_row, s_enc_row, tid, kStripWarps * 32);
    if (NORM || s_enc_col == s_enc_row) code_lut_col = code_lut_row;
    else if (want_col) code_lut_fill<ENCODE_CENTRIC>(code_lut_col, code_base_col, s_enc_col, tid, kStripWarps * 32);
  }
  if constexpr (NORM) {
    for (int q = tid; q < (a.K >> 1); q += kStripWarps * 32) {
      const uint32_t g = __ldg(reinterpret_cast<const uint32_t*>(a.gamma) + q);
      *reinterpret_cast<float2*>(gamma_f + 2 * q) = make_float2(bf16lo_to_f32(g), bf16hi_to_f32(g));
    }
  }
  __syncthreads();

  // loop-invariant geometry
  const int sw = lane & 7;
  int row_off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) row_off[j] = lane * 128 + ((j ^ sw) << 4);
  int col_off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) col_off[j] = j * 128 + ((((lane >> 2) ^ j) << 4) | ((lane & 3) << 2));

  // lane-constant parts of the output addresses
  const int cin = wh * kStripCols + 2 * lane;   // this lane's first column inside the 128-column tile
  const int col_sc_lane0 = scale_tile_offset(cin, 0), col_sc_lane1 = scale_tile_offset(cin + 1, 0);
  const size_t col_pitch = (size_t)(a.M >> 1);
  const size_t row_sc_tiles_per_row_block = (size_t)(a.K >> 6);
  const size_t col_sc_tiles_per_col_block = (size_t)(a.M >> 6);

  float inv_next[halves];
#pragma unroll
  for (int h = 0; h < halves; ++h) inv_next[h] = 0.0f;
  if constexpr (NORM) {
    if (my_units > 0) {
#pragma unroll
      for (int h = 0; h < halves; ++h) inv_next[h] = __ldg(a.inv_rms + cm * kChunk + (wv_base + h) * kStripRows + lane);
    }
  }
  uint32_t held_sc = 0;   // paired: the upper strip's column scale bytes (two per column)
  bool ok = true;

  for (int u = 0; u < my_units && ok; ++u) {
    int nm = cm, nk = ck;
    advance(nm, nk);
    float inv_unit[halves];
#pragma unroll
    for (int h = 0; h < halves; ++h) inv_unit[h] = inv_next[h];
    if constexpr (NORM) {
      if (u + 1 < my_units) {
#pragma unroll
        for (int h = 0; h < halves; ++h) inv_next[h] = __ldg(a.inv_rms + nm * kChunk + (wv_base + h) * kStripRows + lane);
      }
    }
    const int col0 = ck * kChunk + wh * kStripCols;      // first column of the unit
    uint8_t* const row_sc_unit = a.row_sc + (((size_t)cm * row_sc_tiles_per_row_block + (size_t)(col0 >> 6)) << 9) + lane * 16;

#pragma unroll
    for (int half = 0; half < halves; ++half) {
    const int s = PAIR ? half : (u & 1);
    const uint32_t parity = PAIR ? ((uint32_t)u & 1u) : (((uint32_t)u >> 1) & 1u);
    const int wv = wv_base + half;                       // which 32 rows of the chunk
    const int row0 = cm * kChunk + wv * kStripRows;      // first row of the strip
    const float inv = inv_unit[half];
    if (!mbar_wait_bounded(&my_bars[s], parity)) {
      if (lane == 0) atomicExch(a.status, kStatusQuantTmaTimeout);
      ok = false;
      break;
    }
    uint8_t* tile = my_slots + (size_t)s * kStripBytes;

    // ---- row pass: lane = row ----------------------------------------------------------
    {
      uint32_t w[32];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(tile + row_off[j]);
        w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
      }
      if constexpr (NORM) {
        const float2 inv2 = make_float2(inv, inv);
        const float4* g4 = reinterpret_cast<const float4*>(gamma_f + col0);   // same address on all lanes
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float4 g = g4[q];
          float2 t0 = mul2(make_float2(bf16lo_to_f32(w[2 * q]), bf16hi_to_f32(w[2 * q])), inv2);
          float2 t1 = mul2(make_float2(bf16lo_to_f32(w[2 * q + 1]), bf16hi_to_f32(w[2 * q + 1])), inv2);
          t0 = mul2(t0, make_float2(g.x, g.y));
          t1 = mul2(t1, make_float2(g.z, g.w));
          w[2 * q] = f32x2_to_bf16x2(t0.x, t0.y);
          w[2 * q + 1] = f32x2_to_bf16x2(t1.x, t1.y);
        }
        if (want_col) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(tile + row_off[j]) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        }
      }
      uint32_t codes[8];
      uint32_t sc_word = 0;
      if constexpr (OPT != 0) {
        // Stochastic rounding follows the reference kernel's thread/draw order inside the 128x128 chunk
        // (128 threads, four 64x64 stages, per stage a row pass of 2 iterations x 4 words and, when the
        // launch has one, a column pass of 2 x 4 words; quantize_transpose_tuned.cuh:392-528): the word
        // for an element depends only on its position, so any kernel shape reproduces it.
        const int rc = wv * kStripRows + lane;        // row inside the chunk
        // sign vector of the strip's 64 columns: one hash per lane and half, shared through a ballot
        uint32_t row_neg_lo = 0, row_neg_hi = 0;
        if (a.opt_sign && a.opt_rht_row && a.opt_return_row) {
          row_neg_lo = __ballot_sync(0xffffffffu, rht_sign_is_negative(a.sign_seed, a.sign_subseq, (unsigned long long)(col0 + lane)) != 0);
          row_neg_hi = __ballot_sync(0xffffffffu, rht_sign_is_negative(a.sign_seed, a.sign_subseq, (unsigned long long)(col0 + 32 + lane)) != 0);
        }
        if (a.opt_return_row && !kScaleSr && !a.opt_rht_row && !a.opt_sr_row) {
          // a row operand without any of the modes (only the column operand is transformed or rounded
          // stochastically): the round-to-nearest kernel's row arithmetic
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            uint32_t mx = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) mx = absmax_xs(mx, w[8 * b + q]);
            ScaleLut e;
            if constexpr (kCodeLut) {
              const uint32_t am = mx & 0x7FFF7FFFu;
              e = code_lut_lookup<ENCODE_CENTRIC>(code_lut_row, lut_row, code_base_row, s_enc_row, max(am >> 16, am & 0xFFFFu));
            } else {
              e = lut_row[block_code<ENCODE_CENTRIC>(fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx))), s_enc_row)];
            }
            codes[2 * b] = quant8(w + 8 * b, e.coeff);
            codes[2 * b + 1] = quant8(w + 8 * b + 4, e.coeff);
            sc_word |= e.stored << (8 * b);
          }
        } else if (a.opt_return_row) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            float x[16];
#pragma unroll
            for (int q = 0; q < 8; ++q) { x[2 * q] = bf16lo_to_f32(w[8 * b + q]); x[2 * q + 1] = bf16hi_to_f32(w[8 * b + q]); }
            const int lc0 = wh * kStripCols + b * 16;   // first column of the block inside the chunk
            uint32_t wsel[4] = {0, 0, 0, 0};
            uint32_t scale_rbits = 0;
            if (a.opt_sr_row || kScaleSr) {
              const int stage = (rc >> 6) * 2 + (lc0 >> 6);
              const int lr = rc & 63, it_ref = lr >> 5;
              const int tid_ref = (lr & 31) * 4 + ((lc0 & 63) >> 4);
              const unsigned long long seq = (unsigned long long)tid_ref + 128ull * (unsigned long long)ck +
                                             128ull * (unsigned long long)a.chunks_k * (unsigned long long)cm;
              const int bg = (tid_ref & 31) >> 4;
              if constexpr (kScaleSr) {
                // q words per block (scale first, then the data words); the stage holds 2 (row-only launch) or 4 blocks.
                // Earlier blocks of the reference thread that drew no scale word move this block's draws up; a block
                // that draws none itself takes its data words from its first draw on.
                const int q = 1 + (a.opt_sr_row ? 4 : 0);
                const int pos = stage * (a.opt_row_per_stage >> 2) + it_ref;
                uint32_t zm = 0;
                if (ENCODE_CENTRIC && a.ec_zero_row_stream != nullptr) zm = __ldg(a.ec_zero_row_stream + seq);
                const bool own_zero = (zm >> pos) & 1u;
                uint32_t dr[5];
                philox_draws(rng_s[0], seq, rng_s[1], pos * q - __popc(zm & ((1u << pos) - 1u)), q, dr);
                scale_rbits = dr[0];
                const uint32_t d0 = own_zero ? dr[0] : dr[1], d1 = own_zero ? dr[1] : dr[2], d2 = own_zero ? dr[2] : dr[3],
                               d3 = own_zero ? dr[3] : dr[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) wsel[g] = (((g >> 1) - bg) & 1) ? ((g & 1) ? d3 : d2) : ((g & 1) ? d1 : d0);
              } else {
                const uint4 rw = philox4x32_10(rng_s[0], seq,
                                               rng_s[1] + (unsigned long long)((stage * a.opt_row_per_stage + it_ref * 4) >> 2));
                const uint32_t words[4] = {rw.x, rw.y, rw.z, rw.w};
#pragma unroll
                for (int g = 0; g < 4; ++g) wsel[g] = words[2 * (((g >> 1) - bg) & 1) + (g & 1)];
              }
            }
            uint32_t stored;
            const uint32_t neg = ((b < 2 ? row_neg_lo : row_neg_hi) >> (16 * (b & 1))) & 0xFFFFu;
            const uint2 cd = opt_block<ENCODE_CENTRIC>(x, a.opt_rht_row != 0, neg, s_enc_row, lut_row, a.opt_sr_row != 0, wsel,
                                                       stored, kScaleSr, scale_rbits, kCodeLut ? code_lut_row : nullptr, code_base_row);
            codes[2 * b] = cd.x;
            codes[2 * b + 1] = cd.y;
            sc_word |= stored << (8 * b);
          }
        }
      } else {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          uint32_t mx = 0;
#pragma unroll
          for (int q = 0; q < 8; ++q) mx = absmax_xs(mx, w[8 * b + q]);
          ScaleLut e;
          if constexpr (kCodeLut) {
            const uint32_t am = mx & 0x7FFF7FFFu;
            e = code_lut_lookup<ENCODE_CENTRIC>(code_lut_row, lut_row, code_base_row, s_enc_row, max(am >> 16, am & 0xFFFFu));
          } else {
            e = lut_row[block_code<ENCODE_CENTRIC>(fmaxf(fabsf(bf16lo_to_f32(mx)), fabsf(bf16hi_to_f32(mx))), s_enc_row)];
          }
          codes[2 * b] = quant8(w + 8 * b, e.coeff);
          codes[2 * b + 1] = quant8(w + 8 * b + 4, e.coeff);
          sc_word |= e.stored << (8 * b);
        }
      }
      // codes leave through a TMA store (32 bytes per row; one store per unit): per-lane global stores of 32
      // different lines each would cost the L1 as much as all the shared-memory traffic of the strip
      if (!OPT || a.opt_return_row) {
        if (half == 0) {
          if (lane == 0) bulk_wait_group_read0();   // the previous unit's store has left the staging buffer
          __syncwarp();
        }
        uint8_t* stage_row = my_stage + half * kStripStageBytes + lane * 32;
        *reinterpret_cast<uint4*>(stage_row) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
        *reinterpret_cast<uint4*>(stage_row + 16) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
        // 512-byte tile (128 rows x these 4 blocks): row wv*32 + lane, blocks 0..3 are 4 adjacent bytes
        st_cs_u32(row_sc_unit + wv * 4, sc_word);
      }
    }

    // ---- column pass: lane = column pair -----------------------------------------------
    if (want_col) {
      if constexpr (NORM) __syncwarp();   // the normalised rows of all lanes are in the slot
      uint32_t cc0[4], cc1[4];            // codes of columns c and c+1: rows 0..7, 8..15, 16..23, 24..31
      uint32_t sc0 = 0, sc1 = 0;
      uint32_t col_neg = 0;               // sign vector of the strip's 32 rows: one hash per lane, shared through a ballot
      if constexpr (OPT != 0) {
        if (a.opt_sign && a.opt_rht_col)
          col_neg = __ballot_sync(0xffffffffu, rht_sign_is_negative(a.sign_seed, a.sign_subseq, (unsigned long long)(row0 + lane)) != 0);
      }
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint8_t* gbase = tile + g * 16 * 128;
        uint32_t w[16];
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          w[i] = *reinterpret_cast<const uint32_t*>(gbase + (i >> 3) * 1024 + col_off[i & 7]);
          mx = absmax_xs(mx, w[i]);
        }
        if constexpr (OPT != 0) {
          const int grp16 = wv * 2 + g;   // 16-row group inside the chunk (the reference kernel's warp role)
          if (a.opt_rht_col) {
            // the transform of both columns of the pair at once, in packed fp32x2 arithmetic, rounded back to bf16x2
            const uint32_t neg = (col_neg >> (16 * g)) & 0xFFFFu;
            float2 v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              v[i] = make_float2(bf16lo_to_f32(w[i]), bf16hi_to_f32(w[i]));
              if ((neg >> i) & 1u) v[i] = make_float2(-v[i].x, -v[i].y);
            }
            fwht16x2(v);
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = f32x2_to_bf16x2(v[i].x, v[i].y);
          }
#pragma unroll
          for (int wq = 0; wq < 2; ++wq) {
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = wq ? bf16hi_to_f32(w[i]) : bf16lo_to_f32(w[i]);
            uint32_t wsel[4] = {0, 0, 0, 0};
            uint32_t scale_rbits = 0;
            if (a.opt_sr_col || kScaleSr) {
              const int stage = (grp16 >> 2) * 2 + wh;
              const int tid_ref = (((grp16 & 3) - (lane & 3)) & 3) * 32 + lane;
              const unsigned long long seq = (unsigned long long)tid_ref + 128ull * (unsigned long long)ck +
                                             128ull * (unsigned long long)a.chunks_k * (unsigned long long)cm;
              if constexpr (kScaleSr) {
                // the stage's two row blocks (drawn or skipped over by the launch this pass belongs to), then its two column blocks
                const int q = 1 + (a.opt_sr_col ? 4 : 0);
                const int pos = stage * 4 + 2 + wq;
                uint32_t zm = 0;
                if (ENCODE_CENTRIC && a.ec_zero_col_stream != nullptr) zm = __ldg(a.ec_zero_col_stream + seq);
                const bool own_zero = (zm >> pos) & 1u;
                uint32_t dr[5];
                philox_draws(rng_s[0], seq, rng_s[2], pos * q - __popc(zm & ((1u << pos) - 1u)), q, dr);
                scale_rbits = dr[0];
                wsel[0] = own_zero ? dr[0] : dr[1]; wsel[1] = own_zero ? dr[1] : dr[2];
                wsel[2] = own_zero ? dr[2] : dr[3]; wsel[3] = own_zero ? dr[3] : dr[4];
              } else {
                const uint4 rw = philox4x32_10(rng_s[0], seq, rng_s[2] + (unsigned long long)((stage * 16 + 8 + wq * 4) >> 2));
                wsel[0] = rw.x; wsel[1] = rw.y; wsel[2] = rw.z; wsel[3] = rw.w;
              }
            }
            uint32_t stored;
            const uint2 cd = opt_block<ENCODE_CENTRIC>(x, false, 0u, s_enc_col, lut_col,   // (already transformed above)
                                                       a.opt_sr_col != 0, wsel, stored, kScaleSr, scale_rbits,
                                                       kCodeLut ? code_lut_col : nullptr, code_base_col);
            if (wq == 0) { cc0[2 * g] = cd.x; cc0[2 * g + 1] = cd.y; sc0 |= stored << (8 * g); }
            else { cc1[2 * g] = cd.x; cc1[2 * g + 1] = cd.y; sc1 |= stored << (8 * g); }
          }
        } else {
          ScaleLut e0, e1;
          if constexpr (kCodeLut) {
            e0 = code_lut_lookup<ENCODE_CENTRIC>(code_lut_col, lut_col, code_base_col, s_enc_col, mx & 0x7FFFu);
            e1 = code_lut_lookup<ENCODE_CENTRIC>(code_lut_col, lut_col, code_base_col, s_enc_col, (mx >> 16) & 0x7FFFu);
          } else {
            e0 = lut_col[block_code<ENCODE_CENTRIC>(fabsf(bf16lo_to_f32(mx)), s_enc_col)];
            e1 = lut_col[block_code<ENCODE_CENTRIC>(fabsf(bf16hi_to_f32(mx)), s_enc_col)];
          }
          const float2 cc = make_float2(e0.coeff, e1.coeff);
          float2 v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = mul2(make_float2(bf16lo_to_f32(w[i]), bf16hi_to_f32(w[i])), cc);
          cc0[2 * g] = f32x8_to_e2m1x8(v[0].x, v[1].x, v[2].x, v[3].x, v[4].x, v[5].x, v[6].x, v[7].x);
          cc0[2 * g + 1] = f32x8_to_e2m1x8(v[8].x, v[9].x, v[10].x, v[11].x, v[12].x, v[13].x, v[14].x, v[15].x);
          cc1[2 * g] = f32x8_to_e2m1x8(v[0].y, v[1].y, v[2].y, v[3].y, v[4].y, v[5].y, v[6].y, v[7].y);
          cc1[2 * g + 1] = f32x8_to_e2m1x8(v[8].y, v[9].y, v[10].y, v[11].y, v[12].y, v[13].y, v[14].y, v[15].y);
          sc0 |= e0.stored << (8 * g);
          sc1 |= e1.stored << (8 * g);
        }
      }
      // 16 bytes per column straight to [K, M/2]: as a TMA store this would be 64 box rows of 16 bytes,
      // and the TMA unit's rate of box rows (not bytes) is what bounds the kernel once everything goes through it
      if constexpr (!PAIR) {
        uint8_t* cdst = a.col_fp4 + (size_t)(col0 + 2 * lane) * col_pitch + (row0 >> 1);
        st_cs_u4(cdst, make_uint4(cc0[0], cc0[1], cc0[2], cc0[3]));
        st_cs_u4(cdst + col_pitch, make_uint4(cc1[0], cc1[1], cc1[2], cc1[3]));
        // 512-byte tile (128 columns x four 16-row groups of a 64-row band): this strip holds groups
        // (wv & 1) * 2 and (wv & 1) * 2 + 1 of band cm * 2 + (wv >> 1): two adjacent bytes per column
        uint8_t* sdst = a.col_sc + (((size_t)ck * col_sc_tiles_per_col_block + (size_t)(cm * 2 + (wv >> 1))) << 9) + (wv & 1) * 2;
        st_cs_u16(sdst + col_sc_lane0, (uint16_t)sc0);
        st_cs_u16(sdst + col_sc_lane1, (uint16_t)sc1);
      } else {
        // 64 rows of a column are 32 contiguous bytes.  Both strips' codes go to a [64 columns][32 B] tile in
        // shared memory (16-byte units, unit u at u ^ ((u >> 3) & 7): conflict-free both ways); after the lower
        // strip, store k writes columns 16k .. 16k+15, lanes 2j and 2j+1 the two halves of one column, so a
        // store touches 16 whole sectors instead of 32 half sectors.
        auto unit = [](int q) { return (q ^ ((q >> 3) & 7)) << 4; };
        *reinterpret_cast<uint4*>(my_col_stage + unit(4 * lane + half)) = make_uint4(cc0[0], cc0[1], cc0[2], cc0[3]);
        *reinterpret_cast<uint4*>(my_col_stage + unit(4 * lane + 2 + half)) = make_uint4(cc1[0], cc1[1], cc1[2], cc1[3]);
        if (half == 0) {
          held_sc = (sc0 & 0xFFFFu) | (sc1 << 16);
        } else {
          __syncwarp();
          uint8_t* cdst = a.col_fp4 + (size_t)(col0 + (lane >> 1)) * col_pitch + ((row0 - kStripRows) >> 1) + (lane & 1) * 16;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            st_cs_u4(cdst + (size_t)(16 * k) * col_pitch, *reinterpret_cast<const uint4*>(my_col_stage + unit(32 * k + lane)));
          // the four 16-row groups of the 64-row band cm * 2 + (wv >> 1): one 32-bit word per column
          uint8_t* sdst = a.col_sc + (((size_t)ck * col_sc_tiles_per_col_block + (size_t)(cm * 2 + (wv >> 1))) << 9);
          st_cs_u32(sdst + col_sc_lane0, (held_sc & 0xFFFFu) | (sc0 << 16));
          st_cs_u32(sdst + col_sc_lane1, (held_sc >> 16) | (sc1 << 16));
        }
      }
    }

    // the slot is free again: refill it with this half of the next unit to request; after the unit's last strip the
    // staged row codes leave for global memory
    fence_proxy_async_smem();   // this lane's generic-proxy writes (staging, normalised rows) before the TMA engine's accesses
    __syncwarp();
    if (lane == 0) {
      if (half == halves - 1 && (!OPT || a.opt_return_row)) {
        tma_store_2d_hint(&tmap_row, my_stage, col0 >> 1, cm * kChunk + wv_base * kStripRows, use_once);
        bulk_commit_group();
      }
      if (l_idx < my_units) issue_load(lm, lk, half, s);
    }
    }   // halves
    advance(lm, lk);
    ++l_idx;
    cm = nm;
    ck = nk;
  }
  if (lane == 0) bulk_wait_group0();
}

template <bool ENCODE_CENTRIC, bool NORM, int OPT, bool PAIR>
__global__ void __launch_bounds__(kStripWarps * 32, 1)
nvfp4_quantize_strip_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_row,
                            const QuantArgs a) {
  quantize_strip_cta<ENCODE_CENTRIC, NORM, OPT, PAIR>(tmap_x, tmap_row, a, (int)blockIdx.x, (int)gridDim.x);
}

// Three matrices with the same row count in ONE launch (the attention side's dQ, dK, dV): CTAs [0, cta_end[0]) work
// on the first, [cta_end[0], cta_end[1]) on the second, the rest on the third, each range as a launch of its own would.
struct StripProblem {
  CUtensorMap tmap_x, tmap_row;
  QuantArgs a;
};
struct StripGroup3 {
  StripProblem p[3];
  int cta_end[2];
};

template <bool PAIR>
__global__ void __launch_bounds__(kStripWarps * 32, 1)
nvfp4_quantize_strip3_kernel(const __grid_constant__ StripGroup3 g) {
  const int b = (int)blockIdx.x;
  if (b < g.cta_end[0]) {
    quantize_strip_cta<true, false, 0, PAIR>(g.p[0].tmap_x, g.p[0].tmap_row, g.p[0].a, b, g.cta_end[0]);
  } else if (b < g.cta_end[1]) {
    quantize_strip_cta<true, false, 0, PAIR>(g.p[1].tmap_x, g.p[1].tmap_row, g.p[1].a, b - g.cta_end[0],
                                             g.cta_end[1] - g.cta_end[0]);
  } else {
    quantize_strip_cta<true, false, 0, PAIR>(g.p[2].tmap_x, g.p[2].tmap_row, g.p[2].a, b - g.cta_end[1],
                                             (int)gridDim.x - g.cta_end[1]);
  }
}

// Tensor amax of the 16-point Hadamard transform of x (per 16 contiguous elements along K when
// along_k, else per 16 consecutive rows), taken on the fp32 transform output before its bf16
// rounding, as the reference's scan does (tk_quantize.cu:574-664).
__global__ void __launch_bounds__(256)
rht16_amax_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                  const float* __restrict__ inv_rms, float* __restrict__ amax, int64_t M, int64_t K, int along_k,
                  int sign, unsigned long long sign_seed, unsigned long long sign_subseq) {
  const int64_t groups = along_k ? M * (K / 16) : (M / 16) * K;
  float local = 0.0f;
  for (int64_t gidx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < groups; gidx += (int64_t)gridDim.x * blockDim.x) {
    float v[16];
    int64_t coord0;
    if (along_k) {
      const int64_t bpr = K / 16, row = gidx / bpr, cb = gidx - row * bpr;
      const uint4* p = reinterpret_cast<const uint4*>(x + row * K + cb * 16);
      const uint4 a0 = __ldg(p), a1 = __ldg(p + 1);
      const uint32_t w[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
      for (int q = 0; q < 8; ++q) { v[2 * q] = bf16lo_to_f32(w[q]); v[2 * q + 1] = bf16hi_to_f32(w[q]); }
      if (gamma != nullptr) {   // transform of the RMS-normalised, bf16-rounded values
        const float inv = __ldg(inv_rms + row);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          v[i] = __bfloat162float(__float2bfloat16_rn(v[i] * inv * __bfloat162float(gamma[cb * 16 + i])));
      }
      coord0 = cb * 16;
    } else {
      const int64_t rb = gidx / K, col = gidx - rb * K;
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(x[(rb * 16 + i) * K + col]);
      coord0 = rb * 16;
    }
    if (sign) {
      // scan along M: the 32 lanes of a warp hold 32 columns of ONE 16-row group (K is a multiple of 128 and the
      // grid stride a multiple of 32), so sixteen lanes hash one row each and share the mask
      const uint32_t neg = along_k ? rht_sign_mask16(sign_seed, sign_subseq, (unsigned long long)coord0)
                                   : (__ballot_sync(0xffffffffu, (threadIdx.x & 31) < 16 &&
                                          rht_sign_is_negative(sign_seed, sign_subseq, (unsigned long long)(coord0 + (threadIdx.x & 15))) != 0) & 0xFFFFu);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = ((neg >> i) & 1u) ? -v[i] : v[i];
    }
    fwht16(v);
#pragma unroll
    for (int i = 0; i < 16; ++i) local = fmaxf(local, fabsf(v[i]));
  }
  local = warp_max(local);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x < 32) {
    local = threadIdx.x < 8 ? part[threadIdx.x] : 0.0f;
    local = warp_max(local);
    if (threadIdx.x == 0 && local > 0.0f) atomic_max_nonneg(amax, local);
  }
}

// Column scan of the transform's tensor maximum, two columns per thread: a lane reads 32 bits of sixteen consecutive
// rows (a warp covers 128 contiguous bytes of every row), transforms both columns and, when plain_amax is given,
// also takes the maximum of the untransformed values — the row operand's tensor scale when only the column operand is
// transformed, from the same read.  Same arithmetic as rht16_amax_kernel with along_k = 0.
__global__ void __launch_bounds__(256)
rht16_col_amax_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ amax, float* __restrict__ plain_amax,
                      int64_t M, int64_t K, int sign, unsigned long long sign_seed, unsigned long long sign_subseq) {
  const int64_t pairs = K >> 1, groups = (M / 16) * pairs;
  float local = 0.0f;
  uint32_t plain = 0;
  for (int64_t gidx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gidx < groups; gidx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t rb = gidx / pairs, cp = gidx - rb * pairs;
    const uint32_t* p = reinterpret_cast<const uint32_t*>(x + rb * 16 * K) + cp;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = __ldg(p + (size_t)i * pairs);
    float2 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      plain = absmax_xs(plain, w[i]);
      v[i] = make_float2(bf16lo_to_f32(w[i]), bf16hi_to_f32(w[i]));
    }
    if (sign) {
      // the 32 lanes of a warp hold 64 columns of ONE 16-row group (K is a multiple of 128 and the grid stride a
      // multiple of 32), so sixteen lanes hash one row each and share the mask
      const uint32_t neg = __ballot_sync(0xffffffffu, (threadIdx.x & 31) < 16 &&
                               rht_sign_is_negative(sign_seed, sign_subseq, (unsigned long long)(rb * 16 + (threadIdx.x & 15))) != 0) & 0xFFFFu;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if ((neg >> i) & 1u) v[i] = make_float2(-v[i].x, -v[i].y);
      }
    }
    fwht16x2(v);
#pragma unroll
    for (int i = 0; i < 16; ++i) local = fmaxf(local, fmaxf(fabsf(v[i].x), fabsf(v[i].y)));
  }
  float plain_f = fmaxf(fabsf(bf16lo_to_f32(plain)), fabsf(bf16hi_to_f32(plain)));
  local = warp_max(local);
  plain_f = warp_max(plain_f);
  __shared__ float part[2][8];
  if ((threadIdx.x & 31) == 0) { part[0][threadIdx.x >> 5] = local; part[1][threadIdx.x >> 5] = plain_f; }
  __syncthreads();
  if (threadIdx.x < 32) {
    local = threadIdx.x < 8 ? part[0][threadIdx.x] : 0.0f;
    plain_f = threadIdx.x < 8 ? part[1][threadIdx.x] : 0.0f;
    local = warp_max(local);
    plain_f = warp_max(plain_f);
    if (threadIdx.x == 0) {
      if (local > 0.0f) atomic_max_nonneg(amax, local);
      if (plain_amax != nullptr && plain_f > 0.0f) atomic_max_nonneg(plain_amax, plain_f);
    }
  }
}

__global__ void finalize_sg_pair_kernel(float* __restrict__ a, float* __restrict__ b) {
  a[1] = a[0] / 2688.0f;
  if (b != nullptr) b[1] = b[0] / 2688.0f;
}

// ---------------------------------------------------------------------------------------
// Numbering of stochastic launches on the device
// ---------------------------------------------------------------------------------------
//
// The reference numbers its stochastic launches with a device word that a one-thread kernel advances by 2^32 per
// reserved launch, and hands the launch its {key, base} through device memory (tk_quantize.cu:443-481:
// tk_sr_invocation_offset, tk_prepare_advancing_rng_state_kernel), so that a captured CUDA graph draws from a new
// place on every replay.  Same here: one counter per device (a module-scope device word), same stride.
constexpr unsigned long long kSrInvocationStride = 1ull << 32;
__device__ unsigned long long g_sr_invocation_offset = 0;

__global__ void sr_prepare_state_kernel(unsigned long long* __restrict__ rng_state, unsigned long long seed,
                                        unsigned long long subsequence, unsigned long long launches) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const unsigned long long offset = atomicAdd(&g_sr_invocation_offset, kSrInvocationStride * launches);
    rng_state[0] = seed;
    rng_state[1] = subsequence + offset;
  }
}

// The other numbering: a PRODUCER's own persistent pair {seed, next subsequence} (one row of a checkpointed table),
// advanced by the stride per reserved launch right before the launch it feeds, on that launch's stream; independent
// of the order in which different producers are launched (low_bits_training/quantization/localcta_sr_state.py:1-11).
__global__ void sr_reserve_from_state_kernel(unsigned long long* __restrict__ producer_state,
                                             unsigned long long* __restrict__ rng_state, unsigned long long launches) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const unsigned long long next = producer_state[1];
    rng_state[0] = producer_state[0];
    rng_state[1] = next;
    producer_state[1] = next + kSrInvocationStride * launches;
  }
}

__global__ void sr_set_offset_kernel(unsigned long long value) {
  if (threadIdx.x == 0 && blockIdx.x == 0) g_sr_invocation_offset = value;
}

__global__ void sr_get_offset_kernel(unsigned long long* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *out = g_sr_invocation_offset;
}

// ---------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------

// Launch configuration with the programmatic-serialisation attribute (when pdl): the kernel may start
// while the kernel before it on the stream still runs and must call pdl_wait() before touching that
// kernel's results.
struct PdlLaunch {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  PdlLaunch(dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl) {
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
  }
  PdlLaunch(const PdlLaunch&) = delete;
};

// FP4B200_PDL_CHAIN=0: the statistics and amax kernels are launched the ordinary way (A/B runs).
static bool stats_pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("FP4B200_PDL_CHAIN");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// Whether the pass-1 kernels may read their input before the previous kernel on the stream has ended: off unless
// the caller promises (fp4b200_set_pdl_early_reads, or FP4B200_PDL_EARLY_READS=1) that no input of a call is
// written by the kernel launched immediately before it.
static int g_pdl_early_reads = [] {
  const char* e = getenv("FP4B200_PDL_EARLY_READS");
  return (e != nullptr && e[0] == '1') ? 1 : 0;
}();
static int pdl_early_reads() { return g_pdl_early_reads; }

// Reduction of the per-CTA maxima into amax_sg[0..1], launched behind the kernel that produced them.
static int launch_reduce_partials(const float* partials, int n, float* amax_sg, cudaStream_t st) {
  PdlLaunch l(dim3(1), dim3(256), 0, st, true);
  FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, reduce_partials_kernel, partials, n, amax_sg));
  return 0;
}

int launch_amax(const void* x, int64_t n_elems, float* amax_sg, cudaStream_t st, float* scratch,
                AmaxPartials* partials_out) {
  if (scratch == nullptr) scratch = stream_scratch(st);
  if (scratch == nullptr) return -1;
  const size_t n_vec = (size_t)n_elems / 8;
  int grid = (int)std::min<size_t>((n_vec + 255) / 256, std::min<size_t>((size_t)device_sm_count() * 8, kScratchFloats));
  grid = std::max(grid, 1);   // an empty input still leaves one partial (0)
  PdlLaunch l(dim3((unsigned)grid), dim3(256), 0, st, stats_pdl_enabled());
  FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, amax_bf16_kernel, reinterpret_cast<const uint4*>(x), n_vec, scratch,
                                    pdl_early_reads()));
  if (partials_out != nullptr) {
    partials_out->ptr = scratch;
    partials_out->count = grid;
    return 0;
  }
  return launch_reduce_partials(scratch, grid, amax_sg, st);
}

template <bool EC, bool NORM, bool W2D = false, bool OPT = false>
static int launch_quantize_t(const CUtensorMap& tmap, const QuantArgs& args, cudaStream_t st, bool pdl) {
  auto kern = nvfp4_quantize_kernel<EC, NORM, W2D, OPT>;
  const int smem = (int)sizeof(QuantSmem) + 1024;
  FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int n_chunks = args.chunks_m * args.chunks_k;
  const int grid = std::min(n_chunks, (OPT ? 1 : 2) * device_sm_count());
  if (grid == 0) return 0;
  PdlLaunch l(dim3((unsigned)grid), dim3(kQThreads), (size_t)smem, st, pdl);
  FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, kern, tmap, args));
  return 0;
}

// CTA-synchronous kernel for everything when FP4B200_QUANT_STRIP=0 (A/B comparisons)
static bool quant_strip_disabled() {
  static const bool off = [] {
    const char* e = getenv("FP4B200_QUANT_STRIP");
    return e != nullptr && e[0] == '0';
  }();
  return off;
}

// FP4B200_QUANT_PAIR: "0" never pairs strips, "1" pairs them whenever there are column outputs; unset: by size.
static int quant_pair_mode() {
  static const int mode = [] {
    const char* e = getenv("FP4B200_QUANT_PAIR");
    return e == nullptr ? -1 : (e[0] == '0' ? 0 : 1);
  }();
  return mode;
}

// The strip kernel's two tensor maps: the input in strips of 32 rows x 64 columns, and the row-wise codes.
static int make_strip_tmaps(const void* x, const QuantArgs& args, bool pair, CUtensorMap* tmap, CUtensorMap* tmap_row) {
  const bool nhsd = args.nhsd_seq > 0;   // [B * heads * seq, 64] instead of [M, K]
  if (int rc = make_tmap_2d(tmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, nhsd ? 64u : (uint64_t)args.K,
                            nhsd ? (uint64_t)args.M * (uint64_t)args.nhsd_heads : (uint64_t)args.M,
                            nhsd ? 128u : (uint64_t)args.K * 2, kStripCols, kStripRows, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  // row-wise codes as a byte matrix [M, K/2], stored in boxes of 32 (paired: 64) rows x 32 bytes
  *tmap_row = *tmap;   // launches without row-wise outputs never use it
  if (args.row_fp4 != nullptr) {
    if (int rc = make_tmap_2d(tmap_row, args.row_fp4, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)args.K / 2, (uint64_t)args.M,
                              args.row_pitch_bytes > 0 ? (uint64_t)args.row_pitch_bytes : (uint64_t)args.K / 2, kStripCols / 2,
                              kStripRows * (pair ? 2 : 1), CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
  }
  return 0;
}

template <bool EC, bool NORM, int OPT, bool PAIR>
static int launch_quantize_strip_tp(const void* x, const QuantArgs& args, cudaStream_t st, bool pdl) {
  CUtensorMap tmap, tmap_row;
  if (int rc = make_strip_tmaps(x, args, PAIR, &tmap, &tmap_row)) return rc;
  auto kern = nvfp4_quantize_strip_kernel<EC, NORM, OPT, PAIR>;
  const int smem = (int)strip_smem_bytes(NORM ? args.K : 0, PAIR);
  FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int n_chunks = args.chunks_m * args.chunks_k;
  constexpr int groups = PAIR ? 4 : 2;
  const int grid = std::min((n_chunks + groups - 1) / groups, device_sm_count());
  if (grid == 0) return 0;
  PdlLaunch l(dim3((unsigned)grid), dim3(kStripWarps * 32), (size_t)smem, st, pdl);
  FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, kern, tmap, tmap_row, args));
  return 0;
}

// Paired strips when there are column outputs, enough chunks to keep the four groups of every SM busy, and
// room in shared memory for the column staging tiles.
static bool strip_pairing_applies(const QuantArgs& a, bool norm) {
  if (a.col_fp4 == nullptr || strip_smem_bytes(norm ? a.K : 0, true) > 227 * 1024) return false;
  if (norm && a.n_partials == 0 && a.amax_row != a.amax_col) return false;   // the paired NORM form keeps one code table
  const int mode = quant_pair_mode();
  return mode < 0 ? a.chunks_m * a.chunks_k >= 4 * device_sm_count() : mode == 1;
}

template <bool EC, bool NORM, int OPT = 0>
static int launch_quantize_strip_t(const void* x, const QuantArgs& args, cudaStream_t st, bool pdl) {
  // The paired form of the fused-RMSNorm kernel with stochastic data rounding needs more than 128 registers: unpaired.
  if constexpr (NORM && OPT == 1) {
    return launch_quantize_strip_tp<EC, NORM, OPT, false>(x, args, st, pdl);
  } else {
    return strip_pairing_applies(args, NORM) ? launch_quantize_strip_tp<EC, NORM, OPT, true>(x, args, st, pdl)
                                             : launch_quantize_strip_tp<EC, NORM, OPT, false>(x, args, st, pdl);
  }
}

// The strip kernel stores codes by TMA (16-byte aligned outputs) and keeps gamma in shared memory.
static bool strip_kernel_applies(const QuantArgs& a, bool norm) {
  if (quant_strip_disabled()) return false;
  if (((reinterpret_cast<uintptr_t>(a.row_fp4) | reinterpret_cast<uintptr_t>(a.col_fp4)) & 15) != 0) return false;   // TMA / 16-byte stores
  return strip_smem_bytes(norm ? a.K : 0, false) <= 227 * 1024;
}

int launch_quantize(const void* x, int64_t M, int64_t K, const float* amax_row, const float* amax_col,
                           bool encode_centric, const float* inv_rms, const void* gamma, void* row_fp4,
                           void* row_sc, void* col_fp4, void* col_sc, float* sg_out, bool reverse,
                           cudaStream_t st, bool weight_2d, const QuantOpt* opt, const AmaxPartials* partials,
                           float* amax_out, int nhsd_heads, int nhsd_seq, int64_t row_pitch_bytes) {
  const bool behind_pass1 = partials != nullptr;
  CUtensorMap tmap;
  if (int rc = make_tmap_2d(&tmap, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                            (uint64_t)K * 2, 64, kChunk, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  QuantArgs a{};
  a.amax_row = amax_row;
  a.amax_col = amax_col ? amax_col : amax_row;
  a.inv_rms = inv_rms;
  a.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  a.row_fp4 = (uint8_t*)row_fp4; a.row_sc = (uint8_t*)row_sc;
  a.col_fp4 = (uint8_t*)col_fp4; a.col_sc = (uint8_t*)col_sc;
  a.sg_out = sg_out;
  if (partials != nullptr) {
    if (partials->ptr == nullptr || partials->count <= 0 || partials->count > kScratchFloats)
      return set_error("launch_quantize: bad partial-amax descriptor");
    a.partials = partials->ptr;
    a.n_partials = partials->count;
    a.amax_out = amax_out;
  }
  a.status = device_status_ptr();
  if (a.status == nullptr) return -1;
  a.M = (int)M; a.K = (int)K;
  a.chunks_m = (int)(M / kChunk); a.chunks_k = (int)(K / kChunk);
  a.reverse = reverse ? 1 : 0;
  a.nhsd_heads = nhsd_heads; a.nhsd_seq = nhsd_seq;
  a.row_pitch_bytes = (int)row_pitch_bytes;
  const bool norm = inv_rms != nullptr;
  if (row_pitch_bytes > 0 && (weight_2d || !strip_kernel_applies(a, norm)))
    return set_error("row codes into a wider matrix: 1-D blocks into 16-byte aligned outputs only");
  if (nhsd_seq > 0 && (opt != nullptr || weight_2d || norm || !strip_kernel_applies(a, false)))
    return set_error("head-major input: plain quantisation into 16-byte aligned outputs only");
  if (opt != nullptr) {
    a.opt_sr_row = opt->sr_row; a.opt_sr_col = opt->sr_col; a.rng_offset_col = opt->rng_offset_col;
    a.opt_scale_sr = opt->scale_sr;
    a.opt_row_per_stage = opt->row_per_stage ? opt->row_per_stage : (col_fp4 != nullptr ? 16 : 8);
    a.opt_rht_row = opt->rht_row; a.opt_rht_col = opt->rht_col; a.opt_sign = opt->sign;
    a.opt_return_row = opt->return_row; a.rng_seed = opt->rng_seed; a.rng_offset = opt->rng_offset;
    a.rng_state = reinterpret_cast<const unsigned long long*>(opt->rng_state);
    a.sign_seed = opt->sign_seed; a.sign_subseq = opt->sign_subseq;
    if (strip_kernel_applies(a, norm)) {
      if (a.opt_scale_sr && encode_centric && opt->ec_zero_scratch != nullptr) {
        // which blocks draw no scale word, per stream: one launch of the reference (both passes in one stream), or,
        // when one axis only rounds its codes stochastically, its row-only launch and its column launch
        const bool split = opt->row_per_stage == 8 && col_fp4 != nullptr;
        const int n_chunks = a.chunks_m * a.chunks_k;
        uint16_t* masks = reinterpret_cast<uint16_t*>(opt->ec_zero_scratch);
        ec_zero_block_mask_kernel<<<n_chunks, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), (int)K, a.chunks_k,
                                                           a.opt_row_per_stage >> 2, opt->return_row != 0,
                                                           col_fp4 != nullptr && !split, !split && opt->return_row != 0,
                                                           masks, masks + (size_t)n_chunks * 128);
        FP4_CUDA_CHECK(cudaGetLastError());
        a.ec_zero_row_stream = masks;
        a.ec_zero_col_stream = masks + (size_t)n_chunks * 128;
      }
      if (a.opt_scale_sr) {
        if (encode_centric) return norm ? launch_quantize_strip_t<true, true, 2>(x, a, st, behind_pass1)
                                        : launch_quantize_strip_t<true, false, 2>(x, a, st, behind_pass1);
        return norm ? launch_quantize_strip_t<false, true, 2>(x, a, st, behind_pass1)
                    : launch_quantize_strip_t<false, false, 2>(x, a, st, behind_pass1);
      }
      if (encode_centric) return norm ? launch_quantize_strip_t<true, true, 1>(x, a, st, behind_pass1)
                                      : launch_quantize_strip_t<true, false, 1>(x, a, st, behind_pass1);
      return norm ? launch_quantize_strip_t<false, true, 1>(x, a, st, behind_pass1)
                  : launch_quantize_strip_t<false, false, 1>(x, a, st, behind_pass1);
    }
    if (a.opt_scale_sr) return set_error("scale stochastic rounding needs 16-byte aligned outputs (strip quantiser only)");
    if (encode_centric) return norm ? launch_quantize_t<true, true, false, true>(tmap, a, st, behind_pass1)
                                    : launch_quantize_t<true, false, false, true>(tmap, a, st, behind_pass1);
    return norm ? launch_quantize_t<false, true, false, true>(tmap, a, st, behind_pass1)
                : launch_quantize_t<false, false, false, true>(tmap, a, st, behind_pass1);
  }
  if (weight_2d) return launch_quantize_t<false, false, true>(tmap, a, st, behind_pass1);   // decode-centric, as the reference
  if (strip_kernel_applies(a, norm)) {
    if (encode_centric) return norm ? launch_quantize_strip_t<true, true>(x, a, st, behind_pass1)
                                    : launch_quantize_strip_t<true, false>(x, a, st, behind_pass1);
    return norm ? launch_quantize_strip_t<false, true>(x, a, st, behind_pass1)
                : launch_quantize_strip_t<false, false>(x, a, st, behind_pass1);
  }
  if (encode_centric) return norm ? launch_quantize_t<true, true>(tmap, a, st, behind_pass1) : launch_quantize_t<true, false>(tmap, a, st, behind_pass1);
  return norm ? launch_quantize_t<false, true>(tmap, a, st, behind_pass1) : launch_quantize_t<false, false>(tmap, a, st, behind_pass1);
}

// Row slots of the pipelined statistics kernel for rows of K elements (fewer than 4: rows too long for it).
static int stats_slots_for(int64_t K) {
  const int64_t budget = 227 * 1024 - K * 4 - 2048;   // gamma tables, barriers, static shared memory
  return (int)std::max<int64_t>(0, std::min<int64_t>(budget / (K * 2), 64));
}

template <int NV, bool CI, int TREE = 0>
static int launch_stats_t(const __nv_bfloat16* xb, const __nv_bfloat16* gb, float* inv_rms, float* partials, float eps,
                          int64_t M, int64_t K, int slots, int* status, cudaStream_t st, int* grid_out, int want_amax) {
  auto kern = rmsnorm_stats_kernel<NV, CI, TREE>;
  const int warps = std::min(NV <= 16 ? kStatsMaxWarps : 6, slots);
  const size_t smem = (size_t)K * 4 + (size_t)slots * K * 2 + (size_t)slots * 12;
  FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = (int)std::min<int64_t>((M + warps - 1) / warps, (int64_t)device_sm_count());
  PdlLaunch l(dim3((unsigned)grid), dim3((unsigned)warps * 32), smem, st, stats_pdl_enabled());
  FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, kern, xb, gb, inv_rms, partials, eps, (int)M, (int)K, slots, status,
                                    pdl_early_reads(), want_amax));
  *grid_out = grid;
  return 0;
}

// FP4B200_STATS_PAIR=0: one warp per row (the earlier form of the statistics kernel), for A/B runs.
static bool stats_pair_enabled() {
  static const bool on = [] {
    const char* e = getenv("FP4B200_STATS_PAIR");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

template <int NVH, bool CI>
static int launch_stats_pair_t(const __nv_bfloat16* xb, const __nv_bfloat16* gb, float* inv_rms, float* partials, float eps,
                               int64_t M, int64_t K, int* status, cudaStream_t st, int* grid_out, int want_amax) {
  auto kern = rmsnorm_stats_pair_kernel<NVH, CI>;
  const int max_pairs = NVH <= 8 ? 12 : 6;
  const int64_t per_pair = (int64_t)kStatsPairSlots * K * 2 + kStatsPairSlots * 8 + 2 * 2 * 32 * 4;
  const int pairs = (int)std::min<int64_t>(max_pairs, (227 * 1024 - K * 4 - 1024) / per_pair);
  if (pairs < 1) return set_error("rmsnorm statistics: rows of %lld elements do not fit the pipelined kernel", (long long)K);
  const size_t smem = (size_t)K * 4 + (size_t)pairs * per_pair;
  FP4_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = (int)std::min<int64_t>((M + pairs - 1) / pairs, (int64_t)device_sm_count());
  PdlLaunch l(dim3((unsigned)grid), dim3((unsigned)pairs * 64), smem, st, stats_pdl_enabled());
  FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, kern, xb, gb, inv_rms, partials, eps, (int)M, (int)K, status, pdl_early_reads(),
                                    want_amax));
  *grid_out = grid;
  return 0;
}

// RMSNorm statistics of x [M, K]: inv_rms per row (computed, or read when !compute_inv) and the tensor
// amax of bf16(x * inv_rms * gamma).  partials_out == nullptr: amax_sg[0..1] are written on the stream
// (two launches).  Otherwise only the per-CTA maxima are produced, in `scratch`, for the quantiser
// launched next.
static int launch_rmsnorm_stats(const void* x, const void* gamma, float* inv_rms, float* amax_sg, float eps,
                                int64_t M, int64_t K, bool compute_inv, cudaStream_t st, float* scratch = nullptr,
                                AmaxPartials* partials_out = nullptr, int tree = 0) {
  if ((reinterpret_cast<uintptr_t>(gamma) & 15) != 0) return set_error("rmsnorm statistics: gamma must be 16-byte aligned");
  if (scratch == nullptr) scratch = stream_scratch(st);
  if (scratch == nullptr) return -1;
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto gb = reinterpret_cast<const __nv_bfloat16*>(gamma);
  const int slots = stats_slots_for(K);
  int grid = 0;
  // neither a tensor amax nor partial maxima wanted: inverse RMS only (the pipelined kernel skips the second sweep)
  const int want_amax = (amax_sg != nullptr || partials_out != nullptr) ? 1 : 0;
  if (K <= 8192 && slots >= 4) {
    int* status = device_status_ptr();
    if (status == nullptr) return -1;
    int rc;
    if (tree == 1) {   // inverse RMS only, in the MXFP4 producer's summation order: one warp per row
      if (K <= 1024) rc = launch_stats_t<4, true, 1>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
      else if (K <= 2048) rc = launch_stats_t<8, true, 1>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
      else if (K <= 4096) rc = launch_stats_t<16, true, 1>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
      else rc = launch_stats_t<32, true, 1>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
    } else if (tree == 2) {   // the same for the optional-mode NVFP4 producer's
      if (K <= 1024) rc = launch_stats_t<4, true, 2>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
      else if (K <= 2048) rc = launch_stats_t<8, true, 2>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
      else if (K <= 4096) rc = launch_stats_t<16, true, 2>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
      else rc = launch_stats_t<32, true, 2>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, 0);
    } else
    if (stats_pair_enabled()) {
      if (K <= 1024) rc = compute_inv ? launch_stats_pair_t<2, true>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax)
                                      : launch_stats_pair_t<2, false>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax);
      else if (K <= 2048) rc = compute_inv ? launch_stats_pair_t<4, true>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax)
                                           : launch_stats_pair_t<4, false>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax);
      else if (K <= 4096) rc = compute_inv ? launch_stats_pair_t<8, true>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax)
                                           : launch_stats_pair_t<8, false>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax);
      else rc = compute_inv ? launch_stats_pair_t<16, true>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax)
                            : launch_stats_pair_t<16, false>(xb, gb, inv_rms, scratch, eps, M, K, status, st, &grid, want_amax);
    } else
    if (K <= 1024) rc = compute_inv ? launch_stats_t<4, true>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax)
                                    : launch_stats_t<4, false>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax);
    else if (K <= 2048) rc = compute_inv ? launch_stats_t<8, true>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax)
                                         : launch_stats_t<8, false>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax);
    else if (K <= 4096) rc = compute_inv ? launch_stats_t<16, true>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax)
                                         : launch_stats_t<16, false>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax);
    else rc = compute_inv ? launch_stats_t<32, true>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax)
                          : launch_stats_t<32, false>(xb, gb, inv_rms, scratch, eps, M, K, slots, status, st, &grid, want_amax);
    if (rc) return rc;
  } else {
    grid = (int)std::min<int64_t>((M + 7) / 8, std::min<int64_t>((int64_t)device_sm_count() * 8, kScratchFloats));
    if (compute_inv) rmsnorm_stats_generic_kernel<true><<<grid, 256, 0, st>>>(xb, gb, inv_rms, scratch, eps, (int)M, (int)K, tree);
    else rmsnorm_stats_generic_kernel<false><<<grid, 256, 0, st>>>(xb, gb, inv_rms, scratch, eps, (int)M, (int)K, 0);
    FP4_CUDA_CHECK(cudaGetLastError());
  }
  if (partials_out != nullptr) {
    partials_out->ptr = scratch;
    partials_out->count = grid;
    return 0;
  }
  if (!want_amax) return 0;
  return launch_reduce_partials(scratch, grid, amax_sg, st);
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

int fp4b200_set_pdl_early_reads(int enabled) {
  const int before = g_pdl_early_reads;
  g_pdl_early_reads = enabled != 0;
  return before;
}

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
  AmaxPartials part;
  if (int rc = launch_amax(x_bf16, M * K, amax_sg, (cudaStream_t)stream, nullptr, &part)) return rc;
  return launch_quantize(x_bf16, M, K, nullptr, nullptr, encode_centric != 0, nullptr, nullptr, row_fp4, row_sc,
                         return_transpose ? col_fp4 : nullptr, return_transpose ? col_sc : nullptr, nullptr,
                         true, (cudaStream_t)stream, false, nullptr, &part, amax_sg);
}

int fp4b200_nvfp4_quantize_for_gemm_into(const void* x_bf16, int64_t M, int64_t K, int return_transpose, int encode_centric,
                                         void* row_fp4, int64_t row_pitch_bytes, void* row_sc, void* col_fp4, void* col_sc,
                                         float* amax_sg, void* stream) {
  const char* fn = "nvfp4_quantize_for_gemm_into";
  if (int rc = check_quant_shapes(x_bf16, M, K, fn)) return rc;
  if (row_fp4 == nullptr || row_sc == nullptr || amax_sg == nullptr)
    return set_error("%s: row_fp4, row_sc and amax_sg are required", fn);
  if (return_transpose && (col_fp4 == nullptr || col_sc == nullptr))
    return set_error("%s: return_transpose needs col_fp4 and col_sc", fn);
  if (row_pitch_bytes < K / 2 || (row_pitch_bytes % 16) != 0 || row_pitch_bytes > INT32_MAX)
    return set_error("%s: the row pitch must be a multiple of 16 bytes and at least K/2 (got %lld)", fn, (long long)row_pitch_bytes);
  AmaxPartials part;
  if (int rc = launch_amax(x_bf16, M * K, amax_sg, (cudaStream_t)stream, nullptr, &part)) return rc;
  return launch_quantize(x_bf16, M, K, nullptr, nullptr, encode_centric != 0, nullptr, nullptr, row_fp4, row_sc,
                         return_transpose ? col_fp4 : nullptr, return_transpose ? col_sc : nullptr, nullptr, true,
                         (cudaStream_t)stream, false, nullptr, &part, amax_sg, 0, 0, row_pitch_bytes);
}

// Shares of `total` for three weights, each between 1 and cap[i] and as near its exact share as that allows.
static void split_three(const int64_t w[3], const int64_t cap[3], int64_t total, int out[3]) {
  const double sum = (double)(w[0] + w[1] + w[2]);
  double ideal[3];
  int64_t given = 0;
  for (int i = 0; i < 3; ++i) {
    ideal[i] = (double)total * (double)w[i] / sum;
    out[i] = (int)std::max<int64_t>(1, std::min<int64_t>((int64_t)ideal[i], cap[i]));
    given += out[i];
  }
  for (; given < total; ++given) {   // hand the rest to whichever is furthest below its share
    int best = -1;
    for (int i = 0; i < 3; ++i)
      if (out[i] < cap[i] && (best < 0 || ideal[i] - out[i] > ideal[best] - out[best])) best = i;
    if (best < 0) break;
    ++out[best];
  }
  for (; given > total; --given) {   // the minimum of 1 overshot: take from whichever is furthest above
    int best = -1;
    for (int i = 0; i < 3; ++i)
      if (out[i] > 1 && (best < 0 || out[i] - ideal[i] > out[best] - ideal[best])) best = i;
    if (best < 0) break;
    --out[best];
  }
}

int fp4b200_nvfp4_quantize_split3_into(const void* x0, const void* x1, const void* x2, int64_t M, int64_t n0, int64_t n1,
                                       int64_t n2, void* row_fp4_full, void* row_sc0, void* row_sc1, void* row_sc2,
                                       void* col_fp4_full, void* col_sc_cat, float* amax3, float* sg3, void* stream) {
  const char* fn = "nvfp4_quantize_split3_into";
  const void* xs[3] = {x0, x1, x2};
  const int64_t ns[3] = {n0, n1, n2};
  void* row_scs[3] = {row_sc0, row_sc1, row_sc2};
  for (int g = 0; g < 3; ++g)
    if (int rc = check_quant_shapes(xs[g], M, ns[g], fn)) return rc;
  if (!row_fp4_full || !row_sc0 || !row_sc1 || !row_sc2 || !col_fp4_full || !col_sc_cat || !amax3 || !sg3)
    return set_error("%s: every output is required", fn);
  const int64_t n_total = n0 + n1 + n2;
  if (M * n_total / 2 > INT32_MAX) return set_error("%s: outputs of more than 2 GiB are not supported", fn);
  if (((reinterpret_cast<uintptr_t>(row_fp4_full) | reinterpret_cast<uintptr_t>(col_fp4_full)) & 15) != 0)
    return set_error("%s: the code matrices must be 16-byte aligned", fn);
  cudaStream_t st = (cudaStream_t)stream;
  float* scratch = stream_scratch(st);
  int* status = device_status_ptr();
  if (scratch == nullptr || status == nullptr) return -1;
  const int sms = device_sm_count();

  // pass 1: the three tensor maxima as per-CTA partial maxima, one launch
  AmaxGroup3 ag{};
  int64_t w[3], cap[3];
  int amax_ctas[3];
  for (int g = 0; g < 3; ++g) {
    ag.x[g] = reinterpret_cast<const uint4*>(xs[g]);
    ag.n_vec[g] = (size_t)(M * ns[g] / 8);
    w[g] = M * ns[g];
    cap[g] = (int64_t)((ag.n_vec[g] + 255) / 256);
  }
  split_three(w, cap, std::min<int64_t>((int64_t)sms * 8, kScratchFloats), amax_ctas);
  ag.cta_end[0] = amax_ctas[0];
  ag.cta_end[1] = amax_ctas[0] + amax_ctas[1];
  {
    PdlLaunch l(dim3((unsigned)(ag.cta_end[1] + amax_ctas[2])), dim3(256), 0, st, stats_pdl_enabled());
    FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, amax3_bf16_kernel, ag, scratch, pdl_early_reads()));
  }

  // pass 2: one launch, the SMs shared out by the matrices' sizes
  int64_t total_chunks = 0;
  for (int g = 0; g < 3; ++g) total_chunks += (M / kChunk) * (ns[g] / kChunk);
  const int mode = quant_pair_mode();
  const bool pair = strip_smem_bytes(0, true) <= 227 * 1024 && (mode < 0 ? total_chunks >= 4 * (int64_t)sms : mode == 1);
  const int groups = pair ? 4 : 2;
  StripGroup3 sg{};
  int64_t off = 0, partial0 = 0;
  for (int g = 0; g < 3; ++g) {
    QuantArgs& a = sg.p[g].a;
    a.row_fp4 = (uint8_t*)row_fp4_full + off / 2;
    a.row_pitch_bytes = (int)(n_total / 2);
    a.row_sc = (uint8_t*)row_scs[g];
    a.col_fp4 = (uint8_t*)col_fp4_full + off * (M / 2);
    a.col_sc = (uint8_t*)col_sc_cat + (off / 128) * (M / 64) * 512;
    a.partials = scratch + partial0;
    a.n_partials = amax_ctas[g];
    a.amax_scalar_out = amax3 + g;
    a.sg_out = sg3 + g;
    a.status = status;
    a.M = (int)M; a.K = (int)ns[g];
    a.chunks_m = (int)(M / kChunk); a.chunks_k = (int)(ns[g] / kChunk);
    a.reverse = 1;   // pass 1 read each matrix front to back: its tail is what the L2 still holds
    if (int rc = make_strip_tmaps(xs[g], a, pair, &sg.p[g].tmap_x, &sg.p[g].tmap_row)) return rc;
    w[g] = (int64_t)a.chunks_m * a.chunks_k;
    cap[g] = (w[g] + groups - 1) / groups;
    off += ns[g];
    partial0 += amax_ctas[g];
  }
  int ctas[3];
  split_three(w, cap, std::min<int64_t>(cap[0] + cap[1] + cap[2], sms), ctas);
  sg.cta_end[0] = ctas[0];
  sg.cta_end[1] = ctas[0] + ctas[1];
  const int smem = (int)strip_smem_bytes(0, pair);
  PdlLaunch l(dim3((unsigned)(sg.cta_end[1] + ctas[2])), dim3(kStripWarps * 32), (size_t)smem, st, true);
  if (pair) {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(nvfp4_quantize_strip3_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, nvfp4_quantize_strip3_kernel<true>, sg));
  } else {
    FP4_CUDA_CHECK(cudaFuncSetAttribute(nvfp4_quantize_strip3_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    FP4_CUDA_CHECK(cudaLaunchKernelEx(&l.cfg, nvfp4_quantize_strip3_kernel<false>, sg));
  }
  return 0;
}

int fp4b200_nvfp4_quantize_nhsd_wo(const void* x_bf16, int64_t B, int64_t H, int64_t S, int64_t D, int return_transpose,
                                   int encode_centric, void* row_fp4, void* row_sc, void* col_fp4, void* col_sc,
                                   float* amax_sg, void* stream) {
  const char* fn = "nvfp4_quantize_nhsd_wo";
  if (B <= 0 || H <= 0 || S <= 0) return set_error("%s: B, H and S must be positive", fn);
  if (D != 64) return set_error("%s: head_dim must be 64 (got %lld)", fn, (long long)D);
  if ((S % 128) != 0) return set_error("%s: the sequence length must be a multiple of 128 (got %lld)", fn, (long long)S);
  if (B * S > INT32_MAX || H * D > INT32_MAX) return set_error("%s: matrix too large", fn);
  const int64_t M = B * S, K = H * D;
  if (int rc = check_quant_shapes(x_bf16, M, K, fn)) return rc;
  if (row_fp4 == nullptr || row_sc == nullptr || amax_sg == nullptr)
    return set_error("%s: row_fp4, row_sc and amax_sg are required", fn);
  if (return_transpose && (col_fp4 == nullptr || col_sc == nullptr))
    return set_error("%s: return_transpose needs col_fp4 and col_sc", fn);
  AmaxPartials part;
  if (int rc = launch_amax(x_bf16, M * K, amax_sg, (cudaStream_t)stream, nullptr, &part)) return rc;
  return launch_quantize(x_bf16, M, K, nullptr, nullptr, encode_centric != 0, nullptr, nullptr, row_fp4, row_sc,
                         return_transpose ? col_fp4 : nullptr, return_transpose ? col_sc : nullptr, nullptr, true,
                         (cudaStream_t)stream, false, nullptr, &part, amax_sg, (int)H, (int)S);
}

int fp4b200_nvfp4_rht16_amax(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                             int along_k, int with_sign, uint64_t sign_seed, uint64_t sign_subseq, float* amax_sg,
                             float* plain_amax_sg, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_rht16_amax")) return rc;
  if (!amax_sg) return set_error("nvfp4_rht16_amax: amax_sg is required");
  if ((gamma_bf16 == nullptr) != (inv_rms == nullptr) || (gamma_bf16 != nullptr && !along_k))
    return set_error("nvfp4_rht16_amax: fused RMSNorm needs gamma and inv_rms and the transform along K");
  if (plain_amax_sg != nullptr && along_k)
    return set_error("nvfp4_rht16_amax: the untransformed maximum comes with the scan along M only");
  cudaStream_t st = (cudaStream_t)stream;
  FP4_CUDA_CHECK(cudaMemsetAsync(amax_sg, 0, 2 * sizeof(float), st));
  if (!along_k) {
    if (plain_amax_sg != nullptr) FP4_CUDA_CHECK(cudaMemsetAsync(plain_amax_sg, 0, 2 * sizeof(float), st));
    const int64_t groups = M * K / 32;
    const int grid = (int)std::min<int64_t>((groups + 255) / 256, (int64_t)device_sm_count() * 8);
    rht16_col_amax_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x_bf16), amax_sg, plain_amax_sg, M, K,
                                                with_sign != 0, sign_seed, sign_subseq);
    FP4_CUDA_CHECK(cudaGetLastError());
    finalize_sg_pair_kernel<<<1, 1, 0, st>>>(amax_sg, plain_amax_sg);
    FP4_CUDA_CHECK(cudaGetLastError());
    return 0;
  }
  const int64_t groups = M * K / 16;
  const int grid = (int)std::min<int64_t>((groups + 255) / 256, (int64_t)device_sm_count() * 8);
  rht16_amax_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x_bf16),
                                          reinterpret_cast<const __nv_bfloat16*>(gamma_bf16), inv_rms, amax_sg, M, K, along_k != 0,
                                          with_sign != 0, sign_seed, sign_subseq);
  FP4_CUDA_CHECK(cudaGetLastError());
  finalize_sg_kernel<<<1, 1, 0, st>>>(amax_sg);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_nvfp4_quantize_opt_into(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                                    const float* amax_row, const float* amax_col, int encode_centric, int data_sr,
                                    int rht_row, int rht_col, int with_sign, uint64_t sign_seed, uint64_t sign_subseq,
                                    int return_row, uint64_t rng_seed, uint64_t rng_offset, uint64_t rng_offset_col,
                                    const uint64_t* rng_state, int scale_sr, void* row_fp4, int64_t row_pitch_bytes,
                                    void* row_sc, void* col_fp4, void* col_sc, void* ec_zero_scratch, void* stream);

int fp4b200_nvfp4_quantize_opt(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                               const float* amax_row, const float* amax_col, int encode_centric, int data_sr,
                               int rht_row, int rht_col, int with_sign, uint64_t sign_seed, uint64_t sign_subseq,
                               int return_row, uint64_t rng_seed, uint64_t rng_offset, uint64_t rng_offset_col,
                               const uint64_t* rng_state, int scale_sr,
                               void* row_fp4, void* row_sc, void* col_fp4, void* col_sc, void* ec_zero_scratch, void* stream) {
  return fp4b200_nvfp4_quantize_opt_into(x_bf16, gamma_bf16, inv_rms, M, K, amax_row, amax_col, encode_centric, data_sr, rht_row,
                                         rht_col, with_sign, sign_seed, sign_subseq, return_row, rng_seed, rng_offset,
                                         rng_offset_col, rng_state, scale_sr, row_fp4, 0, row_sc, col_fp4, col_sc,
                                         ec_zero_scratch, stream);
}

int fp4b200_nvfp4_quantize_opt_into(const void* x_bf16, const void* gamma_bf16, const float* inv_rms, int64_t M, int64_t K,
                                    const float* amax_row, const float* amax_col, int encode_centric, int data_sr,
                                    int rht_row, int rht_col, int with_sign, uint64_t sign_seed, uint64_t sign_subseq,
                                    int return_row, uint64_t rng_seed, uint64_t rng_offset, uint64_t rng_offset_col,
                                    const uint64_t* rng_state, int scale_sr, void* row_fp4, int64_t row_pitch_bytes,
                                    void* row_sc, void* col_fp4, void* col_sc, void* ec_zero_scratch, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_quantize_opt")) return rc;
  if (reinterpret_cast<uintptr_t>(rng_state) & 7) return set_error("nvfp4_quantize_opt: rng_state must be 8-byte aligned");
  if (reinterpret_cast<uintptr_t>(ec_zero_scratch) & 1) return set_error("nvfp4_quantize_opt: ec_zero_scratch must be 2-byte aligned");
  if (row_pitch_bytes != 0 && (row_pitch_bytes < K / 2 || (row_pitch_bytes % 16) != 0 || row_pitch_bytes > INT32_MAX))
    return set_error("nvfp4_quantize_opt: the row pitch must be 0 or a multiple of 16 bytes and at least K/2 (got %lld)",
                     (long long)row_pitch_bytes);
  if (!amax_row) return set_error("nvfp4_quantize_opt: amax_row is required");
  if ((gamma_bf16 == nullptr) != (inv_rms == nullptr))
    return set_error("nvfp4_quantize_opt: gamma and inv_rms must both be given (fused RMSNorm) or both be null");
  if (return_row && (!row_fp4 || !row_sc)) return set_error("nvfp4_quantize_opt: row outputs are required when return_row");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("nvfp4_quantize_opt: col_fp4 and col_sc must both be given or both be null");
  if (!return_row && !col_fp4) return set_error("nvfp4_quantize_opt: nothing to compute");
  QuantOpt o{};
  if (data_sr < 0 || data_sr > 4)
    return set_error("nvfp4_quantize_opt: data_sr must be 0 (off), 1 (both passes, one stream), 2 (row pass), 3 (column pass) or "
                     "4 (both passes, a stream each)");
  o.sr_row = data_sr == 1 || data_sr == 2 || data_sr == 4; o.sr_col = data_sr == 1 || data_sr == 3 || data_sr == 4;
  // a row-only stochastic launch of the reference draws 8 words per stage, also when this launch adds the column pass
  o.row_per_stage = (data_sr >= 2) ? 8 : 0;
  o.scale_sr = scale_sr != 0;
  o.rng_offset_col = (data_sr == 0 || data_sr == 1) ? rng_offset : rng_offset_col;   // one launch of the reference: one stream
  o.rht_row = rht_row != 0; o.rht_col = rht_col != 0; o.sign = with_sign != 0;
  o.return_row = return_row != 0; o.rng_seed = rng_seed; o.rng_offset = rng_offset;
  o.sign_seed = sign_seed; o.sign_subseq = sign_subseq;
  o.ec_zero_scratch = ec_zero_scratch;
  o.rng_state = rng_state;
  return launch_quantize(x_bf16, M, K, amax_row, amax_col, encode_centric != 0, inv_rms, gamma_bf16, row_fp4, row_sc,
                         col_fp4, col_sc, nullptr, false, (cudaStream_t)stream, false, &o, nullptr, nullptr, 0, 0,
                         row_pitch_bytes);
}

int fp4b200_nvfp4_quantize_weight_2d(const void* w_bf16, int64_t N, int64_t K, void* row_fp4, void* row_sc,
                                     void* col_fp4, void* col_sc, float* amax_sg, void* stream) {
  if (int rc = check_quant_shapes(w_bf16, N, K, "nvfp4_quantize_weight_2d")) return rc;
  if (!row_fp4 || !row_sc || !col_fp4 || !col_sc || !amax_sg)
    return set_error("nvfp4_quantize_weight_2d: all outputs are required");
  AmaxPartials part;
  if (int rc = launch_amax(w_bf16, N * K, amax_sg, (cudaStream_t)stream, nullptr, &part)) return rc;
  return launch_quantize(w_bf16, N, K, nullptr, nullptr, false, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc,
                         nullptr, true, (cudaStream_t)stream, true, nullptr, &part, amax_sg);
}

int fp4b200_nvfp4_quantize_weight_2d_with_amax(const void* w_bf16, int64_t N, int64_t K, const float* amax, void* row_fp4,
                                               void* row_sc, void* col_fp4, void* col_sc, void* stream) {
  if (int rc = check_quant_shapes(w_bf16, N, K, "nvfp4_quantize_weight_2d_with_amax")) return rc;
  if (!amax || !row_fp4 || !row_sc || !col_fp4 || !col_sc)
    return set_error("nvfp4_quantize_weight_2d_with_amax: amax and all outputs are required");
  return launch_quantize(w_bf16, N, K, amax, amax, false, nullptr, nullptr, row_fp4, row_sc, col_fp4, col_sc,
                         nullptr, true, (cudaStream_t)stream, true);
}

int fp4b200_nvfp4_rmsnorm_stats(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                float* inv_rms, int compute_inv_rms, float* amax_sg, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_rmsnorm_stats")) return rc;
  if (gamma_bf16 == nullptr || inv_rms == nullptr)
    return set_error("nvfp4_rmsnorm_stats: gamma and inv_rms are required");
  if (amax_sg == nullptr && !compute_inv_rms) return set_error("nvfp4_rmsnorm_stats: nothing to compute");
  return launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, amax_sg, eps, M, K, compute_inv_rms != 0,
                              (cudaStream_t)stream);
}

int fp4b200_mxfp4_rmsnorm_inv_rms(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                  float* inv_rms, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "mxfp4_rmsnorm_inv_rms")) return rc;
  if (gamma_bf16 == nullptr || inv_rms == nullptr) return set_error("mxfp4_rmsnorm_inv_rms: gamma and inv_rms are required");
  return launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, nullptr, eps, M, K, true, (cudaStream_t)stream, nullptr, nullptr,
                              1);
}

int fp4b200_nvfp4_rmsnorm_inv_rms_opt(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M, int64_t K,
                                      float* inv_rms, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_rmsnorm_inv_rms_opt")) return rc;
  if (gamma_bf16 == nullptr || inv_rms == nullptr) return set_error("nvfp4_rmsnorm_inv_rms_opt: gamma and inv_rms are required");
  return launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, nullptr, eps, M, K, true, (cudaStream_t)stream, nullptr, nullptr,
                              2);
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
  AmaxPartials part;
  if (int rc = launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, amax_sg, eps, M, K, compute_inv_rms != 0,
                                    (cudaStream_t)stream, nullptr, &part))
    return rc;
  return launch_quantize(x_bf16, M, K, nullptr, nullptr, encode_centric != 0, inv_rms, gamma_bf16, row_fp4,
                         row_sc, col_fp4, col_sc, nullptr, true, (cudaStream_t)stream, false, nullptr, &part, amax_sg);
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


// ---- device-side numbering of stochastic launches ---------------------------------------------

int fp4b200_sr_prepare_state(uint64_t* rng_state, uint64_t rng_seed, uint64_t rng_subsequence, uint64_t launches,
                             void* stream) {
  if (rng_state == nullptr || (reinterpret_cast<uintptr_t>(rng_state) & 7))
    return set_error("sr_prepare_state: rng_state must be 8-byte aligned device memory for two 64-bit words");
  if (launches == 0) return set_error("sr_prepare_state: the number of launches to reserve must be positive");
  sr_prepare_state_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<unsigned long long*>(rng_state), rng_seed,
                                                            rng_subsequence, launches);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_sr_reserve_from_state(int64_t* producer_state, uint64_t* rng_state, uint64_t launches, void* stream) {
  if (producer_state == nullptr || (reinterpret_cast<uintptr_t>(producer_state) & 7))
    return set_error("sr_reserve_from_state: producer_state must be 8-byte aligned device memory for two 64-bit words");
  if (rng_state == nullptr || (reinterpret_cast<uintptr_t>(rng_state) & 7))
    return set_error("sr_reserve_from_state: rng_state must be 8-byte aligned device memory for two 64-bit words");
  if (launches == 0) return set_error("sr_reserve_from_state: the number of launches to reserve must be positive");
  sr_reserve_from_state_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<unsigned long long*>(producer_state),
                                                                 reinterpret_cast<unsigned long long*>(rng_state), launches);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_sr_set_invocation_offset(uint64_t value, void* stream) {
  sr_set_offset_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(value);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_sr_get_invocation_offset(uint64_t* out_dev, void* stream) {
  if (out_dev == nullptr || (reinterpret_cast<uintptr_t>(out_dev) & 7))
    return set_error("sr_get_invocation_offset: out must be 8-byte aligned device memory");
  sr_get_offset_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<unsigned long long*>(out_dev));
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// ---- variant that allocates nothing -------------------------------------------------------
// Scratch of the fused producer (inverse RMS per row, per-CTA partial maxima of pass 1) in a fixed
// device array owned by the library, for callers that must not allocate.  Every device that loads
// the library holds (kNoAllocMaxRows + kScratchFloats) * 4 bytes of it until the process exits.
constexpr int64_t kNoAllocMaxRows = 65536;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocMaxRows + kScratchFloats];

// Device address of the scratch array on the current device.  The array's name is only a
// host-side handle, so the address is looked up once per device and cached (host threads that race
// here store the same value).
static float* noalloc_scratch_ptr() {
  static std::atomic<float*> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("nvfp4_fused_norm_quantize_noalloc: cudaGetDevice failed");
    return nullptr;
  }
  float* have = cached[dev].load(std::memory_order_acquire);
  if (have == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("nvfp4_fused_norm_quantize_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    have = static_cast<float*>(p);
    cached[dev].store(have, std::memory_order_release);
  }
  return have;
}

int fp4b200_nvfp4_fused_norm_quantize_noalloc(const void* x_bf16, const void* gamma_bf16, float eps, int64_t M,
                                              int64_t K, void* row_fp4, void* row_sc, void* col_fp4,
                                              void* col_sc, float* sg_out, void* stream) {
  if (int rc = check_quant_shapes(x_bf16, M, K, "nvfp4_fused_norm_quantize_noalloc")) return rc;
  if (M > kNoAllocMaxRows)
    return set_error("nvfp4_fused_norm_quantize_noalloc: M=%lld exceeds the built-in scratch (at most %lld rows); "
                     "use fp4b200_nvfp4_fused_norm_quantize with caller-provided buffers",
                     (long long)M, (long long)kNoAllocMaxRows);
  if (gamma_bf16 == nullptr || row_fp4 == nullptr || row_sc == nullptr || sg_out == nullptr)
    return set_error("nvfp4_fused_norm_quantize_noalloc: gamma, row_fp4, row_sc and sg_out are required");
  if ((col_fp4 == nullptr) != (col_sc == nullptr))
    return set_error("nvfp4_fused_norm_quantize_noalloc: col_fp4 and col_sc must both be given or both be null");
  if ((reinterpret_cast<uintptr_t>(gamma_bf16) & 15) != 0)
    return set_error("nvfp4_fused_norm_quantize_noalloc: gamma must be 16-byte aligned");
  float* scratch = noalloc_scratch_ptr();
  if (scratch == nullptr) return -1;
  float* partials = scratch;                 // [kScratchFloats] per-CTA maxima of the statistics kernel
  float* inv_rms = scratch + kScratchFloats;  // [M]
  AmaxPartials part;
  if (int rc = launch_rmsnorm_stats(x_bf16, gamma_bf16, inv_rms, nullptr, eps, M, K, true, (cudaStream_t)stream, partials,
                                    &part))
    return rc;
  return launch_quantize(x_bf16, M, K, nullptr, nullptr, true, inv_rms, gamma_bf16, row_fp4, row_sc, col_fp4,
                         col_sc, sg_out, true, (cudaStream_t)stream, false, nullptr, &part, nullptr);
}

}  // extern "C"
