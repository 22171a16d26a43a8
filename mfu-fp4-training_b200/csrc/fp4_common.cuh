// Shared device helpers for the sm_100a FP4 hot-path kernels: number-format conversions,
// mbarrier / TMA wrappers with bounded waits, and small vector utilities.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fp4b200 {

constexpr float kFltMax = 3.4028235e+38f;

// Device status words (one array per loaded library, per device).  A kernel whose bounded
// wait runs out records a non-zero code here and returns; the host reads it with
// fp4b200_device_status().
enum StatusCode : int {
  kStatusOk = 0,
  kStatusQuantTmaTimeout = 1,
  kStatusGemmTmaTimeout = 2,
  kStatusGemmMmaTimeout = 3,
  kStatusGemmEpilogueTimeout = 4,
  kStatusGemmTmemTimeout = 5,
  kStatusSelfTestTimeout = 6,
};

// ---------------------------------------------------------------------------------------
// Number formats
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// two floats -> packed bf16x2 (round-to-nearest-even), lo in the low half
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// |a| max |b| element-wise on packed bf16x2 (NaN-free inputs assumed)
__device__ __forceinline__ uint32_t bf16x2_absmax(uint32_t acc, uint32_t v) {
  uint32_t r;
  asm("{.reg .b32 t; abs.bf16x2 t, %2; max.bf16x2 %0, %1, t;}" : "=r"(r) : "r"(acc), "r"(v));
  return r;
}

__device__ __forceinline__ float bf16x2_hmax_to_f32(uint32_t absmax2) {
  return fmaxf(bf16lo_to_f32(absmax2), bf16hi_to_f32(absmax2));
}

// fp32 -> E4M3 byte: round-to-nearest-even, saturate to +-448, subnormals kept.
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// fp32 -> E4M3 with stochastic rounding by the low 16 bits of rbits (the hardware adds them to the 16 leading
// discarded bits of the value's position between its two neighbours and rounds up on carry); saturating.
__device__ __forceinline__ uint8_t f32_to_e4m3_sr(float v, uint32_t rbits) {
  uint32_t p;
  asm("cvt.rs.satfinite.e4m3x4.f32 %0, {%1, %1, %1, %1}, %2;" : "=r"(p) : "f"(v), "r"(rbits));
  return (uint8_t)(p & 0xFFu);
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}

// Two fp32 -> one byte of two E2M1 codes (lo in the low nibble), RN-even, saturating.
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{.reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t;}"
      : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Eight fp32 (already multiplied by the block coefficient) -> 4 bytes of packed codes.
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(float v0, float v1, float v2, float v3,
                                                    float v4, float v5, float v6, float v7) {
  uint32_t r;
  asm("{.reg .b8 a, b, c, d;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 a, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 c, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 d, %8, %7;\n\t"
      "mov.b32 %0, {a, b, c, d};}"
      : "=r"(r)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7));
  return r;
}

// Stochastic rounding of four fp32 with one 32-bit random word -> 2 bytes (v0 lowest nibble).
__device__ __forceinline__ uint32_t f32x4_to_e2m1x4_sr(float v0, float v1, float v2, float v3,
                                                       uint32_t rbits) {
  uint32_t r;
  asm("{.reg .b16 t; cvt.rs.satfinite.e2m1x4.f32 t, {%4, %3, %2, %1}, %5; cvt.u32.u16 %0, t;}"
      : "=r"(r) : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "r"(rbits));
  return r;
}

// ---------------------------------------------------------------------------------------
// NVFP4 scale rules
// ---------------------------------------------------------------------------------------

// S_enc = min(448*6/amax, FLT_MAX); 1 when amax == 0 or the quotient underflows to 0.
__device__ __forceinline__ float nvfp4_global_encode_scale(float amax) {
  float s = fminf((448.0f * 6.0f) / amax, kFltMax);
  return (amax == 0.0f || s == 0.0f) ? 1.0f : s;
}

// Byte offset of scale (row r, block kb) inside its 512-byte tile of 128 rows x 4 blocks.
__device__ __forceinline__ int scale_tile_offset(int r_in_tile, int kb_in_tile) {
  return (r_in_tile & 31) * 16 + (r_in_tile >> 5) * 4 + kb_in_tile;
}

// ---------------------------------------------------------------------------------------
// mbarrier / TMA
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// First 1024-byte boundary at or after p inside the dynamic shared-memory array.  The pad is added to
// the array's own pointer (no round trip through an integer), so that the compiler still knows that
// everything derived from the result is shared memory and emits shared loads and stores, not generic ones.
__device__ __forceinline__ uint8_t* smem_align_1024(uint8_t* p) {
  return p + ((1024u - (smem_u32(p) & 1023u)) & 1023u);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after ~kSpinLimit polls (each poll itself blocks for a
// hardware-defined short time), returning false so that the caller can record a status
// code and leave instead of spinning for ever.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// 2-D tiled TMA store shared -> global of one box; completion is tracked by the thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(tmap), "r"(x), "r"(y), "r"(smem_u32(smem_src))
               : "memory");
}

// the same with an L2 eviction policy for the written lines
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* tmap, const void* smem_src, int x, int y, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;"
               ::"l"(tmap), "r"(x), "r"(y), "r"(smem_u32(smem_src)), "l"(policy)
               : "memory");
}

__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// earlier bulk stores of this thread have finished READING shared memory (the source may be overwritten)
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// earlier bulk stores of this thread are complete
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Programmatic dependent launch: a kernel launched with the programmatic-serialisation attribute may
// start while its predecessor in the stream still runs; everything the predecessor wrote is
// visible only after pdl_wait().  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// L2 eviction policies for bulk copies of data that is touched once (evict first) so that it does not push
// out lines that another part of the same kernel is about to re-read.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ void bulk_load_1d_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar,
                                                  uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
               : "memory");
}

__device__ __forceinline__ void bulk_store_1d_hint(void* gdst, const void* smem_src, uint32_t bytes, uint64_t policy) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes), "l"(policy)
               : "memory");
}

// Contiguous bytes from shared memory to global memory as one bulk copy of the calling thread's
// current bulk group (16-byte aligned addresses, size a multiple of 16).
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

// 2-D tiled TMA load (no multicast): box at element coordinates (x = inner, y = outer).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// the same with an L2 eviction policy for the lines read
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// float max via integer atomics; valid for non-negative, non-NaN values.
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}

// Streaming (evict-first) stores for write-once outputs.
__device__ __forceinline__ void st_cs_u16(void* p, uint16_t v) {
  asm volatile("st.global.cs.u16 [%0], %1;" ::"l"(p), "h"(v) : "memory");
}
__device__ __forceinline__ void st_cs_u32(void* p, uint32_t v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cs_u4(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------------------------------
// Packed fp32x2 arithmetic (one issue slot for two lanes of fp32 work)
// ---------------------------------------------------------------------------------------

// {a.x*b.x, a.y*b.y}, round-to-nearest, denormals kept
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{.reg .b64 x, y, z; mov.b64 x, {%2, %3}; mov.b64 y, {%4, %5}; mul.f32x2 z, x, y; mov.b64 {%0, %1}, z;}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// {a.x + b.x, a.y + b.y} and {a.x - b.x, a.y - b.y}: two IEEE additions per instruction
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{.reg .b64 x, y, z; mov.b64 x, {%2, %3}; mov.b64 y, {%4, %5}; add.rn.f32x2 z, x, y; mov.b64 {%0, %1}, z;}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 sub2(float2 a, float2 b) {
  float2 d;
  asm("{.reg .b64 x, y, z; mov.b64 x, {%2, %3}; mov.b64 y, {%4, %5}; sub.rn.f32x2 z, x, y; mov.b64 {%0, %1}, z;}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// {a.x*b.x + c.x, a.y*b.y + c.y}, each a fused multiply-add (same rounding as fmaf)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{.reg .b64 x, y, z, w; mov.b64 x, {%2, %3}; mov.b64 y, {%4, %5}; mov.b64 z, {%6, %7};"
      " fma.rn.f32x2 w, x, y, z; mov.b64 {%0, %1}, w;}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

// acc + lo(w)^2 and then + hi(w)^2, each one fused multiply-add of the bf16 value with itself into the
// fp32 accumulator (mixed-precision FMA: the bf16 x bf16 product is exact in fp32, so the result is
// bit-identical to fmaf on the converted values, without the conversion instructions).
__device__ __forceinline__ float fma_sq_bf16x2(uint32_t w, float acc) {
  asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1;\n\t"
      "fma.rn.f32.bf16 %0, lo, lo, %0;\n\t"
      "fma.rn.f32.bf16 %0, hi, hi, %0;}"
      : "+f"(acc) : "r"(w));
  return acc;
}

// max(acc, |a|, |b|) for acc >= 0 (written so that the compiler may use a three-input maximum with
// absolute-value operand modifiers)
__device__ __forceinline__ float absmax3(float acc, float a, float b) {
  return fmaxf(acc, fmaxf(fabsf(a), fabsf(b)));
}

// running |.|-max on packed bf16x2; the sign of the result is meaningless
__device__ __forceinline__ uint32_t absmax_xs(uint32_t acc, uint32_t v) {
  uint32_t r;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(acc), "r"(v));
  return r;
}

// four packed bf16x2 words times one coefficient -> 4 bytes of E2M1 codes
__device__ __forceinline__ uint32_t quant8(const uint32_t* w, float coeff) {
  const float2 cc = make_float2(coeff, coeff);
  const float2 a = mul2(make_float2(bf16lo_to_f32(w[0]), bf16hi_to_f32(w[0])), cc);
  const float2 b = mul2(make_float2(bf16lo_to_f32(w[1]), bf16hi_to_f32(w[1])), cc);
  const float2 c = mul2(make_float2(bf16lo_to_f32(w[2]), bf16hi_to_f32(w[2])), cc);
  const float2 d = mul2(make_float2(bf16lo_to_f32(w[3]), bf16hi_to_f32(w[3])), cc);
  return f32x8_to_e2m1x8(a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y);
}

// Philox4x32-10 block: key = seed, counter = {offset (64 bit), sequence (64 bit)}
// (reference generator: nvfp4_v5/util/curanddx.hpp:20-103)
__device__ __forceinline__ uint4 philox4x32_10(unsigned long long seed, unsigned long long sequence,
                                               unsigned long long offset) {
  uint32_t kx = (uint32_t)seed, ky = (uint32_t)(seed >> 32);
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = (uint32_t)sequence, c3 = (uint32_t)(sequence >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ kx, n2 = hi0 ^ c3 ^ ky;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    kx += 0x9E3779B9u; ky += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// Random words of the draws n0 .. n0 + count - 1 (count <= 5) of one thread's stream: draw n is component n & 3 of the
// Philox block at counter offset + (n >> 2) (the reference refills its four words when the fourth has been used,
// core.cuh:116-127).
__device__ __forceinline__ void philox_draws(unsigned long long seed, unsigned long long seq, unsigned long long offset, int n0,
                                             int count, uint32_t (&out)[5]) {
  const uint4 b0 = philox4x32_10(seed, seq, offset + (unsigned long long)(n0 >> 2));
  const bool two = ((n0 + count - 1) >> 2) != (n0 >> 2);
  const uint4 b1 = two ? philox4x32_10(seed, seq, offset + (unsigned long long)((n0 >> 2) + 1)) : b0;
  const uint32_t w[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  const int sh = n0 & 3;
#pragma unroll
  for (int i = 0; i < 5; ++i) out[i] = sh == 0 ? w[i] : (sh == 1 ? w[i + 1] : (sh == 2 ? w[i + 2] : w[i + 3]));   // registers only
}


}  // namespace fp4b200
