// Block-scaled FP4 GEMM for sm_100a: D[M,N] = (A . B^T) * (a_sg * b_sg), A [M,K/2] and
// B [N,K/2] packed E2M1 (K-major), block scales in 512-byte tiles (128 rows x 4 blocks),
// fp32 accumulation in tensor memory.
//
//   NVFP4: 16-element blocks, E4M3 scales, tcgen05.mma kind::mxf4nvf4 scale_vec::4X
//   MXFP4: 32-element blocks, E8M0 scales, tcgen05.mma kind::mxf4     scale_vec::2X,
//          accumulator multiplied by 1/36 (operands were scaled to +-6 rather than +-1)
//
// Replaces nvfp4_gemm::kernel / mxfp4_gemm::kernel of the reference
// (fp4_runtime/ThunderKittens/kernels/gemm/nvfp4_b200/nvfp4_gemm.cuh:490-1012,
//  fp4_runtime/ThunderKittens/kernels/gemm/mxfp4_gb200/mxfp4_gemm.cuh).  Unlike the reference
// there is no cluster-multicast TMA load: every CTA fetches its own operand tiles.
//
// One persistent CTA per SM works through 128 x 256 output tiles (this file), or a pair of CTAs through
// 256 x 256 tiles (gemm_fp4_pair.cuh, the default when M is a multiple of 256).  Warp roles:
//   warp 0      TMA producer: per 256-deep K stage one A box (128 rows x 128 B), one B box
//               (256 rows x 128 B), both 128-byte swizzled, and three bulk copies of scale tiles
//   warp 1      owns tensor memory; one lane issues tcgen05.mma
//   warps 2..5  epilogue: tcgen05.ld the accumulator, scale, (residual), convert, store
//   warps 6..9  scale movers: shared memory -> registers -> tcgen05.st into this quadrant's scale columns
// Both kernels run setup (barriers, tensor-memory allocation, descriptor prefetch) ahead of griddepcontrol.wait,
// so that, launched as a programmatic dependent, it overlaps the previous kernel's tail.
// Every wait on an mbarrier is bounded in time; a wait that runs out records a status code,
// and the CTA drains to the common exit where tensor memory is released.
#include "fp4_common.cuh"
#include "host_util.h"

#include <stdlib.h>
#include <string.h>

namespace fp4b200 {

constexpr int kGemmBM = 128;
constexpr int kGemmBN = 256;
constexpr int kGemmBKBytes = 128;                  // 256 FP4 elements per stage
constexpr int kGemmStages = 3;
constexpr int kGemmThreads = 320;
constexpr int kATileBytes = kGemmBM * kGemmBKBytes;   // 16 KiB
constexpr int kBTileBytes = kGemmBN * kGemmBKBytes;   // 32 KiB
constexpr int kASfBytes = 2048;                    // 4 scale tiles of 512 B (one per K=64 step)
constexpr int kBSfBytes = 4096;                    // two 128-row groups x 4 scale tiles
constexpr int kTmemCols = 512;
constexpr int kSfTmemBase = 256;                   // accumulator occupies columns [0,256)
constexpr int kSfSlotCols = 48;                    // per stage: 16 columns of A scales + 32 of B scales
constexpr long long kWaitLimitCycles = 4000000000LL;   // ~2 s at boost clock

struct GemmSmem {
  alignas(1024) uint8_t a[kGemmStages][kATileBytes];
  alignas(1024) uint8_t b[kGemmStages][kBTileBytes];
  alignas(1024) uint8_t epi[4][2][4096];             // per epilogue warp: two slabs of 32 rows x 128 B
  alignas(128) uint8_t sfa[kGemmStages][kASfBytes];
  alignas(128) uint8_t sfb[kGemmStages][kBSfBytes];
  alignas(8) uint64_t full[kGemmStages];
  alignas(8) uint64_t empty[kGemmStages];
  alignas(8) uint64_t sf_ready[kGemmStages];
  alignas(8) uint64_t acc_full;
  alignas(8) uint64_t acc_empty;
  uint32_t tmem_base;
};

// The K dimension may be the concatenation of up to kMaxKSeg segments, each with its own B tensor,
// its own scale tensors and its own column offset inside the rows of A (one segment = a plain GEMM).
constexpr int kMaxKSeg = 4;
struct GemmBMaps {
  CUtensorMap m[kMaxKSeg];
};

struct GemmArgs {
  int n_seg;
  int seg_stage_end[kMaxKSeg];      // cumulative number of K stages (256 deep; a tail may be 128) at the end of each segment
  int seg_a_col_bytes[kMaxKSeg];    // byte offset of the segment inside a row of A's codes
  const uint8_t* seg_a_sc[kMaxKSeg];   // [M/128, Kseg/(4*block), 512]
  const uint8_t* seg_b_sc[kMaxKSeg];   // [N/128, Kseg/(4*block), 512]
  int seg_sf_tiles_k[kMaxKSeg];     // scale tiles along K per row tile, per segment
  int seg_a_sf_row_tiles[kMaxKSeg]; // scale tiles from one 128-row block of A's scales to the next (= seg_sf_tiles_k unless A is a column slice)
  int seg_tail_half[kMaxKSeg];      // 1: the segment's last stage holds 128 elements only (MXFP4, K an odd multiple of 128)
  // Batched accumulation (kEpiBatchSum): every segment is a GEMM term of its own — its own A tensor (tensor map
  // tmap_a_seg.m[s]) and its own tensor scales; the terms' scaled accumulators are summed in fp32 by the epilogue.
  int a_per_seg;
  int round_terms;          // batched accumulation: every term rounded to bf16, terms added in bf16 left to right
  const float* seg_a_sg[kMaxKSeg];
  const float* seg_b_sg[kMaxKSeg];
  const float* a_sg;        // device scalar (NVFP4) or null
  const float* b_sg;        // device scalar, or per-256-column-tile array when b_sg_per_tile != 0
  int b_sg_per_tile;
  float fixed_scale;        // multiplies the accumulator when a_sg is null (MXFP4: 1/36)
  void* d[3];               // up to three outputs, split by column range
  int d_col_end[3];         // exclusive end column (in N) of each output
  int d_ld[3];              // leading dimension (elements) of each output
  int n_out;
  int out_fp32;             // 0: bf16 output, 1: fp32 output
  const __nv_bfloat16* residual;  // optional [M, N] bf16 added after the bf16 rounding
  int residual_ld;
  const float* accum_f32;   // optional [M, N] fp32 partial sum: fma(acc, scale, partial) before the output rounding
  // optional rotary embedding of the column range [0, rope_col_end) (the Q and K parts of a fused QKV projection)
  // in the bf16 epilogue: pairs of neighbouring columns rotated by the (cos, sin) entry of their token and
  // position inside the head (reference: nvfp4_rope_epilogue.cuh:104-161)
  const float2* rope_cs;    // [seq_len, head_dim/2] (cos, sin)
  int rope_seq_mask, rope_pair_dim, rope_head_mask, rope_col_end;
  int rope_round_bf16;      // round the scaled accumulator to bf16 before the rotation ("packed" forms)
  int silu_col_end;         // > 0: x / (1 + __expf(-x)) on the scaled accumulator of the columns [0, silu_col_end), before any rotation
  int rope_in_tmem;         // pair kernel, heads of 64 or 128: each row's (cos, sin) table row lives in tensor memory
  int M, N, K;              // K = sum of the segments
  int* status;
};

__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity, long long limit_cycles = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > limit_cycles) return false;
  }
  return true;
}

// Exercises the give-up path of mbar_wait_timed in the safe form: one warp, a barrier that nothing will ever arrive
// on, no copy in flight, a limit of the caller's choosing.  The wait runs out, the status word gets its code and the
// kernel returns like any other.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ alignas(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    if (!mbar_wait_timed(&bar, 0, limit_cycles)) atomicExch(status, kStatusSelfTestTimeout);
  }
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// shared-memory matrix descriptor (tcgen05): 14-bit address/offset fields in 16-byte units,
// descriptor version 1 at bit 46, layout type at bits 61..63 (0 none, 2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)((lbo_bytes & 0x3FFFF) >> 4) << 16) |
         ((uint64_t)((sbo_bytes & 0x3FFFF) >> 4) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}

template <bool MX>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (MX) {
    asm volatile(
        "{.reg .pred p; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{.reg .pred p; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// instruction descriptor of the block-scaled kinds: A/B format E2M1 (=1) at bits 7 and 10,
// N>>3 at bit 17, scale type at bit 23 (0 UE4M3, 1 UE8M0), M>>4 at bit 24, scale-factor ids
// at bits 4 (B) and 29 (A), K=64 (bit 31 = 0), both operands K-major, dense.
__host__ __device__ constexpr uint32_t block_scaled_idesc(int M, int N, int ue8m0, int sf_id) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)ue8m0 << 23) |
         ((uint32_t)(M >> 4) << 24) | ((uint32_t)sf_id << 4) | ((uint32_t)sf_id << 29);
}

// Tile order: groups of kRasterGroup row tiles are walked column by column, so that the tiles in
// flight at one time (one per CTA or CTA pair) cover a compact block of the output and re-use a
// small set of A and B rows out of L2.
constexpr int kRasterGroup = 8;
__device__ __forceinline__ void raster_tile(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kRasterGroup * tiles_n;
  const int grp = t / per_group, r = t - grp * per_group;
  const int rows = min(kRasterGroup, tiles_m - grp * kRasterGroup);
  tn = r / rows;
  tm = grp * kRasterGroup + (r - tn * rows);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// registers -> 32 lanes x 16 / 32 columns of tensor memory (this warp's lane quadrant)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

struct GemmOutMaps {
  CUtensorMap m[3];
};

// One lane's share of a stage's scale tiles, shared memory -> registers, in the column order of the stage's scale
// slot in tensor memory: 16 columns of A scales (4 per K step of 64), then 32 of B scales (4 + 4 per K step, the
// two 128-row groups of the tile).  Lane l holds the 16 bytes of tile row l, i.e. the scales of rows l, 32+l,
// 64+l, 96+l.  MXFP4 stages hold two tiles per group; the other columns are zeroed.
template <int kTiles>
__device__ __forceinline__ void load_stage_scales(const uint8_t* sfa, const uint8_t* sfb, int lane, uint32_t (&ra)[16],
                                                  uint32_t (&rb)[32]) {
#pragma unroll
  for (int j = 0; j < kTiles; ++j) {
    const uint4 va = *reinterpret_cast<const uint4*>(sfa + j * 512 + lane * 16);
    ra[4 * j] = va.x; ra[4 * j + 1] = va.y; ra[4 * j + 2] = va.z; ra[4 * j + 3] = va.w;
    const uint4 v0 = *reinterpret_cast<const uint4*>(sfb + j * 512 + lane * 16);
    const uint4 v1 = *reinterpret_cast<const uint4*>(sfb + kTiles * 512 + j * 512 + lane * 16);
    rb[8 * j] = v0.x; rb[8 * j + 1] = v0.y; rb[8 * j + 2] = v0.z; rb[8 * j + 3] = v0.w;
    rb[8 * j + 4] = v1.x; rb[8 * j + 5] = v1.y; rb[8 * j + 6] = v1.z; rb[8 * j + 7] = v1.w;
  }
#pragma unroll
  for (int j = kTiles; j < 4; ++j) {
    ra[4 * j] = ra[4 * j + 1] = ra[4 * j + 2] = ra[4 * j + 3] = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) rb[8 * j + e] = 0;
  }
}


constexpr int kEpiPlain = 0, kEpiRope = 1, kEpiSilu = 2, kEpiGeneral = 3, kEpiBatchSum = 4;

// x / (1 + exp(-x)) with the hardware exponential and approximate division: no slow-path branch, so the
// unrolled uses in the epilogue stay a few instructions each.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Epilogue of NCOLS (64 or 128) accumulator columns by one warp (its 32-lane quadrant of tensor memory).
// The columns are lifted into registers by loads issued back to back (128 columns, 64 KB per SM, leave tensor
// memory in ~300 cycles this way) and release() is called at once: from then on the MMA thread may overwrite
// them, and scaling, rounding, staging and the TMA stores run beside the next tile's MMAs.
//   taddr  tensor-memory address of the first column in this warp's lane quadrant
//   row0   first global row of this warp's 32 rows;  col0  first global column
//   epi    this warp's two staging buffers of 4 KiB (32 rows x 128 bytes, 128-byte swizzle); slab0 = which of them
//          the call's first 128-byte slab goes to (consecutive slabs of consecutive calls alternate)
// EPI selects the form: kEpiPlain bf16 (optional residual), kEpiRope with the rotary embedding, kEpiSilu with a
// SiLU range (rotary or not), kEpiGeneral fp32 outputs or fp32 accumulation.
// (Storing the rounded values straight from registers, 32 bytes per lane and store, instead of through the staging
// buffers and TMA stores was measured: 8 % slower at N 28672, K 4096.)
// What an epilogue warp does once a range of accumulator columns is in its registers: one arrival on the barrier the
// MMA thread waits on (a barrier of this CTA, or of the leader CTA of a pair), or nothing.
struct AccRelease {
  uint64_t* local = nullptr;        // barrier in this CTA's shared memory
  uint32_t cluster_addr = 0;        // or: shared::cluster address of a barrier of another CTA
  __device__ __forceinline__ void operator()(int lane) const {
    if (local == nullptr && cluster_addr == 0) return;
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (cluster_addr != 0) asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
      else mbar_arrive(local);
    }
  }
};

// CS_TMEM: the rotary table's rows come from tensor memory (cs_taddr) instead of global memory.
// Not inlined: with the forms' bodies inlined at every call site the register allocation of the whole kernel suffers
// (the rotary forms spilled a kilobyte per thread).
template <int EPI, int NCOLS, bool CS_TMEM = false>
__device__ __noinline__ void epilogue_region(const GemmArgs& g, const GemmOutMaps& tmap_d, uint32_t taddr, uint8_t* epi,
                                                int row0, int col0, float a_sg, int lane, AccRelease release, int slab0 = 0,
                                                uint32_t cs_taddr = 0) {
  static_assert(NCOLS == 64 || NCOLS == 128, "one or two slabs of 64 columns");
  uint32_t r[NCOLS];
#pragma unroll
  for (int k = 0; k < NCOLS / 32; ++k) tmem_ld32(taddr + (uint32_t)(32 * k), *reinterpret_cast<uint32_t(*)[32]>(&r[32 * k]));
  tmem_ld_wait();
  release(lane);
  if (col0 >= g.N) return;   // second half of the last column tile when N is an odd multiple of 128

  float gs = a_sg;
  if (g.b_sg != nullptr) gs = a_sg * __ldg(g.b_sg + (g.b_sg_per_tile ? (col0 >> 8) : 0));
  const int row = row0 + lane;
  int oi = 0, col_start = 0;   // which output receives this column range
  while (oi + 1 < g.n_out && col0 >= g.d_col_end[oi]) { col_start = g.d_col_end[oi]; ++oi; }
  const int ocol = col0 - col_start;
  uint8_t* rowp = epi + lane * 128;
  const int sw = lane & 7;
  // a staging buffer may be rewritten once the store issued from it two slabs ago has read it
  auto buffer_free = [&]() {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
  };
  auto store_slab = [&](const uint8_t* buf, int x) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(&tmap_d.m[oi], buf, x, row0);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  };

  if constexpr (EPI == kEpiGeneral) {
    // slabs of 128 bytes per row: 32 fp32 columns, or 64 bf16 columns from two 32-column chunks
#pragma unroll
    for (int c = 0; c < NCOLS / 32; ++c) {
      float v[32];
      if (g.accum_f32 != nullptr) {
        // running fp32 sum over a batch of GEMMs: fma(acc, scale, partial), one rounding per term — what the
        // reference's kernel does for every term after the first (its multiply and add contract to a fused
        // multiply-add; checked against its compiled kernel's output bytes)
        const float4* ps = reinterpret_cast<const float4*>(g.accum_f32 + (size_t)row * g.N + col0 + 32 * c);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 pv = __ldg(ps + q);
          v[4 * q] = __fmaf_rn(__uint_as_float(r[32 * c + 4 * q]), gs, pv.x);
          v[4 * q + 1] = __fmaf_rn(__uint_as_float(r[32 * c + 4 * q + 1]), gs, pv.y);
          v[4 * q + 2] = __fmaf_rn(__uint_as_float(r[32 * c + 4 * q + 2]), gs, pv.z);
          v[4 * q + 3] = __fmaf_rn(__uint_as_float(r[32 * c + 4 * q + 3]), gs, pv.w);
        }
      } else {
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] = __fmul_rn(__uint_as_float(r[32 * c + q]), gs);
      }
      if (g.out_fp32) {
        uint8_t* buf = rowp + ((c + slab0) & 1) * 4096;
        buffer_free();
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(buf + ((q ^ sw) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        store_slab(epi + ((c + slab0) & 1) * 4096, ocol + 32 * c);
      } else {
        uint8_t* buf = rowp + (((c >> 1) + slab0) & 1) * 4096;
        if ((c & 1) == 0) buffer_free();
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(buf + ((((c & 1) * 4 + q) ^ sw) << 4)) =
              make_uint4(f32x2_to_bf16x2(v[8 * q], v[8 * q + 1]), f32x2_to_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                         f32x2_to_bf16x2(v[8 * q + 4], v[8 * q + 5]), f32x2_to_bf16x2(v[8 * q + 6], v[8 * q + 7]));
        if (c & 1) store_slab(epi + (((c >> 1) + slab0) & 1) * 4096, ocol + 64 * (c >> 1));
      }
    }
  } else {
    constexpr bool ROPE = EPI == kEpiRope || EPI == kEpiSilu;
    constexpr bool SILU = EPI == kEpiSilu;
    const float2 gs2 = make_float2(gs, gs);
    const __nv_bfloat16* res_row = g.residual != nullptr ? g.residual + (size_t)row * g.residual_ld + col0 : nullptr;
    // rope_col_end is 0 when there is no table (SiLU alone)
    const bool rope_region = ROPE && g.rope_cs != nullptr && col0 < g.rope_col_end;
    const float2* cs_row = (rope_region && !CS_TMEM) ? g.rope_cs + (size_t)(row & g.rope_seq_mask) * g.rope_pair_dim : nullptr;
#pragma unroll
    for (int slab = 0; slab < NCOLS / 64; ++slab) { // 64 columns = 128 bytes per row
      uint32_t w[32];
#pragma unroll
      for (int h = 0; h < 4; ++h) {                 // 16 columns = eight pairs
        const int col = slab * 64 + h * 16;
        const bool silu_here = SILU && col0 + col < g.silu_col_end;
        const bool rope_here = rope_region && col0 + col < g.rope_col_end;
        float4 cs[4];
        if (rope_here) {
          // (cos, sin) of this lane's token and of the pairs' positions inside their head: 64 contiguous bytes of
          // the table — or sixteen columns of this lane's copy of its table row in tensor memory (pair kernel)
          if constexpr (CS_TMEM) {
            uint32_t t[16];
            tmem_ld16(cs_taddr + (uint32_t)((col0 + col) & g.rope_head_mask), t);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q)
              cs[q] = make_float4(__uint_as_float(t[4 * q]), __uint_as_float(t[4 * q + 1]), __uint_as_float(t[4 * q + 2]),
                                  __uint_as_float(t[4 * q + 3]));
          } else {
            const float4* p = reinterpret_cast<const float4*>(cs_row + (((col0 + col) & g.rope_head_mask) >> 1));
#pragma unroll
            for (int q = 0; q < 4; ++q) cs[q] = __ldg(p + q);
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float2 v = mul2(make_float2(__uint_as_float(r[col + 2 * q]), __uint_as_float(r[col + 2 * q + 1])), gs2);
          if constexpr (SILU) { if (silu_here) v = make_float2(silu_fast(v.x), silu_fast(v.y)); }
          uint32_t o = f32x2_to_bf16x2(v.x, v.y);
          if constexpr (ROPE) {
            if (rope_here) {
              // even' = fma(x, cos, -(y*sin)), odd' = fma(y, cos, x*sin); the packed forms rotate the rounded output
              const float x = g.rope_round_bf16 ? bf16lo_to_f32(o) : v.x, y = g.rope_round_bf16 ? bf16hi_to_f32(o) : v.y;
              const float cc = (q & 1) ? cs[q >> 1].z : cs[q >> 1].x, sn = (q & 1) ? cs[q >> 1].w : cs[q >> 1].y;
              o = f32x2_to_bf16x2(__fmaf_rn(x, cc, -__fmul_rn(y, sn)), __fmaf_rn(y, cc, __fmul_rn(x, sn)));
            }
          }
          w[h * 8 + q] = o;
        }
      }
      if (res_row != nullptr) {
        const uint4* rs = reinterpret_cast<const uint4*>(res_row + slab * 64);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint4 rv = __ldg(rs + q);
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t d = w[4 * q + e];
            w[4 * q + e] = f32x2_to_bf16x2(bf16lo_to_f32(d) + bf16lo_to_f32(rw[e]), bf16hi_to_f32(d) + bf16hi_to_f32(rw[e]));
          }
        }
      }
      uint8_t* buf = rowp + ((slab + slab0) & 1) * 4096;
      buffer_free();
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(buf + ((q ^ sw) << 4)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
      store_slab(epi + ((slab + slab0) & 1) * 4096, ocol + slab * 64);
    }
  }
}

// A region of 128 accumulator columns in the width the epilogue form's register budget affords: the plain and
// general forms lift all 128 columns at once; the rotary and SiLU forms work on 64 at a time (with 128 raw values
// live they spill, and with ~5 KB of L1 beside 222 KB of shared memory every spill is an L2 round trip), so their
// release comes after the second half's loads.
template <int EPI>
__device__ __forceinline__ void epilogue_region128(const GemmArgs& g, const GemmOutMaps& tmap_d, uint32_t taddr, uint8_t* epi,
                                                   int row0, int col0, float a_sg, int lane, AccRelease release,
                                                   uint32_t cs_taddr = 0) {
  if constexpr (EPI == kEpiRope || EPI == kEpiSilu) {
    if (cs_taddr != 0) {
      epilogue_region<EPI, 64, true>(g, tmap_d, taddr, epi, row0, col0, a_sg, lane, AccRelease{}, 0, cs_taddr);
      epilogue_region<EPI, 64, true>(g, tmap_d, taddr + 64, epi, row0, col0 + 64, a_sg, lane, release, 1, cs_taddr);
    } else {
      epilogue_region<EPI, 64>(g, tmap_d, taddr, epi, row0, col0, a_sg, lane, AccRelease{}, 0);
      epilogue_region<EPI, 64>(g, tmap_d, taddr + 64, epi, row0, col0 + 64, a_sg, lane, release, 1);
    }
  } else {
    epilogue_region<EPI, 128>(g, tmap_d, taddr, epi, row0, col0, a_sg, lane, release, 0);
  }
}

// Rotary / SiLU epilogue of the pair kernel's wide form: eight epilogue warps per CTA, two per lane quadrant, each
// owning 128 of the tile's 256 columns.  A warp lifts all its 128 accumulator columns into registers at once and
// releases them; the MMA thread then starts the next tile while the rotation (about 1400 instructions per lane and
// 256 columns: too many to sit between two tiles on one warp per scheduler) runs beside that tile's MMAs.  The
// registers for this come from the other warps of the CTA (setmaxnreg in the kernel).  Sixteen columns at a time:
// table values from this lane's copy of its table row in tensor memory (cs_taddr != 0) or from global memory, scale,
// SiLU, rotate, round, stage (one buffer of 32 rows x 128 bytes per warp, 128-byte swizzle), TMA store per 64 columns.
template <int EPI>
__device__ __forceinline__ void epilogue_wide(const GemmArgs& g, const GemmOutMaps& tmap_d, uint32_t taddr, uint8_t* epi,
                                              int row0, int col0, float a_sg, int lane, uint32_t release_cluster_addr,
                                              uint32_t cs_taddr) {
  constexpr bool SILU = EPI == kEpiSilu;
  uint32_t r[128];
#pragma unroll
  for (int k = 0; k < 4; ++k) tmem_ld32(taddr + (uint32_t)(32 * k), *reinterpret_cast<uint32_t(*)[32]>(&r[32 * k]));
  tmem_ld_wait();
  AccRelease{nullptr, release_cluster_addr}(lane);
  if (col0 >= g.N) return;   // second half of the last column tile when N is an odd multiple of 128

  float gs = a_sg;
  if (g.b_sg != nullptr) gs = a_sg * __ldg(g.b_sg + (g.b_sg_per_tile ? (col0 >> 8) : 0));
  const float2 gs2 = make_float2(gs, gs);
  const int row = row0 + lane;
  int oi = 0, col_start = 0;   // which output receives this column range
  while (oi + 1 < g.n_out && col0 >= g.d_col_end[oi]) { col_start = g.d_col_end[oi]; ++oi; }
  const int ocol = col0 - col_start;
  uint8_t* rowp = epi + lane * 128;
  const int sw = lane & 7;
  const __nv_bfloat16* res_row = g.residual != nullptr ? g.residual + (size_t)row * g.residual_ld + col0 : nullptr;
  const bool rope_region = g.rope_cs != nullptr && col0 < g.rope_col_end;
  const float2* cs_row = (rope_region && cs_taddr == 0) ? g.rope_cs + (size_t)(row & g.rope_seq_mask) * g.rope_pair_dim : nullptr;
#pragma unroll
  for (int slab = 0; slab < 2; ++slab) {          // 64 columns = 128 bytes per row
    // the staging buffer may be rewritten once the previous slab's store has read it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
#pragma unroll
    for (int h = 0; h < 4; ++h) {                 // 16 columns = eight pairs
      const int col = slab * 64 + h * 16;
      const bool silu_here = SILU && col0 + col < g.silu_col_end;
      const bool rope_here = rope_region && col0 + col < g.rope_col_end;
      uint32_t t[16];
      if (rope_here) {
        if (cs_taddr != 0) {
          tmem_ld16(cs_taddr + (uint32_t)((col0 + col) & g.rope_head_mask), t);
          tmem_ld_wait();
        } else {
          const uint4* p = reinterpret_cast<const uint4*>(cs_row + (((col0 + col) & g.rope_head_mask) >> 1));
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 f = __ldg(p + q);
            t[4 * q] = f.x; t[4 * q + 1] = f.y; t[4 * q + 2] = f.z; t[4 * q + 3] = f.w;
          }
        }
      }
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float2 v = mul2(make_float2(__uint_as_float(r[col + 2 * q]), __uint_as_float(r[col + 2 * q + 1])), gs2);
        if constexpr (SILU) { if (silu_here) v = make_float2(silu_fast(v.x), silu_fast(v.y)); }
        uint32_t o = f32x2_to_bf16x2(v.x, v.y);
        if (rope_here) {
          // even' = fma(x, cos, -(y*sin)), odd' = fma(y, cos, x*sin); the packed forms rotate the rounded output
          const float x = g.rope_round_bf16 ? bf16lo_to_f32(o) : v.x, y = g.rope_round_bf16 ? bf16hi_to_f32(o) : v.y;
          const float cc = __uint_as_float(t[2 * q]), sn = __uint_as_float(t[2 * q + 1]);
          o = f32x2_to_bf16x2(__fmaf_rn(x, cc, -__fmul_rn(y, sn)), __fmaf_rn(y, cc, __fmul_rn(x, sn)));
        }
        w[q] = o;
      }
      if (res_row != nullptr) {
        const uint4* rs = reinterpret_cast<const uint4*>(res_row + col);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint4 rv = __ldg(rs + q);
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t d = w[4 * q + e];
            w[4 * q + e] = f32x2_to_bf16x2(bf16lo_to_f32(d) + bf16lo_to_f32(rw[e]), bf16hi_to_f32(d) + bf16hi_to_f32(rw[e]));
          }
        }
      }
      *reinterpret_cast<uint4*>(rowp + (((2 * h) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(rowp + (((2 * h + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(&tmap_d.m[oi], epi, ocol + slab * 64, row0);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
}

// Batched accumulation in the pair kernel's wide structure (eight epilogue warps, 128 columns each): the MMA thread
// hands over one accumulator per term; a warp folds it into a register sum — term 0: acc * scale (rounded), later
// terms: fma(acc, scale, sum), the reference's order (nvfp4_batched_accum_gemm.cuh:293-310 as compiled) — 16 columns
// at a time, releases the accumulator, and after the last term rounds the sum to bf16 and stores it.
// acc_phase: the parity the warp waits for next; returns false when a wait ran out.
__device__ __forceinline__ float bf16_round_f32(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ bool epilogue_batch_sum(const GemmArgs& g, const GemmOutMaps& tmap_d, uint64_t* acc_full, uint32_t& acc_phase,
                                                   uint32_t taddr, uint8_t* epi, int row0, int col0, int lane,
                                                   uint32_t release_cluster_addr) {
  float sum[128];
  for (int term = 0; term < g.n_seg; ++term) {
    if (!mbar_wait_timed(acc_full, acc_phase)) {
      if (lane == 0) atomicExch(g.status, kStatusGemmTmemTimeout);
      return false;
    }
    acc_phase ^= 1;
    tc_fence_after();
    const float gs = __ldg(g.seg_a_sg[term]) * __ldg(g.seg_b_sg[term]);
#pragma unroll
    for (int c = 0; c < 8; ++c) {          // sixteen columns at a time: the sum already holds 128 registers
      uint32_t r[16];
      tmem_ld16(taddr + (uint32_t)(16 * c), r);
      tmem_ld_wait();
      if (g.round_terms) {
        // every term as the bf16 matrix a GEMM of its own would have written, added to the bf16 sum so far
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float t = bf16_round_f32(__fmul_rn(__uint_as_float(r[q]), gs));
          sum[16 * c + q] = term == 0 ? t : bf16_round_f32(__fadd_rn(sum[16 * c + q], t));
        }
      } else if (term == 0) {
#pragma unroll
        for (int q = 0; q < 16; ++q) sum[16 * c + q] = __fmul_rn(__uint_as_float(r[q]), gs);
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) sum[16 * c + q] = __fmaf_rn(__uint_as_float(r[q]), gs, sum[16 * c + q]);
      }
    }
    AccRelease{nullptr, release_cluster_addr}(lane);
  }
  if (col0 >= g.N) return true;   // second half of the last column tile when N is an odd multiple of 128
  uint8_t* rowp = epi + lane * 128;
  const int sw = lane & 7;
#pragma unroll
  for (int slab = 0; slab < 2; ++slab) {          // 64 columns = 128 bytes per row
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float* v = sum + slab * 64 + 8 * q;
      *reinterpret_cast<uint4*>(rowp + ((q ^ sw) << 4)) =
          make_uint4(f32x2_to_bf16x2(v[0], v[1]), f32x2_to_bf16x2(v[2], v[3]), f32x2_to_bf16x2(v[4], v[5]), f32x2_to_bf16x2(v[6], v[7]));
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(&tmap_d.m[0], epi, col0 + slab * 64, row0);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  return true;
}

// K-segment bookkeeping of the producer: which segment a K stage belongs to and its index inside the segment.
struct SegCursor {
  int seg = -1, seg_end = 0, kl = 0;
  __device__ __forceinline__ bool enter(const GemmArgs& g, int ks) {   // true at a segment's first stage
    if (ks != seg_end) { ++kl; return false; }
    ++seg;
    seg_end = g.seg_stage_end[seg];
    kl = 0;
    return true;
  }
};

// EPI: one epilogue form per instantiation, chosen by the host.  Several forms inside one kernel cost every one of
// them a few percent.
template <bool MX, int EPI = kEpiPlain>
__global__ void __launch_bounds__(kGemmThreads, 1)
fp4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ GemmBMaps tmap_b,
                const __grid_constant__ GemmOutMaps tmap_d, const GemmArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  GemmSmem& sm = *reinterpret_cast<GemmSmem*>(smem_align_1024(smem_raw));

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int tiles_m = g.M / kGemmBM, tiles_n = (g.N + kGemmBN - 1) / kGemmBN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_stages = g.seg_stage_end[g.n_seg - 1];   // stages of 256 elements (the very last may hold 128)
  const bool k_tail_half = g.seg_tail_half[g.n_seg - 1] != 0;   // only a plain MXFP4 GEMM (one segment) can have one

  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); mbar_init(&sm.sf_ready[s], 4); }
    mbar_init(&sm.acc_full, 1);
    mbar_init(&sm.acc_empty, 4);   // one arrival per epilogue warp
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    for (int s = 0; s < g.n_seg; ++s) tma_prefetch_desc(&tmap_b.m[s]);
  }
  if (warp == 1) {   // tensor-memory allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  // Launched as a programmatic dependent, everything above ran beside the previous kernel's tail; nothing below
  // touches global memory before that kernel's writes are visible.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        int tm, tn;
        raster_tile(t, tiles_m, tiles_n, tm, tn);
        SegCursor cur;
        int a_col = 0;
        const CUtensorMap* bmap = nullptr;
        const uint8_t *sfa_src = nullptr, *sfb_src0 = nullptr, *sfb_src1 = nullptr;
        for (int ks = 0; ks < k_stages; ++ks) {
          if (cur.enter(g, ks)) {   // first stage of the next K segment
            a_col = g.seg_a_col_bytes[cur.seg];
            bmap = &tmap_b.m[cur.seg];
            const size_t tiles_k = (size_t)g.seg_sf_tiles_k[cur.seg];
            sfa_src = g.seg_a_sc[cur.seg] + (size_t)tm * (size_t)g.seg_a_sf_row_tiles[cur.seg] * 512;
            sfb_src0 = g.seg_b_sc[cur.seg] + (size_t)(2 * tn) * tiles_k * 512;
            // the last column tile of an N that is an odd multiple of 128 has no second group of B rows
            sfb_src1 = (2 * tn + 1) * 128 < g.N ? sfb_src0 + tiles_k * 512 : sfb_src0;
          }
          if (!mbar_wait_timed(&sm.empty[stage], phase ^ 1)) {
            atomicExch(g.status, kStatusGemmTmaTimeout);
            ok = false;
            break;
          }
          constexpr int kSfPerStage = MX ? 1024 : 2048;
          const uint32_t sf_bytes = (MX && k_tail_half && ks + 1 == k_stages) ? kSfPerStage / 2 : kSfPerStage;
          mbar_expect_tx(&sm.full[stage], kATileBytes + kBTileBytes + 3 * sf_bytes);
          tma_load_2d(sm.a[stage], &tmap_a, a_col + cur.kl * kGemmBKBytes, tm * kGemmBM, &sm.full[stage]);
          tma_load_2d(sm.b[stage], bmap, cur.kl * kGemmBKBytes, tn * kGemmBN, &sm.full[stage]);
          // scale tiles of this stage: NVFP4 4 tiles (256/64), MXFP4 2 tiles (256/128) per row tile
          bulk_load_1d(sm.sfa[stage], sfa_src + (size_t)cur.kl * kSfPerStage, sf_bytes, &sm.full[stage]);
          bulk_load_1d(sm.sfb[stage], sfb_src0 + (size_t)cur.kl * kSfPerStage, sf_bytes, &sm.full[stage]);
          bulk_load_1d(sm.sfb[stage] + kSfPerStage, sfb_src1 + (size_t)cur.kl * kSfPerStage, sf_bytes, &sm.full[stage]);
          if (++stage == kGemmStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
        // the epilogue must have lifted the previous tile's accumulator out of tensor memory
        if (!mbar_wait_timed(&sm.acc_empty, acc_phase ^ 1)) {
          atomicExch(g.status, kStatusGemmEpilogueTimeout);
          ok = false;
          break;
        }
        tc_fence_after();
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait_timed(&sm.sf_ready[stage], phase)) {   // operands landed and scales are in tensor memory
            atomicExch(g.status, kStatusGemmMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sf_cols = tmem + kSfTmemBase + stage * kSfSlotCols;
          const uint32_t a_base = smem_u32(sm.a[stage]);
          const uint32_t b_base = smem_u32(sm.b[stage]);
          // MXFP4 with K an odd multiple of 128: the very last stage holds 128 elements, two MMAs instead of four
          // (a branch of its own: a run-time MMA count in the unrolled loop cost every stage of every shape ~4 %)
          if (MX && k_tail_half && ks + 1 == k_stages) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tc_mma<true>(tmem, smem_desc(a_base + j * 32, 16, 1024, 2), smem_desc(b_base + j * 32, 16, 1024, 2),
                          block_scaled_idesc(kGemmBM, kGemmBN, 1, j * 2), sf_cols, sf_cols + 16, (ks | j) != 0);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint64_t adesc = smem_desc(a_base + j * 32, 16, 1024, 2);
              const uint64_t bdesc = smem_desc(b_base + j * 32, 16, 1024, 2);
              if constexpr (!MX) {
                tc_mma<false>(tmem, adesc, bdesc, block_scaled_idesc(kGemmBM, kGemmBN, 0, 0), sf_cols + j * 4,
                             sf_cols + 16 + j * 8, (ks | j) != 0);
              } else {
                const int sf_id = (j & 1) * 2;   // bytes 0..1 or 2..3 of the scale column
                tc_mma<true>(tmem, adesc, bdesc, block_scaled_idesc(kGemmBM, kGemmBN, 1, sf_id),
                            sf_cols + (j >> 1) * 4, sf_cols + 16 + (j >> 1) * 8, (ks | j) != 0);
              }
            }
          }
          tc_commit(&sm.empty[stage]);   // frees the shared-memory stage once these MMAs have read it
          if (++stage == kGemmStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&sm.acc_full);
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------ scale movers ------------------------------------------
    // Four warps, one per tensor-memory lane quadrant, move each stage's scale tiles from shared
    // memory into tensor memory through registers (tcgen05.st), which keeps the tensor pipe free
    // for MMAs (a tcgen05.cp per 512-byte tile would serialise with them).  Every quadrant gets
    // the same 16 bytes per lane: row l of a tile, i.e. the scales of tile rows l, 32+l, 64+l, 96+l.
    const int quad = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    constexpr int kTiles = MX ? 2 : 4;            // scale tiles per 128-row group per stage
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_timed(&sm.full[stage], phase)) {
          if (lane == 0) atomicExch(g.status, kStatusGemmMmaTimeout);
          ok = false;
          break;
        }
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + kSfTmemBase + stage * kSfSlotCols;
        uint32_t ra[16], rb[32];
        load_stage_scales<kTiles>(sm.sfa[stage], sm.sfb[stage], lane, ra, rb);
        tmem_st16(taddr, ra);
        tmem_st32(taddr + 16, rb);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.sf_ready[stage]);
        if (++stage == kGemmStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------------------
    const int quad = warp & 3;                 // tensor-memory lane quadrant this warp may read
    uint32_t acc_phase = 0;
    float a_sg = g.fixed_scale;
    if (g.a_sg != nullptr) a_sg = __ldg(g.a_sg);
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      int tm, tn;
      raster_tile(t, tiles_m, tiles_n, tm, tn);
      if (!mbar_wait_timed(&sm.acc_full, acc_phase)) {
        if (lane == 0) atomicExch(g.status, kStatusGemmTmemTimeout);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t tq = tmem + ((uint32_t)(quad * 32) << 16);
      uint8_t* epi = &sm.epi[warp - 2][0][0];
      const int row0 = tm * kGemmBM + quad * 32;
      epilogue_region128<EPI>(g, tmap_d, tq, epi, row0, tn * kGemmBN, a_sg, lane, AccRelease{});
      // both halves are out of tensor memory: let the MMA warp start the next tile
      epilogue_region128<EPI>(g, tmap_d, tq + 128, epi, row0, tn * kGemmBN + 128, a_sg, lane, AccRelease{&sm.acc_empty, 0});
      acc_phase ^= 1;
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // staged stores have left shared memory
  }

  // common exit: every role arrives here (also after a timeout); release tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace fp4b200

#include "gemm_fp4_pair.cuh"

namespace fp4b200 {

// FP4B200_GEMM_PAIR=0 in the environment selects the one-CTA kernel for every shape (A/B comparisons).
static bool gemm_pair_disabled() {
  static const bool off = [] { const char* e = getenv("FP4B200_GEMM_PAIR"); return e != nullptr && e[0] == '0'; }();
  return off;
}

// Programmatic dependent launch of the GEMM kernels: on unless FP4B200_GEMM_PDL=0 or the calling thread has switched
// it off with fp4b200_set_gemm_pdl(0) (the mirrors' *_nopdl entry points do, around their one call).
static thread_local int t_gemm_pdl = 1;
static bool gemm_pdl_enabled() {
  static const bool env_off = [] { const char* e = getenv("FP4B200_GEMM_PDL"); return e != nullptr && e[0] == '0'; }();
  return !env_off && t_gemm_pdl != 0;
}

// K segments of one GEMM launch on the host side: D = sum_s A[:, off_s : off_s + k_s] * B_s^T, all
// accumulated in tensor memory before the one epilogue.  a_width = elements per row of A's code matrix.
struct KSegments {
  int n = 0;
  int64_t a_width = 0;
  int64_t a_col_off[kMaxKSeg] = {0, 0, 0, 0};   // elements
  int64_t k[kMaxKSeg] = {0, 0, 0, 0};           // elements, multiples of 256
  const void* a_sc[kMaxKSeg] = {nullptr, nullptr, nullptr, nullptr};
  const void* b[kMaxKSeg] = {nullptr, nullptr, nullptr, nullptr};
  const void* b_sc[kMaxKSeg] = {nullptr, nullptr, nullptr, nullptr};
  // batched accumulation (two-CTA kernel only): every segment is a term with its own A tensor [M, k/2] and tensor scales,
  // summed in fp32 by the epilogue instead of in tensor memory
  bool batch_sum = false;
  bool round_terms = false;   // with batch_sum: bf16(term) summed in bf16, left to right, instead of one fp32 sum
  const void* a[kMaxKSeg] = {nullptr, nullptr, nullptr, nullptr};
  const float* a_sg[kMaxKSeg] = {nullptr, nullptr, nullptr, nullptr};
  const float* b_sg[kMaxKSeg] = {nullptr, nullptr, nullptr, nullptr};
  // a term's A may be a column slice of a wider code matrix: row pitch of its codes in bytes (0: k/2) and scale tiles
  // from one 128-row block of its scale tensor to the next (0: k/64)
  int64_t a_pitch_bytes[kMaxKSeg] = {0, 0, 0, 0};
  int64_t a_sc_row_tiles[kMaxKSeg] = {0, 0, 0, 0};
};

// Rotary embedding applied by the bf16 epilogue to the output columns [0, col_end).
struct RopeDesc {
  const float2* cs;   // [seq_len, head_dim/2] (cos, sin), seq_len and head_dim powers of two; null: no rotation
  int seq_len, head_dim, col_end, round_bf16;
  int silu_col_end;   // SiLU on the columns [0, silu_col_end) before the rotation; 0: none
};

static int launch_gemm_segs(bool mx, const void* A, const KSegments& segs, const float* A_sg, const float* B_sg,
                            int b_sg_per_tile, void* const* D, const int* d_col_end, const int* d_ld, int n_out,
                            int out_fp32, const void* residual, int residual_ld, int64_t M, int64_t N, cudaStream_t st,
                            const float* accum_f32 = nullptr, const RopeDesc* rope = nullptr) {
  const bool pair = (M % 256) == 0 && !gemm_pair_disabled();
  CUtensorMap tmap_a;
  GemmBMaps tmap_b, tmap_a_seg;
  memset(&tmap_b, 0, sizeof(tmap_b));
  memset(&tmap_a_seg, 0, sizeof(tmap_a_seg));
  if (segs.batch_sum && (!pair || mx || out_fp32 || residual != nullptr || accum_f32 != nullptr || rope != nullptr || n_out != 1))
    return set_error("batched accumulation in one kernel: NVFP4, M a multiple of 256, one bf16 output");
  if (segs.batch_sum) {
    for (int s = 0; s < segs.n; ++s)
      if (int rc = make_tmap_2d(&tmap_a_seg.m[s], segs.a[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)segs.k[s] / 2, (uint64_t)M,
                                segs.a_pitch_bytes[s] > 0 ? (uint64_t)segs.a_pitch_bytes[s] : (uint64_t)segs.k[s] / 2, kGemmBKBytes,
                                kGemmBM, CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    tmap_a = tmap_a_seg.m[0];
  } else if (int rc = make_tmap_2d(&tmap_a, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)segs.a_width / 2, (uint64_t)M,
                                   (uint64_t)segs.a_width / 2, kGemmBKBytes, kGemmBM, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  int64_t K = 0, stages = 0;
  GemmArgs g{};
  g.n_seg = segs.n;
  for (int s = 0; s < segs.n; ++s) {
    // the pair kernel loads B in halves of 128 rows per CTA
    if (int rc = make_tmap_2d(&tmap_b.m[s], segs.b[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)segs.k[s] / 2, (uint64_t)N,
                              (uint64_t)segs.k[s] / 2, kGemmBKBytes, pair ? 128 : kGemmBN, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
    K += segs.k[s];
    stages += (segs.k[s] + 255) / 256;
    g.seg_stage_end[s] = (int)stages;
    g.seg_tail_half[s] = (segs.k[s] % 256) != 0;
    g.seg_a_col_bytes[s] = (int)(segs.a_col_off[s] / 2);
    g.seg_a_sc[s] = (const uint8_t*)segs.a_sc[s];
    g.seg_b_sc[s] = (const uint8_t*)segs.b_sc[s];
    g.seg_sf_tiles_k[s] = (int)(segs.k[s] / (mx ? 128 : 64));
    g.seg_a_sf_row_tiles[s] = segs.a_sc_row_tiles[s] > 0 ? (int)segs.a_sc_row_tiles[s] : g.seg_sf_tiles_k[s];
    g.seg_a_sg[s] = segs.a_sg[s];
    g.seg_b_sg[s] = segs.b_sg[s];
  }
  g.a_per_seg = segs.batch_sum ? 1 : 0;
  g.round_terms = (segs.batch_sum && segs.round_terms) ? 1 : 0;
  GemmOutMaps omaps;
  memset(&omaps, 0, sizeof(omaps));
  for (int i = 0; i < n_out; ++i) {
    const uint64_t cols = (uint64_t)d_ld[i];
    if (int rc = make_tmap_2d(&omaps.m[i], D[i], out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                              out_fp32 ? 4 : 2, cols, (uint64_t)M, cols * (out_fp32 ? 4 : 2), out_fp32 ? 32 : 64, 32,
                              CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  g.a_sg = A_sg; g.b_sg = B_sg; g.b_sg_per_tile = b_sg_per_tile;
  g.fixed_scale = mx ? (1.0f / 36.0f) : 1.0f;
  for (int i = 0; i < 3; ++i) { g.d[i] = i < n_out ? D[i] : nullptr; g.d_col_end[i] = i < n_out ? d_col_end[i] : 0; g.d_ld[i] = i < n_out ? d_ld[i] : 0; }
  g.n_out = n_out; g.out_fp32 = out_fp32;
  g.residual = (const __nv_bfloat16*)residual; g.residual_ld = residual_ld;
  g.accum_f32 = accum_f32;
  if (rope != nullptr) {
    g.rope_cs = rope->cs; g.rope_seq_mask = rope->seq_len - 1; g.rope_pair_dim = rope->head_dim / 2;
    g.rope_head_mask = rope->head_dim - 1; g.rope_col_end = rope->cs != nullptr ? rope->col_end : 0;
    g.rope_round_bf16 = rope->round_bf16; g.silu_col_end = rope->silu_col_end;
  }
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.rope_in_tmem = pair && g.rope_cs != nullptr && (rope->head_dim == 64 || rope->head_dim == 128);
  g.status = device_status_ptr();
  if (g.status == nullptr) return -1;
  const int epi = segs.batch_sum ? kEpiBatchSum
                  : (g.out_fp32 || g.accum_f32 != nullptr) ? kEpiGeneral
                  : g.silu_col_end > 0 ? kEpiSilu : g.rope_cs != nullptr ? kEpiRope : kEpiPlain;
  if (pair) {
    // two-CTA clusters: one 256 x 256 tile per pair of SMs
    const int psmem = (int)sizeof(GemmPairSmem) + 1024;
    const int pair_tiles = (int)((M / 256) * ((N + kGemmBN - 1) / kGemmBN));
    const int clusters = std::min(pair_tiles, device_sm_count() / 2);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * clusters, 1, 1);
    // the MXFP4 kernels with another epilogue form than the rotary one are instantiated as kEpiPlain / kEpiGeneral
    cfg.blockDim = dim3(pair_form_is_wide(epi) && (!mx || epi == kEpiRope) ? kPairWideThreads : kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = psmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemm_pdl_enabled() ? 2 : 1;
#define FP4_LAUNCH_PAIR(MXF, EPI)                                                                                          \
  do {                                                                                                                   \
    FP4_CUDA_CHECK(cudaFuncSetAttribute(fp4_gemm_pair_kernel<MXF, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, psmem)); \
    FP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, fp4_gemm_pair_kernel<MXF, EPI>, tmap_a, tmap_b, omaps, g, tmap_a_seg));       \
  } while (0)
    if (mx) {
      if (epi == kEpiGeneral) FP4_LAUNCH_PAIR(true, kEpiGeneral);
      else if (epi == kEpiRope) FP4_LAUNCH_PAIR(true, kEpiRope);
      else FP4_LAUNCH_PAIR(true, kEpiPlain);
    } else if (epi == kEpiGeneral) FP4_LAUNCH_PAIR(false, kEpiGeneral);
    else if (epi == kEpiBatchSum) FP4_LAUNCH_PAIR(false, kEpiBatchSum);
    else if (epi == kEpiSilu) FP4_LAUNCH_PAIR(false, kEpiSilu);
    else if (epi == kEpiRope) FP4_LAUNCH_PAIR(false, kEpiRope);
    else FP4_LAUNCH_PAIR(false, kEpiPlain);
#undef FP4_LAUNCH_PAIR
    return 0;
  }
  const int smem = (int)sizeof(GemmSmem) + 1024;
  const int n_tiles = (int)((M / kGemmBM) * ((N + kGemmBN - 1) / kGemmBN));
  const int grid = std::min(n_tiles, device_sm_count());
  if (grid == 0) return 0;
  cudaLaunchConfig_t cfg1{};
  cfg1.gridDim = dim3(grid, 1, 1);
  cfg1.blockDim = dim3(kGemmThreads, 1, 1);
  cfg1.dynamicSmemBytes = smem;
  cfg1.stream = st;
  cudaLaunchAttribute attr1[1];
  attr1[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr1[0].val.programmaticStreamSerializationAllowed = 1;
  cfg1.attrs = attr1;
  cfg1.numAttrs = gemm_pdl_enabled() ? 1 : 0;
#define FP4_LAUNCH_ONE(MXF, EPI)                                                                                      \
  do {                                                                                                               \
    FP4_CUDA_CHECK(cudaFuncSetAttribute(fp4_gemm_kernel<MXF, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    FP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg1, fp4_gemm_kernel<MXF, EPI>, tmap_a, tmap_b, omaps, g));                   \
  } while (0)
  if (mx) {
    if (epi == kEpiGeneral) FP4_LAUNCH_ONE(true, kEpiGeneral);
    else if (epi == kEpiRope) FP4_LAUNCH_ONE(true, kEpiRope);
    else FP4_LAUNCH_ONE(true, kEpiPlain);
  } else if (epi == kEpiGeneral) FP4_LAUNCH_ONE(false, kEpiGeneral);
  else if (epi == kEpiSilu) FP4_LAUNCH_ONE(false, kEpiSilu);
  else if (epi == kEpiRope) FP4_LAUNCH_ONE(false, kEpiRope);
  else FP4_LAUNCH_ONE(false, kEpiPlain);
#undef FP4_LAUNCH_ONE
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// plain GEMM = one K segment covering all of A
static int launch_gemm(bool mx, const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                       const float* B_sg, int b_sg_per_tile, void* const* D, const int* d_col_end, const int* d_ld,
                       int n_out, int out_fp32, const void* residual, int residual_ld, int64_t M, int64_t N,
                       int64_t K, cudaStream_t st, const float* accum_f32 = nullptr, const RopeDesc* rope = nullptr) {
  KSegments segs;
  segs.n = 1;
  segs.a_width = K;
  segs.k[0] = K;
  segs.a_sc[0] = A_sc;
  segs.b[0] = B;
  segs.b_sc[0] = B_sc;
  return launch_gemm_segs(mx, A, segs, A_sg, B_sg, b_sg_per_tile, D, d_col_end, d_ld, n_out, out_fp32, residual, residual_ld,
                          M, N, st, accum_f32, rope);
}

}  // namespace fp4b200

using namespace fp4b200;

// k_mult: 256 (NVFP4: a K stage is four scale tiles of 64 elements) or 128 (MXFP4: a half-depth last stage)
static int check_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, int64_t M, int64_t N,
                      int64_t K, const char* who, int k_mult = 256) {
  if (!A || !A_sc || !B || !B_sc) return set_error("%s: operand pointer is null", who);
  if (M <= 0 || N <= 0 || K <= 0 || (M % kGemmBM) || (N % 128) || (K % k_mult))
    return set_error("%s: needs M %% 128 == 0, N %% 128 == 0, K %% %d == 0 (got M=%lld N=%lld K=%lld)", who, k_mult,
                     (long long)M, (long long)N, (long long)K);
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return set_error("%s: dimension too large", who);
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(A_sc) |
       reinterpret_cast<uintptr_t>(B_sc)) & 15)
    return set_error("%s: operands and scales must be 16-byte aligned", who);
  return 0;
}

extern "C" {

int fp4b200_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
  if (limit_cycles < 1 || limit_cycles > 100000000) return set_error("selftest_bounded_wait: the limit must be 1 to 1e8 cycles");
  int* status = device_status_ptr();
  if (status == nullptr) return -1;
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (long long)limit_cycles);
  FP4_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int fp4b200_set_gemm_pdl(int enabled) {
  const int before = t_gemm_pdl;
  t_gemm_pdl = enabled != 0;
  return before;
}

int fp4b200_nvfp4_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                       const float* B_sg, void* D, int out_fp32, const void* residual_bf16, int64_t M, int64_t N,
                       int64_t K, void* stream) {
  if (int rc = check_gemm(A, A_sc, B, B_sc, M, N, K, "nvfp4_gemm")) return rc;
  if (!A_sg || !B_sg || !D) return set_error("nvfp4_gemm: A_sg, B_sg and D are required");
  if (residual_bf16 && out_fp32) return set_error("nvfp4_gemm: the residual epilogue writes bf16 only");
  void* d[1] = {D};
  int ce[1] = {(int)N}, ld[1] = {(int)N};
  return launch_gemm(false, A, A_sc, A_sg, B, B_sc, B_sg, 0, d, ce, ld, 1, out_fp32, residual_bf16, (int)N, M, N, K,
                     (cudaStream_t)stream);
}

int fp4b200_nvfp4_gemm_accum(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                             const float* B_sg, const float* partial_f32, void* D, int out_fp32, int64_t M, int64_t N,
                             int64_t K, void* stream) {
  if (int rc = check_gemm(A, A_sc, B, B_sc, M, N, K, "nvfp4_gemm_accum")) return rc;
  if (!A_sg || !B_sg || !D || !partial_f32) return set_error("nvfp4_gemm_accum: A_sg, B_sg, partial_f32 and D are required");
  void* d[1] = {D};
  int ce[1] = {(int)N}, ld[1] = {(int)N};
  return launch_gemm(false, A, A_sc, A_sg, B, B_sc, B_sg, 0, d, ce, ld, 1, out_fp32, nullptr, 0, M, N, K,
                     (cudaStream_t)stream, partial_f32);
}

int fp4b200_nvfp4_batched_accum_gemm(int n_terms, const void* const* A, const void* const* A_sc, const float* const* A_sg,
                                     const void* const* B, const void* const* B_sc, const float* const* B_sg,
                                     const int64_t* K, const int64_t* A_pitch_bytes, const int64_t* A_sc_row_tiles, void* D,
                                     int64_t M, int64_t N, int round_each_term, void* stream) {
  const char* fn = "nvfp4_batched_accum_gemm";
  if (n_terms < 1 || n_terms > kMaxKSeg) return set_error("%s: 1 to %d terms (got %d)", fn, kMaxKSeg, n_terms);
  if (!A || !A_sc || !A_sg || !B || !B_sc || !B_sg || !K || !D) return set_error("%s: null argument", fn);
  if ((M % 256) != 0 || gemm_pair_disabled())
    return set_error("%s: the one-kernel form needs M to be a multiple of 256 (two-CTA kernel); use the chain of "
                     "fp4b200_nvfp4_gemm_accum launches otherwise", fn);
  KSegments segs;
  segs.n = n_terms;
  segs.batch_sum = true;
  segs.round_terms = round_each_term != 0;
  for (int i = 0; i < n_terms; ++i) {
    if (int rc = check_gemm(A[i], A_sc[i], B[i], B_sc[i], M, N, K[i], fn)) return rc;
    if (!A_sg[i] || !B_sg[i]) return set_error("%s: every term needs its tensor scales", fn);
    segs.k[i] = K[i];
    if (A_pitch_bytes != nullptr) {
      if (A_pitch_bytes[i] != 0 && (A_pitch_bytes[i] < K[i] / 2 || (A_pitch_bytes[i] % 16)))
        return set_error("%s: a row pitch of A must be 0 or a multiple of 16 bytes and at least K/2", fn);
      segs.a_pitch_bytes[i] = A_pitch_bytes[i];
    }
    if (A_sc_row_tiles != nullptr) {
      if (A_sc_row_tiles[i] != 0 && A_sc_row_tiles[i] < K[i] / 64)
        return set_error("%s: the scale tiles per row block of A must be 0 or at least K/64", fn);
      segs.a_sc_row_tiles[i] = A_sc_row_tiles[i];
    }
    segs.a[i] = A[i]; segs.a_sc[i] = A_sc[i]; segs.a_sg[i] = A_sg[i];
    segs.b[i] = B[i]; segs.b_sc[i] = B_sc[i]; segs.b_sg[i] = B_sg[i];
  }
  segs.a_width = K[0];
  void* d[1] = {D};
  int ce[1] = {(int)N}, ld[1] = {(int)N};
  return launch_gemm_segs(false, A[0], segs, nullptr, nullptr, 0, d, ce, ld, 1, 0, nullptr, 0, M, N, (cudaStream_t)stream);
}

int fp4b200_nvfp4_grouped_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                               const float* B_sg_per_tile, int n_out, void* const* D, const int64_t* D_cols,
                               int64_t M, int64_t N, int64_t K, void* stream) {
  if (int rc = check_gemm(A, A_sc, B, B_sc, M, N, K, "nvfp4_grouped_gemm")) return rc;
  if (!A_sg || !B_sg_per_tile || !D || !D_cols) return set_error("nvfp4_grouped_gemm: null argument");
  if (n_out < 1 || n_out > 3) return set_error("nvfp4_grouped_gemm: 1 to 3 outputs are supported");
  int ce[3] = {0, 0, 0}, ld[3] = {0, 0, 0};
  int64_t acc = 0;
  for (int i = 0; i < n_out; ++i) {
    if (!D[i] || D_cols[i] <= 0 || (D_cols[i] % kGemmBN))
      return set_error("nvfp4_grouped_gemm: every output needs a column count that is a multiple of 256");
    acc += D_cols[i];
    ce[i] = (int)acc;
    ld[i] = (int)D_cols[i];
  }
  if (acc != N) return set_error("nvfp4_grouped_gemm: output columns must add up to N");
  return launch_gemm(false, A, A_sc, A_sg, B, B_sc, B_sg_per_tile, 1, D, ce, ld, n_out, 0, nullptr, 0, M, N, K,
                     (cudaStream_t)stream);
}

int fp4b200_nvfp4_grouped_gemm_rope(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                                    const float* B_sg_per_tile, int n_out, void* const* D, const int64_t* D_cols,
                                    const float* rope_cs, int64_t rope_seq_len, int64_t rope_head_dim, int64_t rope_cols,
                                    int round_input_bf16, int64_t silu_dim, int64_t M, int64_t N, int64_t K, void* stream) {
  const char* fn = "nvfp4_grouped_gemm_rope";
  if (int rc = check_gemm(A, A_sc, B, B_sc, M, N, K, fn)) return rc;
  if (!A_sg || !B_sg_per_tile || !D || !D_cols) return set_error("%s: null argument", fn);
  if (n_out < 1 || n_out > 3) return set_error("%s: 1 to 3 outputs are supported", fn);
  if (rope_cs == nullptr && silu_dim <= 0) return set_error("%s: neither a rotation table nor a SiLU range was given", fn);
  if (silu_dim < 0 || silu_dim > N || (silu_dim % 32))
    return set_error("%s: silu_dim must be a multiple of 32 between 0 and N (got %lld)", fn, (long long)silu_dim);
  if (rope_cs != nullptr) {
    if (rope_seq_len <= 0 || (rope_seq_len & (rope_seq_len - 1)) || (M % rope_seq_len))
      return set_error("%s: rope_seq_len must be a power of two that divides M (got %lld)", fn, (long long)rope_seq_len);
    if (rope_head_dim < 16 || (rope_head_dim & (rope_head_dim - 1)) || rope_head_dim > 256)
      return set_error("%s: rope_head_dim must be a power of two between 16 and 256 (got %lld)", fn, (long long)rope_head_dim);
    if (reinterpret_cast<uintptr_t>(rope_cs) & 15) return set_error("%s: rope_cs must be 16-byte aligned", fn);
    if (rope_cols <= 0 || rope_cols > N || (rope_cols % 32) || (rope_cols % rope_head_dim))
      return set_error("%s: the rotated column range must be head-aligned, a multiple of 32 and at most N (got %lld)", fn,
                       (long long)rope_cols);
  }
  int ce[3] = {0, 0, 0}, ld[3] = {0, 0, 0};
  int64_t acc = 0;
  for (int i = 0; i < n_out; ++i) {
    if (!D[i] || D_cols[i] <= 0 || (D_cols[i] % kGemmBN))
      return set_error("%s: every output needs a column count that is a multiple of 256", fn);
    acc += D_cols[i];
    ce[i] = (int)acc;
    ld[i] = (int)D_cols[i];
  }
  if (acc != N) return set_error("%s: output columns must add up to N", fn);
  RopeDesc rope{reinterpret_cast<const float2*>(rope_cs), rope_cs ? (int)rope_seq_len : 1, rope_cs ? (int)rope_head_dim : 2,
                (int)rope_cols, round_input_bf16 != 0, (int)silu_dim};
  return launch_gemm(false, A, A_sc, A_sg, B, B_sc, B_sg_per_tile, 1, D, ce, ld, n_out, 0, nullptr, 0, M, N, K,
                     (cudaStream_t)stream, nullptr, &rope);
}

int fp4b200_mxfp4_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int out_fp32,
                       const void* residual_bf16, int64_t M, int64_t N, int64_t K, void* stream) {
  if (int rc = check_gemm(A, A_sc, B, B_sc, M, N, K, "mxfp4_gemm", 128)) return rc;
  if (!D) return set_error("mxfp4_gemm: D is required");
  if (residual_bf16 && out_fp32) return set_error("mxfp4_gemm: the residual epilogue writes bf16 only");
  void* d[1] = {D};
  int ce[1] = {(int)N}, ld[1] = {(int)N};
  return launch_gemm(true, A, A_sc, nullptr, B, B_sc, nullptr, 0, d, ce, ld, 1, out_fp32, residual_bf16, (int)N, M, N,
                     K, (cudaStream_t)stream);
}

int fp4b200_mxfp4_gemm_rope(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, const float* rope_cs,
                            int64_t rope_seq_len, int64_t rope_head_dim, int64_t M, int64_t N, int64_t K, void* stream) {
  const char* fn = "mxfp4_gemm_rope";
  if (int rc = check_gemm(A, A_sc, B, B_sc, M, N, K, fn, 128)) return rc;
  if (!D || !rope_cs) return set_error("%s: D and rope_cs are required", fn);
  if (rope_seq_len <= 0 || (rope_seq_len & (rope_seq_len - 1)) || (M % rope_seq_len))
    return set_error("%s: rope_seq_len must be a power of two that divides M (got %lld)", fn, (long long)rope_seq_len);
  if (rope_head_dim < 16 || (rope_head_dim & (rope_head_dim - 1)) || rope_head_dim > 256 || (N % rope_head_dim))
    return set_error("%s: rope_head_dim must be a power of two between 16 and 256 that divides N (got %lld)", fn,
                     (long long)rope_head_dim);
  if (reinterpret_cast<uintptr_t>(rope_cs) & 15) return set_error("%s: rope_cs must be 16-byte aligned", fn);
  void* d[1] = {D};
  int ce[1] = {(int)N}, ld[1] = {(int)N};
  RopeDesc rope{reinterpret_cast<const float2*>(rope_cs), (int)rope_seq_len, (int)rope_head_dim, (int)N, false, 0};
  return launch_gemm(true, A, A_sc, nullptr, B, B_sc, nullptr, 0, d, ce, ld, 1, 0, nullptr, 0, M, N, K, (cudaStream_t)stream,
                     nullptr, &rope);
}

int fp4b200_mxfp4_gemm_ksplit_strided(const void* A_full, int64_t a_width, int n_seg, const int64_t* a_col_offsets,
                                      const int64_t* a_col_widths, const void* const* A_sc_list,
                                      const int64_t* a_sc_row_tiles, const void* const* B_list,
                                      const void* const* B_sc_list, void* D, int out_fp32, int64_t M, int64_t N, void* stream) {
  if (!A_full || !a_col_offsets || !a_col_widths || !A_sc_list || !B_list || !B_sc_list || !D)
    return set_error("mxfp4_gemm_ksplit: null pointer");
  if (n_seg < 1 || n_seg > kMaxKSeg) return set_error("mxfp4_gemm_ksplit: 1 to %d K segments are supported", kMaxKSeg);
  if (a_width <= 0 || (a_width % 32)) return set_error("mxfp4_gemm_ksplit: the row width of A must be a positive multiple of 32");
  KSegments segs;
  segs.n = n_seg;
  segs.a_width = a_width;
  int64_t K = 0;
  for (int s = 0; s < n_seg; ++s) {
    const int64_t off = a_col_offsets[s], w = a_col_widths[s];
    if (w <= 0 || (w % 256) || off < 0 || (off % 32) || off + w > a_width)
      return set_error("mxfp4_gemm_ksplit: segment %d (offset %lld, width %lld) must be a multiple of 256 wide, start at a "
                       "multiple of 32 and lie inside the %lld columns of A", s, (long long)off, (long long)w, (long long)a_width);
    segs.a_col_off[s] = off; segs.k[s] = w;
    segs.a_sc[s] = A_sc_list[s]; segs.b[s] = B_list[s]; segs.b_sc[s] = B_sc_list[s];
    if (int rc = check_gemm(A_full, A_sc_list[s], B_list[s], B_sc_list[s], M, N, w, "mxfp4_gemm_ksplit")) return rc;
    if (a_sc_row_tiles != nullptr && a_sc_row_tiles[s] != 0) {
      if (a_sc_row_tiles[s] < w / 128 || a_sc_row_tiles[s] > INT32_MAX)
        return set_error("mxfp4_gemm_ksplit: segment %d: %lld scale tiles per row block cannot hold its %lld", s,
                         (long long)a_sc_row_tiles[s], (long long)(w / 128));
      segs.a_sc_row_tiles[s] = a_sc_row_tiles[s];
    }
    K += w;
  }
  void* d[1] = {D};
  int ce[1] = {(int)N}, ld[1] = {(int)N};
  return launch_gemm_segs(true, A_full, segs, nullptr, nullptr, 0, d, ce, ld, 1, out_fp32, nullptr, 0, M, N,
                          (cudaStream_t)stream);
}

int fp4b200_mxfp4_gemm_ksplit(const void* A_full, int64_t a_width, int n_seg, const int64_t* a_col_offsets,
                              const int64_t* a_col_widths, const void* const* A_sc_list, const void* const* B_list,
                              const void* const* B_sc_list, void* D, int out_fp32, int64_t M, int64_t N, void* stream) {
  return fp4b200_mxfp4_gemm_ksplit_strided(A_full, a_width, n_seg, a_col_offsets, a_col_widths, A_sc_list, nullptr, B_list,
                                           B_sc_list, D, out_fp32, M, N, stream);
}

}  // extern "C"
