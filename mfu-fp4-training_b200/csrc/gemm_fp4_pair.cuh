// Two-CTA ("pair") variant of the block-scaled FP4 GEMM: a cluster of two CTAs on neighbouring SMs
// computes one 256 x 256 output tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows
// of A and its own half (128 rows) of the B tile, so a K stage costs 38 KB of L2 -> SM traffic per SM
// instead of 54 KB for the same MMA work — operand delivery, not the tensor pipe, bounds the
// one-CTA kernel.  No multicast loads: the second CTA's data arrives through its own TMA.
//
// Tensor-memory plan (512 columns per SM): consecutive tiles of a pair alternate between the accumulator
// columns [0, 256) and [128, 384), so that only the middle 128 columns are shared between a tile and the next.
// The epilogue lifts that shared half into registers first (~300 cycles) and releases it; the MMA thread then
// starts the next tile while the private half is drained, scaled, rounded and stored.  The block scales of two
// K stages (2 x 48 columns from column 384) fit beside the accumulators.
//
// What bounds this kernel is shared-memory bandwidth (128 B per clock and SM for reads and writes together): at
// the tensor pipe's full rate the operands alone need 64 B per clock to arrive and 64 B per clock to be read;
// scale tiles (written once, read by four mover warps) and staged outputs come on top.  Measured per 256-deep
// stage: ~760 cycles where the MMAs alone take 512.  Moving the scales with tcgen05.cp (one read per tile,
// replicated to the four lane quadrants by the copy) was measured too and is slower: twelve copies per stage
// cost ~1100 cycles of the tensor pipe when the MMA thread issues them and ~600 when a thread of their own does.
// Included by gemm_fp4.cu after the shared helpers.
#pragma once

namespace fp4b200 {

constexpr int kPairStages = 5;
constexpr int kPairBHalfBytes = 128 * kGemmBKBytes;   // this CTA's half of the B tile: 16 KiB
// K stages whose scales are resident in tensor memory, and the columns of one such slot.  NVFP4: 16 columns of A
// scales + 32 of B scales per stage, two slots in the 128 columns beside the accumulators.  MXFP4 has half the scale
// bytes: 8 + 16 columns, one slot per shared-memory stage, so its movers may run as far ahead of the MMA thread as the
// TMA producer does instead of one stage.  With two slots the hand-over of a stage — scales written, waited for,
// announced across the cluster, MMAs issued — has to fit inside one stage's MMA time, and it does not quite: five slots
// took the MXFP4 GEMM at K = 14336 from 5.34 to 5.80 PFLOP/s.  NVFP4 in five HALF-stage slots of the same 24 columns
// (two MMAs each, a completion barrier per half) was built and measured as well: correct, and 8 % slower — the
// hand-over's fixed cost is paid twice per stage then; five whole-stage NVFP4 slots behind the single accumulator of the
// batched-accumulation form: 1 % slower (with twice the scale bytes the shared-memory port binds first).
constexpr int kPairSfSlotsNv = 2, kPairSfSlotsMx = 5;
constexpr int kPairSfSlotsMax = 5;
constexpr int kPairSfSlotColsMx = 24;
constexpr int kPairSfBase = 384;                      // accumulators occupy columns [0, 384)
constexpr int kPairThreads = kGemmThreads;            // producer, MMA thread, four epilogue warps, four scale movers
// The rotary / SiLU forms ("wide"): four warpgroups — {producer, MMA thread, two idle warps}, four scale movers, and two
// groups of four epilogue warps — with the register file re-divided between them (setmaxnreg), because an epilogue
// warp there holds 128 raw accumulator columns while it rotates them.  56 + 88 + 2 x 184 = 512 = 4 x 128.
constexpr int kPairWideThreads = 512;
constexpr int kWideRegsControl = 56, kWideRegsMovers = 88, kWideRegsEpilogue = 184;
// batched accumulation: the producer and the MMA thread track segments as well (56 + 72 + 2 x 192 = 512)
constexpr int kSumRegsControl = 56, kSumRegsMovers = 72, kSumRegsEpilogue = 192;
__host__ __device__ constexpr bool pair_form_is_wide(int epi) { return epi == kEpiRope || epi == kEpiSilu || epi == kEpiBatchSum; }

struct GemmPairSmem {
  alignas(1024) uint8_t a[kPairStages][kATileBytes];
  alignas(1024) uint8_t b[kPairStages][kPairBHalfBytes];
  alignas(1024) uint8_t epi[4][2][4096];       // per epilogue warp: two slabs of 32 rows x 128 bytes
  alignas(128) uint8_t sfa[kPairStages][kASfBytes];
  alignas(128) uint8_t sfb[kPairStages][kBSfBytes];
  alignas(8) uint64_t full[kPairStages];       // this CTA's TMA data of the stage has landed
  alignas(8) uint64_t empty[kPairStages];      // the pair's MMAs have finished reading the stage (and its scale slot)
  alignas(8) uint64_t sf_ready[kPairSfSlotsMax];  // leader only: operands + scales of BOTH CTAs are in place
  alignas(8) uint64_t acc_full;                // accumulator of the tile is complete
  alignas(8) uint64_t acc_empty_shared;        // leader only: both CTAs have lifted columns [128, 256) out
  alignas(8) uint64_t acc_empty_priv[2];       // leader only: columns [0, 128) / [256, 384)
  uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// Arrival on a barrier of any CTA of the pair.  Relaxed: the arriving threads publish no generic-proxy
// writes (tensor-memory stores and loads are ordered by tcgen05.wait + tcgen05.fence, operand tiles by the
// TMA's own mbarrier), and a cluster-scope release was measured at ~1200 cycles per arrival while TMA
// traffic is in flight.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// completion of all earlier tcgen05 operations of this thread -> one arrival on the barrier at this offset in
// BOTH CTAs of the pair (one instruction in the tensor pipe's queue, no forwarding hop)
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}

// Which tiles a CTA pair works through, and in which order.  Default: tile t = pair + i * pairs in the grouped
// raster order (compact blocks of the output in flight at a time).  With the rotary table in tensor memory
// (rope_in_tmem): a contiguous run of tiles in row-major order, so that a pair stays on one row block of the output
// for many tiles in a row and re-fills its (cos, sin) rows once or twice per launch; the accumulator then does not
// alternate (columns [256, 384) hold the table rows).
struct PairTiles {
  int first, step, count, tiles_m, tiles_n;
  bool row_major;
  __device__ __forceinline__ PairTiles(const GemmArgs& g, int pair, int pairs, int tiles_m_, int tiles_n_)
      : tiles_m(tiles_m_), tiles_n(tiles_n_), row_major(g.rope_in_tmem != 0) {
    const int n = tiles_m * tiles_n;
    if (row_major) {
      first = (int)((long long)pair * n / pairs);
      step = 1;
      count = (int)((long long)(pair + 1) * n / pairs) - first;
    } else {
      first = pair;
      step = pairs;
      count = pair < n ? (n - pair + pairs - 1) / pairs : 0;
    }
  }
  __device__ __forceinline__ void get(int i, int& tm, int& tn) const {
    const int t = first + i * step;
    if (row_major) { tm = t / tiles_n; tn = t - tm * tiles_n; }
    else raster_tile(t, tiles_m, tiles_n, tm, tn);
  }
};

template <bool MX>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (MX) {
    asm volatile(
        "{.reg .pred p; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{.reg .pred p; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// EPI: one epilogue form per instantiation, chosen by the host (see epilogue_region).
template <bool MX, int EPI = kEpiPlain>
__global__ void __launch_bounds__(pair_form_is_wide(EPI) ? kPairWideThreads : kPairThreads, 1)
fp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ GemmBMaps tmap_b,
                     const __grid_constant__ GemmOutMaps tmap_d, const GemmArgs g,
                     const __grid_constant__ GemmBMaps tmap_a_seg) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  GemmPairSmem& sm = *reinterpret_cast<GemmPairSmem*>(smem_align_1024(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int tiles_m = g.M / 256, tiles_n = (g.N + kGemmBN - 1) / kGemmBN;
  const PairTiles tiles(g, cluster_id, n_clusters, tiles_m, tiles_n);
  constexpr bool kWide = pair_form_is_wide(EPI);
  constexpr bool kBatchSum = EPI == kEpiBatchSum;   // every K segment is a term with an accumulator hand-over of its own
  constexpr int kRegsControl = kBatchSum ? kSumRegsControl : kWideRegsControl, kRegsMovers = kBatchSum ? kSumRegsMovers : kWideRegsMovers,
                kRegsEpilogue = kBatchSum ? kSumRegsEpilogue : kWideRegsEpilogue;
  // roles by warp: 0 producer, 1 MMA thread; scale movers and epilogue warps in lane-quadrant order (warp & 3)
  constexpr int kMoverWarp0 = kWide ? 4 : 6, kEpiWarp0 = kWide ? 8 : 2, kEpiWarps = kWide ? 8 : 4;
  const int kind_toggle = (kWide || g.rope_in_tmem) ? 0 : 1;      // 0: the accumulator stays at columns [0, 256)
  const int k_stages = g.seg_stage_end[g.n_seg - 1];
  const bool k_tail_half = g.seg_tail_half[g.n_seg - 1] != 0;   // only a plain MXFP4 GEMM (one segment) can have one
  constexpr int kSfPerStage = MX ? 1024 : 2048;
  constexpr int kPairSfSlots = MX ? kPairSfSlotsMx : kPairSfSlotsNv;
  constexpr int kSlotCols = MX ? kPairSfSlotColsMx : kSfSlotCols;
  constexpr int kSfbOff = MX ? 8 : 16;          // B scales behind the A scales of the slot
  static_assert(kPairSfBase + kPairSfSlots * kSlotCols <= 512, "scale slots must fit beside the accumulators");
  static_assert(!MX || kPairSfSlots == kPairStages, "MXFP4: the scale slot of a stage is the stage");

  if (tid == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int s = 0; s < kPairSfSlots; ++s) mbar_init(&sm.sf_ready[s], 8);   // four mover warps of each CTA
    mbar_init(&sm.acc_full, 1);
    mbar_init(&sm.acc_empty_shared, 2 * kEpiWarps);                          // the epilogue warps of each CTA
    mbar_init(&sm.acc_empty_priv[0], 8);
    mbar_init(&sm.acc_empty_priv[1], 8);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    for (int s = 0; s < g.n_seg; ++s) tma_prefetch_desc(&tmap_b.m[s]);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before any remote arrival
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  // Launched as a programmatic dependent, everything above ran beside the previous kernel's tail; nothing below
  // touches global memory before that kernel's writes are visible.
  pdl_launch_dependents();
  pdl_wait();

  if (kWide && warp >= 2 && warp < 4) {
    // idle warps of the first warpgroup: they only hand their registers over
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
  } else if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) --------------------------------
    if constexpr (kWide) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int ti = 0; ti < tiles.count && ok; ++ti) {
        int tm, tn;
        tiles.get(ti, tm, tn);
        SegCursor cur;
        int a_col = 0;
        const CUtensorMap* bmap = nullptr;
        const CUtensorMap* amap = &tmap_a;
        const uint8_t *sfa_src = nullptr, *sfb_src0 = nullptr, *sfb_src1 = nullptr;
        for (int ks = 0; ks < k_stages; ++ks) {
          if (cur.enter(g, ks)) {   // first stage of the next K segment
            a_col = g.seg_a_col_bytes[cur.seg];
            bmap = &tmap_b.m[cur.seg];
            if (g.a_per_seg) amap = &tmap_a_seg.m[cur.seg];
            const size_t tiles_k = (size_t)g.seg_sf_tiles_k[cur.seg];
            sfa_src = g.seg_a_sc[cur.seg] + (size_t)(2 * tm + rank) * (size_t)g.seg_a_sf_row_tiles[cur.seg] * 512;
            sfb_src0 = g.seg_b_sc[cur.seg] + (size_t)(2 * tn) * tiles_k * 512;
            // the last column tile of an N that is an odd multiple of 128 has no second group of B rows
            sfb_src1 = (2 * tn + 1) * 128 < g.N ? sfb_src0 + tiles_k * 512 : sfb_src0;
          }
          if (!mbar_wait_timed(&sm.empty[stage], phase ^ 1)) {
            atomicExch(g.status, kStatusGemmTmaTimeout);
            ok = false;
            break;
          }
          const uint32_t sf_bytes = (MX && k_tail_half && ks + 1 == k_stages) ? kSfPerStage / 2 : kSfPerStage;
          mbar_expect_tx(&sm.full[stage], kATileBytes + kPairBHalfBytes + 3 * sf_bytes);
          tma_load_2d(sm.a[stage], amap, a_col + cur.kl * kGemmBKBytes, tm * 256 + (int)rank * 128, &sm.full[stage]);
          tma_load_2d(sm.b[stage], bmap, cur.kl * kGemmBKBytes, tn * kGemmBN + (int)rank * 128, &sm.full[stage]);
          bulk_load_1d(sm.sfa[stage], sfa_src + (size_t)cur.kl * kSfPerStage, sf_bytes, &sm.full[stage]);
          bulk_load_1d(sm.sfb[stage], sfb_src0 + (size_t)cur.kl * kSfPerStage, sf_bytes, &sm.full[stage]);
          bulk_load_1d(sm.sfb[stage] + kSfPerStage, sfb_src1 + (size_t)cur.kl * kSfPerStage, sf_bytes, &sm.full[stage]);
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ----------------------------
    if constexpr (kWide) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t gk = 0;                       // K stages issued so far, over all tiles
      uint32_t shared_phase = 0, priv_phase = 0;   // priv_phase: bit `kind`
      int kind = 0;                          // 0: accumulator at columns [0, 256), 1: at [128, 384)
      bool ok = true;
      for (int ti = 0; ti < tiles.count && ok; ++ti, kind ^= kind_toggle) {
       // One accumulator hand-over per tile — or, batched accumulation, per term (= K segment) of the tile.
       const int n_groups = kBatchSum ? g.n_seg : 1;
       for (int grp = 0; grp < n_groups && ok; ++grp) {
        const int ks_begin = (kBatchSum && grp > 0) ? g.seg_stage_end[grp - 1] : 0;
        const int ks_end = kBatchSum ? g.seg_stage_end[grp] : k_stages;
        // the private half was released two tiles ago, the shared half by the previous tile's epilogue
        // (wide forms: one accumulator, every epilogue warp arrives on the one barrier)
        if ((!kWide && !mbar_wait_timed(&sm.acc_empty_priv[kind], ((priv_phase >> kind) & 1u) ^ 1u)) ||
            !mbar_wait_timed(&sm.acc_empty_shared, shared_phase ^ 1)) {
          atomicExch(g.status, kStatusGemmEpilogueTimeout);
          ok = false;
          break;
        }
        priv_phase ^= 1u << kind;
        shared_phase ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem + (uint32_t)kind * 128;
        for (int ks = ks_begin; ks < ks_end; ++ks, ++gk) {
          // operands of both CTAs have landed and the movers have put the stage's scales into tensor memory
          const uint32_t slot = gk % kPairSfSlots;
          if (!mbar_wait_timed(&sm.sf_ready[slot], (gk / kPairSfSlots) & 1u)) {
            atomicExch(g.status, kStatusGemmMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sf_cols = tmem + kPairSfBase + slot * kSlotCols;
          const uint32_t a_base = smem_u32(sm.a[stage]);
          const uint32_t b_base = smem_u32(sm.b[stage]);
          const int ka = ks - ks_begin;          // 0 at the first stage of this accumulator
          // MXFP4 with K an odd multiple of 128: the very last stage holds 128 elements, two MMAs instead of four
          // (a branch of its own: a run-time MMA count in the unrolled loop cost every stage of every shape ~4 %)
          if (MX && k_tail_half && ks + 1 == k_stages) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tc_mma_pair<true>(d_tmem, smem_desc(a_base + j * 32, 16, 1024, 2), smem_desc(b_base + j * 32, 16, 1024, 2),
                          block_scaled_idesc(256, kGemmBN, 1, j * 2), sf_cols, sf_cols + kSfbOff, (ka | j) != 0);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint64_t adesc = smem_desc(a_base + j * 32, 16, 1024, 2);
              const uint64_t bdesc = smem_desc(b_base + j * 32, 16, 1024, 2);
              if constexpr (!MX) {
                tc_mma_pair<false>(d_tmem, adesc, bdesc, block_scaled_idesc(256, kGemmBN, 0, 0), sf_cols + j * 4,
                             sf_cols + 16 + j * 8, (ka | j) != 0);
              } else {
                const int sf_id = (j & 1) * 2;   // bytes 0..1 or 2..3 of the scale column
                tc_mma_pair<true>(d_tmem, adesc, bdesc, block_scaled_idesc(256, kGemmBN, 1, sf_id),
                            sf_cols + (j >> 1) * 4, sf_cols + kSfbOff + (j >> 1) * 8, (ka | j) != 0);
              }
            }
          }
          tc_commit_pair(&sm.empty[stage]);   // both CTAs: the stage may be refilled
          if (++stage == kPairStages) stage = 0;
        }
        if (ok) tc_commit_pair(&sm.acc_full);   // both CTAs' epilogues
       }
      }
    }
  } else if (warp >= kMoverWarp0 && warp < kMoverWarp0 + 4) {
    // ------------------------------ scale movers (both CTAs) --------------------------------
    if constexpr (kWide) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsMovers));
    // A scale slot is rewritten as soon as the MMAs of the stage two steps back have completed, which the
    // leader's tcgen05.commit announces to both CTAs at once (multicast arrival on that stage's `empty` barrier).
    const int quad = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t gk = 0;
    bool ok = true;
    constexpr int kTiles = MX ? 2 : 4;
    uint32_t sf_ready_leader[kPairSfSlots];       // the leader's barrier of each slot
#pragma unroll
    for (int s = 0; s < kPairSfSlots; ++s) sf_ready_leader[s] = map_to_cta(&sm.sf_ready[s], 0);
    for (int ti = 0; ti < tiles.count && ok; ++ti) {
      for (int ks = 0; ks < k_stages; ++ks, ++gk) {
        if (!mbar_wait_timed(&sm.full[stage], phase)) {
          if (lane == 0) atomicExch(g.status, kStatusGemmMmaTimeout);
          ok = false;
          break;
        }
        uint32_t ra[16], rb[32];
        load_stage_scales<kTiles>(sm.sfa[stage], sm.sfb[stage], lane, ra, rb);
        const uint32_t slot = gk % kPairSfSlots;
        if (gk >= kPairSfSlots) {
          const uint32_t pg = gk - kPairSfSlots;
          if (!mbar_wait_timed(&sm.empty[pg % kPairStages], (pg / kPairStages) & 1u)) {
            if (lane == 0) atomicExch(g.status, kStatusGemmMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after();
        }
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + kPairSfBase + slot * kSlotCols;
        if constexpr (MX) {
          tmem_st8(taddr, ra);
          tmem_st8(taddr + 8, rb);
          tmem_st8(taddr + 16, rb + 8);
        } else {
          tmem_st16(taddr, ra);
          tmem_st32(taddr + 16, rb);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        // tell the leader: this CTA's operands have landed and this quadrant's scales are in place
        if (lane == 0) {
          uint32_t leader = sf_ready_leader[0];
#pragma unroll
          for (int s = 1; s < kPairSfSlots; ++s) leader = slot == (uint32_t)s ? sf_ready_leader[s] : leader;
          mbar_arrive_cluster(leader);
        }
        if (++stage == kPairStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + kEpiWarps) {
    // ------------------------------ epilogue (both CTAs) -------------------------------------
    if constexpr (kWide) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    const int quad = warp & 3;
    uint32_t acc_phase = 0;
    int kind = 0;
    float a_sg = g.fixed_scale;
    if (g.a_sg != nullptr) a_sg = __ldg(g.a_sg);
    const uint32_t empty_shared_leader = map_to_cta(&sm.acc_empty_shared, 0);
    const uint32_t empty_priv_leader0 = map_to_cta(&sm.acc_empty_priv[0], 0), empty_priv_leader1 = map_to_cta(&sm.acc_empty_priv[1], 0);
    bool ok = true;
    int cs_tm = -1;                                   // row block whose table rows are in tensor memory
    const uint32_t cs_taddr = g.rope_in_tmem ? tmem + ((uint32_t)(quad * 32) << 16) + 256u : 0u;
    const int half = kWide ? (warp - kEpiWarp0) >> 2 : 0;   // wide: which 128 of the tile's 256 columns
    for (int ti = 0; ti < tiles.count && ok; ++ti, kind ^= kind_toggle) {
      int tm, tn;
      tiles.get(ti, tm, tn);
      if constexpr (kWide) {
        if (g.rope_in_tmem && tm != cs_tm) {
          // This lane's row of the (cos, sin) table, 2 * pair_dim floats, into columns [256, 256 + 2 * pair_dim) of
          // its tensor-memory lane: once per row block, while the tile's MMAs run.  Every later tile of the row
          // block reads the sixteen columns it needs from there instead of 64 scattered bytes per lane from L2.
          // The quadrant's two warps write half of the row each, after both have finished with the previous row
          // block's values and before either reads the new ones (named barrier 1 + quad, 64 threads).
          asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
          const int row = tm * 256 + (int)rank * 128 + quad * 32 + lane;
          const float4* src = reinterpret_cast<const float4*>(g.rope_cs + (size_t)(row & g.rope_seq_mask) * g.rope_pair_dim);
          const int chunks = g.rope_pair_dim >> 4;            // stores of 32 floats = 16 pairs: 2 (heads of 64) or 4
          for (int c = half * (chunks >> 1); c < (half + 1) * (chunks >> 1); ++c) {
            uint32_t v[32];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 f = __ldg(src + c * 8 + q);
              v[4 * q] = __float_as_uint(f.x); v[4 * q + 1] = __float_as_uint(f.y);
              v[4 * q + 2] = __float_as_uint(f.z); v[4 * q + 3] = __float_as_uint(f.w);
            }
            tmem_st32(cs_taddr + (uint32_t)(32 * c), v);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          tc_fence_before();
          asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
          tc_fence_after();
          cs_tm = tm;
        }
      }
      const uint32_t tq = tmem + ((uint32_t)(quad * 32) << 16);
      const int row0 = tm * 256 + (int)rank * 128 + quad * 32;
      const int col0 = tn * kGemmBN;
      if constexpr (kBatchSum) {
        uint8_t* epi = &sm.epi[0][0][0] + (size_t)(warp - kEpiWarp0) * 4096;   // one staging buffer per warp
        ok = epilogue_batch_sum(g, tmap_d, &sm.acc_full, acc_phase, tq + (uint32_t)(half * 128), epi, row0, col0 + half * 128,
                                lane, empty_shared_leader);
        continue;
      }
      if (!mbar_wait_timed(&sm.acc_full, acc_phase)) {
        if (lane == 0) atomicExch(g.status, kStatusGemmTmemTimeout);
        ok = false;
        break;
      }
      tc_fence_after();
      if constexpr (kWide) {
        uint8_t* epi = &sm.epi[0][0][0] + (size_t)(warp - kEpiWarp0) * 4096;   // one staging buffer per warp
        epilogue_wide<EPI>(g, tmap_d, tq + (uint32_t)(half * 128), epi, row0, col0 + half * 128, a_sg, lane,
                           empty_shared_leader, cs_taddr);
      } else {
        uint8_t* epi = &sm.epi[warp - kEpiWarp0][0][0];
        // tensor-memory columns [128, 256) hold output columns [128, 256) of a tile at [0, 256) and output
        // columns [0, 128) of a tile at [128, 384): lift them out first, the next tile needs them
        epilogue_region128<EPI>(g, tmap_d, tq + 128, epi, row0, col0 + (kind ? 0 : 128), a_sg, lane,
                                AccRelease{nullptr, empty_shared_leader}, cs_taddr);
        epilogue_region128<EPI>(g, tmap_d, tq + (kind ? 256 : 0), epi, row0, col0 + (kind ? 128 : 0), a_sg, lane,
                                AccRelease{nullptr, kind ? empty_priv_leader1 : empty_priv_leader0}, cs_taddr);
      }
      acc_phase ^= 1;
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // common exit: neither CTA may leave while the other can still signal its barriers or read its memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace fp4b200
