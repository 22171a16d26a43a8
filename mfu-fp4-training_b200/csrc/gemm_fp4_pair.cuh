// Two-CTA ("pair") variant of the block-scaled FP4 GEMM: a cluster of two CTAs on neighbouring SMs
// computes one 256 x 256 output tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows
// of A and its own half (128 rows) of the B tile, so a K stage costs 38 KB of L2 -> SM traffic per SM
// instead of 54 KB for the same MMA work — operand delivery, not the tensor pipe, bounds the
// one-CTA kernel.  No multicast loads: the second CTA's data arrives through its own TMA and its
// readiness is forwarded with remote mbarrier arrivals; the leader's tcgen05.commit signals the
// barriers of both CTAs one by one.  Included by gemm_fp4.cu after the shared helpers.
#pragma once

namespace fp4b200 {

constexpr int kPairStages = 5;
constexpr int kPairBHalfBytes = 128 * kGemmBKBytes;   // this CTA's half of the B tile: 16 KiB

struct GemmPairSmem {
  alignas(1024) uint8_t a[kPairStages][kATileBytes];
  alignas(1024) uint8_t b[kPairStages][kPairBHalfBytes];
  alignas(1024) uint8_t epi[4][2][4096];
  alignas(128) uint8_t sfa[kPairStages][kASfBytes];
  alignas(128) uint8_t sfb[kPairStages][kBSfBytes];
  alignas(8) uint64_t full[kPairStages];       // this CTA's TMA data of the stage has landed
  alignas(8) uint64_t empty[kPairStages];      // the pair's MMAs have finished reading the stage
  alignas(8) uint64_t sf_ready[kPairStages];   // leader only: operands + scales of BOTH CTAs are in place
  alignas(8) uint64_t acc_full;                // accumulator of the tile is complete
  alignas(8) uint64_t acc_empty;               // leader only: both CTAs' epilogues have drained it
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
// writes (tensor-memory stores are ordered by tcgen05.wait::st + tcgen05.fence, operand tiles by the
// TMA's own mbarrier), and a cluster-scope release was measured at ~1200 cycles per arrival while TMA
// traffic is in flight.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// completion of all earlier tcgen05 operations of this thread -> one arrival on a barrier of any CTA of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

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

// EPI: one epilogue form per instantiation, chosen by the host (kEpiPlain: bf16 outputs, optional residual;
// kEpiRope: with the rotary embedding; kEpiSilu: with a SiLU range, rotary or not; kEpiGeneral: fp32 outputs or
// accumulation).  Several forms inside one kernel cost every one of them a few percent.
template <bool MX, int EPI = kEpiPlain>
__global__ void __launch_bounds__(kGemmThreads, 1)
fp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ GemmBMaps tmap_b,
                     const __grid_constant__ GemmOutMaps tmap_d, const GemmArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  GemmPairSmem& sm = *reinterpret_cast<GemmPairSmem*>(smem_align_1024(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  const int tiles_m = g.M / 256, tiles_n = g.N / kGemmBN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_stages = g.K / (2 * kGemmBKBytes);
  constexpr int kSfPerStage = MX ? 1024 : 2048;

  if (tid == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
      mbar_init(&sm.sf_ready[s], 8);   // four mover warps of each CTA
    }
    mbar_init(&sm.acc_full, 1);
    mbar_init(&sm.acc_empty, 8);       // four epilogue warps of each CTA
    fence_mbar_init();
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

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) --------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      for (int s = 0; s < g.n_seg; ++s) tma_prefetch_desc(&tmap_b.m[s]);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t empty_peer[kPairStages];
#pragma unroll
      for (int s = 0; s < kPairStages; ++s) empty_peer[s] = map_to_cta(&sm.empty[s], 1);
      int filled = 0;
      for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
        int tm, tn;
        raster_tile(t, tiles_m, tiles_n, tm, tn);
        int seg = -1, seg_end = 0, kl = 0, a_col = 0;
        const CUtensorMap* bmap = nullptr;
        const uint8_t *sfa_src = nullptr, *sfb_src0 = nullptr, *sfb_src1 = nullptr;
        for (int ks = 0; ks < k_stages; ++ks, ++kl) {
          if (ks == seg_end) {   // first stage of the next K segment
            ++seg;
            seg_end = g.seg_stage_end[seg];
            kl = 0;
            a_col = g.seg_a_col_bytes[seg];
            bmap = &tmap_b.m[seg];
            const size_t tiles_k = (size_t)g.seg_sf_tiles_k[seg];
            sfa_src = g.seg_a_sc[seg] + (size_t)(2 * tm + rank) * tiles_k * 512;
            sfb_src0 = g.seg_b_sc[seg] + (size_t)(2 * tn) * tiles_k * 512;
            sfb_src1 = sfb_src0 + tiles_k * 512;
          }
          const bool first_fill = filled < kPairStages;   // the first use of a stage waits for nothing
          ++filled;
          if (!mbar_wait_timed(&sm.empty[stage], phase ^ 1)) {
            atomicExch(g.status, kStatusGemmTmaTimeout);
            ok = false;
            break;
          }
          // the leader's barrier is signalled by tcgen05.commit; it passes the news on to the other CTA
          // (one commit per stage instead of two keeps the tensor pipe's queue short)
          if (rank == 0 && !first_fill) mbar_arrive_cluster(empty_peer[stage]);
          mbar_expect_tx(&sm.full[stage], kATileBytes + kPairBHalfBytes + 3 * kSfPerStage);
          tma_load_2d(sm.a[stage], &tmap_a, a_col + kl * kGemmBKBytes, tm * 256 + (int)rank * 128, &sm.full[stage]);
          tma_load_2d(sm.b[stage], bmap, kl * kGemmBKBytes, tn * kGemmBN + (int)rank * 128, &sm.full[stage]);
          bulk_load_1d(sm.sfa[stage], sfa_src + (size_t)kl * kSfPerStage, kSfPerStage, &sm.full[stage]);
          bulk_load_1d(sm.sfb[stage], sfb_src0 + (size_t)kl * kSfPerStage, kSfPerStage, &sm.full[stage]);
          bulk_load_1d(sm.sfb[stage] + kSfPerStage, sfb_src1 + (size_t)kl * kSfPerStage, kSfPerStage, &sm.full[stage]);
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ----------------------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      const uint32_t acc_full_remote = map_to_cta(&sm.acc_full, 1);
      for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
        if (!mbar_wait_timed(&sm.acc_empty, acc_phase ^ 1)) {
          atomicExch(g.status, kStatusGemmEpilogueTimeout);
          ok = false;
          break;
        }
        tc_fence_after();
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait_timed(&sm.sf_ready[stage], phase)) {
            atomicExch(g.status, kStatusGemmMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sf_cols = tmem + kSfTmemBase + stage * kSfSlotCols;
          const uint32_t a_base = smem_u32(sm.a[stage]);
          const uint32_t b_base = smem_u32(sm.b[stage]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t adesc = smem_desc(a_base + j * 32, 16, 1024, 2);
            const uint64_t bdesc = smem_desc(b_base + j * 32, 16, 1024, 2);
            if constexpr (!MX) {
              tc_mma_pair<false>(tmem, adesc, bdesc, block_scaled_idesc(256, kGemmBN, 0, 0), sf_cols + j * 4,
                                 sf_cols + 16 + j * 8, (ks | j) != 0);
            } else {
              const int sf_id = (j & 1) * 2;
              tc_mma_pair<true>(tmem, adesc, bdesc, block_scaled_idesc(256, kGemmBN, 1, sf_id),
                                sf_cols + (j >> 1) * 4, sf_cols + 16 + (j >> 1) * 8, (ks | j) != 0);
            }
          }
          tc_commit_pair(smem_u32(&sm.empty[stage]));   // the producer forwards it to the other CTA
          if (++stage == kPairStages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          // once per tile: signal both CTAs' epilogues directly (a forwarded arrival would add a hop)
          tc_commit_pair(smem_u32(&sm.acc_full));
          tc_commit_pair(acc_full_remote);
        }
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------ scale movers (both CTAs) --------------------------------
    const int quad = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    constexpr int kTiles = MX ? 2 : 4;
    for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_timed(&sm.full[stage], phase)) {
          if (lane == 0) atomicExch(g.status, kStatusGemmMmaTimeout);
          ok = false;
          break;
        }
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + kSfTmemBase + stage * kSfSlotCols;
        uint32_t ra[16], rb[32];
#pragma unroll
        for (int j = 0; j < kTiles; ++j) {
          const uint4 va = *reinterpret_cast<const uint4*>(&sm.sfa[stage][j * 512 + lane * 16]);
          ra[4 * j] = va.x; ra[4 * j + 1] = va.y; ra[4 * j + 2] = va.z; ra[4 * j + 3] = va.w;
          const uint4 v0 = *reinterpret_cast<const uint4*>(&sm.sfb[stage][j * 512 + lane * 16]);
          const uint4 v1 = *reinterpret_cast<const uint4*>(&sm.sfb[stage][kTiles * 512 + j * 512 + lane * 16]);
          rb[8 * j] = v0.x; rb[8 * j + 1] = v0.y; rb[8 * j + 2] = v0.z; rb[8 * j + 3] = v0.w;
          rb[8 * j + 4] = v1.x; rb[8 * j + 5] = v1.y; rb[8 * j + 6] = v1.z; rb[8 * j + 7] = v1.w;
        }
#pragma unroll
        for (int j = kTiles; j < 4; ++j) {
          ra[4 * j] = ra[4 * j + 1] = ra[4 * j + 2] = ra[4 * j + 3] = 0;
#pragma unroll
          for (int e = 0; e < 8; ++e) rb[8 * j + e] = 0;
        }
        tmem_st16(taddr, ra);
        tmem_st32(taddr + 16, rb);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        // tell the leader: this CTA's operands have landed and this quadrant's scales are in place
        if (lane == 0) mbar_arrive_cluster(map_to_cta(&sm.sf_ready[stage], 0));
        if (++stage == kPairStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) -------------------------------------
    const int quad = warp & 3;
    uint32_t acc_phase = 0;
    float a_sg = g.fixed_scale;
    if (g.a_sg != nullptr) a_sg = __ldg(g.a_sg);
    const uint32_t acc_empty_leader = map_to_cta(&sm.acc_empty, 0);
    bool ok = true;
    for (int t = cluster_id; t < n_tiles && ok; t += n_clusters) {
      int tm, tn;
        raster_tile(t, tiles_m, tiles_n, tm, tn);
      if (!mbar_wait_timed(&sm.acc_full, acc_phase)) {
        if (lane == 0) atomicExch(g.status, kStatusGemmTmemTimeout);
        ok = false;
        break;
      }
      tc_fence_after();
      // this CTA's half of the accumulator is drained: tell the leader's MMA thread
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
      };
      if constexpr (EPI == kEpiGeneral) {
        epilogue_tile(g, tmap_d, tmem, &sm.epi[warp - 2][0][0], tm * 256 + (int)rank * 128, tn, a_sg, quad, lane);
        release();
      } else if constexpr (EPI == kEpiSilu) {
        epilogue_tile_bf16<true, true>(g, tmap_d, tmem, &sm.epi[warp - 2][0][0], tm * 256 + (int)rank * 128, tn, a_sg, quad,
                                   lane, release);
      } else if constexpr (EPI == kEpiRope) {
        epilogue_tile_bf16<true, false>(g, tmap_d, tmem, &sm.epi[warp - 2][0][0], tm * 256 + (int)rank * 128, tn, a_sg, quad,
                                   lane, release);
      } else {
        epilogue_tile_bf16<false, false>(g, tmap_d, tmem, &sm.epi[warp - 2][0][0], tm * 256 + (int)rank * 128, tn, a_sg, quad,
                                   lane, release);
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
