// CTA-pair variant of the persistent TF32 GEMM: two CTAs on neighbouring SMs (a cluster of 2)
// compute one 256 x block_n tile with tcgen05.mma cta_group::2.
//
// Each CTA loads its own 128 rows of A and HALF of the B tile (block_n / 2 columns) and keeps
// its own 128 x block_n half of the accumulator in its own TMEM; the tensor cores of both SMs
// read the two B halves from both shared memories.  Against two independent 128 x block_n
// tiles this halves the shared-memory bytes read per MMA for B and cuts the L2 -> SM traffic
// per output element by a third, which is what the MN-major (transposed) operand layouts need
// to keep the tensor pipe fed.
//
// Wide tiles (block_n = 512): the pair computes 256 x 512 as TWO 256-wide MMA groups that share the
// A stage -- per 32-deep k-block a CTA then loads 16 KiB of A and 2 x 16 KiB of B for 1024 cycles of
// tensor work, 48 B/clk, where the 256 x 256 tile needs 64 B/clk: exactly what one SM can take in
// from L2, so that form waits for its loads whenever anything jitters.  The 512 accumulator
// columns are all of a CTA's tensor memory: one accumulator set, the epilogue of a tile and the
// main loop of the next no longer overlap (a per cent or two at the K this form is chosen for).
//
// Roles per CTA as in the single-CTA kernel; differences:
//   * both producers credit the LEADER CTA's (cluster rank 0) full barrier, which therefore
//     expects two arrivals per stage;
//   * only the leader issues MMAs; its commits arrive on the empty / accumulator-full barriers
//     of both CTAs (one commit per destination CTA);
//   * the epilogue warps of both CTAs arrive on the leader's accumulator-empty barrier (8);
//   * every producer ends by waiting for the last stage releases, and both CTAs meet at a
//     cluster barrier before freeing TMEM, so no arrival targets a CTA that has exited.
#pragma once
#include "gemm_tcgen05.cuh"

namespace fnn {

constexpr int kPairBlockM = 2 * kBlockM;

__device__ __forceinline__ Unit decode_unit_pair(const GemmParams& p, int u) {
  // identical rasterisation, with tiles_m counting 256-row tiles (set by the host)
  return decode_unit(p, u);
}

constexpr int kPairMmaWarpB = 6;                     // second MMA-issuing warp (wide tiles)
constexpr int kNumThreadsPair = kNumThreads + 32;    // producer, MMA issuer, four epilogue warps, second MMA issuer

// kGather: every finished tile is also stored through p.n_peers extra tensor maps (see PeerMaps).
template <bool kGather>
__device__ __forceinline__ void gemm_tf32_pair_body(const CUtensorMap& tmA, const CUtensorMap& tmB,
                                                    const CUtensorMap& tmC, const GemmParams& p,
                                                    const CUtensorMap* peers) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();          // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  // one MMA group is at most 256 columns wide; a 512-wide tile is two groups over the same A
  // MMA groups over the same A stage, each with an issuing thread of its own: the two 256-column
  // halves of a wide tile, or the two 128-column halves of a 256-wide one
  const int n_sub = p.mma_groups;
  const int mma_n = p.block_n / n_sub;                   // N of one tcgen05.mma
  const int half_n = mma_n >> 1;                         // B columns of one group this CTA loads
  const int n_acc = p.block_n > kMaxBlockN ? 1 : 2;      // accumulator sets that fit 512 TMEM columns

  // A stage holds kb_per_stage consecutive 32-deep k-blocks, each as [A 16 KiB][B half]; one
  // barrier round trip (wait, commit) then covers 4 * kb_per_stage MMAs.
  const int R = p.kb_per_stage;
  const uint32_t half_bytes = static_cast<uint32_t>(half_n) * kBlockK * 4;
  const uint32_t sub_bytes = kStageABytes + static_cast<uint32_t>(n_sub) * half_bytes;
  const uint32_t stage_bytes = static_cast<uint32_t>(R) * sub_bytes;
  const uint32_t staging_base = smem_base + p.num_stages * stage_bytes;
  const uint32_t bar_base = staging_base + kStagingBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 64u + 8u * s; };
  auto tfull_bar = [&](int a) { return bar_base + 128u + 8u * a; };
  auto tempty_bar = [&](int a) { return bar_base + 144u + 8u * a; };
  const uint32_t tmem_slot = bar_base + 160u;
  uint8_t* bar_gen = smem_gen + (bar_base - smem_base);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(bar_gen + 160);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 168);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.num_stages; ++s) {
      ptx::mbar_init(full_bar(s), 2);          // one arrive.expect_tx from each CTA's producer
      ptx::mbar_init(empty_bar(s), n_sub);     // one commit per MMA-issuing thread (two for a wide tile)
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), n_sub);
      ptx::mbar_init(tempty_bar(a), 8);        // four epilogue warps of each CTA
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    if (p.store_mode == 0) ptx::prefetch_tensormap(&tmC);
    if constexpr (kGather) {
      for (int i = 0; i < p.n_peers; ++i) ptx::prefetch_tensormap(peers + i);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc_2cta(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_2cta();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  // the peer's barriers must exist before anything arrives on them
  ptx::cluster_arrive_release();
  ptx::cluster_wait_acquire();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ------------------------------------------------------------- producer ---
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = ptx::make_l2_policy(p.l2_a);
      const uint64_t pol_b = ptx::make_l2_policy(p.l2_b);
      for (int u = cluster_id; u < p.total_units && ok; u += num_clusters) {
        const Unit w = decode_unit_pair(p, u);
        const int m0 = w.mt * kPairBlockM + static_cast<int>(rank) * kBlockM;
        const int n_tile = w.nt * p.block_n + static_cast<int>(rank) * half_n;
        const int kb0 = w.s * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; kb += R) {
          ok = wait_barrier(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusProducerTimeout);
          if (!ok) break;
          const int nsub = min(R, kb1 - kb);          // k-blocks of this unit left for the stage
          const uint32_t fb = ptx::mapa_shared(full_bar(stage), 0);     // leader's barrier
          ptx::mbar_expect_tx_cluster(fb, static_cast<uint32_t>(nsub) * sub_bytes);
          for (int r = 0; r < nsub; ++r) {
          const uint32_t sa = smem_base + stage * stage_bytes + r * sub_bytes;
          const uint32_t sb = sa + kStageABytes;
          const int k0 = (kb + r) * kBlockK;
          if (!p.a_mn_major) {
            ptx::tma_load_3d_pair(sa, &tmA, fb, k0, m0, w.b, pol_a);
          } else if (p.a_chunked) {
            ptx::tma_load_4d_pair(sa, &tmA, fb, 0, k0, m0 >> 5, w.b, pol_a);
          } else {
#pragma unroll
            for (int c = 0; c < kBlockM / 32; ++c)
              ptx::tma_load_3d_pair(sa + c * kChunkBytes, &tmA, fb, m0 + 32 * c, k0, w.b, pol_a);
          }
          for (int h = 0; h < n_sub; ++h) {
            const int n0 = n_tile + h * mma_n;              // this CTA's half of MMA group h
            const uint32_t sbh = sb + h * half_bytes;
            if (!p.b_mn_major) {
              ptx::tma_load_3d_pair(sbh, &tmB, fb, k0, n0, w.b, pol_b);  // box 32 x half_n
            } else if (p.b_chunked) {
              ptx::tma_load_4d_pair(sbh, &tmB, fb, 0, k0, n0 >> 5, w.b, pol_b);
            } else {
              for (int c = 0; c < half_n / 32; ++c)
                ptx::tma_load_3d_pair(sbh + c * kChunkBytes, &tmB, fb, n0 + 32 * c, k0, w.b, pol_b);
            }
          }
          }
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
      }
      // tail: every release the leader's commits still owe this CTA must land before exit
      for (int i = 0; i < p.num_stages && ok; ++i) {
        ok = wait_barrier(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusProducerTimeout);
        if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1 || warp == kPairMmaWarpB) {
    // ------------------------------------------------ MMA issuers (leader only) ---
    // With two MMA groups there are two issuing threads: warp 1 issues the group of the tile's lower
    // columns, warp 6 the group of the upper ones, over the same A stage, each into its own
    // accumulator columns -- one thread issues a tcgen05.mma only every 100-170 clocks, and eight
    // instructions per k-block from one thread left the tensor pipe 85 % busy.
    const int my_group = warp == 1 ? 0 : 1;
    if (lane == 0 && rank == 0 && my_group < n_sub) {
      const uint32_t idesc = ptx::idesc_tf32(kPairBlockM, mma_n, p.a_mn_major, p.b_mn_major);
      const uint64_t a_desc0 = ptx::smem_desc_sw128(
          smem_base, p.a_mn_major ? kChunkBytes : 16u, p.a_mn_major ? 512u : 1024u,
          p.a_mn_major ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128);
      const uint64_t b_desc0 = ptx::smem_desc_sw128(
          smem_base + kStageABytes, p.b_mn_major ? kChunkBytes : 16u, p.b_mn_major ? 512u : 1024u,
          p.b_mn_major ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128);
      const uint64_t a_kstep = (p.a_mn_major ? 1024u : kUmmaK * 4u) >> 4;
      const uint64_t b_kstep = (p.b_mn_major ? 1024u : kUmmaK * 4u) >> 4;
      const uint64_t stage_step = stage_bytes >> 4;
      const uint64_t sub_step = sub_bytes >> 4;
      const uint64_t half_step = half_bytes >> 4;
      // the two CTAs' copies of a barrier differ by a constant in the cluster address space
      const uint32_t bar0 = ptx::mapa_shared(bar_base, 0);
      const uint32_t bar1 = ptx::mapa_shared(bar_base, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = cluster_id; u < p.total_units && ok; u += num_clusters) {
        const Unit w = decode_unit_pair(p, u);
        const int kb0 = w.s * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        ok = wait_barrier(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p, kStatusMmaTmemTimeout);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kMaxBlockN);
        uint32_t accumulate = 0u;                     // 0 on the unit's first k-block: overwrite
        for (int kb = kb0; kb < kb1; kb += R) {
          ok = wait_barrier(full_bar(stage), phase, abort_flag, p, kStatusMmaTimeout);
          if (!ok) break;
          const int nsub = min(R, kb1 - kb);
          for (int r = 0; r < nsub; ++r) {
            const uint64_t da = a_desc0 + stage * stage_step + r * sub_step;
            const uint64_t db = b_desc0 + stage * stage_step + r * sub_step;
            {                                         // this thread's MMA group over the A stage
              const int h = my_group;
              const uint32_t td = tmem_d + static_cast<uint32_t>(h * mma_n);
              const uint64_t dbh = db + h * half_step;
              ptx::mma_tf32_2cta(td, da, dbh, idesc, accumulate);
#pragma unroll
              for (int ks = 1; ks < kBlockK / kUmmaK; ++ks)
                ptx::mma_tf32_2cta(td, da + ks * a_kstep, dbh + ks * b_kstep, idesc, 1u);
            }
            accumulate = 1u;
          }
          ptx::mma_commit_2cta(bar0 + 64u + 8u * stage);    // empty[stage], leader
          ptx::mma_commit_2cta(bar1 + 64u + 8u * stage);    // empty[stage], peer
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit_2cta(bar0 + 128u + 8u * acc);       // accumulator full, leader
        ptx::mma_commit_2cta(bar1 + 128u + 8u * acc);       // accumulator full, peer
        if (++acc == n_acc) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp < kPairMmaWarpB) {
    // -------------------------------------------------------------- epilogue ---
    const int q = warp & 3;
    const uint32_t staging = staging_base + (warp - kEpilogueWarp0) * kStagingBytesPerWarp;
    uint8_t* staging_gen = smem_gen + (staging - smem_base);
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    long long t_prev_full = clock64();
    const bool raw = p.split_k > 1;
    for (int u = cluster_id; u < p.total_units && ok; u += num_clusters) {
      const Unit w = decode_unit_pair(p, u);
      const int m0 = w.mt * kPairBlockM + static_cast<int>(rank) * kBlockM + q * 32;
      const int n0 = w.nt * p.block_n;
      ok = wait_barrier(tfull_bar(acc), acc_phase, abort_flag, p, kStatusEpilogueTimeout);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * kMaxBlockN);
      const int cz = raw ? (w.b * p.split_k + w.s) : w.b;
      Pace pace;
      if constexpr (kGather) {
        // as in the single-CTA kernel: the tiles of all waves but the last leave over 7/8 of a
        // main loop's time; only with two accumulators, where the drain is off the critical path
        const long long now = clock64();
        if (p.pace_gather && n_acc == 2 && u / num_clusters < (p.total_units - 1) / num_clusters) {
          pace.t0 = now;
          pace.step = (now - t_prev_full) * p.pace_gather / (8 * (p.block_n / 32));
        }
        t_prev_full = now;
      }
      epilogue_drain_tile(p, &tmC, taddr0, staging, staging_gen, buf, m0, n0, cz, w.b, raw, lane, 0, 1, 2,
                          kGather ? peers : nullptr, kGather ? p.n_peers : 0, pace);
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(tempty_bar(acc), 0));
      if (++acc == n_acc) { acc = 0; acc_phase ^= 1u; }
    }
    if (p.store_mode == 0 && lane == 0) ptx::tma_store_wait_all<0>();
    if (p.mc_c != nullptr) __threadfence_system();
  }

  // ---------------------------------------------------------------- teardown ---
  __syncwarp();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_arrive_release();
  ptx::cluster_wait_acquire();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_2cta(tmem_base, kTmemCols);
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreadsPair, 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const __grid_constant__ GemmParams p) {
  gemm_tf32_pair_body<false>(tmA, tmB, tmC, p, nullptr);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreadsPair, 1)
gemm_tf32_pair_gather_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const __grid_constant__ CUtensorMap tmC, const __grid_constant__ PeerMaps peers,
                             const __grid_constant__ GemmParams p) {
  gemm_tf32_pair_body<true>(tmA, tmB, tmC, p, peers.m);
}

// Dynamic shared memory per CTA of the pair kernel.
inline size_t gemm_pair_smem_bytes(int block_n, int num_stages, int kb_per_stage) {
  return 1024 + static_cast<size_t>(num_stages) * kb_per_stage *
                    (kStageABytes + (block_n / 2) * kBlockK * 4) +
         kStagingBytes + kBarrierBytes;
}
constexpr int kPairWideBlockN = 2 * kMaxBlockN;      // 256 x 512 tiles: two MMA groups per A stage

}  // namespace fnn
