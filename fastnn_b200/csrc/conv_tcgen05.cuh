// Conv2d forward as an implicit GEMM on the tcgen05 main loop (sm_100a).
//
//   out[n, co, oh, ow] = bias[co] + sum over (ci, ki, kj) of
//                        w[co, ci, ki, kj] * x[n, ci, oh*sh + ki - ph, ow*sw + kj - pw]
// FastNN's Conv2d::forward runs these loops on the CPU (src/nn/conv.rs:97-123); its unbound CUDA
// entry builds an im2col matrix per image and calls cuBLAS (cuda/kernels.cu:836-946).  Here the
// im2col matrix never exists: as a GEMM  D[position, co] = A[position, k] . W[co, k]^T  with
// position = (n, oh, ow) and k = (ci, ki, kj),
//   warps 6-21 gather A: a thread owns one output position of the tile and a quarter of the
//              k-block; it reads its 8 inputs (consecutive lanes = consecutive ow, so each load
//              instruction is one coalesced row segment; padding and the K tail are zeros), one
//              k-block ahead of the one it writes, into row r of a K-major 128B-swizzled stage,
//              exactly what TMA would have produced.  What depends on k alone (offset of the tap,
//              its bit in the tap mask) is read from a table written by conv_ktab_kernel just
//              before.  Measured: the gather, not the tensor core, sets the pace, and it is bound
//              by instruction issue;
//   warp 0     loads the weight tile W[co-tile, k-block] by TMA (weights are [co, k] row-major,
//              i.e. already K-major; the host pads k to a multiple of 4 when TMA needs it);
//   warp 1     one lane issues tcgen05.mma kind::tf32 (M = 128 positions, N = block_n channels);
//   warps 2-5  drain the accumulator: lane = position, column = channel, so for one channel a
//              warp's 32 lanes write 32 consecutive NCHW elements (coalesced), bias (+ReLU) fused.
// One persistent CTA per SM, two accumulators in TMEM, every wait bounded as in the GEMM kernels.
//
// Slab form (conv2d_tf32_slab_kernel), taken when the shape allows: position tiles lie inside one
// image, and the input rows a tile needs -- 32 channels at a time, every row padded by four zero
// columns on either side -- are brought into shared memory by ONE TMA load per chunk (x coordinate
// -4: 16-byte aligned; rows above and below the image and the side columns arrive as zeros, so no
// tap mask is needed).  The gather warps then read shared memory instead of L2: per element one
// add and one load, the tap offsets from a table in shared memory that is the same for every
// chunk (k = (ci, ki, kj), so 32 channels are exactly kh*kw k-blocks).  Two slab slots take turns;
// the weight producer loads chunk j + 1 when the main loop reaches chunk j.  The gathered rows do
// not pass through shared memory again: a gather thread holds a whole row of 32 k's and writes it
// with one tcgen05.st into the stage's A slot in TENSOR memory, from where the MMA takes its A
// operand (a shared-memory A stage needed a fence.proxy.async per fill, ~900 clocks); a stage of
// shared memory holds the weight tile alone.  The sixteen gather warps form four groups that take
// every fourth k-block.  For channel tiles of at most 64 columns (conv2d_tf32_slab_dual_kernel)
// two threads issue the MMAs, taking k-blocks in turn.
#pragma once
#include "gemm_tcgen05.cuh"

namespace fnn {

struct ConvParams {
  int batch, ci, co, h, w, kh, kw, sh, sw, ph, pw, oh, ow;
  int k;               // ci * kh * kw
  int num_kb;          // ceil(k / 32)
  long long positions; // batch * oh * ow
  int tiles_p, tiles_n, total_units;
  int block_n, num_stages;
  const float* x;
  const int4* ktab;    // [num_kb * 32] per k: {offset ci*H*W + ki*W + kj, tap bit (low word),
                       // tap bit (high word), 0}; all zero for k >= ci*kh*kw (conv_ktab_kernel)
  const float* bias;   // [co] or null
  float* out;
  // Where output position (oy, ox) of image n, channel c lands:
  //   out + ((n * co + c) * dst_h + dst_y0 + oy * dst_sy) * dst_w + dst_x0 + ox * dst_sx
  // The convolution itself writes a dense [oh, ow] plane (dst_h = oh, dst_w = ow, strides 1,
  // offsets 0); a phase of a strided input gradient writes every dst_sy-th row and dst_sx-th column
  // of the full gradient plane.
  int dst_h, dst_w, dst_y0, dst_x0, dst_sy, dst_sx;
  int act;             // 0 none, 1 ReLU
  // slab form only
  int tiles_pi;        // position tiles per image: ceil(oh * ow / 128)
  int taps;            // kh * kw = k-blocks per chunk of 32 channels
  int n_chunks;        // ceil(ci / 32)
  int slab_rows;       // input rows one tile can need: (output rows a tile can touch - 1) * sh + kh
  int slab_pitch;      // floats per row in shared memory: w + 8 (four zero columns on either side)
  int slab_bytes;      // 32 * slab_rows * slab_pitch * 4
  unsigned int* status;
  long long spin_budget;
};

enum : unsigned int { kStatusConvGather = 0x301, kStatusConvSlab = 0x302, kStatusConvSlabFull = 0x303 };
constexpr int kConvSlabChannels = 32;
constexpr int kConvSlabHalo = 4;      // zero columns either side of a row (keeps the TMA x coordinate aligned)
constexpr int kConvSlabMinStages = 4;  // the slab form needs one stage per group of gather warps at least
// Tensor-memory column of the A slot of stage s: four slots of 32 columns between the two accumulators
// (which are at most 128 columns wide in this form), four more after the second one.
__host__ __device__ constexpr uint32_t conv_slab_tmem_a(int s) {
  return s < 4 ? 128u + 32u * static_cast<uint32_t>(s) : 384u + 32u * static_cast<uint32_t>(s - 4);
}
constexpr int kConvGatherWarps = 16;     // four groups of four in the slab forms (a group = one warp per lane quadrant)
static_assert(kConvGatherWarps == 16, "the slab forms take k-blocks in turns of four groups of four warps");
constexpr int kConvThreads = 32 * (6 + kConvGatherWarps);   // producer, MMA issuer, 4 epilogue warps, gather warps
constexpr int kConvKPerThread = kBlockK / (kConvGatherWarps / 4);   // k's of a stage row one gather thread fills
constexpr int kConvGatherWarp0 = 6;
// The slab form for channel tiles of at most 64 columns (conv2d_tf32_slab_dual_kernel) has TWO threads
// that issue MMAs (warps 1 and 22), taking k-blocks in turn, each into a 64-column accumulator of its
// own; the epilogue adds the two.  One thread cannot issue a tcgen05.mma of M 128, K 8 more often than
// every ~100-120 clocks whatever its N (measured: 96-121 clocks per instruction at N = 32 ... 128, for
// 16-64 clocks of tensor work); two threads together reach 60-70 clocks per instruction.  Wider tiles
// keep one issuing thread: four 128-column accumulators and the A slots do not fit tensor memory, and
// with a single accumulator set the drain no longer overlaps the next tile (measured slower).
constexpr int kConvSlabDualThreads = kConvThreads + 32;
constexpr int kConvSlabMmaWarpB = kConvGatherWarp0 + kConvGatherWarps;

// *ptr when cond != 0, else 0, as ONE predicated load: no branch, and no access when cond is 0
// (the address may then lie outside the tensor).
__device__ __forceinline__ float ldg_if(const float* ptr, uint32_t cond) {
  float v;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %2, 0;\n\t"
      "mov.f32 %0, 0f00000000;\n\t"
      "@p ld.global.nc.f32 %0, [%1];\n\t}"
      : "=f"(v)
      : "l"(ptr), "r"(cond));
  return v;
}

// Bounded wait, as in the GEMM kernels.  sleep_ns > 0: the waiter sleeps between probes -- for the
// roles that wait long and are not on the critical path (22 warps share four schedulers here, and a
// warp that probes at full rate takes issue slots from the thread that issues the MMAs).
__device__ __forceinline__ bool conv_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          const ConvParams& p, unsigned int code, unsigned int sleep_ns = 0) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (true) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++it & 63) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > p.spin_budget) {
        atomicCAS(p.status, 0u, code);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
}

template <bool kSlab, bool kDual = false>
__device__ __forceinline__ void conv2d_tf32_body(const CUtensorMap& tmW, const CUtensorMap& tmX,
                                                 const ConvParams& p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t stage_b_bytes = static_cast<uint32_t>(p.block_n) * kBlockK * 4;
  // slab form: the A operand goes from the gather warps' registers into tensor memory (32 columns
  // per stage beside the accumulators), so a stage of shared memory holds the weight tile alone
  const uint32_t stage_a_bytes = kSlab ? 0u : static_cast<uint32_t>(kStageABytes);
  const uint32_t stage_bytes = stage_a_bytes + stage_b_bytes;
  // slab form: [stages][slab slot 0][slab slot 1][tap offsets, taps * 32 ints][barriers]
  const uint32_t slab_base = smem_base + p.num_stages * stage_bytes;
  const uint32_t tab_base = slab_base + (kSlab ? 2u * static_cast<uint32_t>(p.slab_bytes) : 0u);
  const uint32_t bar_base = tab_base + (kSlab ? ((static_cast<uint32_t>(p.taps) * 128u + 127u) & ~127u) : 0u);
  // barriers: full[8] @0, empty[8] @64, tmem_full[2] @128, tmem_empty[2] @144 | tmem slot @160 | abort @168
  //           | slab_full[2] @176, slab_empty[2] @192
  auto slab_full_bar = [&](int s) { return bar_base + 176u + 8u * s; };
  auto slab_empty_bar = [&](int s) { return bar_base + 192u + 8u * s; };
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
      // the weight load's expect_tx + the gather warps that fill the stage: all sixteen (a quarter of
      // each row's k's each), or in the slab form the four (one per tensor-memory lane quadrant) of
      // the group that owns this k-block
      ptx::mbar_init(full_bar(s), kSlab ? 1 + 4 : 1 + kConvGatherWarps);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), kDual ? 2 : 1);   // two MMA threads: both commit
      ptx::mbar_init(tempty_bar(a), 4);
      if constexpr (kSlab) {
        ptx::mbar_init(slab_full_bar(a), 1);
        ptx::mbar_init(slab_empty_bar(a), kConvGatherWarps);
      }
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmW);
    if constexpr (kSlab) ptx::prefetch_tensormap(&tmX);
  }
  if constexpr (kSlab) {
    // byte offset of local k = c * taps + (ki * kw + kj) inside a slab: the same for every chunk
    int* tab = reinterpret_cast<int*>(smem_gen + (tab_base - smem_base));
    for (int e = threadIdx.x; e < p.taps * kBlockK; e += blockDim.x) {
      const int c = e / p.taps;
      const int tap = e - c * p.taps;
      const int ki = tap / p.kw, kj = tap - ki * p.kw;
      tab[e] = ((c * p.slab_rows + ki) * p.slab_pitch + kj) * 4;
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc_1cta(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_1cta();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  // dependents of this grid may be scheduled only now that this CTA holds its TMEM columns
  ptx::grid_dep_launch_dependents();
  // unit u -> (position tile, channel tile); channel tiles of one position tile are neighbours
  auto tile_p = [&](int u) { return u / p.tiles_n; };
  auto tile_n = [&](int u) { return u % p.tiles_n; };
  // slab form: position tile tp = (image, tile inside the image)
  const int plane_i = p.oh * p.ow;

  if (warp == 0) {
    // ------------------------------------------------------- weight producer ---
    if (lane == 0) {
      ptx::grid_dep_wait();
      const uint64_t pol = ptx::make_l2_policy(3);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // slab form: the next chunk to load, as (unit, chunk) with a running count for slot and parity
      int slab_u = blockIdx.x, slab_j = 0, slab_count = 0;
      auto issue_slab = [&]() -> bool {
        if (slab_u >= p.total_units) return true;
        const int slot = slab_count & 1;
        if (!conv_wait(slab_empty_bar(slot), ((slab_count >> 1) & 1u) ^ 1u, abort_flag, p, kStatusConvSlab, 64))
          return false;
        const int tp = tile_p(slab_u);
        const int img = tp / p.tiles_pi;
        const int oy_first = ((tp - img * p.tiles_pi) * kBlockM) / p.ow;
        ptx::mbar_expect_tx(slab_full_bar(slot), static_cast<uint32_t>(p.slab_bytes));
        ptx::tma_load_4d_hint(slab_base + slot * p.slab_bytes, &tmX, slab_full_bar(slot), -kConvSlabHalo,
                              oy_first * p.sh - p.ph, slab_j * kConvSlabChannels, img, pol);
        ++slab_count;
        if (++slab_j == p.n_chunks) { slab_j = 0; slab_u += gridDim.x; }
        return true;
      };
      if constexpr (kSlab) ok = issue_slab();
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const int n0 = tile_n(u) * p.block_n;
        int next_chunk_kb = 0;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if constexpr (kSlab) {
            if (kb == next_chunk_kb) {               // the main loop enters a chunk: fetch the one after it
              next_chunk_kb += p.taps;
              ok = issue_slab();
              if (!ok) break;
            }
          }
          ok = conv_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusProducerTimeout, kSlab ? 32 : 0);
          if (!ok) break;
          const uint32_t sb = smem_base + stage * stage_bytes + stage_a_bytes;
          ptx::mbar_expect_tx(full_bar(stage), stage_b_bytes);
          ptx::tma_load_3d_hint(sb, &tmW, full_bar(stage), kb * kBlockK, n0, 0, pol);
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (kDual && (warp == 1 || warp == kConvSlabMmaWarpB)) {
    // ------------------------------------------------------ the two MMA issuers ---
    // Thread `who` takes the k-blocks whose running count (over all units) has its parity, into its own
    // 64-column accumulator of the set; a tile's first k-block of each thread overwrites it.
    if (lane == 0) {
      const int who = warp == 1 ? 0 : 1;
      const uint32_t idesc = ptx::idesc_tf32(kBlockM, p.block_n, 0, 0);
      const uint64_t db0 = ptx::smem_desc_sw128(smem_base, 16u, 1024u);
      const uint64_t db_step = stage_bytes >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      int count = 0;                                                 // k-blocks passed, over all units
      bool ok = true;
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        ok = conv_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p, kStatusMmaTmemTimeout);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kMaxBlockN) + static_cast<uint32_t>(who) * 64u;
        uint32_t first = 0u;
        for (int kb = 0; kb < p.num_kb; ++kb, ++count) {
          if ((count & 1) == who) {
            ok = conv_wait(full_bar(stage), phase, abort_flag, p, kStatusMmaTimeout);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t acol = tmem_base + conv_slab_tmem_a(stage);
            const uint64_t db = db0 + static_cast<uint64_t>(stage) * db_step;
            ptx::mma_tf32_1cta_ts(tmem_d, acol, db, idesc, first);
            first = 1u;
#pragma unroll
            for (int ks = 1; ks < kBlockK / kUmmaK; ++ks)
              ptx::mma_tf32_1cta_ts(tmem_d, acol + ks * kUmmaK, db + ks * 2u, idesc, 1u);
            ptx::mma_commit_1cta(empty_bar(stage));
          }
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit_1cta(tfull_bar(acc));          // this thread's part of the tile is complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer ---
    if (lane == 0) {
      const uint32_t idesc = ptx::idesc_tf32(kBlockM, p.block_n, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // slab form: state of the current stage
      const uint64_t s_db0 = ptx::smem_desc_sw128(smem_base + stage_a_bytes, 16u, 1024u);
      const uint64_t s_db_step = stage_bytes >> 4;
      uint64_t s_db = s_db0;
      uint32_t s_full = full_bar(0);
      uint32_t s_acol = tmem_base + conv_slab_tmem_a(0);
      uint32_t ready = 0;
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        ok = conv_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p, kStatusMmaTmemTimeout);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kMaxBlockN);
        uint32_t first = 0u;
        if constexpr (kSlab) {
          // A from tensor memory.  Everything that depends on the stage alone (barrier addresses, the
          // weight tile's descriptor, the A slot's column) advances by a constant, so a k-block costs
          // this thread a dozen instructions.
          for (int kb = 0; kb < p.num_kb; ++kb) {
            // `ready`: a non-suspending probe of this stage's barrier made one k-block earlier, so its
            // latency ran under the previous k-block's MMA issue
            if (!ready) {
              ok = conv_wait(s_full, phase, abort_flag, p, kStatusMmaTimeout);
              if (!ok) break;
            }
            const uint32_t cur_empty = s_full + 64u;
            const uint32_t cur_acol = s_acol;
            const uint64_t cur_db = s_db;
            if (++stage == p.num_stages) {
              stage = 0; phase ^= 1u;
              s_full = full_bar(0); s_db = s_db0; s_acol = tmem_base + conv_slab_tmem_a(0);
            } else {
              s_full += 8u; s_db += s_db_step;
              s_acol += (stage == 4) ? 160u : 32u;     // slots 0-3 at columns 128.., slots 4-7 at 384..
            }
            ready = ptx::mbar_test_wait(s_full, phase);
            ptx::tc_fence_after_sync();
            ptx::mma_tf32_1cta_ts(tmem_d, cur_acol, cur_db, idesc, first);
            first = 1u;
#pragma unroll
            for (int ks = 1; ks < kBlockK / kUmmaK; ++ks)
              ptx::mma_tf32_1cta_ts(tmem_d, cur_acol + ks * kUmmaK, cur_db + ks * 2u, idesc, 1u);
            ptx::mma_commit_1cta(cur_empty);
          }
        } else
        for (int kb = 0; kb < p.num_kb; ++kb) {
          ok = conv_wait(full_bar(stage), phase, abort_flag, p, kStatusMmaTimeout);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + stage_a_bytes;
#pragma unroll
          for (int ks = 0; ks < kBlockK / kUmmaK; ++ks) {
            const uint64_t db = ptx::smem_desc_sw128(sb + ks * 32u, 16u, 1024u);
            if constexpr (kSlab) {
              // A: 128 lanes x 8 columns of this stage's tensor-memory slot
              ptx::mma_tf32_1cta_ts(tmem_d, tmem_base + conv_slab_tmem_a(stage) + ks * kUmmaK, db, idesc, first);
            } else {
              const uint64_t da = ptx::smem_desc_sw128(sa + ks * 32u, 16u, 1024u);
              ptx::mma_tf32_1cta(tmem_d, da, db, idesc, first);
            }
            first = 1u;
          }
          ptx::mma_commit_1cta(empty_bar(stage));
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit_1cta(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp < kConvGatherWarp0) {
    // -------------------------------------------------------------- epilogue ---
    ptx::grid_dep_wait();
    const int q = warp & 3;
    const long long plane = static_cast<long long>(p.oh) * p.ow;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int kb_seen = 0;       // two MMA threads: the running k-block count tells which took a tile's first k-block
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const int n0 = tile_n(u) * p.block_n;
      bool row_ok;
      long long img;
      int rem;
      if constexpr (kSlab) {
        const int tp = tile_p(u);
        img = tp / p.tiles_pi;
        rem = (tp - static_cast<int>(img) * p.tiles_pi) * kBlockM + q * 32 + lane;
        row_ok = rem < plane_i;
        if (!row_ok) rem = 0;
      } else {
        const long long pos = static_cast<long long>(tile_p(u)) * kBlockM + q * 32 + lane;
        row_ok = pos < p.positions;
        img = row_ok ? pos / plane : 0;
        rem = row_ok ? static_cast<int>(pos - img * plane) : 0;
      }
      const int e_oy = rem / p.ow, e_ox = rem - e_oy * p.ow;
      const long long dplane = static_cast<long long>(p.dst_h) * p.dst_w;           // channel stride
      float* obase = p.out + (img * p.co) * dplane +
                     static_cast<long long>(p.dst_y0 + e_oy * p.dst_sy) * p.dst_w + p.dst_x0 + e_ox * p.dst_sx;
      ok = conv_wait(tfull_bar(acc), acc_phase, abort_flag, p, kStatusEpilogueTimeout, kSlab ? 256 : 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * kMaxBlockN);
      // two MMA threads: their two accumulators are added; with a single k-block only the thread whose
      // turn it was has written one
      const int first_who = kb_seen & 1;
      const bool both = p.num_kb >= 2;
      kb_seen += p.num_kb;
      for (int c = 0; c < p.block_n / 32; ++c) {
        const int co0 = n0 + c * 32;
        if (co0 >= p.co) break;
        uint32_t r[32];
        if constexpr (kDual) {
          ptx::tmem_ld_32x32(taddr0 + static_cast<uint32_t>(first_who) * 64u + c * 32, r);
          if (both) {                                // warp-uniform
            uint32_t r2[32];
            ptx::tmem_ld_32x32(taddr0 + static_cast<uint32_t>(first_who ^ 1) * 64u + c * 32, r2);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
          } else {
            ptx::tmem_ld_wait();
          }
        } else {
          ptx::tmem_ld_32x32(taddr0 + c * 32, r);
          ptx::tmem_ld_wait();
        }
        if (co0 + 32 <= p.co) {                      // whole chunk: no per-channel bound checks
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(p.bias + co0 + j));
          }
          if (p.act == kActRelu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(fmaxf(__uint_as_float(r[j]), 0.0f));
          }
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) obase[(co0 + j) * dplane] = __uint_as_float(r[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (co0 + j < p.co && row_ok) {
              float v = __uint_as_float(r[j]);
              if (p.bias != nullptr) v += __ldg(p.bias + co0 + j);
              if (p.act == kActRelu) v = fmaxf(v, 0.0f);
              obase[(co0 + j) * dplane] = v;
            }
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else if (kDual && warp == kConvSlabMmaWarpB) {
    // (the second MMA thread's warp: handled above)
  } else {
    // ---------------------------------------------------------------- gather ---
    // Sixteen warps: warp g fills rows (g & 3) * 32 + lane, k sub-range (g >> 2) * 8 .. + 8 of the
    // stage.  The gather is bound by instruction issue, so the per-element work is cut to a
    // broadcast table read, a mask test, one add and the load:
    //  * per unit a thread builds a bit mask over the kernel taps (ki * kw + kj) that fall inside
    //    the image for its position, and the pointer to tap (0, 0) of channel 0;
    //  * what depends on k alone -- the offset ci*H*W + ki*W + kj and the tap's bit -- comes from a
    //    table a small kernel wrote before this one (all lanes read the same entry).
    ptx::grid_dep_wait();
    const int g = warp - kConvGatherWarp0;
    // row of the A stage = position.  The slab form writes its rows into tensor memory, where a
    // warp reaches the 32 lanes of quadrant warp % 4 only
    const int r = (kSlab ? (warp & 3) : (g & 3)) * 32 + lane;
    const int part = g >> 2;                                      // which k sub-range of the row (slab form: which k-blocks)
    const long long plane = static_cast<long long>(p.oh) * p.ow;
    const int hw = p.h * p.w;
    const bool taps_fit_32 = p.kh * p.kw <= 32;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // waits for a free stage, writes this thread's part of the row, hands the stage over
    auto emit = [&](const float (&e)[kConvKPerThread]) -> bool {
      // one lane per warp polls; the shuffle orders the other lanes' writes after its observation
      int okw = 1;
      if (lane == 0) okw = conv_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusConvGather) ? 1 : 0;
      if (__shfl_sync(0xffffffffu, okw, 0) == 0) return false;
      // 32-bit shared-window addresses: row r of the stage, 16-byte chunk c at c ^ (r & 7)
      const uint32_t row = smem_base + stage * stage_bytes + r * 128;
#pragma unroll
      for (int j = 0; j < kConvKPerThread / 4; ++j)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                         row + (((part * (kConvKPerThread / 4) + j) ^ (r & 7)) << 4)),
                     "f"(e[4 * j]), "f"(e[4 * j + 1]), "f"(e[4 * j + 2]), "f"(e[4 * j + 3])
                     : "memory");
      ptx::fence_proxy_async_smem();               // generic writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(full_bar(stage));
      if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
      return true;
    };
    if constexpr (kSlab) {
      // ------------------------------------------- gather from the slab in shared memory ---
      const int* tab = reinterpret_cast<const int*>(smem_gen + (tab_base - smem_base));
      int chunk_count = 0;                           // chunks consumed: slot and parity of the slab barriers
      int kb_count = 0;                              // k-blocks passed, over all units: whose turn a stage is
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const int tp = tile_p(u);
        const int img = tp / p.tiles_pi;
        const int p0 = (tp - img * p.tiles_pi) * kBlockM;
        const int oy_first = p0 / p.ow;
        const int rem = p0 + r;
        // rows past the end of the image read the tile's first position: their products are never stored
        const int oy = rem < plane_i ? rem / p.ow : oy_first;
        const int ox = rem < plane_i ? rem - oy * p.ow : 0;
        // byte offset, inside a slab, of tap (0, 0) of channel 0 for this position (column 0 of the
        // image is column kConvSlabHalo of the slab row)
        const uint32_t pos_off = static_cast<uint32_t>(((oy - oy_first) * p.sh * p.slab_pitch +
                                                        ox * p.sw - p.pw + kConvSlabHalo) * 4);
        int kb = 0;
        for (int j = 0; j < p.n_chunks && ok; ++j) {
          const int slot = chunk_count & 1;
          int okw = 1;
          if (lane == 0)
            okw = conv_wait(slab_full_bar(slot), (chunk_count >> 1) & 1u, abort_flag, p, kStatusConvSlabFull, 32) ? 1 : 0;
          if (__shfl_sync(0xffffffffu, okw, 0) == 0) { ok = false; break; }
          const uint32_t base = slab_base + static_cast<uint32_t>(slot) * p.slab_bytes + pos_off;
          for (int t = 0; t < p.taps && kb < p.num_kb; ++t, ++kb) {
            // A warp fills 32 rows (its tensor-memory lane quadrant) of every fourth k-block
            // (g >> 2 = k-block count mod 4), all 32 k's of a row per thread, with one tcgen05.st.
            // Written through shared memory instead, every fill needed a fence.proxy.async, which
            // took ~900 clocks and held up the MMA issue as well: the tensor pipe stayed at 23 %.
            if ((kb_count & 3) == part) {
              // the row's 32 values into registers first: the loads need nothing but the slab
              const int4* t4 = reinterpret_cast<const int4*>(tab + t * kBlockK);
              uint32_t e[kBlockK];
#pragma unroll
              for (int i = 0; i < kBlockK / 4; ++i) {
                const int4 o = t4[i];
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(e[4 * i]) : "r"(base + o.x));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(e[4 * i + 1]) : "r"(base + o.y));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(e[4 * i + 2]) : "r"(base + o.z));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(e[4 * i + 3]) : "r"(base + o.w));
              }
              int okw2 = 1;
              if (lane == 0)
                okw2 = conv_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusConvGather, 32) ? 1 : 0;
              if (__shfl_sync(0xffffffffu, okw2, 0) == 0) { ok = false; break; }
              // the tensor core has read this slot's previous contents (its commit released the stage)
              ptx::tc_fence_after_sync();
              ptx::tmem_st_32x32(tmem_base + (static_cast<uint32_t>(r & ~31) << 16) + conv_slab_tmem_a(stage), e);
              ptx::tmem_st_wait();                     // in tensor memory before the tensor core is told
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(full_bar(stage));
            }
            ++kb_count;
            if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
          }
          // the slab has been read (its values went through this warp's stores above): hand it back
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(slab_empty_bar(slot));
          ++chunk_count;
        }
      }
    } else
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const long long pos = static_cast<long long>(tile_p(u)) * kBlockM + r;
      const bool row_ok = pos < p.positions;
      const long long img = row_ok ? pos / plane : 0;
      const int rem = row_ok ? static_cast<int>(pos - img * plane) : 0;
      const int oy = rem / p.ow, ox = rem - oy * p.ow;
      const int iy0 = oy * p.sh - p.ph, ix0 = ox * p.sw - p.pw;
      unsigned long long tapmask = 0;
      if (row_ok) {
        for (int ki = 0; ki < p.kh; ++ki)
          for (int kj = 0; kj < p.kw; ++kj)
            if (static_cast<unsigned>(iy0 + ki) < static_cast<unsigned>(p.h) &&
                static_cast<unsigned>(ix0 + kj) < static_cast<unsigned>(p.w))
              tapmask |= 1ull << (ki * p.kw + kj);
      }
      // never dereferenced for a tap outside the image
      const float* xp = p.x + img * p.ci * hw + static_cast<long long>(iy0) * p.w + ix0;
      const uint32_t mlo = static_cast<uint32_t>(tapmask), mhi = static_cast<uint32_t>(tapmask >> 32);
      // The loads of k-block kb + 1 are issued before k-block kb is written out, so their latency
      // (L2, mostly) runs under the write, the fence and the wait for the next free stage.  Two
      // register buffers take turns (the loop is unrolled by two so that both are indexed
      // statically and nothing is copied).
      float na[kConvKPerThread], nb[kConvKPerThread];
      auto issue_loads = [&](int kb, float (&dst)[kConvKPerThread]) {
        const int4* tab = p.ktab + kb * kBlockK + part * kConvKPerThread;
        if (taps_fit_32) {                           // warp-uniform: kernels up to 32 taps (1x1 .. 5x5)
#pragma unroll
          for (int i = 0; i < kConvKPerThread; ++i) {
            const int4 t = __ldg(tab + i);
            dst[i] = ldg_if(xp + t.x, mlo & static_cast<uint32_t>(t.y));
          }
        } else {
#pragma unroll
          for (int i = 0; i < kConvKPerThread; ++i) {
            const int4 t = __ldg(tab + i);
            dst[i] = ldg_if(xp + t.x, (mlo & static_cast<uint32_t>(t.y)) | (mhi & static_cast<uint32_t>(t.z)));
          }
        }
      };
      issue_loads(0, na);
      for (int kb = 0; kb < p.num_kb; kb += 2) {
        if (kb + 1 < p.num_kb) issue_loads(kb + 1, nb);
        ok = emit(na);
        if (!ok || kb + 1 >= p.num_kb) break;
        if (kb + 2 < p.num_kb) issue_loads(kb + 2, na);
        ok = emit(nb);
        if (!ok) break;
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_1cta(tmem_base, kTmemCols);
  }
}

__global__ void __launch_bounds__(kConvThreads, 1)
conv2d_tf32_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ ConvParams p) {
  conv2d_tf32_body<false>(tmW, tmW, p);
}

// tmX: the input as a 4-D tensor (w, h, ci, batch) with box (w + 8, slab_rows, 32, 1).
__global__ void __launch_bounds__(kConvThreads, 1)
conv2d_tf32_slab_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                        const __grid_constant__ ConvParams p) {
  conv2d_tf32_body<true>(tmW, tmX, p);
}

// The slab form with two MMA-issuing threads, for channel tiles of at most 64 columns.
__global__ void __launch_bounds__(kConvSlabDualThreads, 1)
conv2d_tf32_slab_dual_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                             const __grid_constant__ ConvParams p) {
  conv2d_tf32_body<true, true>(tmW, tmX, p);
}

// What the gather needs per k = (ci, ki, kj): the offset of that tap from tap (0, 0) of channel 0
// and the tap's bit in the 64-bit tap mask; zeros past the end of k (never inside the image).
__global__ void __launch_bounds__(256)
conv_ktab_kernel(int4* __restrict__ tab, int entries, int k, int kh, int kw, int h, int w) {
  const int khw = kh * kw;
  for (int e = blockIdx.x * 256 + threadIdx.x; e < entries; e += 256 * gridDim.x) {
    int4 t = make_int4(0, 0, 0, 0);
    if (e < k) {
      const int ci = e / khw;
      const int rk = e - ci * khw;
      const int ki = rk / kw, kj = rk - ki * kw;
      t.x = ci * h * w + ki * w + kj;
      if (rk < 32) t.y = static_cast<int>(1u << rk); else t.z = static_cast<int>(1u << (rk - 32));
    }
    tab[e] = t;
  }
}

// weights [co, k] -> [co, k_pad] with zero fill, for k that TMA cannot stride over (k % 4 != 0)
__global__ void __launch_bounds__(256)
pad_weights_kernel(const float* __restrict__ w, float* __restrict__ wp, int co, int k, int k_pad) {
  const long long total = static_cast<long long>(co) * k_pad;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const long long c = e / k_pad;
    const int kk = static_cast<int>(e - c * k_pad);
    wp[e] = kk < k ? w[c * k + kk] : 0.0f;
  }
}

// w [ic, oc, kh, kw] -> wp [oc, k_pad] with k = (ic, a, b) and wp[oc][(ic*kh + a)*kw + b] =
// w[ic][oc][kh-1-a][kw-1-b], zero fill past k: the weights of the convolution that maps an output
// gradient back to the input gradient.
__global__ void __launch_bounds__(256)
flip_weights_kernel(const float* __restrict__ w, float* __restrict__ wp, int ic, int oc, int kh, int kw,
                    int k_pad) {
  const int khw = kh * kw;
  const int k = ic * khw;
  const long long total = static_cast<long long>(oc) * k_pad;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const int o = static_cast<int>(e / k_pad);
    const int kk = static_cast<int>(e - static_cast<long long>(o) * k_pad);
    float v = 0.0f;
    if (kk < k) {
      const int i = kk / khw;
      const int r = kk - i * khw;
      const int a = r / kw, b = r - a * kw;
      v = w[((static_cast<long long>(i) * oc + o) * kh + (kh - 1 - a)) * kw + (kw - 1 - b)];
    }
    wp[e] = v;
  }
}

// The same for one phase (ry, rx) of a strided input gradient: only the taps ki = ry + sh * t,
// kj = rx + sw * u reach the input rows iy with (iy + pad_h) % sh == ry (likewise columns), so the
// phase is a stride-1 convolution of the output gradient with the sub-kernel [ty, tx], reversed:
// wp[oc][(ic*ty + a)*tx + b] = w[ic][oc][ry + sh*(ty-1-a)][rx + sw*(tx-1-b)], zero fill past k.
__global__ void __launch_bounds__(256)
flip_weights_phase_kernel(const float* __restrict__ w, float* __restrict__ wp, int ic, int oc, int kh, int kw,
                          int ry, int rx, int sh, int sw, int ty, int tx, int k_pad) {
  const int tt = ty * tx;
  const int k = ic * tt;
  const long long total = static_cast<long long>(oc) * k_pad;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const int o = static_cast<int>(e / k_pad);
    const int kk = static_cast<int>(e - static_cast<long long>(o) * k_pad);
    float v = 0.0f;
    if (kk < k) {
      const int i = kk / tt;
      const int r = kk - i * tt;
      const int a = r / tx, b = r - a * tx;
      v = w[((static_cast<long long>(i) * oc + o) * kh + (ry + sh * (ty - 1 - a))) * kw + (rx + sw * (tx - 1 - b))];
    }
    wp[e] = v;
  }
}

// Explicit im2col for the weight gradient, tap-major: col[(n * K + k) * ldp + p] = the input under
// tap k = (c, ki, kj) of output position p of image n (0 in the padding and for p in [P, ldp)).
// FastNN's kernel_im2col uses the same [K, P] layout per image (cuda/kernels.cu:836-861); here one
// launch covers all images, a block walks whole rows (the tap is decoded once per row), a thread
// writes four consecutive positions as one float4 and reads along the image row, so both sides
// are coalesced.  Both operands of the GEMM that follows are then contiguous along its
// contraction (the positions).
__global__ void __launch_bounds__(256)
im2col_taps_kernel(const float* __restrict__ x, float* __restrict__ col, int batch, int ci, int h, int w,
                   int kh, int kw, int sh, int sw, int ph, int pw, int oh, int ow, int ldp) {
  const int khw = kh * kw;
  const int k_all = ci * khw;
  const int plane = oh * ow;
  const long long rows = static_cast<long long>(batch) * k_all;
  const int n4 = ldp >> 2;
  // 64 threads walk one row (a row of 56 x 56 positions is 784 float4s: 12.25 turns of 64, where
  // 256 threads on one row idled through a quarter of their turns); four rows per block and turn
  const int sub = threadIdx.x >> 6, lane64 = threadIdx.x & 63;
  const int step_y = 256 / ow, step_x = 256 - step_y * ow;      // 64 float4s = 256 positions on
  for (long long row = 4ll * blockIdx.x + sub; row < rows; row += 4ll * gridDim.x) {
    const long long n = row / k_all;
    const int k = static_cast<int>(row - n * k_all);
    const int c = k / khw;
    const int r = k - c * khw;
    const int ki = r / kw, kj = r - ki * kw;
    const float* xc = x + (n * ci + c) * static_cast<long long>(h) * w;
    float4* dst = reinterpret_cast<float4*>(col + row * ldp);
    int oy0 = (lane64 * 4) / ow, ox0 = lane64 * 4 - oy0 * ow;
    for (int p4 = lane64; p4 < n4; p4 += 64) {
      const int p = p4 * 4;
      int oy = oy0, ox = ox0;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int iy = oy * sh - ph + ki, ix = ox * sw - pw + kj;
        v[j] = (p + j < plane && static_cast<unsigned>(iy) < static_cast<unsigned>(h) &&
                static_cast<unsigned>(ix) < static_cast<unsigned>(w))
                   ? __ldg(xc + static_cast<long long>(iy) * w + ix) : 0.0f;
        if (++ox == ow) { ox = 0; ++oy; }
      }
      dst[p4] = make_float4(v[0], v[1], v[2], v[3]);
      ox0 += step_x; oy0 += step_y;
      if (ox0 >= ow) { ox0 -= ow; ++oy0; }
    }
  }
}

// Direct convolution, one thread per output element, FP32 FMA: serves the shapes the implicit-GEMM
// kernel's gather cannot encode (64 kernel taps or more, images of 2^25 elements or more).  With
// flip != 0 `wt` is [ci, co, kh, kw] and is read with both kernel axes reversed (the stride-1 input
// gradient written as a convolution of the output gradient; channel roles already swapped by the
// caller), otherwise [co, ci, kh, kw].  Loop order ci, ki, kj as Conv2d::forward
// (src/nn/conv.rs:97-123).
__global__ void __launch_bounds__(256)
conv2d_direct_kernel(const float* __restrict__ x, const float* __restrict__ wt,
                     const float* __restrict__ bias, float* __restrict__ out, int batch, int ci, int co,
                     int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int oh, int ow, int act,
                     int flip) {
  const long long total = static_cast<long long>(batch) * co * oh * ow;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const int ox = static_cast<int>(e % ow);
    const int oy = static_cast<int>((e / ow) % oh);
    const int c = static_cast<int>((e / (static_cast<long long>(ow) * oh)) % co);
    const long long n = e / (static_cast<long long>(ow) * oh * co);
    float acc = 0.0f;
    for (int i = 0; i < ci; ++i) {
      const float* xi = x + (n * ci + i) * static_cast<long long>(h) * w;
      for (int ki = 0; ki < kh; ++ki) {
        const int iy = oy * sh - ph + ki;
        if (static_cast<unsigned>(iy) >= static_cast<unsigned>(h)) continue;
        for (int kj = 0; kj < kw; ++kj) {
          const int ix = ox * sw - pw + kj;
          if (static_cast<unsigned>(ix) >= static_cast<unsigned>(w)) continue;
          const float wv = flip ? __ldg(wt + ((static_cast<long long>(i) * co + c) * kh + (kh - 1 - ki)) * kw +
                                        (kw - 1 - kj))
                                : __ldg(wt + ((static_cast<long long>(c) * ci + i) * kh + ki) * kw + kj);
          acc = fmaf(__ldg(xi + static_cast<long long>(iy) * w + ix), wv, acc);
        }
      }
    }
    if (bias != nullptr) acc += __ldg(bias + c);
    if (act == kActRelu) acc = fmaxf(acc, 0.0f);
    out[e] = acc;
  }
}

// Input gradient of a convolution with any stride and padding, gather form: the thread that owns
// grad_input[n, c, iy, ix] adds grad_output[n, o, oy, ox] * weight[o, c, ki, kj] over all (o, ki, kj)
// with oy * stride_h = iy + pad_h - ki and ox * stride_w = ix + pad_w - kj inside the output.  The
// same terms FastNN's GEMM + col2im adds (cuda/kernels.cu:862-893, 949-987); every element is
// written exactly once, so the output needs no clearing and no atomics.
__global__ void __launch_bounds__(256)
conv2d_backward_data_direct_kernel(const float* __restrict__ go, const float* __restrict__ wt,
                                   float* __restrict__ gi, int batch, int ci, int co, int h, int w, int oh,
                                   int ow, int kh, int kw, int sh, int sw, int ph, int pw) {
  const long long total = static_cast<long long>(batch) * ci * h * w;
  const long long oplane = static_cast<long long>(oh) * ow;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const int ix = static_cast<int>(e % w);
    const int iy = static_cast<int>((e / w) % h);
    const int c = static_cast<int>((e / (static_cast<long long>(w) * h)) % ci);
    const long long n = e / (static_cast<long long>(w) * h * ci);
    float acc = 0.0f;
    for (int ki = 0; ki < kh; ++ki) {
      const int ty = iy + ph - ki;
      if (ty < 0 || ty % sh != 0) continue;
      const int oy = ty / sh;
      if (oy >= oh) continue;
      for (int kj = 0; kj < kw; ++kj) {
        const int tx = ix + pw - kj;
        if (tx < 0 || tx % sw != 0) continue;
        const int ox = tx / sw;
        if (ox >= ow) continue;
        const float* gp = go + n * co * oplane + static_cast<long long>(oy) * ow + ox;
        const float* wp = wt + (static_cast<long long>(c) * kh + ki) * kw + kj;
        const long long wstep = static_cast<long long>(ci) * kh * kw;
        for (int o = 0; o < co; ++o) acc = fmaf(__ldg(gp + o * oplane), __ldg(wp + o * wstep), acc);
      }
    }
    gi[e] = acc;
  }
}

inline size_t conv_smem_bytes(int block_n, int num_stages) {
  return 1024 + static_cast<size_t>(num_stages) * (kStageABytes + block_n * kBlockK * 4) + kBarrierBytes;
}

// The slab form: the stage ring (weight tiles only), two slabs, the tap-offset table, the barriers.
inline size_t conv_slab_smem_bytes(int block_n, int num_stages, int slab_bytes, int taps) {
  return 1024 + static_cast<size_t>(num_stages) * (block_n * kBlockK * 4) +
         2 * static_cast<size_t>(slab_bytes) + ((static_cast<size_t>(taps) * 128 + 127) & ~static_cast<size_t>(127)) +
         kBarrierBytes;
}

}  // namespace fnn
