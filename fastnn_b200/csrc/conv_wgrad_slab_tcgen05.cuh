// Conv2d weight gradient as an implicit GEMM with the gathered operand in TENSOR memory (sm_100a).
//
//   dW[co, ci, ki, kj] = sum over (n, oy, ox) of dY[n, co, oy, ox] * x[n, ci, oy*sh + ki - ph, ox*sw + kj - pw]
// (Conv2dBackward, src/autograd/backward_ops.rs:753-770; FastNN's CUDA entry does im2col + cuBLAS per
// image, cuda/kernels.cu:989-1026.)  The product is turned round: D[tap, co] = A[tap, k] . B[co, k]^T with
// tap = (ci, ki, kj) as the M dimension and k = output positions,
//   * a k-block is 32 consecutive ox of ONE output row (n, oy) -- rows shorter than a multiple of 32 leave
//     columns that TMA fills with zeros on the dY side -- so B, the dY tile [co, 32 positions], is K-major
//     as stored and arrives by one 4-D TMA load, and the 32 values a tap needs are 32 consecutive (strided
//     by sw) words of one input row;
//   * the input rows of a group of output rows come into shared memory as a slab -- the channels of the
//     tap tile x rows x (w + 12) columns, one TMA load, zero halo columns and zero rows outside the image,
//     so no masks -- and a gather thread (= one tap = one row of A = one tensor-memory lane) reads its 32
//     words and writes them with ONE tcgen05.st into the stage's A slot in tensor memory: no shared-memory
//     A stage and so no fence.proxy.async per fill;
//   * two threads issue the MMAs, taking k-blocks in turn, each into its own accumulator (one thread issues
//     a tcgen05.mma of N <= 128 only every 100-120 clocks); the epilogue adds the two;
//   * the positions are cut into slices (one unit per SM); a unit leaves its [taps, co] tile transposed in
//     partial[slice][co][tap], i.e. already in dW's layout, and the split-K reduce kernel adds the slices
//     in ascending order: deterministic, no atomics, no column matrix.
// Roles: warp 0 producer (dY tiles, slabs), warps 1 and 22 MMA issuers, warps 2-5 epilogue, warps 6-21
// gather (four groups of four warps, a group takes every fourth k-block, a warp the 32 taps of its
// tensor-memory lane quadrant).  Every wait is bounded as in the other kernels.
#pragma once
#include "conv_tcgen05.cuh"

namespace fnn {

struct WgradSlabParams {
  int batch, ci, co, h, w, kh, kw, sh, sw, ph, pw, oh, ow;
  int k_taps;            // ci * kh * kw: rows of the product
  int taps;              // kh * kw
  int tiles_m;           // ceil(k_taps / 128)
  int tiles_n, block_n;  // channel tiles of dY
  int g_rows;            // output rows per slab
  int slabs_per_image;   // ceil(oh / g_rows)
  int kb_per_row;        // ceil(ow / 32)
  int total_slabs;       // batch * slabs_per_image
  int slices;            // K slices (each a run of slabs)
  int slab_ch;           // channels in a slab: those the 128 taps of a tile can touch
  int slab_rows;         // (g_rows - 1) * sh + kh
  int slab_pitch;        // floats per row in shared memory
  int slab_bytes;
  int num_stages;
  int total_units;       // slices * tiles_m * tiles_n
  float* partial;        // [slices][co][k_taps] (or dW itself when slices == 1)
  unsigned int* status;
  long long spin_budget;
};

enum : unsigned int { kStatusWgradSlab = 0x311 };
constexpr int kWgradSlabThreads = kConvThreads + 32;       // + the second MMA warp
constexpr int kWgradSlabMmaWarpB = kConvGatherWarp0 + kConvGatherWarps;
constexpr int kWgradSlabHalo = 4;
constexpr int kWgradSlabTailBytes = 2048;                  // zeroed bytes after the slabs (reads past a row's end)
// tensor memory: accumulators of the two MMA threads at columns 0 and 128, eight A slots of 32 columns from 256
__host__ __device__ constexpr uint32_t wgrad_slab_tmem_a(int s) { return 256u + 32u * static_cast<uint32_t>(s); }

__device__ __forceinline__ bool wgs_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                         const WgradSlabParams& p, unsigned int code, unsigned int sleep_ns = 0) {
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

// tmG: dY as (ow, oh, co, batch), box (32, 1, block_n, 1), 128B swizzle.
// tmX: x as (w, h, ci, batch), box (slab_pitch, slab_rows, slab_ch, 1), no swizzle.
__global__ void __launch_bounds__(kWgradSlabThreads, 1)
conv2d_wgrad_slab_kernel(const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmX,
                         const __grid_constant__ WgradSlabParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t stage_bytes = static_cast<uint32_t>(p.block_n) * kBlockK * 4;       // the dY tile
  // [stages][slab 0][slab 1][zeroed tail][barriers]
  const uint32_t slab_base = smem_base + p.num_stages * stage_bytes;
  const uint32_t bar_base = slab_base + 2u * static_cast<uint32_t>(p.slab_bytes) + kWgradSlabTailBytes;
  // barriers: full[8] @0, empty[8] @64, tmem_full @128, tmem_empty @144 | tmem slot @160 | abort @168
  //           | slab_full[2] @176, slab_empty[2] @192
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 64u + 8u * s; };
  const uint32_t tfull_bar = bar_base + 128u;
  const uint32_t tempty_bar = bar_base + 144u;
  auto slab_full_bar = [&](int s) { return bar_base + 176u + 8u * s; };
  auto slab_empty_bar = [&](int s) { return bar_base + 192u + 8u * s; };
  const uint32_t tmem_slot = bar_base + 160u;
  uint8_t* bar_gen = smem_gen + (bar_base - smem_base);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(bar_gen + 160);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 168);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.num_stages; ++s) {
      ptx::mbar_init(full_bar(s), 1 + 4);      // the dY load's expect_tx + the four warps of the owning group
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(tfull_bar, 2);              // both MMA threads commit
    ptx::mbar_init(tempty_bar, 4);
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(slab_full_bar(a), 1);
      ptx::mbar_init(slab_empty_bar(a), kConvGatherWarps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmG);
    ptx::prefetch_tensormap(&tmX);
  }
  // the slabs and the tail after them start as zeros: a read that runs past the end of a slab row (the
  // positions past the end of an output row, whose dY columns are zeros) must meet finite values
  {
    uint32_t* z = reinterpret_cast<uint32_t*>(smem_gen + (slab_base - smem_base));
    const int words = (2 * p.slab_bytes + kWgradSlabTailBytes) / 4;
    for (int i = threadIdx.x; i < words; i += blockDim.x) z[i] = 0u;
  }
  ptx::fence_proxy_async_smem();               // before TMA writes the same bytes
  if (warp == 1) {
    ptx::tmem_alloc_1cta(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_1cta();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  ptx::grid_dep_launch_dependents();

  // unit u -> (slice, tap tile, channel tile): the tiles of one slice are neighbours (they share dY and x)
  const int tiles = p.tiles_m * p.tiles_n;
  auto unit_slice = [&](int u) { return u / tiles; };
  auto unit_mt = [&](int u) { return (u % tiles) / p.tiles_n; };
  auto unit_nt = [&](int u) { return (u % tiles) % p.tiles_n; };
  auto slab_lo = [&](int slice) { return static_cast<int>(static_cast<long long>(slice) * p.total_slabs / p.slices); };
  // rows of slab q that exist
  auto slab_rows_of = [&](int q) {
    const int oy0 = (q % p.slabs_per_image) * p.g_rows;
    return min(p.g_rows, p.oh - oy0);
  };

  if (warp == 0) {
    // ------------------------------------------------------------- producer ---
    if (lane == 0) {
      ptx::grid_dep_wait();
      const uint64_t pol = ptx::make_l2_policy(3);
      int stage = 0;
      uint32_t phase = 0;
      int slab_count = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const int slice = unit_slice(u);
        const int c_first = (unit_mt(u) * kBlockM) / p.taps;        // first channel the tap tile touches
        const int co0 = unit_nt(u) * p.block_n;
        const int q0 = slab_lo(slice), q1 = slab_lo(slice + 1);
        for (int q = q0; q < q1 && ok; ++q) {
          const int n = q / p.slabs_per_image;
          const int oy0 = (q - n * p.slabs_per_image) * p.g_rows;
          {
            const int slot = slab_count & 1;
            ok = wgs_wait(slab_empty_bar(slot), ((slab_count >> 1) & 1u) ^ 1u, abort_flag, p, kStatusWgradSlab, 64);
            if (!ok) break;
            ptx::mbar_expect_tx(slab_full_bar(slot), static_cast<uint32_t>(p.slab_bytes));
            ptx::tma_load_4d_hint(slab_base + slot * p.slab_bytes, &tmX, slab_full_bar(slot), -kWgradSlabHalo,
                                  oy0 * p.sh - p.ph, c_first, n, pol);
            ++slab_count;
          }
          const int g = slab_rows_of(q);
          for (int rr = 0; rr < g && ok; ++rr)
            for (int xb = 0; xb < p.kb_per_row; ++xb) {
              ok = wgs_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusProducerTimeout, 32);
              if (!ok) break;
              ptx::mbar_expect_tx(full_bar(stage), stage_bytes);
              ptx::tma_load_4d_hint(smem_base + stage * stage_bytes, &tmG, full_bar(stage), xb * kBlockK, oy0 + rr,
                                    co0, n, pol);
              if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
            }
        }
      }
    }
  } else if (warp == 1 || warp == kWgradSlabMmaWarpB) {
    // ------------------------------------------------------ the two MMA issuers ---
    if (lane == 0) {
      const int who = warp == 1 ? 0 : 1;
      const uint32_t idesc = ptx::idesc_tf32(kBlockM, p.block_n, 0, 0);
      const uint64_t db0 = ptx::smem_desc_sw128(smem_base, 16u, 1024u);
      const uint64_t db_step = stage_bytes >> 4;
      const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(who) * 128u;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int count = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const int slice = unit_slice(u);
        int n_kb = 0;
        for (int q = slab_lo(slice); q < slab_lo(slice + 1); ++q) n_kb += slab_rows_of(q) * p.kb_per_row;
        ok = wgs_wait(tempty_bar, acc_phase ^ 1u, abort_flag, p, kStatusMmaTmemTimeout);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        uint32_t first = 0u;
        for (int kb = 0; kb < n_kb; ++kb, ++count) {
          if ((count & 1) == who) {
            ok = wgs_wait(full_bar(stage), phase, abort_flag, p, kStatusMmaTimeout);
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t acol = tmem_base + wgrad_slab_tmem_a(stage);
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
        ptx::mma_commit_1cta(tfull_bar);
        acc_phase ^= 1u;
      }
    }
  } else if (warp < kConvGatherWarp0) {
    // -------------------------------------------------------------- epilogue ---
    ptx::grid_dep_wait();
    const int q4 = warp & 3;
    uint32_t acc_phase = 0;
    int kb_seen = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const int slice = unit_slice(u);
      int n_kb = 0;
      for (int q = slab_lo(slice); q < slab_lo(slice + 1); ++q) n_kb += slab_rows_of(q) * p.kb_per_row;
      const int first_who = kb_seen & 1;
      const bool both = n_kb >= 2;
      kb_seen += n_kb;
      const int tap = unit_mt(u) * kBlockM + q4 * 32 + lane;      // this lane's row of the tile
      const int co0 = unit_nt(u) * p.block_n;
      float* obase = p.partial + (static_cast<long long>(slice) * p.co + co0) * p.k_taps + tap;
      ok = wgs_wait(tfull_bar, acc_phase, abort_flag, p, kStatusEpilogueTimeout, 256);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16);
      for (int c = 0; c < p.block_n / 32; ++c) {
        if (co0 + c * 32 >= p.co) break;
        uint32_t r[32];
        ptx::tmem_ld_32x32(taddr0 + static_cast<uint32_t>(first_who) * 128u + c * 32, r);
        if (both) {                                    // warp-uniform
          uint32_t r2[32];
          ptx::tmem_ld_32x32(taddr0 + static_cast<uint32_t>(first_who ^ 1) * 128u + c * 32, r2);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        } else {
          ptx::tmem_ld_wait();
        }
        if (tap < p.k_taps) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (co0 + c * 32 + j < p.co) obase[static_cast<long long>(c * 32 + j) * p.k_taps] = __uint_as_float(r[j]);
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar);
      acc_phase ^= 1u;
    }
  } else {
    // ---------------------------------------------------------------- gather ---
    ptx::grid_dep_wait();
    const int g = warp - kConvGatherWarp0;
    const int r = (warp & 3) * 32 + lane;            // row of the tile = tap = lane of tensor memory
    const int part = g >> 2;                         // this warp's k-blocks: those with count % 4 == part
    const uint32_t step = static_cast<uint32_t>(p.sw) * 4u;      // bytes between the inputs of neighbouring ox
    int stage = 0;
    uint32_t phase = 0;
    int chunk_count = 0;
    int kb_count = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const int slice = unit_slice(u);
      const int t0 = unit_mt(u) * kBlockM;
      const int c_first = t0 / p.taps;
      // this thread's tap; rows past the last tap read tap 0 of the tile's first channel (never stored)
      int tap = t0 + r;
      if (tap >= p.k_taps) tap = c_first * p.taps;
      const int ci = tap / p.taps;
      const int rk = tap - ci * p.taps;
      const int ki = rk / p.kw, kj = rk - ki * p.kw;
      // byte offset, inside a slab, of this tap's input for output position (row 0 of the slab, ox 0)
      const uint32_t tap_off = static_cast<uint32_t>((((ci - c_first) * p.slab_rows + ki) * p.slab_pitch + kj - p.pw +
                                                      kWgradSlabHalo) * 4);
      for (int q = slab_lo(slice); q < slab_lo(slice + 1) && ok; ++q) {
        const int slot = chunk_count & 1;
        int okw = 1;
        if (lane == 0)
          okw = wgs_wait(slab_full_bar(slot), (chunk_count >> 1) & 1u, abort_flag, p, kStatusWgradSlab, 32) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, okw, 0) == 0) { ok = false; break; }
        const uint32_t base = slab_base + static_cast<uint32_t>(slot) * p.slab_bytes + tap_off;
        const int grows = slab_rows_of(q);
        for (int rr = 0; rr < grows && ok; ++rr)
          for (int xb = 0; xb < p.kb_per_row; ++xb) {
            if ((kb_count & 3) == part) {
              // 32 inputs, one per ox of this k-block: words `step` bytes apart in one slab row
              const uint32_t a0 = base + static_cast<uint32_t>(rr * p.sh * p.slab_pitch) * 4u +
                                  static_cast<uint32_t>(xb * kBlockK) * step;
              uint32_t e[kBlockK];
#pragma unroll
              for (int j = 0; j < kBlockK; ++j)
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(e[j]) : "r"(a0 + j * step));
              // positions past the end of the output row: zeros (their dY columns are zeros too, but a
              // non-finite input next to the row must not turn the product into NaN)
              const int n_valid = p.ow - xb * kBlockK;
              if (n_valid < kBlockK) {                 // warp-uniform
#pragma unroll
                for (int j = 0; j < kBlockK; ++j)
                  if (j >= n_valid) e[j] = 0u;
              }
              int okw2 = 1;
              if (lane == 0)
                okw2 = wgs_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusConvGather, 32) ? 1 : 0;
              if (__shfl_sync(0xffffffffu, okw2, 0) == 0) { ok = false; break; }
              ptx::tc_fence_after_sync();
              ptx::tmem_st_32x32(tmem_base + (static_cast<uint32_t>(r & ~31) << 16) + wgrad_slab_tmem_a(stage), e);
              ptx::tmem_st_wait();
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(full_bar(stage));
            }
            ++kb_count;
            if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
          }
        // the slab has been read: hand it back
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(slab_empty_bar(slot));
        ++chunk_count;
      }
    }
  }

  // ---------------------------------------------------------------- teardown ---
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

inline size_t wgrad_slab_smem_bytes(int block_n, int num_stages, int slab_bytes) {
  return 1024 + static_cast<size_t>(num_stages) * (block_n * kBlockK * 4) + 2 * static_cast<size_t>(slab_bytes) +
         kWgradSlabTailBytes + kBarrierBytes;
}

}  // namespace fnn
