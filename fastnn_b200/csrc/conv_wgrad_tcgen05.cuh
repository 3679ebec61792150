// Conv2d weight gradient as an implicit GEMM on the tcgen05 main loop (sm_100a).
//
//   grad_weight[co, k] = sum over images n and output positions p of
//                        grad_output[n, co, p] * x[n, ci, oy*sh + ki - ph, ox*sw + kj - pw]
// with k = (ci, ki, kj) and p = (oy, ox): Conv2dBackward (src/autograd/backward_ops.rs:753-770).
// FastNN's CUDA entry builds an im2col matrix per image and calls cuBLAS with beta = 1
// (cuda/kernels.cu:989-1026).  Here the column matrix never exists: as a GEMM
//   D[co, k] = A[co, (n, p)] . B[k, (n, p)]^T        contraction over all positions of all images
//   warp 0      loads the A stage -- 128 channels x 32 positions of grad_output, contiguous along
//               the positions as stored -- by TMA;
//   warps 6-21  gather the B stage: row r = tap k0 + r, 32 consecutive positions of one image.  A
//               lane owns one position (consecutive lanes = consecutive ox, so a load instruction
//               is one coalesced row segment), a warp takes every sixteenth tap row; what depends
//               on the tap alone (offset, ki, kj) comes from a table; rows are written in the
//               K-major 128B-swizzled layout TMA would have produced, one k-block ahead;
//   warp 1      one lane issues tcgen05.mma kind::tf32 (M = 128 channels, N = block_n taps);
//   warps 2-5   drain the accumulator: lane = channel row, 32 taps per chunk, to grad_weight or to
//               a partial-sum slab when the contraction is cut into slices.
// Work unit = (channel tile, tap tile, slice of the global k-block sequence); a k-block lies inside
// one image (positions past the end of an image are zero in A by TMA's fill and zero in B by the
// gather).  Slices are added in ascending order by the split-K reduce kernel: deterministic.
#pragma once
#include "conv_tcgen05.cuh"

namespace fnn {

struct WgradParams {
  int batch, ci, co, h, w, kh, kw, sh, sw, ph, pw, oh, ow;
  int k;                 // ci * kh * kw
  int plane;             // oh * ow
  int kb_per_image;      // ceil(plane / 32)
  long long total_kb;    // batch * kb_per_image
  int slices;            // K slices; unit u -> slice u % slices
  long long kb_per_slice;
  int tiles_m, tiles_n, total_units;
  int block_n, num_stages;
  const float* x;
  const int4* ktab;      // [tiles_n * block_n] per tap: {offset ci*H*W + ki*W + kj, ki, kj, 1}; zeros past k
  float* out;            // slices == 1: grad_weight [co, k]; else partials [slices][co][k]
  unsigned int* status;
  long long spin_budget;
};

constexpr int kWgradGatherWarps = 16;
constexpr int kWgradThreads = 32 * (6 + kWgradGatherWarps);
constexpr int kWgradGatherWarp0 = 6;
constexpr int kWgradMaxRowsPerWarp = kMaxBlockN / kWgradGatherWarps;      // 16

__device__ __forceinline__ bool wgrad_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                           const WgradParams& p, unsigned int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (true) {
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

// tmG: grad_output as (position, channel, image), box 32 x 128 x 1, 128-byte swizzle, zero fill.
__global__ void __launch_bounds__(kWgradThreads, 1)
conv2d_wgrad_tf32_kernel(const __grid_constant__ CUtensorMap tmG, const __grid_constant__ WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t stage_b_bytes = static_cast<uint32_t>(p.block_n) * kBlockK * 4;
  const uint32_t stage_bytes = kStageABytes + stage_b_bytes;
  const uint32_t bar_base = smem_base + p.num_stages * stage_bytes;
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
      ptx::mbar_init(full_bar(s), 1 + kWgradGatherWarps);   // the TMA load's expect_tx + gather warps
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmG);
  }
  if (warp == 1) {
    ptx::tmem_alloc_1cta(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_1cta();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  ptx::grid_dep_launch_dependents();        // only now that this CTA holds its TMEM columns

  // unit u -> slice (fastest), tap tile, channel tile; the k-blocks of a slice
  auto slice_of = [&](int u) { return u % p.slices; };
  auto tile_n = [&](int u) { return (u / p.slices) % p.tiles_n; };
  auto tile_m = [&](int u) { return u / (p.slices * p.tiles_n); };
  auto kb_range = [&](int u, long long& kb0, long long& kb1) {
    kb0 = slice_of(u) * p.kb_per_slice;
    kb1 = kb0 + p.kb_per_slice < p.total_kb ? kb0 + p.kb_per_slice : p.total_kb;
    if (kb0 > kb1) kb0 = kb1;
  };

  if (warp == 0) {
    // ------------------------------------------------- grad_output producer ---
    if (lane == 0) {
      ptx::grid_dep_wait();
      const uint64_t pol = ptx::make_l2_policy(3);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const int m0 = tile_m(u) * kBlockM;
        long long kb0, kb1;
        kb_range(u, kb0, kb1);
        int img = static_cast<int>(kb0 / p.kb_per_image);           // one division per unit
        int kbi = static_cast<int>(kb0 - static_cast<long long>(img) * p.kb_per_image);
        for (long long kb = kb0; kb < kb1; ++kb) {
          ok = wgrad_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusProducerTimeout);
          if (!ok) break;
          const uint32_t sa = smem_base + stage * stage_bytes;
          ptx::mbar_expect_tx(full_bar(stage), kStageABytes);
          ptx::tma_load_3d_hint(sa, &tmG, full_bar(stage), kbi * kBlockK, m0, img, pol);
          if (++kbi == p.kb_per_image) { kbi = 0; ++img; }
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
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
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        long long kb0, kb1;
        kb_range(u, kb0, kb1);
        if (kb0 >= kb1) continue;               // an empty slice: the epilogue writes zeros on its own
        ok = wgrad_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p, kStatusMmaTmemTimeout);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kMaxBlockN);
        uint32_t first = 0u;
        for (long long kb = kb0; kb < kb1; ++kb) {
          ok = wgrad_wait(full_bar(stage), phase, abort_flag, p, kStatusMmaTimeout);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * stage_bytes;
          const uint32_t sb = sa + kStageABytes;
#pragma unroll
          for (int ks = 0; ks < kBlockK / kUmmaK; ++ks) {
            const uint64_t da = ptx::smem_desc_sw128(sa + ks * 32u, 16u, 1024u);
            const uint64_t db = ptx::smem_desc_sw128(sb + ks * 32u, 16u, 1024u);
            ptx::mma_tf32_1cta(tmem_d, da, db, idesc, first);
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
  } else if (warp < kWgradGatherWarp0) {
    // -------------------------------------------------------------- epilogue ---
    ptx::grid_dep_wait();
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const int row = tile_m(u) * kBlockM + q * 32 + lane;            // output channel
      const int n0 = tile_n(u) * p.block_n;
      long long kb0, kb1;
      kb_range(u, kb0, kb1);
      const bool empty = kb0 >= kb1;            // a slice past the end of the k-blocks: zeros
      if (!empty) {
        ok = wgrad_wait(tfull_bar(acc), acc_phase, abort_flag, p, kStatusEpilogueTimeout);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after_sync();
      }
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * kMaxBlockN);
      float* orow = p.out + (static_cast<long long>(slice_of(u)) * p.co + row) * p.k;
      for (int c = 0; c < p.block_n / 32; ++c) {
        const int k0 = n0 + c * 32;
        if (k0 >= p.k) break;                   // warp-uniform
        uint32_t r[32];
        if (!empty) {                           // warp-uniform
          ptx::tmem_ld_32x32(taddr0 + c * 32, r);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (row < p.co) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (k0 + j < p.k) orow[k0 + j] = __uint_as_float(r[j]);
        }
      }
      if (!empty) {
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------------------------------------------------------- gather ---
    // The gather is bound by instruction issue, so what can be hoisted is: the warp's table entries
    // sit in shared memory (one broadcast read with an immediate offset per element), rows go in
    // groups of four with nothing but the group test between them, and a row's shared-memory
    // address is a per-warp constant plus 2 KiB per step (row r = g + 16 i has r & 7 = g & 7, so
    // the swizzle term does not change from row to row).
    ptx::grid_dep_wait();
    const int g = warp - kWgradGatherWarp0;
    const int row_groups = p.block_n / (4 * kWgradGatherWarps);      // block_n is a multiple of 64
    const int hw = p.h * p.w;
    const int step_y = kBlockK / p.ow, step_x = kBlockK - step_y * p.ow;   // 32 positions further on
    const int lane_oy0 = lane / p.ow, lane_ox0 = lane - lane_oy0 * p.ow;
    const uint32_t tab_s = bar_base + kBarrierBytes + static_cast<uint32_t>(g) * (kWgradMaxRowsPerWarp * 16u);
    const uint32_t row_off = kStageABytes + static_cast<uint32_t>(g) * 128u +
                             ((static_cast<uint32_t>(lane >> 2) ^ static_cast<uint32_t>(g & 7)) << 4) +
                             (static_cast<uint32_t>(lane & 3) << 2);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const int n0 = tile_n(u) * p.block_n;
      long long kb0, kb1;
      kb_range(u, kb0, kb1);
      if (kb0 >= kb1) continue;
      // this warp's rows g, g + 16, ... of the tap table -> its slice of shared memory
      __syncwarp();
      if (lane < 4 * row_groups) {
        const int4 t = __ldg(p.ktab + n0 + g + lane * kWgradGatherWarps);
        asm volatile("st.shared.v4.s32 [%0], {%1, %2, %3, %4};" ::"r"(tab_s + lane * 16u), "r"(t.x), "r"(t.y),
                     "r"(t.z), "r"(t.w)
                     : "memory");
      }
      __syncwarp();
      float na[kWgradMaxRowsPerWarp], nb[kWgradMaxRowsPerWarp];
      // Cursor over the k-blocks the loads are issued for (one ahead of the one being written):
      // image, k-block inside it and this lane's output position, stepped without divisions.
      int c_img = static_cast<int>(kb0 / p.kb_per_image);           // one division per unit
      int c_kbi = static_cast<int>(kb0 - static_cast<long long>(c_img) * p.kb_per_image);
      int c_pos = c_kbi * kBlockK + lane;
      int c_oy = c_pos / p.ow, c_ox = c_pos - c_oy * p.ow;
      // loads of one k-block: this lane's position under every tap row of this warp
      auto issue_loads = [&](float (&dst)[kWgradMaxRowsPerWarp]) {
        const int iy0 = c_oy * p.sh - p.ph, ix0 = c_ox * p.sw - p.pw;
        // a position past the end of the image fails every row test
        const unsigned hlim = c_pos < p.plane ? static_cast<unsigned>(p.h) : 0u;
        // never dereferenced for a tap outside the image
        const float* xp = p.x + static_cast<long long>(c_img) * p.ci * hw + iy0 * p.w + ix0;
#pragma unroll
        for (int grp = 0; grp < kWgradMaxRowsPerWarp / 4; ++grp) {
          if (grp < row_groups) {               // warp-uniform
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = grp * 4 + j;
              int tx, ty, tz, tw;
              asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(tx), "=r"(ty), "=r"(tz), "=r"(tw)
                           : "r"(tab_s + i * 16u));
              // tw = 1 for a real tap, 0 for the padding rows past k
              const uint32_t in = (static_cast<unsigned>(iy0 + ty) < hlim ? 1u : 0u) &
                                  (static_cast<unsigned>(ix0 + tz) < static_cast<unsigned>(p.w) ? 1u : 0u) &
                                  static_cast<uint32_t>(tw);
              dst[i] = ldg_if(xp + tx, in);
            }
          }
        }
        // next k-block: 32 positions on, or the first positions of the next image
        if (++c_kbi == p.kb_per_image) {
          c_kbi = 0; ++c_img; c_pos = lane; c_oy = lane_oy0; c_ox = lane_ox0;
        } else {
          c_pos += kBlockK; c_ox += step_x; c_oy += step_y;
          if (c_ox >= p.ow) { c_ox -= p.ow; ++c_oy; }
        }
      };
      // waits for a free stage, writes this warp's rows, hands the stage over
      auto emit = [&](const float (&e)[kWgradMaxRowsPerWarp]) -> bool {
        int okw = 1;
        if (lane == 0) okw = wgrad_wait(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusConvGather) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, okw, 0) == 0) return false;
        // row r = g + 16 i of the B stage: 32 floats, 16-byte chunk c at c ^ (r & 7); this lane's
        // float is chunk lane / 4, word lane % 4
        const uint32_t dst0 = smem_base + stage * stage_bytes + row_off;
#pragma unroll
        for (int grp = 0; grp < kWgradMaxRowsPerWarp / 4; ++grp) {
          if (grp < row_groups) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = grp * 4 + j;
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst0 + i * (kWgradGatherWarps * 128u)), "f"(e[i])
                           : "memory");
            }
          }
        }
        ptx::fence_proxy_async_smem();               // generic writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(full_bar(stage));
        if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        return true;
      };
      issue_loads(na);
      for (long long kb = kb0; kb < kb1; kb += 2) {
        if (kb + 1 < kb1) issue_loads(nb);
        ok = emit(na);
        if (!ok || kb + 1 >= kb1) break;
        if (kb + 2 < kb1) issue_loads(na);
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

// Per tap k = (ci, ki, kj): the offset of that tap from tap (0, 0) of channel 0, its ki and kj, and
// a valid flag; zeros past the end of k (such rows gather zeros and their outputs are not stored).
__global__ void __launch_bounds__(256)
wgrad_ktab_kernel(int4* __restrict__ tab, int entries, int k, int kh, int kw, int h, int w) {
  const int khw = kh * kw;
  for (int e = blockIdx.x * 256 + threadIdx.x; e < entries; e += 256 * gridDim.x) {
    int4 t = make_int4(0, 0, 0, 0);
    if (e < k) {
      const int ci = e / khw;
      const int rk = e - ci * khw;
      const int ki = rk / kw, kj = rk - ki * kw;
      t = make_int4(ci * h * w + ki * w + kj, ki, kj, 1);
    }
    tab[e] = t;
  }
}

// Dynamic shared memory of the weight-gradient kernel: stages, barriers, the gather warps' table slices.
constexpr int kWgradTableBytes = kWgradGatherWarps * kWgradMaxRowsPerWarp * 16;     // 4 KiB
inline size_t wgrad_smem_bytes(int block_n, int num_stages) {
  return conv_smem_bytes(block_n, num_stages) + kWgradTableBytes;
}

}  // namespace fnn
