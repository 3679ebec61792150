// Fused attention core for sm_100a:  O = softmax(scale * Q.K^T + causal mask) . V  per head,
// without writing the [heads, Tq, Tk] score matrix to memory.
//
// What FastNN does for this (src/nn/transformer.rs:87-115): batched matmul Q.K^T, mul_scalar,
// additive mask (0 / -1e9 above the diagonal, :22-27), row softmax (src/tensor/ops.rs:273-284),
// batched matmul with V -- five launches and three [heads, Tq, Tk] temporaries.  Here one
// persistent CTA per SM walks (head, 128-query tile) units as a software pipeline:
//   warp 0     TMA: Q tile, all keys K and values V of the head into one of two buffer sets
//   warp 1     one lane issues  S = Q.K^T   (tcgen05.mma kind::tf32, M=128, N=Tk padded) into one
//              of two score tiles in TMEM, and  O = P.V  with the A operand P read FROM TMEM
//              (V is the MN-major B operand in shared memory) into one of two O tiles
//   warps 2-9  two groups of four warps, one thread per query row, taking alternate units: read S
//              from TMEM, scale + mask, row max, exp2, row sum, write the unnormalised
//              probabilities P back over S in TMEM (tcgen05.st); then read O from TMEM, divide
//              by the row sum and store through a swizzled staging tile + TMA store.
// While one group waits for P.V of unit i and writes it out, the other runs the softmax of unit
// i+1 and the tensor core the products on either side.
// Limits: head_dim a multiple of 32 up to 128, Tk up to 256, scale > 0, and the operand sets must
// fit shared memory (checked on the host).  Every mbarrier wait is bounded as in the GEMM kernels.
#pragma once
#include "gemm_tcgen05.cuh"

namespace fnn {

struct AttnParams {
  int heads, tq, tk, d;          // batch*heads, query length, key length, head dim
  int tk_pad;                    // tk rounded up to 32
  int q_tiles;                   // ceil(tq / 128)
  int total_units;               // heads * q_tiles
  float scale;
  int causal;
  int nsets;                     // Q/K/V buffer sets in shared memory, 1..4 as fit and are useful
  const float* mask;             // null, or an additive [tq, tk] mask shared by all heads (added to
                                 // scale * q.k before the softmax, src/nn/transformer.rs:99-105)
  unsigned int* status;
  long long spin_budget;
};

enum : unsigned int {
  kStatusAttnProducer = 0x201,
  kStatusAttnMma = 0x202,
  kStatusAttnSoftmax = 0x203,
};

// shared-memory plan (bytes); every region is 1024-byte aligned
struct AttnSmem {
  uint32_t q_bytes, k_bytes, v_bytes, set_bytes, staging_bufs, staging_bytes, total;
};
constexpr int kAttnSoftmaxWarps = 8;                         // two groups of four
constexpr int kAttnThreads = 64 + 32 * kAttnSoftmaxWarps;
constexpr uint32_t kAttnSmemLimit = 232448u;                 // 227 KiB per CTA
constexpr int kAttnMaxSets = 4;                              // Q/K/V sets in flight per CTA
__host__ __device__ inline AttnSmem attn_smem_plan(int d, int tk_pad, int nsets) {
  AttnSmem s;
  const uint32_t kb = static_cast<uint32_t>(d / 32);
  s.q_bytes = kb * 128u * 128u;                              // [d/32][128 rows][128 B]
  s.k_bytes = kb * static_cast<uint32_t>(tk_pad) * 128u;     // [d/32][tk_pad rows][128 B]
  s.v_bytes = kb * static_cast<uint32_t>(tk_pad) * 128u;     // [d/32 chunks][tk_pad rows][128 B]
  s.set_bytes = s.q_bytes + s.k_bytes + s.v_bytes;
  // one 32x32 output staging tile per softmax warp, two when they fit
  s.staging_bufs = 2u;
  s.staging_bytes = kAttnSoftmaxWarps * s.staging_bufs * 4096u;
  s.total = 1024u + static_cast<uint32_t>(nsets) * s.set_bytes + s.staging_bytes + 256u;
  if (s.total > kAttnSmemLimit) {
    s.staging_bufs = 1u;
    s.staging_bytes = kAttnSoftmaxWarps * 4096u;
    s.total = 1024u + static_cast<uint32_t>(nsets) * s.set_bytes + s.staging_bytes + 256u;
  }
  return s;
}

__device__ __forceinline__ bool attn_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          const AttnParams& p, unsigned int code) {
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

__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tf32_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                      const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const AttnSmem sm = attn_smem_plan(p.d, p.tk_pad, p.nsets);
  const uint32_t staging_base = smem_base + static_cast<uint32_t>(p.nsets) * sm.set_bytes;
  const uint32_t bar_base = staging_base + sm.staging_bytes;
  // barriers (8 bytes each): full[4] @0, empty[4] @32, s_full[2] @64, p_full[2] @80,
  //                          o_full[2] @96, o_free[2] @112 | tmem slot @128 | abort @136
  auto full_bar = [&](int b) { return bar_base + 8u * b; };
  auto empty_bar = [&](int b) { return bar_base + 32u + 8u * b; };
  auto s_full = [&](int b) { return bar_base + 64u + 8u * b; };
  auto p_full = [&](int b) { return bar_base + 80u + 8u * b; };
  auto o_full = [&](int b) { return bar_base + 96u + 8u * b; };
  auto o_free = [&](int b) { return bar_base + 112u + 8u * b; };
  const uint32_t tmem_slot = bar_base + 128u;
  uint8_t* bar_gen = smem_gen + (bar_base - smem_base);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(bar_gen + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 136);
  // Two score tiles when they fit beside the two output tiles in TMEM and two operand sets fit in
  // shared memory; otherwise one score tile and the two products of a unit run back to back.
  const bool dbl = (p.nsets >= 2) && (2 * p.tk_pad <= 256);

  if (threadIdx.x == 0) {
    for (int b = 0; b < kAttnMaxSets; ++b) {
      ptx::mbar_init(full_bar(b), 1); ptx::mbar_init(empty_bar(b), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(s_full(b), 1);   ptx::mbar_init(p_full(b), 4);
      ptx::mbar_init(o_full(b), 1);   ptx::mbar_init(o_free(b), 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmQ); ptx::prefetch_tensormap(&tmK);
    ptx::prefetch_tensormap(&tmV); ptx::prefetch_tensormap(&tmO);
  }
  if (warp == 1) {
    ptx::tmem_alloc_1cta(tmem_slot, kTmemCols);
    ptx::tmem_relinquish_1cta();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  // the next kernel of the stream may set itself up on SMs this grid has left -- only now that
  // this CTA holds its tensor-memory columns (a dependent may not take them first)
  ptx::grid_dep_launch_dependents();
  // score / probability tiles at columns [0, tk_pad) and [tk_pad, 2 tk_pad); O tiles at 256 + b*d
  auto tmem_s = [&](int b) { return tmem_base + static_cast<uint32_t>(b * p.tk_pad); };
  auto tmem_o = [&](int b) { return tmem_base + 256u + static_cast<uint32_t>(b * p.d); };
  const int kblocks = p.d / 32;
  const int n_units = (p.total_units - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                      static_cast<int>(gridDim.x);
  // Where this CTA's i-th unit lives.  The s_full / p_full / o_full / o_free barriers and the O
  // tile are indexed by i & 1 with phase (i >> 1) & 1, so that each softmax group waits only on
  // its own barriers and is never more than one phase behind them.  Nothing guards the reuse of a
  // score tile by a later Q.K^T: the tensor core runs one thread's MMAs in issue order, so that
  // product follows the P.V that read the tile.
  auto tile_of = [&](int i) { return dbl ? (i & 1) : 0; };
  auto set_of = [&](int i) { return i % p.nsets; };
  auto set_phase = [&](int i) { return static_cast<uint32_t>(i / p.nsets) & 1u; };
  auto out_phase = [&](int i) { return static_cast<uint32_t>(i >> 1) & 1u; };

  if (warp == 0) {
    // ------------------------------------------------------------- producer ---
    if (lane == 0) {
      ptx::grid_dep_wait();          // earlier kernels of the stream are complete from here on
      // Q is read once; K and V are read once per query tile of the head
      const uint64_t pol_q = ptx::make_l2_policy(1);
      const uint64_t pol_kv = ptx::make_l2_policy(p.q_tiles > 1 ? 3 : 1);
      for (int i = 0; i < n_units; ++i) {
        const int u = blockIdx.x + i * gridDim.x;
        const int head = u / p.q_tiles, qt = u - head * p.q_tiles;
        const int buf = set_of(i);
        if (!attn_wait(empty_bar(buf), set_phase(i) ^ 1u, abort_flag, p, kStatusAttnProducer)) break;
        const uint32_t sq = smem_base + buf * sm.set_bytes;
        const uint32_t sk = sq + sm.q_bytes;
        const uint32_t sv = sk + sm.k_bytes;
        const uint32_t fb = full_bar(buf);
        ptx::mbar_expect_tx(fb, sm.set_bytes);
        for (int kb = 0; kb < kblocks; ++kb) {
          ptx::tma_load_3d_hint(sq + kb * 16384u, &tmQ, fb, kb * 32, qt * 128, head, pol_q);
          ptx::tma_load_3d_hint(sk + kb * p.tk_pad * 128u, &tmK, fb, kb * 32, 0, head, pol_kv);
          ptx::tma_load_3d_hint(sv + kb * p.tk_pad * 128u, &tmV, fb, kb * 32, 0, head, pol_kv);
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer ---
    if (lane == 0) {
      const uint32_t idesc_s = ptx::idesc_tf32(128, p.tk_pad, 0, 0);     // Q, K both K-major
      const uint32_t idesc_o = ptx::idesc_tf32(128, p.d, 0, 1);          // P from TMEM, V MN-major
      bool ok = true;
      // S(i) = Q.K^T of this CTA's i-th unit into its score tile
      auto issue_scores = [&](int i) {
        const int buf = set_of(i), sb = tile_of(i);
        const uint32_t sq = smem_base + buf * sm.set_bytes;
        const uint32_t sk = sq + sm.q_bytes;
        ok = attn_wait(full_bar(buf), set_phase(i), abort_flag, p, kStatusAttnMma);
        if (!ok) return;
        ptx::tc_fence_after_sync();
        uint32_t acc = 0u;
        for (int kb = 0; kb < kblocks; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t da = ptx::smem_desc_sw128(sq + kb * 16384u + ks * 32u, 16u, 1024u);
            const uint64_t db = ptx::smem_desc_sw128(sk + kb * p.tk_pad * 128u + ks * 32u, 16u, 1024u);
            ptx::mma_tf32_1cta(tmem_s(sb), da, db, idesc_s, acc);
            acc = 1u;
          }
        ptx::mma_commit_1cta(s_full(i & 1));
      };
      if (n_units > 0) issue_scores(0);
      int issued = 0;                                          // last unit whose scores are issued
      for (int i = 0; i < n_units && ok; ++i) {
        // Early start of the next unit's scores into the other tile, but only if its operands
        // have already landed: blocking here would hold back unit i's second product.
        if (dbl && i + 1 < n_units && issued == i &&
            ptx::mbar_test_wait(full_bar(set_of(i + 1)), set_phase(i + 1))) {
          issue_scores(i + 1);
          issued = i + 1;
        }
        if (!ok) break;
        const int buf = set_of(i), sb = tile_of(i), ob = i & 1;
        const uint32_t sv = smem_base + buf * sm.set_bytes + sm.q_bytes + sm.k_bytes;
        // O(i) = P(i) . V once the probabilities are in TMEM and that O tile has been drained
        ok = attn_wait(p_full(ob), out_phase(i), abort_flag, p, kStatusAttnMma);
        if (ok) ok = attn_wait(o_free(ob), out_phase(i) ^ 1u, abort_flag, p, kStatusAttnMma);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        uint32_t acc = 0u;
        for (int ks = 0; ks < p.tk_pad / 8; ++ks) {
          const uint64_t db = ptx::smem_desc_sw128(sv + ks * 1024u, p.tk_pad * 128u, 512u,
                                                   ptx::kLayoutSw128Base32);
          ptx::mma_tf32_1cta_ts(tmem_o(ob), tmem_s(sb) + ks * 8, db, idesc_o, acc);
          acc = 1u;
        }
        ptx::mma_commit_1cta(o_full(ob));
        ptx::mma_commit_1cta(empty_bar(buf));        // the operand set may be refilled
        if (i + 1 < n_units && issued == i) { issue_scores(i + 1); issued = i + 1; }
      }
    }
  } else {
    // ------------------------------------------------- softmax + output warps ---
    ptx::grid_dep_wait();            // before the first store of O
    // Two groups of four warps; group g takes this CTA's units g, g+2, ...  A warp may touch the
    // TMEM lane quarter (warp index mod 4) only, so each group covers all 128 rows.
    const int group = (warp - 2) >> 2;
    const int q = warp & 3;
    const uint32_t nbufs = sm.staging_bufs;
    const uint32_t staging = staging_base + (warp - 2) * nbufs * 4096u;
    uint8_t* staging_gen = smem_gen + (staging - smem_base);
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int row_in_tile = q * 32 + lane;
    const float sl2 = p.scale * 1.4426950408889634f;            // scale * log2(e)
    const int nchunks = p.tk_pad / 32;
    int sbuf = 0;
    bool ok = true;

    // One thread owns one query row.  e = 2^(scale*log2e*(s - max)) over the visible keys
    // replaces the scores in TMEM, unnormalised; the row sum divides the output instead.
    // ex2.approx is good to 2^-22, far inside TF32 rounding.  Returns 1 / row sum.
    auto softmax_unit = [&](int i) -> float {
      const int u = blockIdx.x + i * gridDim.x;
      const int qt = u % p.q_tiles;
      const int qi = qt * 128 + row_in_tile;                     // query index in the sequence
      const int jmax = p.causal ? min(p.tk, qi + 1) : p.tk;      // keys j < jmax are visible
      const int sb = tile_of(i);
      const uint32_t ts = tmem_s(sb) + lane_off;
      ok = attn_wait(s_full(i & 1), out_phase(i), abort_flag, p, kStatusAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return 0.0f;
      ptx::tc_fence_after_sync();
      // pass 1 finds the row maximum, pass 2 re-reads the scores for the exponentials
      float sum = 0.0f;
      // The branch below must be warp-uniform (tcgen05.ld / .st are .sync.aligned: every lane of the
      // warp has to execute the same one), so it depends on the launch alone; lanes whose row lies
      // past the last query read the last query's mask row and their results are never stored.
      const float* mrow = p.mask != nullptr
                              ? p.mask + static_cast<long long>(min(qi, p.tq - 1)) * p.tk : nullptr;
      if (p.mask == nullptr) {
        float mx = -INFINITY;
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(ts + c * 32, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c * 32 + j < jmax) mx = fmaxf(mx, __uint_as_float(r[j]));
        }
        const float mx2 = (jmax > 0) ? mx * sl2 : 0.0f;
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(ts + c * 32, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float x = ptx::ex2_approx(fmaf(__uint_as_float(r[j]), sl2, -mx2));
            const float e = (c * 32 + j < jmax) ? x : 0.0f;
            sum += e;
            r[j] = __float_as_uint(e);
          }
          ptx::tmem_st_32x32(ts + c * 32, r);
        }
      } else {
        // additive mask: logits are scale * s + mask, here in the base-2 domain.  The mask row is
        // read twice (it is small and stays in L1/L2; lanes hold different rows).
        constexpr float kLog2e = 1.4426950408889634f;
        float mx = -INFINITY;
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(ts + c * 32, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c * 32 + j < jmax)
              mx = fmaxf(mx, fmaf(__uint_as_float(r[j]), sl2, __ldg(mrow + c * 32 + j) * kLog2e));
        }
        const float mx2 = (jmax > 0) ? mx : 0.0f;
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(ts + c * 32, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float e = 0.0f;
            if (c * 32 + j < jmax)
              e = ptx::ex2_approx(fmaf(__uint_as_float(r[j]), sl2, __ldg(mrow + c * 32 + j) * kLog2e) - mx2);
            sum += e;
            r[j] = __float_as_uint(e);
          }
          ptx::tmem_st_32x32(ts + c * 32, r);
        }
      }
      ptx::tmem_st_wait();                            // P is in TMEM before the tensor core is told
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(p_full(i & 1));
      return sum > 0.0f ? 1.0f / sum : 0.0f;
    };
    // output of unit i: O / row sum through the staging tile
    auto output_unit = [&](int i, float inv) {
      const int u = blockIdx.x + i * gridDim.x;
      const int head = u / p.q_tiles, qt = u - head * p.q_tiles;
      const int ob = i & 1;
      ok = attn_wait(o_full(ob), out_phase(i), abort_flag, p, kStatusAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      ptx::tc_fence_after_sync();
      const int m0 = qt * 128 + q * 32;
      for (int c = 0; c < p.d / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_o(ob) + lane_off + c * 32, r);
        ptx::tmem_ld_wait();
        if (m0 >= p.tq) continue;
        if (lane == 0) {                      // the staging tile about to be overwritten is read
          if (nbufs == 2) ptx::tma_store_wait_read<1>(); else ptx::tma_store_wait_read<0>();
        }
        __syncwarp();
        uint8_t* dst = staging_gen + sbuf * 4096 + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(dst + ((j ^ (lane & 7)) << 4)) =
              make_float4(__uint_as_float(r[4 * j]) * inv, __uint_as_float(r[4 * j + 1]) * inv,
                          __uint_as_float(r[4 * j + 2]) * inv, __uint_as_float(r[4 * j + 3]) * inv);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_3d(&tmO, staging + sbuf * 4096, c * 32, m0, head);
          ptx::tma_store_commit();
        }
        if (nbufs == 2) sbuf ^= 1;
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(o_free(ob));
    };

    // While this group waits for and writes out O(i), the other group runs the softmax of
    // unit i+1 and the tensor core the products around it.
    for (int i = group; i < n_units && ok; i += 2) {
      const float inv = softmax_unit(i);
      if (!ok) break;
      output_unit(i, inv);
    }
    if (lane == 0) ptx::tma_store_wait_all<0>();
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

// Row softmax of scale-d, masked scores in place, one warp per row of a [rows_total, tk] matrix
// whose rows cycle through tq query positions: x_j = s_j + mask[qi, j] (mask null = none), keys
// j > qi hidden when causal; p_j = exp(x_j - max) / sum, the order of Tensor::softmax
// (src/tensor/ops.rs:273-284).  For the attention shapes the fused kernel does not take.
__global__ void __launch_bounds__(256)
masked_softmax_rows_kernel(float* __restrict__ s, const float* __restrict__ mask, long long rows_total,
                           int tq, int tk, int causal) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp0; row < rows_total; row += nwarps) {
    const int qi = static_cast<int>(row % tq);
    float* x = s + row * tk;
    const float* m = mask != nullptr ? mask + static_cast<long long>(qi) * tk : nullptr;
    const int jmax = causal ? min(tk, qi + 1) : tk;
    float mx = -INFINITY;
    for (int j = lane; j < jmax; j += 32) {
      const float v = x[j] + (m != nullptr ? __ldg(m + j) : 0.0f);
      x[j] = v;
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (int j = lane; j < jmax; j += 32) {
      const float e = expf(x[j] - mx);
      x[j] = e;
      sum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (int j = lane; j < tk; j += 32) x[j] = j < jmax ? x[j] * inv : 0.0f;
  }
}

}  // namespace fnn
