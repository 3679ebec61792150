// Fused attention core for sm_100a:  O = softmax(scale * Q.K^T + causal mask) . V  per head,
// without writing the [heads, Tq, Tk] score matrix to memory.
//
// What FastNN does for this (src/nn/transformer.rs:87-115): batched matmul Q.K^T, mul_scalar,
// additive mask (0 / -1e9 above the diagonal, :22-27), row softmax (src/tensor/ops.rs:273-284),
// batched matmul with V -- five launches and three [heads, Tq, Tk] temporaries.  Here one
// persistent CTA per SM walks (head, 128-query tile) units:
//   warp 0     TMA: Q tile, all keys K and values V of the head into one of two buffer sets
//   warp 1     one lane issues  S = Q.K^T   (tcgen05.mma kind::tf32, M=128, N=Tk padded, TMEM)
//              and later        O = P.V     (A = P from shared memory, B = V MN-major)
//   warps 2-5  one thread per query row: read S from TMEM, scale + mask, row max, exp, row
//              sum; write the unnormalised probabilities P to shared memory in the K-major
//              128B-swizzled layout the second MMA reads; afterwards read O from TMEM,
//              divide by the row sum and store through a swizzled staging tile + TMA store.
// Limits: head_dim a multiple of 32 up to 128, Tk up to 256 (one softmax pass, no rescaling),
// and the working set must fit 227 KiB of shared memory (checked on the host).
// All mbarrier waits are bounded as in the GEMM kernels.
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
  int nsets;                     // Q/K/V buffer sets in shared memory: 2 when they fit, else 1
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
  uint32_t q_bytes, k_bytes, v_bytes, set_bytes, p_bytes, staging_bytes, total;
};
__host__ __device__ inline AttnSmem attn_smem_plan(int d, int tk_pad, int nsets) {
  AttnSmem s;
  const uint32_t kb = static_cast<uint32_t>(d / 32);
  s.q_bytes = kb * 128u * 128u;                              // [d/32][128 rows][128 B]
  s.k_bytes = kb * static_cast<uint32_t>(tk_pad) * 128u;     // [d/32][tk_pad rows][128 B]
  s.v_bytes = kb * static_cast<uint32_t>(tk_pad) * 128u;     // [d/32 chunks][tk_pad rows][128 B]
  s.set_bytes = s.q_bytes + s.k_bytes + s.v_bytes;
  s.p_bytes = static_cast<uint32_t>(tk_pad / 32) * 128u * 128u;   // [tk_pad/32][128 rows][128 B]
  s.staging_bytes = 4u * 2u * 4096u;
  s.total = 1024u + static_cast<uint32_t>(nsets) * s.set_bytes + s.p_bytes + s.staging_bytes + 256u;
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

__global__ void __launch_bounds__(kNumThreads, 1)
attention_tf32_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                      const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const AttnSmem sm = attn_smem_plan(p.d, p.tk_pad, p.nsets);
  const uint32_t p_base = smem_base + static_cast<uint32_t>(p.nsets) * sm.set_bytes;
  const uint32_t staging_base = p_base + sm.p_bytes;
  const uint32_t bar_base = staging_base + sm.staging_bytes;
  // barriers: full[2] @0, empty[2] @16, s_full[2] @32, s_empty[2] @48, p_full @64, p_empty @72,
  //           o_full @80, o_empty @88 | tmem slot @96 | abort @104
  auto full_bar = [&](int b) { return bar_base + 8u * b; };
  auto empty_bar = [&](int b) { return bar_base + 16u + 8u * b; };
  auto s_full = [&](int b) { return bar_base + 32u + 8u * b; };
  auto s_empty = [&](int b) { return bar_base + 48u + 8u * b; };
  const uint32_t p_full = bar_base + 64u, p_empty = bar_base + 72u, o_full = bar_base + 80u,
                 o_empty = bar_base + 88u;
  const uint32_t tmem_slot = bar_base + 96u;
  uint8_t* bar_gen = smem_gen + (bar_base - smem_base);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(bar_gen + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 104);
  // With two operand sets in shared memory and room for two score tiles in TMEM, the scores of
  // unit i+1 are computed while unit i is still in its softmax / second product.
  const bool dbl = (p.nsets == 2) && (2 * p.tk_pad <= 256);

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(full_bar(b), 1); ptx::mbar_init(empty_bar(b), 1);
      ptx::mbar_init(s_full(b), 1);   ptx::mbar_init(s_empty(b), 4);
    }
    ptx::mbar_init(p_full, 4);  ptx::mbar_init(p_empty, 1);
    ptx::mbar_init(o_full, 1);  ptx::mbar_init(o_empty, 4);
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
  // score tiles at columns [0, tk_pad) and, when doubled, [tk_pad, 2 tk_pad); O at [256, 256 + d)
  auto tmem_s = [&](int b) { return tmem_base + static_cast<uint32_t>(b * p.tk_pad); };
  const uint32_t tmem_o = tmem_base + 256u;
  const int kblocks = p.d / 32;

  if (warp == 0) {
    // ------------------------------------------------------------- producer ---
    if (lane == 0) {
      int buf = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const int head = u / p.q_tiles, qt = u - head * p.q_tiles;
        ok = attn_wait(empty_bar(buf), phase ^ 1u, abort_flag, p, kStatusAttnProducer);
        if (!ok) break;
        const uint32_t sq = smem_base + buf * sm.set_bytes;
        const uint32_t sk = sq + sm.q_bytes;
        const uint32_t sv = sk + sm.k_bytes;
        const uint32_t fb = full_bar(buf);
        ptx::mbar_expect_tx(fb, sm.set_bytes);
        for (int kb = 0; kb < kblocks; ++kb) {
          ptx::tma_load_3d(sq + kb * 16384u, &tmQ, fb, kb * 32, qt * 128, head);
          ptx::tma_load_3d(sk + kb * p.tk_pad * 128u, &tmK, fb, kb * 32, 0, head);
          ptx::tma_load_3d(sv + kb * p.tk_pad * 128u, &tmV, fb, kb * 32, 0, head);
        }
        if (++buf == p.nsets) { buf = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer ---
    if (lane == 0) {
      const uint32_t idesc_s = ptx::idesc_tf32(128, p.tk_pad, 0, 0);     // Q, K both K-major
      const uint32_t idesc_o = ptx::idesc_tf32(128, p.d, 0, 1);          // P K-major, V MN-major
      const int n_units = (p.total_units - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                          static_cast<int>(gridDim.x);
      bool ok = true;
      // S(i) = Q.K^T of this CTA's i-th unit into score tile i & 1 (or tile 0 when not doubled)
      auto issue_scores = [&](int i) {
        const int buf = i % p.nsets;
        const uint32_t set_phase = static_cast<uint32_t>(i / p.nsets) & 1u;
        const int sb = dbl ? (i & 1) : 0;
        const uint32_t s_phase = static_cast<uint32_t>(dbl ? (i >> 1) : i) & 1u;
        const uint32_t sq = smem_base + buf * sm.set_bytes;
        const uint32_t sk = sq + sm.q_bytes;
        ok = attn_wait(full_bar(buf), set_phase, abort_flag, p, kStatusAttnMma);
        if (ok) ok = attn_wait(s_empty(sb), s_phase ^ 1u, abort_flag, p, kStatusAttnMma);
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
        ptx::mma_commit_1cta(s_full(sb));
      };
      if (n_units > 0) issue_scores(0);
      int issued = 0;                                          // last unit whose scores are issued
      for (int i = 0; i < n_units && ok; ++i) {
        // Early start of the next unit's scores (they then run under unit i's softmax), but only
        // if its operands have already landed: waiting here would hold back unit i's P.V.
        if (dbl && i + 1 < n_units && issued == i) {
          const int nb = (i + 1) % p.nsets;
          const uint32_t nphase = static_cast<uint32_t>((i + 1) / p.nsets) & 1u;
          if (ptx::mbar_test_wait(full_bar(nb), nphase)) { issue_scores(i + 1); issued = i + 1; }
        }
        if (!ok) break;
        const int buf = i % p.nsets;
        const uint32_t tphase = static_cast<uint32_t>(i) & 1u;
        const uint32_t sv = smem_base + buf * sm.set_bytes + sm.q_bytes + sm.k_bytes;
        // second product once the probabilities are in shared memory
        ok = attn_wait(p_full, tphase, abort_flag, p, kStatusAttnMma);
        if (ok) ok = attn_wait(o_empty, tphase ^ 1u, abort_flag, p, kStatusAttnMma);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        uint32_t acc = 0u;
        for (int ks = 0; ks < p.tk_pad / 8; ++ks) {
          const uint64_t da = ptx::smem_desc_sw128(p_base + (ks >> 2) * 16384u + (ks & 3) * 32u, 16u, 1024u);
          const uint64_t db = ptx::smem_desc_sw128(sv + ks * 1024u, p.tk_pad * 128u, 512u,
                                                   ptx::kLayoutSw128Base32);
          ptx::mma_tf32_1cta(tmem_o, da, db, idesc_o, acc);
          acc = 1u;
        }
        ptx::mma_commit_1cta(o_full);
        ptx::mma_commit_1cta(p_empty);
        ptx::mma_commit_1cta(empty_bar(buf));
        if (i + 1 < n_units && issued == i) { issue_scores(i + 1); issued = i + 1; }
      }
    }
  } else {
    // ------------------------------------------------- softmax + output warps ---
    const int q = warp & 3;
    const uint32_t staging = staging_base + (warp - kEpilogueWarp0) * 8192u;
    uint8_t* staging_gen = smem_gen + (staging - smem_base);
    uint8_t* p_gen = smem_gen + (p_base - smem_base);
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int row_in_tile = q * 32 + lane;
    int sbuf = 0;
    bool ok = true;
    const float sl2 = p.scale * 1.4426950408889634f;            // scale * log2(e)
    const int nchunks = p.tk_pad / 32;
    int i = 0;                                                   // this CTA's unit counter
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x, ++i) {
      const int head = u / p.q_tiles, qt = u - head * p.q_tiles;
      const int qi = qt * 128 + row_in_tile;                     // query index in the sequence
      // keys this row may see: j < tk and (not causal or j <= qi)
      const int jmax = p.causal ? min(p.tk, qi + 1) : p.tk;
      const uint32_t tphase = static_cast<uint32_t>(i) & 1u;
      const int sb = dbl ? (i & 1) : 0;
      const uint32_t s_phase = static_cast<uint32_t>(dbl ? (i >> 1) : i) & 1u;
      const uint32_t ts = tmem_s(sb) + lane_off;
      ok = attn_wait(s_full(sb), s_phase, abort_flag, p, kStatusAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      // One thread owns one query row.  e = 2^(scale*log2e*(s - max)) over the visible keys goes
      // to shared memory unnormalised (K-major, 128B-swizzled: the A operand of P.V); the row
      // sum divides the output instead.  ex2.approx is good to 2^-22, far inside TF32 rounding.
      auto store_p = [&](int c, const float (&e)[32]) {
        uint8_t* dst = p_gen + c * 16384 + row_in_tile * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(dst + ((j ^ (row_in_tile & 7)) << 4)) =
              make_float4(e[4 * j], e[4 * j + 1], e[4 * j + 2], e[4 * j + 3]);
      };
      float sum = 0.0f;
      {
      // pass 1 finds the row maximum, pass 2 re-reads the scores from TMEM for the exponentials
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
      ok = attn_wait(p_empty, tphase ^ 1u, abort_flag, p, kStatusAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      for (int c = 0; c < nchunks; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(ts + c * 32, r);
        ptx::tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float x = ptx::ex2_approx(fmaf(__uint_as_float(r[j]), sl2, -mx2));
          e[j] = (c * 32 + j < jmax) ? x : 0.0f;
          sum += e[j];
        }
        store_p(c, e);
      }
      }
      ptx::tc_fence_before_sync();
      ptx::fence_proxy_async_smem();                 // P visible to the tensor core
      __syncwarp();
      if (lane == 0) { ptx::mbar_arrive(s_empty(sb)); ptx::mbar_arrive(p_full); }
      const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
      // output: O / row sum
      ok = attn_wait(o_full, tphase, abort_flag, p, kStatusAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const int m0 = qt * 128 + q * 32;
      for (int c = 0; c < p.d / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_o + lane_off + c * 32, r);
        ptx::tmem_ld_wait();
        if (m0 >= p.tq) continue;
        if (lane == 0) ptx::tma_store_wait_read<1>();
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
        sbuf ^= 1;
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(o_empty);
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

}  // namespace fnn
