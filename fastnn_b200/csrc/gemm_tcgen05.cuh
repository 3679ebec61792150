// Persistent, warp-specialised TF32 GEMM for sm_100a.
//
//   C[b] = epilogue( A[b] (m x k) . B[b] (k x n) ),  FP32 in memory, TF32 multiply,
//   FP32 accumulate in tensor memory.
//
// One CTA owns one SM and walks a static list of work units (batch, k-split, tile).
//   warp 0     TMA producer: fills a ring of shared-memory stages (A 128 x 32, B block_n x 32).
//   warp 1     allocates TMEM; one lane issues tcgen05.mma kind::tf32 (M=128, N=block_n, K=8),
//              four per stage, into one of two TMEM accumulators.
//   warps 2-5  epilogue: tcgen05.ld 32 lanes x 32 columns, scale / bias / activation, then
//              either a 128B-swizzled staging tile + TMA store, or predicated global stores.
// The transposed layouts never materialise a transpose: an operand whose contiguous
// dimension is M or N is loaded as 32 x 32 boxes (inner dimension M/N) and handed to the
// tensor core through an MN-major shared-memory descriptor.
//
// Every wait on an mbarrier is bounded: when the budget runs out the waiting role records
// a code in the status word, raises a CTA-wide abort flag and every role falls through to
// the common teardown (which frees TMEM), so a bad launch ends with an error, not a hang.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace fnn {

constexpr int kBlockM = 128;          // rows of C per tile = UMMA M = TMEM lanes
constexpr int kBlockK = 32;           // floats per stage along K = one 128-byte swizzle row
constexpr int kUmmaK = 8;             // K of one tcgen05.mma kind::tf32
constexpr int kMaxBlockN = 256;       // columns of one accumulator
constexpr int kTmemCols = 512;        // two accumulators
constexpr int kNumThreads = 192;      // 6 warps: producer, MMA issuer, four epilogue warps
constexpr int kNumThreadsWide = 320;  // the same with eight epilogue warps (single-CTA kernel)
constexpr int kEpilogueWarp0 = 2;
constexpr int kStageABytes = kBlockM * kBlockK * 4;            // 16 KiB
constexpr int kChunkBytes = 32 * kBlockK * 4;                  // one 32 x 32 MN-major box, 4 KiB
constexpr int kStagingBytesPerWarp = 2 * 32 * 32 * 4;          // two 32 x 32 output tiles
constexpr int kStagingBytes = 4 * kStagingBytesPerWarp;        // 32 KiB
constexpr int kMaxStages = 8;
constexpr int kGroupM = 16;           // tile rows per rasterisation group
constexpr int kBarrierBytes = 256;

// status codes written by a role whose wait ran out
enum : unsigned int {
  kStatusOk = 0,
  kStatusProducerTimeout = 0x101,
  kStatusMmaTimeout = 0x102,
  kStatusEpilogueTimeout = 0x103,
  kStatusMmaTmemTimeout = 0x104,
  kStatusSelfTest = 0x1F0,          // bounded_wait_selftest_kernel: the wait gave up, as it must
};

// 1, 2: forward activations.  3, 4: the output is multiplied by the activation's derivative at
// aux[row, col] (the saved pre-activation), as FastNN's ReluBackward / GeluBackward do
// (src/autograd/backward_ops.rs:136-160, 194-218; cuda/kernels.cu:244-252).
enum : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActReluGrad = 3, kActGeluGrad = 4 };

struct GemmParams {
  int m, n, k, batch;
  int block_n;         // 32..256, multiple of 32
  int num_stages;
  int tiles_m, tiles_n;
  int num_kb;          // 32-deep k-blocks in all: ceil(k / 32), or that of both operand pairs
  int num_kb1;         // k-blocks read through the first pair of tensor maps (= num_kb normally)
  int split_k;         // >= 1
  int kb_per_split;
  int cluster_k;       // 1: the split_k CTAs of a tile form a thread-block cluster and add their
                       // partial tiles through distributed shared memory (gemm_tf32_clusterk_kernel)
  int cluster_vec;     // that kernel may store float4s: n, ldc, batch stride multiples of 4, C aligned
  int tmem_cols;       // that kernel's TMEM allocation: one accumulator, a power of two >= block_n
  int n_peers;         // gather kernels: every finished tile is also stored through this many extra
                       // tensor maps (the same rows of C in other GPUs' memory); 0 elsewhere
  float* mc_c;         // gather kernels, instead of the tensor maps: the NVLink multicast address of
                       // C (same ldc and batch stride as c); every finished tile is written ONCE, with
                       // multimem.st, and the switch delivers it to every GPU's C, this one's included
  int pace_gather;     // gather kernels: spread each tile's stores over this many eighths of the time its
                       // main loop took (0: send every tile at once)
  int kb_per_stage;    // 32-deep k-blocks per pipeline stage (CTA-pair kernel only; else 1)
  int mma_groups;      // CTA-pair kernel: MMA groups (and issuing threads) per stage: 1 or 2
  int total_units;     // batch * tiles_m * tiles_n * split_k
  int a_mn_major;      // A stored [k, m]
  int b_mn_major;      // B stored [k, n]
  int a_chunked;       // MN-major A through a 4-D map (32, k, m/32, batch): one box per stage
  int b_chunked;       // same for B; needs the M (N) extent to be a multiple of 32
  int store_mode;      // 0: TMA store through tmC, 1: predicated global stores
  int group_m;         // tile rows per rasterisation group (>= 1)
  int l2_a, l2_b;      // L2 eviction policy of the A / B loads (kinds of ptx::make_l2_policy)
  int l2_c;            // and of the TMA stores of C
  float alpha, beta;
  const float* bias;   // [n] or null (ignored when split_k > 1: applied by the reduce pass)
  const float* bias2;  // a second [n] vector added with it, or null (tensor-core kernels only)
  int act;
  const float* aux;    // [m, n] pre-activations for act 3 / 4, row stride ld_aux
  long long ld_aux;
  float* colsum;       // null, or [ceil(m/32)][n] partial column sums of the output, one row per
                       // 32-row slab (added up in slab order by a second kernel)
  float* c;            // direct-store target
  long long ldc, c_batch_stride;   // elements
  unsigned int* status;
  long long spin_budget;           // clock64 ticks a single wait may last
};

// Extra destinations of a gather launch: tensor maps over the rows this GPU computes, as they lie
// in the full C of up to seven other GPUs (peer-mapped memory).  Stores only -- nothing is ever
// loaded through these maps.
constexpr int kMaxPeers = 7;
struct PeerMaps {
  CUtensorMap m[kMaxPeers];
};

struct Unit {
  int b, s, mt, nt;
};

__device__ __forceinline__ Unit decode_unit(const GemmParams& p, int u) {
  Unit w;
  w.s = u % p.split_k;
  int t = u / p.split_k;
  const int tiles = p.tiles_m * p.tiles_n;
  w.b = t / tiles;
  t -= w.b * tiles;
  const int group_sz = p.group_m * p.tiles_n;
  const int g = t / group_sz;
  const int first_m = g * p.group_m;
  const int gm = min(p.tiles_m - first_m, p.group_m);
  const int r = t - g * group_sz;
  w.mt = first_m + r % gm;
  w.nt = r / gm;
  return w;
}

// 0.5 x (1 + erf(x / sqrt 2)) with the library erff, the form FastNN's CPU path (libm erff,
// src/tensor/ops.rs:220-230) and its CUDA kernel (cuda/kernels.cu:236-242) both evaluate; every
// epilogue of this library -- by-column, split-K reduce, cluster reduce -- goes through here.
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.7071067811865475f));
}

__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == kActRelu) return fmaxf(x, 0.0f);
  if (act == kActGelu) return gelu_erf(x);
  return x;
}

// d act / dx at the saved pre-activation x: 1 or 0 for ReLU; Phi(x) + x phi(x) for erf-GELU, term
// by term as FastNN's kernel_gelu_backward (cuda/kernels.cu:244-252).
__device__ __forceinline__ float apply_act_grad(float x, int act) {
  if (act == kActReluGrad) return x > 0.0f ? 1.0f : 0.0f;
  const float cdf = 0.5f * (1.0f + erff(x * 0.7071067811865475f));
  const float pdf = __expf(-0.5f * x * x) * 0.3989422804014327f;
  return cdf + x * pdf;
}

// Bounded wait.  Returns false when the CTA is aborting (this role's budget ran out, or
// another role's did).
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             const GemmParams& p, unsigned int code) {
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

// Before a staging tile is overwritten: all but the newest nbuf - 1 stores of this thread have
// read their source (nbuf = staging tiles the warp cycles through: 1 or 2).
__device__ __forceinline__ void staging_wait(int nbuf) {
  if (nbuf == 2) ptx::tma_store_wait_read<1>();
  else ptx::tma_store_wait_read<0>();
}

// A finished 32 x 32 staging tile (128B-swizzled, 16-byte chunk j of row r at chunk j ^ (r & 7)) sent
// once through the multicast address of C: every lane reads 16 bytes back, eight lanes cover one
// 128-byte row segment, four rows per step.  n is a multiple of 4 (checked on the host).
__device__ __forceinline__ void multicast_store_tile(const GemmParams& p, const uint8_t* tile, int m0,
                                                     int col0, int cz, int lane) {
  float* base = p.mc_c + static_cast<long long>(cz) * p.c_batch_stride;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = it * 32 + lane;
    const int r = idx >> 3, c = idx & 7;
    const float4 v = *reinterpret_cast<const float4*>(tile + r * 128 + ((c ^ (r & 7)) << 4));
    const int grow = m0 + r, gcol = col0 + c * 4;
    if (grow < p.m && gcol < p.n)
      ptx::multimem_st_f4(base + static_cast<long long>(grow) * p.ldc + gcol, v);
  }
}

// Pacing of a gather epilogue: chunk i of a tile is not started before t0 + i * step (SM clock
// ticks).  All CTAs finish their tiles at about the same time; sent at once, the peer tiles of a
// whole wave fill the queues towards NVLink, and the operand loads of the next tile wait behind
// them.  Spread over most of the next tile's main loop they never queue.  step = 0: no pacing.
struct Pace {
  long long t0 = 0, step = 0;
};
__device__ __forceinline__ void pace_chunk(const Pace& pace, int i, int lane) {
  if (pace.step > 0) {
    if (lane == 0) {
      const long long due = pace.t0 + static_cast<long long>(i) * pace.step;
      while (clock64() < due) __nanosleep(128);
    }
    __syncwarp();
  }
}

// Drains one accumulator tile (this warp's 32 TMEM lanes x block_n columns) when nothing but
// alpha / beta applies: a swizzled staging tile + TMA store, or predicated global stores.
// m0 is the first output row of this warp, n0 the first column of the tile, cz the outer
// (batch or batch*split) coordinate, cb the batch index used for the beta read.  The warp takes
// the 32-column chunks c_first, c_first + c_step, ... of the tile and owns nbuf (1 or 2) staging
// tiles of 4 KiB.
__device__ __forceinline__ void epilogue_drain_plain(const GemmParams& p, const CUtensorMap* tmC,
                                                     uint32_t taddr0, uint32_t staging,
                                                     uint8_t* staging_gen, int& buf, int m0, int n0,
                                                     int cz, int cb, bool raw, int lane, int c_first,
                                                     int c_step, int nbuf,
                                                     const CUtensorMap* peers, int n_peers,
                                                     const Pace& pace) {
  const int row = m0 + lane;
  int ci = 0;
  for (int c = c_first; c < p.block_n / 32; c += c_step) {
    const int col0 = n0 + c * 32;
    if (col0 >= p.n) break;                      // warp-uniform
    pace_chunk(pace, ci++, lane);
    uint32_t r[32];
    ptx::tmem_ld_32x32(taddr0 + c * 32, r);
    ptx::tmem_ld_wait();
    if (m0 >= p.m) continue;                     // warp-uniform: rows all out of range
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (!raw) {
      if (p.alpha != 1.0f) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
      }
      if (p.beta != 0.0f && row < p.m) {         // only reachable in direct-store mode
        const float* crow = p.c + cb * p.c_batch_stride + static_cast<long long>(row) * p.ldc;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.n) v[j] += p.beta * crow[col0 + j];
      }
    }
    if (p.store_mode == 0) {
      // staging tile: 32 rows x 128 B, 16-byte chunk j of row r at chunk (j ^ (r & 7))
      if (lane == 0) staging_wait(nbuf);             // the tile about to be overwritten is read
      __syncwarp();
      uint8_t* dst_row = staging_gen + buf * 4096 + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 f = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        *reinterpret_cast<float4*>(dst_row + ((j ^ (lane & 7)) << 4)) = f;
      }
      if (p.mc_c != nullptr) {                      // warp-uniform
        __syncwarp();                               // the tile is complete before any lane reads it back
        multicast_store_tile(p, staging_gen + buf * 4096, m0, col0, cz, lane);
        __syncwarp();                               // and read by every lane before it is overwritten
      } else {
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (p.l2_c != 0) ptx::tma_store_3d_hint(tmC, staging + buf * 4096, col0, m0, cz,
                                                   ptx::make_l2_policy(p.l2_c));
          else ptx::tma_store_3d(tmC, staging + buf * 4096, col0, m0, cz);
          // gather launches: the same tile into the same rows of C on every other GPU, one bulk
          // group with the local store, so the staging tile is free once all of them have read it
          for (int i = 0; i < n_peers; ++i) ptx::tma_store_3d(peers + i, staging + buf * 4096, col0, m0, cz);
          ptx::tma_store_commit();
        }
      }
      buf = (buf + 1) & (nbuf - 1);
    } else if (row < p.m) {
      float* crow = p.c + static_cast<long long>(cz) * p.c_batch_stride +
                    static_cast<long long>(row) * p.ldc;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.n) crow[col0 + j] = v[j];
    }
  }
}

// The same with bias, activation, the backward derivative at aux and the column sums, which run
// as a second, column-wise pass over the staging tile: lane j then owns column j of all 32 rows,
// so the bias is one register, the aux reads (L2-prefetched at the start of the tile) and any
// direct stores are coalesced, and the column sum is a register.  A loop of its own, apart from
// the plain one: as branches inside one shared loop its code sat between the hot instructions of
// the plain path and slowed every GEMM that skipped it by 5-18 %.
__device__ __forceinline__ void epilogue_drain_by_column(const GemmParams& p, const CUtensorMap* tmC,
                                                      uint32_t taddr0, uint32_t staging,
                                                      uint8_t* staging_gen, int& buf, int m0, int n0,
                                                      int cz, int cb, bool raw, int lane,
                                                      int c_first, int c_step, int nbuf,
                                                      const CUtensorMap* peers, int n_peers,
                                                      const Pace& pace) {
  const int row = m0 + lane;
  const bool grad = !raw && (p.act == kActReluGrad || p.act == kActGeluGrad);
  const bool want_colsum = p.colsum != nullptr && !raw;
  const bool by_column = !raw && (p.bias != nullptr || p.act != kActNone || p.colsum != nullptr);
  const int nchunks = p.block_n / 32;
  // aux[m0 + r][first column of chunk c + lane], r = 0..31: one coalesced row segment per load
  auto load_aux = [&](int c, float (&dst)[32]) {
    const int col = n0 + c * 32 + lane;
    const float* acol = p.aux + static_cast<long long>(m0) * p.ld_aux + col;
    if (m0 + 32 <= p.m) {                        // whole slab: 32 back-to-back loads
      if (col < p.n) {
#pragma unroll
        for (int r = 0; r < 32; ++r) dst[r] = __ldg(acol + r * p.ld_aux);
      } else {
#pragma unroll
        for (int r = 0; r < 32; ++r) dst[r] = 0.0f;
      }
    } else {
#pragma unroll
      for (int r = 0; r < 32; ++r)
        dst[r] = (col < p.n && m0 + r < p.m) ? __ldg(acol + r * p.ld_aux) : 0.0f;
    }
  };
  int ci = 0;
  for (int c = c_first; c < nchunks; c += c_step) {
    const int col0 = n0 + c * 32;
    if (col0 >= p.n) break;                      // warp-uniform
    pace_chunk(pace, ci++, lane);
    const bool col_ok = col0 + lane < p.n;
    // aux of this chunk: the lines were prefetched into L2 when the tile's main loop started, and
    // these loads have the TMEM read and the row-wise staging write to complete under
    float x[32];
    if (grad && m0 < p.m) load_aux(c, x);
    float bias_col = (p.bias != nullptr && col_ok) ? __ldg(p.bias + col0 + lane) : 0.0f;
    if (p.bias2 != nullptr && col_ok) bias_col += __ldg(p.bias2 + col0 + lane);
    uint32_t r[32];
    ptx::tmem_ld_32x32(taddr0 + c * 32, r);
    ptx::tmem_ld_wait();
    if (m0 >= p.m) continue;                     // warp-uniform: rows all out of range
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (!raw) {
      if (p.alpha != 1.0f) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
      }
      if (p.beta != 0.0f && row < p.m) {         // only reachable in direct-store mode
        const float* crow = p.c + cb * p.c_batch_stride + static_cast<long long>(row) * p.ldc;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.n) v[j] += p.beta * crow[col0 + j];
      }
    }
    if (p.store_mode == 0 || by_column) {
      // staging tile: 32 rows x 128 B, 16-byte chunk j of row r at chunk (j ^ (r & 7))
      if (lane == 0) staging_wait(nbuf);             // the tile about to be overwritten is read
      __syncwarp();
      uint8_t* tile = staging_gen + buf * 4096;
      uint8_t* dst_row = tile + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 f = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        *reinterpret_cast<float4*>(dst_row + ((j ^ (lane & 7)) << 4)) = f;
      }
      float colsum = 0.0f;
      if (by_column) {
        // Second pass: lane j owns column j of the tile (no bank conflicts: the swizzle spreads
        // one row's columns over all banks).  Bias is then one register, the derivative's
        // operand a coalesced load, the column sum a register, direct stores coalesced.  All
        // loads, then arithmetic, then all stores, so that nothing serialises on aliasing.
        __syncwarp();
        float t[32];
#pragma unroll
        for (int rr = 0; rr < 32; ++rr)
          t[rr] = *reinterpret_cast<const float*>(tile + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) +
                                                  ((lane & 3) << 2));
        // One dense unrolled loop per kind of work, chosen outside the loops: a per-element
        // choice inside one unrolled loop scatters the few executed instructions over tens of
        // KiB of code and the pass then runs at instruction-cache-miss speed (measured: 14x).
        if (p.bias != nullptr) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) t[rr] += bias_col;
        }
        if (p.act == kActRelu) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) t[rr] = fmaxf(t[rr], 0.0f);
        } else if (p.act == kActGelu) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) t[rr] = gelu_erf(t[rr]);
        } else if (p.act == kActReluGrad) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) t[rr] = x[rr] > 0.0f ? t[rr] : 0.0f;
        } else if (p.act == kActGeluGrad) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) t[rr] *= apply_act_grad(x[rr], kActGeluGrad);
        }
        if (m0 + 32 > p.m) {                         // rows past the end add nothing to a column
#pragma unroll
          for (int rr = 0; rr < 32; ++rr)
            if (m0 + rr >= p.m) t[rr] = 0.0f;
        }
        if (want_colsum) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) colsum += t[rr];
        }
        if (p.bias != nullptr || p.act != kActNone) {
#pragma unroll
          for (int rr = 0; rr < 32; ++rr)
            *reinterpret_cast<float*>(tile + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) +
                                      ((lane & 3) << 2)) = t[rr];
        }
        if (p.store_mode != 0 && col_ok) {
          float* ccol = p.c + static_cast<long long>(cz) * p.c_batch_stride +
                        static_cast<long long>(m0) * p.ldc + col0 + lane;
#pragma unroll
          for (int rr = 0; rr < 32; ++rr)
            if (m0 + rr < p.m) ccol[rr * p.ldc] = t[rr];
        }
      }
      if (p.store_mode == 0 && p.mc_c != nullptr) {  // warp-uniform
        __syncwarp();
        multicast_store_tile(p, tile, m0, col0, cz, lane);
        __syncwarp();
      } else if (p.store_mode == 0) {
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (p.l2_c != 0) ptx::tma_store_3d_hint(tmC, staging + buf * 4096, col0, m0, cz,
                                                   ptx::make_l2_policy(p.l2_c));
          else ptx::tma_store_3d(tmC, staging + buf * 4096, col0, m0, cz);
          for (int i = 0; i < n_peers; ++i) ptx::tma_store_3d(peers + i, staging + buf * 4096, col0, m0, cz);
          ptx::tma_store_commit();
        }
      }
      // after the store has been issued: a global write ahead of the proxy fence would hold it up
      if (want_colsum && col_ok) p.colsum[static_cast<long long>(m0 >> 5) * p.n + col0 + lane] = colsum;
      buf = (buf + 1) & (nbuf - 1);
    } else if (row < p.m) {
      float* crow = p.c + static_cast<long long>(cz) * p.c_batch_stride +
                    static_cast<long long>(row) * p.ldc;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.n) crow[col0 + j] = v[j];
    }
  }
}

__device__ __forceinline__ void epilogue_drain_tile(const GemmParams& p, const CUtensorMap* tmC,
                                                    uint32_t taddr0, uint32_t staging,
                                                    uint8_t* staging_gen, int& buf, int m0, int n0,
                                                    int cz, int cb, bool raw, int lane,
                                                    int c_first = 0, int c_step = 1, int nbuf = 2,
                                                    const CUtensorMap* peers = nullptr,
                                                    int n_peers = 0, const Pace& pace = Pace()) {
  const bool by_column = !raw && (p.bias != nullptr || p.act != kActNone || p.colsum != nullptr);
  if (by_column)
    epilogue_drain_by_column(p, tmC, taddr0, staging, staging_gen, buf, m0, n0, cz, cb, raw, lane,
                             c_first, c_step, nbuf, peers, n_peers, pace);
  else
    epilogue_drain_plain(p, tmC, taddr0, staging, staging_gen, buf, m0, n0, cz, cb, raw, lane,
                         c_first, c_step, nbuf, peers, n_peers, pace);
}

// Pitch in bytes of one row of the partial tile a cluster split-K CTA leaves in shared memory:
// four floats of padding keep both the row-per-lane writes and the row-wise reads conflict-free.
__host__ __device__ constexpr uint32_t cluster_partial_pitch(int block_n) {
  return static_cast<uint32_t>(block_n + 4) * 4u;
}

// kClusterK = false: the persistent kernel described at the top of this file.
// kClusterK = true: one work unit per CTA, launched with cluster dimension split_k.  The CTAs
// of a cluster hold the K slices of one output tile; each leaves its accumulator in its own
// shared memory, and after a cluster barrier CTA r adds rows [r, r+1) * 128 / split_k of all
// slices in ascending slice order (deterministic) over distributed shared memory, applies
// alpha / beta / bias / activation and writes C.  No workspace, no second kernel.
// kGather = true (persistent form only): every finished tile is also stored through the
// p.n_peers tensor maps of `peers`, i.e. into the same rows of C on the other GPUs.
template <bool kClusterK, bool kGather = false>
__device__ __forceinline__ void gemm_tf32_body(const CUtensorMap& tmA, const CUtensorMap& tmB,
                                               const CUtensorMap& tmC, const CUtensorMap& tmA2,
                                               const CUtensorMap& tmB2, const GemmParams& p,
                                               const CUtensorMap* peers = nullptr) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle pattern repeats every 8 rows x 128 B.
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_epi_warps = static_cast<int>(blockDim.x >> 5) - kEpilogueWarp0;     // 4 or 8
  const uint32_t stage_b_bytes = static_cast<uint32_t>(p.block_n) * kBlockK * 4;
  const uint32_t stage_bytes = kStageABytes + stage_b_bytes;
  const uint32_t staging_base = smem_base + p.num_stages * stage_bytes;
  const uint32_t staging_total = kClusterK ? 0u : static_cast<uint32_t>(kStagingBytes);   // none there
  const uint32_t bar_base = staging_base + staging_total;
  // barrier layout: full[8] empty[8] tmem_full[2] tmem_empty[2] | tmem address | abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 64u + 8u * s; };
  auto tfull_bar = [&](int a) { return bar_base + 128u + 8u * a; };
  auto tempty_bar = [&](int a) { return bar_base + 144u + 8u * a; };
  const uint32_t tmem_slot = bar_base + 160u;
  uint8_t* bar_gen = smem_gen + (bar_base - smem_base);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(bar_gen + 160);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 168);

  // One pipeline stage of unit w: announce the bytes, then one box per operand (or per 32-wide
  // chunk of an MN-major operand the chunked view does not cover).  Producer thread only.
  auto issue_stage = [&](const Unit& w, int kb, int stage, uint64_t pol_a, uint64_t pol_b) {
    const int m0 = w.mt * kBlockM;
    const int n0 = w.nt * p.block_n;
    const uint32_t sa = smem_base + stage * stage_bytes;
    const uint32_t sb = sa + kStageABytes;
    const uint32_t fb = full_bar(stage);
    ptx::mbar_expect_tx(fb, stage_bytes);
    // k-blocks [0, num_kb1) come from the first operand pair, the rest from the second
    // (C = A1.B1 + A2.B2 in one accumulator); an ordinary GEMM has num_kb1 = num_kb.
    const bool second = kb >= p.num_kb1;
    const CUtensorMap* mA = second ? &tmA2 : &tmA;
    const CUtensorMap* mB = second ? &tmB2 : &tmB;
    const int k0 = (second ? kb - p.num_kb1 : kb) * kBlockK;
    if (!p.a_mn_major) {
      ptx::tma_load_3d_hint(sa, mA, fb, k0, m0, w.b, pol_a);             // 32 x 128 box
    } else if (p.a_chunked) {
      ptx::tma_load_4d_hint(sa, mA, fb, 0, k0, m0 >> 5, w.b, pol_a);     // 32 x 32 x 4 box
    } else {
#pragma unroll
      for (int c = 0; c < kBlockM / 32; ++c)
        ptx::tma_load_3d_hint(sa + c * kChunkBytes, mA, fb, m0 + 32 * c, k0, w.b, pol_a);
    }
    if (!p.b_mn_major) {
      ptx::tma_load_3d_hint(sb, mB, fb, k0, n0, w.b, pol_b);             // 32 x block_n box
    } else if (p.b_chunked) {
      ptx::tma_load_4d_hint(sb, mB, fb, 0, k0, n0 >> 5, w.b, pol_b);     // 32 x 32 x bn/32
    } else {
      for (int c = 0; c < p.block_n / 32; ++c)
        ptx::tma_load_3d_hint(sb + c * kChunkBytes, mB, fb, n0 + 32 * c, k0, w.b, pol_b);
    }
  };

  // k-blocks [kb0, kb1) of unit w.  The cluster form spreads them evenly (every slice non-empty
  // whenever num_kb >= split_k, which the host guarantees).
  auto kb_range = [&](const Unit& w, int& kb0, int& kb1) {
    if constexpr (kClusterK) {
      kb0 = static_cast<int>(static_cast<long long>(w.s) * p.num_kb / p.split_k);
      kb1 = static_cast<int>(static_cast<long long>(w.s + 1) * p.num_kb / p.split_k);
    } else {
      kb0 = w.s * p.kb_per_split;
      kb1 = min(p.num_kb, kb0 + p.kb_per_split);
    }
  };

  int pre_issued = 0;                 // stages of the first unit loaded before the CTA-wide sync
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.num_stages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), n_epi_warps);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    if (p.store_mode == 0) ptx::prefetch_tensormap(&tmC);
    if (p.num_kb1 < p.num_kb) {
      ptx::prefetch_tensormap(&tmA2);
      ptx::prefetch_tensormap(&tmB2);
    }
    if constexpr (kGather) {
      for (int i = 0; i < p.n_peers; ++i) ptx::prefetch_tensormap(peers + i);
    }
    // Everything above touched no global data; from here on the kernels before this one in
    // the stream must be complete (a no-op unless launched as a programmatic dependent).
    ptx::grid_dep_wait();
    // This thread is also the producer: every stage is free, so the first unit's loads start
    // now and their DRAM latency overlaps the TMEM allocation and the sync below.
    if (static_cast<int>(blockIdx.x) < p.total_units) {
      const uint64_t pol_a = ptx::make_l2_policy(p.l2_a);
      const uint64_t pol_b = ptx::make_l2_policy(p.l2_b);
      const Unit w = decode_unit(p, blockIdx.x);
      int kb0, kb1;
      kb_range(w, kb0, kb1);
      pre_issued = min(p.num_stages, kb1 - kb0);
      for (int i = 0; i < pre_issued; ++i) issue_stage(w, kb0 + i, i, pol_a, pol_b);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc_1cta(tmem_slot, kClusterK ? static_cast<uint32_t>(p.tmem_cols) : kTmemCols);
    ptx::tmem_relinquish_1cta();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  // From here the next kernel of the stream (if launched as a programmatic dependent) may place
  // its CTAs on SMs this grid has left, so its set-up overlaps this grid's last tiles.  Issued
  // only now, after this CTA holds its tensor-memory columns: a dependent CTA that became
  // resident beside a CTA still waiting in tcgen05.alloc could take the columns that CTA needs
  // and then sit in griddepcontrol.wait for it -- with the trigger here, every CTA of this grid
  // has its allocation before any dependent can be scheduled.
  ptx::grid_dep_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------- producer ---
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = ptx::make_l2_policy(p.l2_a);
      const uint64_t pol_b = ptx::make_l2_policy(p.l2_b);
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const Unit w = decode_unit(p, u);
        int kb0, kb1;
        kb_range(w, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (pre_issued > 0) {
            --pre_issued;                         // loaded before the sync, into this same stage
          } else {
            ok = wait_barrier(empty_bar(stage), phase ^ 1u, abort_flag, p, kStatusProducerTimeout);
            if (!ok) break;
            issue_stage(w, kb, stage, pol_a, pol_b);
          }
          if (++stage == p.num_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer ---
    // One lane issues.  Descriptors are a per-stage constant plus the stage's address (>> 4),
    // so the loop body is two 64-bit adds per MMA.
    if (lane == 0) {
      const uint32_t idesc = ptx::idesc_tf32(kBlockM, p.block_n, p.a_mn_major, p.b_mn_major);
      // K-major: rows of 128 B swizzled in 16-byte units, 8-row groups 1024 B apart (SBO);
      //          one MMA advances 32 B along K inside the row.
      // MN-major: 32-element chunks, each [32 k-rows][128 B] swizzled in 32-byte units over
      //          4 rows; chunks kChunkBytes apart (LBO), 4-k-row groups 512 B apart (SBO);
      //          one MMA (K = 8) covers two groups and advances 1024 B.
      const uint64_t a_desc0 = ptx::smem_desc_sw128(
          smem_base, p.a_mn_major ? kChunkBytes : 16u, p.a_mn_major ? 512u : 1024u,
          p.a_mn_major ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128);
      const uint64_t b_desc0 = ptx::smem_desc_sw128(
          smem_base + kStageABytes, p.b_mn_major ? kChunkBytes : 16u, p.b_mn_major ? 512u : 1024u,
          p.b_mn_major ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128);
      const uint64_t a_kstep = (p.a_mn_major ? 1024u : kUmmaK * 4u) >> 4;   // in 16-byte units
      const uint64_t b_kstep = (p.b_mn_major ? 1024u : kUmmaK * 4u) >> 4;
      const uint64_t stage_step = stage_bytes >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      uint32_t full_addr = full_bar(0);            // barrier, descriptors of the current stage
      uint64_t da = a_desc0, db = b_desc0;
      uint32_t ready = 0;                          // early probe result for the current stage
      for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
        const Unit w = decode_unit(p, u);
        int kb0, kb1;
        kb_range(w, kb0, kb1);
        ok = wait_barrier(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p, kStatusMmaTmemTimeout);
        if (!ok) break;
        ptx::tc_fence_after_sync();                  // orders the epilogue's TMEM reads before us
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kMaxBlockN);
        uint32_t first = 0u;                          // 0 on the unit's first MMA: overwrite
        for (int kb = kb0; kb < kb1; ++kb) {
          // `ready` is a probe of this stage's barrier issued one iteration earlier, so its
          // latency is hidden behind the previous stage's MMA issue
          if (!ready) {
            ok = wait_barrier(full_addr, phase, abort_flag, p, kStatusMmaTimeout);
            if (!ok) break;
          }
          const uint32_t cur_empty = full_addr + 64u;
          const uint64_t cda = da, cdb = db;
          if (++stage == p.num_stages) {
            stage = 0; phase ^= 1u; full_addr = full_bar(0); da = a_desc0; db = b_desc0;
          } else {
            full_addr += 8u; da += stage_step; db += stage_step;
          }
          ready = ptx::mbar_test_wait(full_addr, phase);          // next stage, non-blocking
          ptx::mma_tf32_1cta(tmem_d, cda, cdb, idesc, first);
          first = 1u;
#pragma unroll
          for (int ks = 1; ks < kBlockK / kUmmaK; ++ks)
            ptx::mma_tf32_1cta(tmem_d, cda + ks * a_kstep, cdb + ks * b_kstep, idesc, 1u);
          ptx::mma_commit_1cta(cur_empty);            // stage reusable once these MMAs retire
        }
        if (!ok) break;
        ptx::mma_commit_1cta(tfull_bar(acc));       // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue ---
    // Four epilogue warps, or eight when the epilogue carries an activation or its derivative
    // (launch with kNumThreadsWide): the two warps of a TMEM lane quadrant then take alternate
    // 32-column chunks of every tile and one staging tile each instead of two.
    ptx::grid_dep_wait();                            // before the first read or write of global data
    const int q = warp & 3;                          // TMEM lane quadrant this warp may read
    const int groups = n_epi_warps >> 2;             // 1 or 2
    const int group = (warp - kEpilogueWarp0) >> 2;
    const uint32_t staging_per_warp = staging_total / static_cast<uint32_t>(n_epi_warps);
    const int nbuf = static_cast<int>(staging_per_warp >> 12);          // 4 KiB tiles: 2, or 1 with eight warps
    const uint32_t staging = staging_base + (warp - kEpilogueWarp0) * staging_per_warp;
    uint8_t* staging_gen = smem_gen + (staging - smem_base);
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    long long t_prev_full = clock64();              // gather pacing: when the previous accumulator was complete
    const bool raw = p.split_k > 1;                 // partial sums: no scale / bias / activation
    if constexpr (kClusterK) {
      // One unit.  The accumulator goes, unscaled, to a row-major partial tile at the start of
      // the stage ring: every stage has been consumed once the accumulator is complete.
      ok = wait_barrier(tfull_bar(0), 0u, abort_flag, p, kStatusEpilogueTimeout);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        ptx::tc_fence_after_sync();
        const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        uint8_t* prow = smem_gen + static_cast<size_t>(q * 32 + lane) * cluster_partial_pitch(p.block_n);
        for (int c = group; c < p.block_n / 32; c += groups) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(taddr0 + c * 32, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(prow + c * 128 + j * 16) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        ptx::tc_fence_before_sync();
      }
    } else
    for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
      const Unit w = decode_unit(p, u);
      const int m0 = w.mt * kBlockM + q * 32;
      const int n0 = w.nt * p.block_n;
      if (p.aux != nullptr && !raw && m0 + lane < p.m) {
        // the derivative's operand for this tile: into L2 while the main loop runs
        const float* arow = p.aux + static_cast<long long>(m0 + lane) * p.ld_aux + n0;
        for (int c = group; c < p.block_n / 32 && n0 + c * 32 < p.n; c += groups)
          ptx::prefetch_l2(arow + c * 32);
      }
      ok = wait_barrier(tfull_bar(acc), acc_phase, abort_flag, p, kStatusEpilogueTimeout);
      ok = __all_sync(0xffffffffu, ok);              // keep the warp converged for tcgen05.ld
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * kMaxBlockN);
      const int cz = raw ? (w.b * p.split_k + w.s) : w.b;   // outer coordinate of the store
      Pace pace;
      if constexpr (kGather) {
        // every tile of every wave but the grid's last is drained over 7/8 of the time the main
        // loop took to produce it (the next wave takes as long, on this SM or on others); the
        // last wave has nothing left to hide behind
        const long long now = clock64();
        if (p.pace_gather && u / static_cast<int>(gridDim.x) < (p.total_units - 1) / static_cast<int>(gridDim.x)) {
          const int my_chunks = (p.block_n / 32 + groups - 1) / groups;
          pace.t0 = now;
          pace.step = (now - t_prev_full) * p.pace_gather / (8 * my_chunks);
        }
        t_prev_full = now;
      }
      epilogue_drain_tile(p, &tmC, taddr0, staging, staging_gen, buf, m0, n0, cz, w.b, raw, lane,
                          group, groups, nbuf, kGather ? peers : nullptr, kGather ? p.n_peers : 0, pace);
      // accumulator drained: hand it back to the MMA warp
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (p.store_mode == 0 && lane == 0) ptx::tma_store_wait_all<0>();
    if (p.mc_c != nullptr) __threadfence_system();   // multicast stores are ordered before the kernel's end
  }

  if constexpr (kClusterK) {
    // ------------------------------------------- cluster reduction + epilogue ---
    // Every thread of every CTA of the cluster passes both barriers, aborting or not, so no CTA
    // waits for one that has left, and none leaves while its shared memory is still being read.
    __syncwarp();
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
    if (warp >= kEpilogueWarp0 && !*abort_flag) {
      const int split = p.split_k;                         // = cluster size: 2, 4, 8 or 16
      const int rank = static_cast<int>(ptx::cluster_ctarank());
      const int rows_per = kBlockM / split;
      const int n4 = p.block_n >> 2;
      const int nthr = n_epi_warps * 32;
      const Unit w = decode_unit(p, blockIdx.x);
      const uint32_t pitch = cluster_partial_pitch(p.block_n);
      float* cbase = p.c + static_cast<long long>(w.b) * p.c_batch_stride;
      for (int idx = static_cast<int>(threadIdx.x) - kEpilogueWarp0 * 32; idx < rows_per * n4; idx += nthr) {
        const int rr = rank * rows_per + idx / n4;
        const int c4 = idx - (idx / n4) * n4;
        const int gr = w.mt * kBlockM + rr;
        const int gc = w.nt * p.block_n + c4 * 4;
        if (gr >= p.m || gc >= p.n) continue;
        const uint32_t local = smem_base + static_cast<uint32_t>(rr) * pitch + static_cast<uint32_t>(c4) * 16u;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < split; ++s) {
          const float4 t = ptx::ld_shared_cluster_f4(ptx::mapa_shared(local, static_cast<uint32_t>(s)));
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        float v[4] = {p.alpha * acc.x, p.alpha * acc.y, p.alpha * acc.z, p.alpha * acc.w};
        float* dst = cbase + static_cast<long long>(gr) * p.ldc + gc;
        if (p.cluster_vec) {
          if (p.beta != 0.0f) {
            const float4 o = *reinterpret_cast<const float4*>(dst);
            v[0] += p.beta * o.x; v[1] += p.beta * o.y; v[2] += p.beta * o.z; v[3] += p.beta * o.w;
          }
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] += __ldg(p.bias + gc + j);
          }
          if (p.bias2 != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] += __ldg(p.bias2 + gc + j);
          }
          *reinterpret_cast<float4*>(dst) = make_float4(apply_act(v[0], p.act), apply_act(v[1], p.act),
                                                        apply_act(v[2], p.act), apply_act(v[3], p.act));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (gc + j >= p.n) break;
            float x = v[j];
            if (p.beta != 0.0f) x += p.beta * dst[j];
            if (p.bias != nullptr) x += __ldg(p.bias + gc + j);
            if (p.bias2 != nullptr) x += __ldg(p.bias2 + gc + j);
            dst[j] = apply_act(x, p.act);
          }
        }
      }
    }
    __syncwarp();
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
  }

  // ---------------------------------------------------------------- teardown ---
  __syncwarp();
  if (*abort_flag) {
    // give loads that are still in flight towards this CTA's shared memory time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_1cta(tmem_base, kClusterK ? static_cast<uint32_t>(p.tmem_cols) : kTmemCols);
  }
}

__global__ void __launch_bounds__(kNumThreadsWide, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ GemmParams p) {
  gemm_tf32_body<false>(tmA, tmB, tmC, tmA2, tmB2, p);
}

__global__ void __launch_bounds__(kNumThreadsWide, 1)
gemm_tf32_clusterk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmA2,
                          const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ GemmParams p) {
  gemm_tf32_body<true>(tmA, tmB, tmC, tmA2, tmB2, p);
}

// The persistent kernel whose epilogue also stores every tile into other GPUs' copies of C (an
// all-gather of C fused into the GEMM: no collective afterwards, only a barrier between ranks).
__global__ void __launch_bounds__(kNumThreadsWide, 1)
gemm_tf32_gather_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, const __grid_constant__ PeerMaps peers,
                        const __grid_constant__ GemmParams p) {
  gemm_tf32_body<false, true>(tmA, tmB, tmC, tmA, tmB, p, peers.m);
}

// One warp, one mbarrier that nothing ever arrives on, and the GEMM kernels' own bounded wait:
// the wait must give up after p.spin_budget clock ticks, leave `code` in the status word and
// return false.  No TMA, no tensor memory, nothing in flight -- the kernel cannot fault or hang.
// out[0] = 1 when the wait returned false (as it must), out[1] = ticks it lasted (low 32 bits).
__global__ void __launch_bounds__(32, 1)
bounded_wait_selftest_kernel(const __grid_constant__ GemmParams p, unsigned int code,
                             unsigned int* out) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ volatile int abort_storage;
  const uint32_t bar = ptx::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    abort_storage = 0;
    ptx::fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool got = wait_barrier(bar, 0u, &abort_storage, p, code);
    const long long dt = clock64() - t0;
    if (out != nullptr) {
      out[0] = got ? 0u : 1u;
      out[1] = static_cast<unsigned int>(dt);
    }
  }
}

// Bytes of dynamic shared memory the cluster split-K kernel needs (no staging tiles).
inline size_t gemm_clusterk_smem_bytes(int block_n, int num_stages) {
  return 1024 + static_cast<size_t>(num_stages) * (kStageABytes + block_n * kBlockK * 4) + kBarrierBytes;
}

// Bytes of dynamic shared memory a launch with these parameters needs.
inline size_t gemm_smem_bytes(int block_n, int num_stages) {
  return 1024 + static_cast<size_t>(num_stages) * (kStageABytes + block_n * kBlockK * 4) +
         kStagingBytes + kBarrierBytes;
}

}  // namespace fnn
