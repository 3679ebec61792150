// Plain-SIMT kernels that sit beside the tensor-core GEMM:
//   * gemm_simt_kernel   -- strided FP32 GEMM for operands that TMA cannot address
//                           (base or leading dimension not 16-byte aligned, k == 0).
//   * splitk_reduce_kernel -- fixed-order sum of split-K partial tiles + the epilogue.
#pragma once
#include <cuda_runtime.h>

#include "gemm_tcgen05.cuh"   // apply_act, activation codes

namespace fnn {

struct SimtParams {
  const float* a;
  const float* b;
  float* c;
  const float* bias;
  int m, n, k, batch;
  long long a_rs, a_cs, a_bs;   // element strides of A(i,p): row, column, batch
  long long b_rs, b_cs, b_bs;   // element strides of B(p,j)
  long long ldc, c_bs;
  float alpha, beta;
  int act;
};

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;

// 256 threads, 64 x 64 tile of C, 4 x 4 outputs per thread, p ascending.
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  __shared__ float As[kSimtK][kSimtTile + 4];
  __shared__ float Bs[kSimtK][kSimtTile + 4];
  const int bz = blockIdx.z;
  const float* a = p.a + bz * p.a_bs;
  const float* b = p.b + bz * p.b_bs;
  float* c = p.c + bz * p.c_bs;
  const int i0 = blockIdx.y * kSimtTile;
  const int j0 = blockIdx.x * kSimtTile;
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int s = 0; s < 4; ++s) acc[r][s] = 0.0f;

  for (int p0 = 0; p0 < p.k; p0 += kSimtK) {
    for (int e = threadIdx.x; e < kSimtTile * kSimtK; e += 256) {
      const int ii = e / kSimtK, pp = e % kSimtK;           // A tile: 64 rows x 16 k
      const int gi = i0 + ii, gp = p0 + pp;
      As[pp][ii] = (gi < p.m && gp < p.k) ? a[gi * p.a_rs + gp * p.a_cs] : 0.0f;
      const int pj = e / kSimtTile, jj = e % kSimtTile;     // B tile: 16 k x 64 cols
      const int gq = p0 + pj, gj = j0 + jj;
      Bs[pj][jj] = (gq < p.k && gj < p.n) ? b[gq * p.b_rs + gj * p.b_cs] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int pp = 0; pp < kSimtK; ++pp) {
      float av[4], bv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) av[r] = As[pp][ty * 4 + r];
#pragma unroll
      for (int s = 0; s < 4; ++s) bv[s] = Bs[pp][tx * 4 + s];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int s = 0; s < 4; ++s) acc[r][s] = fmaf(av[r], bv[s], acc[r][s]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int gi = i0 + ty * 4 + r;
    if (gi >= p.m) continue;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int gj = j0 + tx * 4 + s;
      if (gj >= p.n) continue;
      float v = p.alpha * acc[r][s];
      if (p.beta != 0.0f) v += p.beta * c[gi * p.ldc + gj];
      if (p.bias != nullptr) v += p.bias[gj];
      c[gi * p.ldc + gj] = apply_act(v, p.act);
    }
  }
}

// Workspace layout: [(b * split + s)][m][n] dense.  Partials are added in s-ascending order,
// so the result does not depend on which CTA finished first.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, float* __restrict__ c, const float* __restrict__ bias,
                     int m, int n, int batch, int split, long long ldc, long long c_bs, float alpha,
                     float beta, int act, const float* __restrict__ bias2 = nullptr) {
  ptx::grid_dep_launch_dependents();     // see gemm_tf32_kernel: no-ops for an ordinary launch
  ptx::grid_dep_wait();
  const long long per = static_cast<long long>(m) * n;
  const long long total = per * batch;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const long long b = e / per;
    const long long r = e - b * per;
    const int i = static_cast<int>(r / n);
    const int j = static_cast<int>(r - static_cast<long long>(i) * n);
    const float* src = ws + b * split * per + r;
    float acc = 0.0f;
    for (int s = 0; s < split; ++s) acc += src[s * per];
    float v = alpha * acc;
    float* dst = c + b * c_bs + static_cast<long long>(i) * ldc + j;
    if (beta != 0.0f) v += beta * *dst;
    if (bias != nullptr) v += bias[j];
    if (bias2 != nullptr) v += bias2[j];
    *dst = apply_act(v, act);
  }
}

// float4 form for n % 4 == 0 and 16-byte aligned C rows.
__global__ void __launch_bounds__(256)
splitk_reduce_vec4_kernel(const float4* __restrict__ ws, float* __restrict__ c,
                          const float* __restrict__ bias, int m, int n, int batch, int split,
                          long long ldc, long long c_bs, float alpha, float beta, int act,
                          const float* __restrict__ bias2 = nullptr) {
  ptx::grid_dep_launch_dependents();
  ptx::grid_dep_wait();
  const int n4 = n >> 2;
  const long long per4 = static_cast<long long>(m) * n4;
  const long long total = per4 * batch;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const long long b = e / per4;
    const long long r = e - b * per4;
    const int i = static_cast<int>(r / n4);
    const int j4 = static_cast<int>(r - static_cast<long long>(i) * n4);
    const float4* src = ws + b * split * per4 + r;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < split; ++s) {
      const float4 t = src[s * per4];
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    float4 v = make_float4(alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w);
    float4* dst = reinterpret_cast<float4*>(c + b * c_bs + static_cast<long long>(i) * ldc) + j4;
    if (beta != 0.0f) {
      const float4 o = *dst;
      v.x += beta * o.x; v.y += beta * o.y; v.z += beta * o.z; v.w += beta * o.w;
    }
    if (bias != nullptr) {
      const float4 bb = *reinterpret_cast<const float4*>(bias + 4 * j4);
      v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
    }
    if (bias2 != nullptr) {
      const float4 bb = *reinterpret_cast<const float4*>(bias2 + 4 * j4);
      v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
    }
    v.x = apply_act(v.x, act); v.y = apply_act(v.y, act);
    v.z = apply_act(v.z, act); v.w = apply_act(v.w, act);
    *dst = v;
  }
}

// Backward epilogue for products that went through the SIMT kernel: c *= act'(aux) in place ...
__global__ void __launch_bounds__(256)
act_grad_inplace_kernel(float* __restrict__ c, const float* __restrict__ aux, int m, int n,
                        long long ldc, long long ld_aux, int act) {
  const long long total = static_cast<long long>(m) * n;
  for (long long e = blockIdx.x * 256ll + threadIdx.x; e < total; e += 256ll * gridDim.x) {
    const long long i = e / n;
    const long long j = e - i * n;
    c[i * ldc + j] *= apply_act_grad(aux[i * ld_aux + j], act);
  }
}

// Adds the per-slab partial column sums [slabs][n] written by the GEMM epilogue.  A block owns 32
// columns; thread (ty, tx) adds slabs ty, ty+32, ... of column tx, then the 32 partial sums of a
// column are added in ty order: a fixed summation tree, so the result is reproducible.
__global__ void __launch_bounds__(1024)
colsum_slabs_kernel(const float* __restrict__ partials, float* __restrict__ out, int slabs, int n) {
  __shared__ float part[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.0f;
  if (j < n)
    for (int r = ty; r < slabs; r += 32) s += partials[static_cast<long long>(r) * n + j];
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < n) {
    float t = 0.0f;
#pragma unroll
    for (int r = 0; r < 32; ++r) t += part[r][tx];
    out[j] = t;
  }
}

// ... and its column sums, one thread per column, rows added in order.
__global__ void __launch_bounds__(256)
colsum_kernel(const float* __restrict__ c, float* __restrict__ out, int m, int n, long long ldc) {
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= n) return;
  float s = 0.0f;
  for (int i = 0; i < m; ++i) s += c[static_cast<long long>(i) * ldc + j];
  out[j] = s;
}

}  // namespace fnn
