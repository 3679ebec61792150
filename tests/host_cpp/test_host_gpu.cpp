// GPU test of the C++ host layer through the real library: Tensor::matmul / matmul_nt /
// matmul_tn (2-D and batched) and Linear::forward(+GELU) against the CPU oracle
// (oracle/fastnn_cpu_oracle.c, linked into this test binary only).
#include <array>
#include <cmath>
#include <cstdio>
#include <random>

#include "../../fastnn_b200/host/fastnn_host.hpp"

extern "C" {
void oracle_matmul_batched(const float*, const float*, float*, size_t, size_t, size_t, size_t, size_t);
int oracle_matmul_nt(const float*, const float*, float*, size_t, size_t, size_t, size_t);
int oracle_matmul_tn(const float*, const float*, float*, size_t, size_t, size_t, size_t);
int oracle_linear(const float*, const float*, const float*, float*, size_t, size_t, size_t, int);
}

using namespace fastnn::host;

static int failures = 0;
// TF32 tolerance: relative Frobenius <= 5e-3, max-abs <= 1e-2 sqrt(K) max|A| max|B|
static void check(const char* what, const std::vector<float>& got, const std::vector<float>& want,
                  size_t k, float amax, float bmax) {
  double num = 0, den = 0, mx = 0;
  for (size_t i = 0; i < want.size(); ++i) {
    const double e = double(got[i]) - double(want[i]);
    num += e * e; den += double(want[i]) * want[i];
    if (std::fabs(e) > mx) mx = std::fabs(e);
  }
  const double rel = std::sqrt(num / (den > 0 ? den : 1));
  const double bound = 1e-2 * std::sqrt(double(k)) * amax * bmax;
  const bool ok = got.size() == want.size() && rel <= 5e-3 && mx <= bound;
  std::printf("%s %-28s rel=%.2e max=%.2e bound=%.2e\n", ok ? "ok  " : "FAIL", what, rel, mx, bound);
  if (!ok) ++failures;
}
static std::vector<float> randn(size_t n, unsigned seed, float* amax) {
  std::mt19937 g(seed);
  std::normal_distribution<float> d(0.f, 1.f);
  std::vector<float> v(n);
  *amax = 0;
  for (auto& x : v) { x = d(g); if (std::fabs(x) > *amax) *amax = std::fabs(x); }
  return v;
}

int main() {
  if (CudaContext::device_count() < 1) { std::printf("no CUDA device\n"); return 2; }
  CudaContext::ensure(0);
  float am, bm;
  {  // 2-D, tensor-core path (aligned) and SIMT path (ragged)
    for (auto dims : {std::array<size_t, 3>{256, 192, 160}, std::array<size_t, 3>{33, 17, 9}}) {
      const size_t m = dims[0], n = dims[1], k = dims[2];
      auto a = randn(m * k, 1, &am), b = randn(k * n, 2, &bm);
      std::vector<float> want(m * n);
      oracle_matmul_batched(a.data(), b.data(), want.data(), m, n, k, 1, 1);
      check("matmul 2-D", Tensor::from_vec(a, {m, k}).matmul(Tensor::from_vec(b, {k, n})).to_vec(), want, k, am, bm);
      auto bt = randn(n * k, 3, &bm);
      oracle_matmul_nt(a.data(), bt.data(), want.data(), m, n, k, 1);
      check("matmul_nt 2-D", Tensor::from_vec(a, {m, k}).matmul_nt(Tensor::from_vec(bt, {n, k})).to_vec(), want, k, am, bm);
      auto at = randn(k * m, 4, &am);
      oracle_matmul_tn(at.data(), b.data(), want.data(), m, n, k, 1);
      check("matmul_tn 2-D", Tensor::from_vec(at, {k, m}).matmul_tn(Tensor::from_vec(b, {k, n})).to_vec(), want, k, am, bm);
    }
  }
  {  // batched attention shapes
    const size_t bh = 16, t = 128, d = 32;
    auto q = randn(bh * t * d, 5, &am), kk = randn(bh * t * d, 6, &bm);
    std::vector<float> want(bh * t * t);
    oracle_matmul_nt(q.data(), kk.data(), want.data(), t, t, d, bh);
    Tensor S = Tensor::from_vec(q, {bh, t, d}).matmul_nt(Tensor::from_vec(kk, {bh, t, d}));
    check("batched Q.K^T", S.to_vec(), want, d, am, bm);
    auto v = randn(bh * t * d, 7, &bm);
    std::vector<float> want2(bh * t * d);
    float sm = 0;
    for (float x : want) if (std::fabs(x) > sm) sm = std::fabs(x);
    oracle_matmul_batched(want.data(), v.data(), want2.data(), t, d, t, bh, bh);
    check("batched S.V", Tensor::from_vec(want, {bh, t, t}).matmul(Tensor::from_vec(v, {bh, t, d})).to_vec(), want2, t, sm, bm);
  }
  {  // Linear + GELU, leading dims kept
    const size_t rows = 96, in = 64, out = 80;
    auto x = randn(rows * in, 8, &am), w = randn(out * in, 9, &bm);
    float tmp;
    auto bias = randn(out, 10, &tmp);
    std::vector<float> want(rows * out);
    oracle_linear(x.data(), w.data(), bias.data(), want.data(), rows, in, out, 2);
    Linear lin(Tensor::from_vec(w, {out, in}), Tensor::from_vec(bias, {out}));
    Tensor y = lin.forward(Tensor::from_vec(x, {4, 24, in}), FASTNN_B200_ACT_GELU);
    if (y.shape() != std::vector<size_t>{4, 24, out}) { std::printf("FAIL linear shape\n"); ++failures; }
    check("Linear+GELU", y.to_vec(), want, in, am, bm);
  }
  {  // buffers are recycled across operations
    BufferCache& c = BufferCache::instance();
    const size_t h0 = c.hits();
    for (int i = 0; i < 4; ++i) {
      auto a = randn(64 * 64, 11, &am);
      Tensor::from_vec(a, {64, 64}).matmul(Tensor::from_vec(a, {64, 64}));
    }
    if (c.hits() <= h0) { std::printf("FAIL cache never hit\n"); ++failures; }
  }
  CudaContext::synchronize();
  unsigned int status = 1;
  if (fastnn_b200_device_status(&status) != 0 || status != 0) { std::printf("FAIL device status %x\n", status); ++failures; }
  std::printf(failures ? "host GPU tests: %d FAILED\n" : "host GPU tests: ok\n", failures);
  return failures ? 1 : 0;
}
