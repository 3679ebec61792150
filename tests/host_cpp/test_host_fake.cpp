// CPU unit test of the C++ host layer against a fake device: host memory stands in for device
// memory and the GEMM entries are computed with a plain loop.  Exercises what FastNN's
// src/cuda/memory.rs and src/tensor/ops.rs promise: exact-size recycling, at most 32 spares per
// size, dirty recycled buffers, error mapping, shape checks, 2-D / batched dispatch.
#define FASTNN_HOST_NO_LIBRARY
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>

#include "../../fastnn_b200/host/fastnn_host.hpp"

using namespace fastnn::host;

static int g_mallocs = 0, g_frees = 0, g_fail_malloc = 0, g_fail_gemm = 0, g_inits = 0;
static std::set<float*> g_live;

static int f_init(int) { ++g_inits; return 0; }
static int f_count() { return 1; }
static int f_sync() { return 0; }
static void f_mem(size_t* f, size_t* t) { *f = 1; *t = 2; }
static int f_malloc(float** p, size_t bytes) {
  if (g_fail_malloc) return -1;
  *p = static_cast<float*>(std::malloc(bytes ? bytes : 4));
  g_live.insert(*p);
  ++g_mallocs;
  return 0;
}
static int f_free(float* p) { g_live.erase(p); std::free(p); ++g_frees; return 0; }
static int f_copy(float* d, const float* s, size_t n) { std::memcpy(d, s, n); return 0; }
static int f_memset(float* d, int v, size_t n) { std::memset(d, v, n); return 0; }
static void ref_gemm(int layout, const float* a, const float* b, float* c, int m, int n, int k, int batch) {
  for (int z = 0; z < batch; ++z)
    for (int i = 0; i < m; ++i)
      for (int j = 0; j < n; ++j) {
        float s = 0;
        for (int p = 0; p < k; ++p) {
          const float av = layout == 2 ? a[(size_t)z * k * m + (size_t)p * m + i] : a[(size_t)z * m * k + (size_t)i * k + p];
          const float bv = layout == 1 ? b[(size_t)z * n * k + (size_t)j * k + p] : b[(size_t)z * k * n + (size_t)p * n + j];
          s += av * bv;
        }
        c[(size_t)z * m * n + (size_t)i * n + j] = s;
      }
}
static int f_mm(const float* a, const float* b, float* c, int m, int n, int k, int, int, int, float, float) {
  if (g_fail_gemm) return -1;
  ref_gemm(0, a, b, c, m, n, k, 1); return 0;
}
static int f_mmb(const float* a, const float* b, float* c, int m, int n, int k, int bt, float, float) { ref_gemm(0, a, b, c, m, n, k, bt); return 0; }
static int f_nt(const float* a, const float* b, float* c, int m, int n, int k) { ref_gemm(1, a, b, c, m, n, k, 1); return 0; }
static int f_tn(const float* a, const float* b, float* c, int m, int n, int k) { ref_gemm(2, a, b, c, m, n, k, 1); return 0; }
static int f_bnt(const float* a, const float* b, float* c, int m, int n, int k, int bt) { ref_gemm(1, a, b, c, m, n, k, bt); return 0; }
static int f_btn(const float* a, const float* b, float* c, int m, int n, int k, int bt) { ref_gemm(2, a, b, c, m, n, k, bt); return 0; }
static int f_lin(int layout, const float* x, const float* w, const float* bias, float* y, int rows, int in, int out, int act) {
  ref_gemm(layout, x, w, y, rows, out, in, 1);
  for (int i = 0; i < rows; ++i)
    for (int j = 0; j < out; ++j) {
      float v = y[(size_t)i * out + j] + (bias ? bias[j] : 0.f);
      if (act == 1 && v < 0) v = 0;
      y[(size_t)i * out + j] = v;
    }
  return 0;
}

static int failures = 0;
#define CHECK(cond)                                                         \
  do {                                                                      \
    if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++failures; } \
  } while (0)
template <class F> static bool throws_invalid(F f) { try { f(); } catch (const std::invalid_argument&) { return true; } catch (...) {} return false; }
template <class F> static bool throws_cuda(F f) { try { f(); } catch (const CudaError&) { return true; } catch (...) {} return false; }

int main() {
  static const DeviceApi fake = {f_init, f_count, f_sync, f_mem, f_malloc, f_free, f_copy, f_copy, f_copy,
                                 f_memset, f_mm, f_mmb, f_nt, f_tn, f_bnt, f_btn, f_lin};
  bind_api(&fake);
  BufferCache& cache = BufferCache::instance();

  // recycling by exact element count; recycled buffers are handed back dirty
  float* first;
  {
    CudaBuffer b(100);
    first = b.ptr();
    std::vector<float> ones(100, 1.f);
    b.copy_from_host(ones.data(), 100);
  }
  CHECK(g_mallocs == 1 && g_frees == 0 && cache.spare(100) == 1);
  {
    CudaBuffer b(100);
    CHECK(b.ptr() == first && g_mallocs == 1);
    CHECK(b.to_vec()[7] == 1.f);                     // not zeroed
    CudaBuffer other(101);                           // a different size class allocates
    CHECK(other.ptr() != first && g_mallocs == 2);
    CudaBuffer z = CudaBuffer::zeros(100);
    CHECK(z.to_vec()[3] == 0.f);
  }
  // at most 32 spares per size: the 33rd release goes back to the device
  {
    std::vector<CudaBuffer> many;
    for (int i = 0; i < 40; ++i) many.emplace_back(7);
  }
  CHECK(cache.spare(7) == BufferCache::kMaxPerSize);
  CHECK(g_frees == 40 - (int)BufferCache::kMaxPerSize);
  // move semantics do not double-release
  {
    CudaBuffer a(9);
    CudaBuffer b(std::move(a));
    CHECK(a.ptr() == nullptr && b.len() == 9);
    CudaBuffer c = b.clone();
    CHECK(c.ptr() != b.ptr());
  }
  CHECK(cache.spare(9) == 2);
  // allocation failure maps to CudaError, size misuse to invalid_argument
  g_fail_malloc = 1;
  CHECK(throws_cuda([] { CudaBuffer b(123456); }));
  g_fail_malloc = 0;
  CHECK(throws_invalid([] { CudaBuffer b(4); float x[8] = {0}; b.copy_from_host(x, 8); }));

  // context initialises once per device
  CudaContext::ensure(0); CudaContext::ensure(0); CudaContext::ensure(1);
  CHECK(g_inits == 2);
  CHECK(CudaContext::memory_info().second == 2);

  // tensor dispatch: 2-D and batched, three layouts, shapes of the result
  std::vector<float> a(2 * 3 * 4), b(2 * 4 * 5);
  for (size_t i = 0; i < a.size(); ++i) a[i] = float(i % 7) - 3.f;
  for (size_t i = 0; i < b.size(); ++i) b[i] = float(i % 5) - 2.f;
  Tensor A = Tensor::from_vec(a, {2, 3, 4}), B = Tensor::from_vec(b, {2, 4, 5});
  Tensor C = A.matmul(B);
  CHECK((C.shape() == std::vector<size_t>{2, 3, 5}));
  std::vector<float> want(2 * 3 * 5);
  ref_gemm(0, a.data(), b.data(), want.data(), 3, 5, 4, 2);
  CHECK(C.to_vec() == want);
  Tensor A2 = Tensor::from_vec(std::vector<float>(a.begin(), a.begin() + 12), {3, 4});
  Tensor Bt = Tensor::from_vec(std::vector<float>(b.begin(), b.begin() + 20), {5, 4});
  CHECK((A2.matmul_nt(Bt).shape() == std::vector<size_t>{3, 5}));
  Tensor At = Tensor::from_vec(std::vector<float>(a.begin(), a.begin() + 12), {4, 3});
  Tensor B2 = Tensor::from_vec(std::vector<float>(b.begin(), b.begin() + 20), {4, 5});
  CHECK((At.matmul_tn(B2).shape() == std::vector<size_t>{3, 5}));
  CHECK(throws_invalid([&] { A2.matmul(Bt); }));                    // k mismatch
  CHECK(throws_invalid([&] { A.matmul(B2.reshape({1, 4, 5})); }));  // batch mismatch (no broadcast)
  g_fail_gemm = 1;
  CHECK(throws_cuda([&] { A2.matmul(B2); }));
  g_fail_gemm = 0;

  // Linear: one fused call, bias + ReLU, leading dims preserved
  Tensor W = Tensor::from_vec(std::vector<float>(b.begin(), b.begin() + 20), {5, 4});
  Tensor bias = Tensor::from_vec({1, 2, 3, 4, 5}, {5});
  Linear lin(W, bias);
  Tensor Y = lin.forward(A, FASTNN_B200_ACT_RELU);
  CHECK((Y.shape() == std::vector<size_t>{2, 3, 5}));
  for (float v : Y.to_vec()) CHECK(v >= 0.f);
  CHECK(throws_invalid([&] { lin.forward(B2); }));

  cache.trim();
  CHECK(cache.spare(100) == 0);
  std::printf(failures ? "host fake-device tests: %d FAILED\n" : "host fake-device tests: ok\n", failures);
  return failures ? 1 : 0;
}
