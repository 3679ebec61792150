// C++ host layer above the C ABI: the device-buffer cache, the once-per-device context and the
// tensor-level matmul dispatch that FastNN implements in Rust
//   src/cuda/memory.rs   (CudaBuffer + size-keyed free list, :23-173)
//   src/cuda/context.rs  (CudaContext, :13-54)
//   src/tensor/ops.rs    (Tensor::matmul / matmul_nt / matmul_tn, :341-518)
//   src/nn/linear.rs     (Linear::forward, :55-88)
// with the same observable behaviour: buffers are recycled by exact element count, at most 32
// spare buffers per size, recycled buffers are NOT zeroed, everything runs on the legacy
// default stream, a non-zero status from the C ABI becomes an error, a shape mismatch is a
// programming error.  Header-only; all device access goes through a table of function
// pointers so the logic can be unit-tested on a machine without a GPU.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/fastnn_b200_kernels.h"

namespace fastnn {
namespace host {

// Thrown where FastNN returns Err(String) and the caller `.expect()`s it.
struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// The slice of the C ABI this layer uses.
struct DeviceApi {
  int (*init)(int);
  int (*device_count)();
  int (*synchronize)();
  void (*memory_info)(size_t*, size_t*);
  int (*malloc_)(float**, size_t);
  int (*free_)(float*);
  int (*h2d)(float*, const float*, size_t);
  int (*d2h)(float*, const float*, size_t);
  int (*d2d)(float*, const float*, size_t);
  int (*memset_)(float*, int, size_t);
  int (*matmul)(const float*, const float*, float*, int, int, int, int, int, int, float, float);
  int (*matmul_batched)(const float*, const float*, float*, int, int, int, int, float, float);
  int (*matmul_nt)(const float*, const float*, float*, int, int, int);
  int (*matmul_tn)(const float*, const float*, float*, int, int, int);
  int (*matmul_batched_nt)(const float*, const float*, float*, int, int, int, int);
  int (*matmul_batched_tn)(const float*, const float*, float*, int, int, int, int);
  int (*linear_forward)(int, const float*, const float*, const float*, float*, int, int, int, int);
};

#ifndef FASTNN_HOST_NO_LIBRARY
// The real library (link against libfastnn_b200.so).
inline const DeviceApi& library_api() {
  static const DeviceApi api = {
      fastnn_cuda_init, fastnn_cuda_device_count, fastnn_cuda_synchronize,
      fastnn_cuda_get_memory_info, fastnn_cuda_malloc, fastnn_cuda_free, fastnn_cuda_memcpy_h2d,
      fastnn_cuda_memcpy_d2h, fastnn_cuda_memcpy_d2d, fastnn_cuda_memset, fastnn_cuda_matmul,
      fastnn_cuda_matmul_batched, fastnn_cuda_matmul_nt, fastnn_cuda_matmul_tn,
      fastnn_cuda_matmul_batched_nt, fastnn_cuda_matmul_batched_tn, fastnn_b200_linear_forward};
  return api;
}
#endif

// Process-wide binding of the device functions (set once, before first use).
inline const DeviceApi*& api_slot() {
  static const DeviceApi* slot = nullptr;
  return slot;
}
inline void bind_api(const DeviceApi* api) { api_slot() = api; }
inline const DeviceApi& api() {
  const DeviceApi* a = api_slot();
#ifndef FASTNN_HOST_NO_LIBRARY
  if (a == nullptr) a = &library_api();
#endif
  if (a == nullptr) throw CudaError("no device API bound");
  return *a;
}

// ------------------------------------------------------------------ buffer cache ---
// Free list keyed by exact element count.  Safe to hand a just-released buffer to the next
// operation because every operation is ordered on the same (default) stream.
class BufferCache {
 public:
  static constexpr size_t kMaxPerSize = 32;

  static BufferCache& instance() {
    static BufferCache c;
    return c;
  }
  // A spare buffer of exactly `len` floats, or nullptr.
  float* take(size_t len) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = free_.find(len);
    if (it == free_.end() || it->second.empty()) {
      ++misses_;
      return nullptr;
    }
    float* p = it->second.back();
    it->second.pop_back();
    ++hits_;
    return p;
  }
  // Keep `ptr` for reuse, or release it to the device when this size class is full.
  void give(size_t len, float* ptr) {
    if (ptr == nullptr) return;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto& list = free_[len];
      if (list.size() < kMaxPerSize) {
        list.push_back(ptr);
        return;
      }
    }
    api().free_(ptr);
  }
  // Release every spare buffer (not in FastNN; useful before measuring free memory).
  void trim() {
    std::unordered_map<size_t, std::vector<float*>> drop;
    {
      std::lock_guard<std::mutex> g(mu_);
      drop.swap(free_);
    }
    for (auto& kv : drop)
      for (float* p : kv.second) api().free_(p);
  }
  size_t spare(size_t len) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = free_.find(len);
    return it == free_.end() ? 0 : it->second.size();
  }
  size_t hits() const { return hits_; }
  size_t misses() const { return misses_; }

 private:
  std::mutex mu_;
  std::unordered_map<size_t, std::vector<float*>> free_;
  size_t hits_ = 0, misses_ = 0;
};

// ------------------------------------------------------------------- CudaBuffer ---
class CudaBuffer {
 public:
  CudaBuffer() = default;
  // `len` floats on the device: a recycled buffer (contents undefined) or a fresh allocation.
  explicit CudaBuffer(size_t len) : len_(len) {
    ptr_ = BufferCache::instance().take(len);
    if (ptr_ == nullptr) {
      const size_t bytes = len * sizeof(float);
      if (api().malloc_(&ptr_, bytes) != 0) {
        ptr_ = nullptr;
        throw CudaError("Failed to allocate " + std::to_string(bytes) + " bytes on GPU");
      }
    }
  }
  CudaBuffer(const CudaBuffer&) = delete;
  CudaBuffer& operator=(const CudaBuffer&) = delete;
  CudaBuffer(CudaBuffer&& o) noexcept : ptr_(o.ptr_), len_(o.len_) { o.ptr_ = nullptr; o.len_ = 0; }
  CudaBuffer& operator=(CudaBuffer&& o) noexcept {
    if (this != &o) {
      release();
      ptr_ = o.ptr_; len_ = o.len_;
      o.ptr_ = nullptr; o.len_ = 0;
    }
    return *this;
  }
  ~CudaBuffer() { release(); }

  static CudaBuffer zeros(size_t len) {
    CudaBuffer b(len);
    if (api().memset_(b.ptr_, 0, len * sizeof(float)) != 0) throw CudaError("Failed to zero GPU memory");
    return b;
  }
  static CudaBuffer from_host(const float* data, size_t len) {
    CudaBuffer b(len);
    b.copy_from_host(data, len);
    return b;
  }
  void copy_from_host(const float* data, size_t n) {
    if (n > len_) throw std::invalid_argument("Source data larger than GPU buffer");
    if (n && api().h2d(ptr_, data, n * sizeof(float)) != 0) throw CudaError("H2D memcpy failed");
  }
  void copy_to_host(float* data, size_t n) const {
    if (n > len_) throw std::invalid_argument("Destination buffer smaller than GPU buffer");
    if (n && api().d2h(data, ptr_, n * sizeof(float)) != 0) throw CudaError("D2H memcpy failed");
  }
  std::vector<float> to_vec() const {
    std::vector<float> v(len_);
    copy_to_host(v.data(), len_);
    return v;
  }
  CudaBuffer clone() const {
    CudaBuffer b(len_);
    if (len_ && api().d2d(b.ptr_, ptr_, len_ * sizeof(float)) != 0) throw CudaError("D2D memcpy failed");
    return b;
  }
  float* ptr() const { return ptr_; }
  size_t len() const { return len_; }
  bool empty() const { return len_ == 0; }
  size_t size_bytes() const { return len_ * sizeof(float); }

 private:
  void release() {
    if (ptr_ != nullptr) BufferCache::instance().give(len_, ptr_);
    ptr_ = nullptr;
  }
  float* ptr_ = nullptr;
  size_t len_ = 0;
};

// ------------------------------------------------------------------ CudaContext ---
class CudaContext {
 public:
  // Initialises the device on first use; later calls for the same device are free.
  static void ensure(int device_id = 0) {
    static std::mutex mu;
    static std::unordered_map<int, bool> done;
    std::lock_guard<std::mutex> g(mu);
    if (done[device_id]) return;
    if (api().init(device_id) != 0)
      throw CudaError("Failed to initialize CUDA device " + std::to_string(device_id));
    done[device_id] = true;
  }
  static int device_count() { return api().device_count(); }
  static void synchronize() {
    if (api().synchronize() != 0) throw CudaError("CUDA synchronize failed");
  }
  static std::pair<size_t, size_t> memory_info() {
    size_t f = 0, t = 0;
    api().memory_info(&f, &t);
    return {f, t};
  }
};

// ----------------------------------------------------------------------- Tensor ---
// A dense row-major float32 device tensor: shape + shared storage.  Only what the matmul
// path needs.
class Tensor {
 public:
  Tensor() = default;
  Tensor(std::shared_ptr<CudaBuffer> buf, std::vector<size_t> shape)
      : buf_(std::move(buf)), shape_(std::move(shape)) {}

  static Tensor from_vec(const std::vector<float>& data, const std::vector<size_t>& shape) {
    size_t n = 1;
    for (size_t s : shape) n *= s;
    if (n != data.size()) throw std::invalid_argument("shape does not match data length");
    CudaContext::ensure(0);
    return Tensor(std::make_shared<CudaBuffer>(CudaBuffer::from_host(data.data(), n)), shape);
  }
  std::vector<float> to_vec() const { return buf_->to_vec(); }
  const std::vector<size_t>& shape() const { return shape_; }
  size_t ndim() const { return shape_.size(); }
  size_t numel() const {
    size_t n = 1;
    for (size_t s : shape_) n *= s;
    return n;
  }
  const float* data() const { return buf_->ptr(); }
  // A view with another shape of the same element count (shares storage).
  Tensor reshape(const std::vector<size_t>& shape) const {
    size_t n = 1;
    for (size_t s : shape) n *= s;
    if (n != numel()) throw std::invalid_argument("reshape changes the element count");
    return Tensor(buf_, shape);
  }

  // a[..,m,k] . b[..,k,n]
  Tensor matmul(const Tensor& o) const { return product(o, 0); }
  // a[..,m,k] . b[..,n,k]^T
  Tensor matmul_nt(const Tensor& o) const { return product(o, 1); }
  // a[..,k,m]^T . b[..,k,n]
  Tensor matmul_tn(const Tensor& o) const { return product(o, 2); }

 private:
  static size_t batch_of(const std::vector<size_t>& s) {
    size_t b = 1;
    for (size_t i = 0; i + 2 < s.size(); ++i) b *= s[i];
    return b;
  }
  Tensor product(const Tensor& o, int layout) const {
    if (ndim() < 2 || o.ndim() < 2) throw std::invalid_argument("matmul requires at least 2D tensors");
    const size_t ra = shape_[ndim() - 2], ca = shape_[ndim() - 1];
    const size_t rb = o.shape_[o.ndim() - 2], cb = o.shape_[o.ndim() - 1];
    const size_t m = layout == 2 ? ca : ra, k = layout == 2 ? ra : ca;
    const size_t kb = layout == 1 ? cb : rb, n = layout == 1 ? rb : cb;
    if (k != kb) throw std::invalid_argument("Matmul shape mismatch");
    const bool two_d = ndim() == 2 && o.ndim() == 2;
    const size_t batch = batch_of(shape_);
    if (!two_d && batch != batch_of(o.shape_))
      throw std::invalid_argument("Batch dimensions must match on CUDA tensors");
    if (m > 0x7fffffffu || n > 0x7fffffffu || k > 0x7fffffffu || batch > 0x7fffffffu)
      throw std::invalid_argument("dimension exceeds the C ABI's int range");
    auto out = std::make_shared<CudaBuffer>(batch * m * n);
    const DeviceApi& d = api();
    const int M = static_cast<int>(m), N = static_cast<int>(n), K = static_cast<int>(k);
    const int B = static_cast<int>(batch);
    int rc;
    if (two_d) {
      rc = layout == 0 ? d.matmul(data(), o.data(), out->ptr(), M, N, K, K, N, N, 1.0f, 0.0f)
         : layout == 1 ? d.matmul_nt(data(), o.data(), out->ptr(), M, N, K)
                       : d.matmul_tn(data(), o.data(), out->ptr(), M, N, K);
    } else {
      rc = layout == 0 ? d.matmul_batched(data(), o.data(), out->ptr(), M, N, K, B, 1.0f, 0.0f)
         : layout == 1 ? d.matmul_batched_nt(data(), o.data(), out->ptr(), M, N, K, B)
                       : d.matmul_batched_tn(data(), o.data(), out->ptr(), M, N, K, B);
    }
    if (rc != 0) throw CudaError(layout == 0 ? "CUDA matmul failed" : layout == 1 ? "CUDA matmul_nt failed"
                                                                                  : "CUDA matmul_tn failed");
    std::vector<size_t> shape(shape_.begin(), shape_.end() - 2);
    shape.push_back(m);
    shape.push_back(n);
    return Tensor(std::move(out), std::move(shape));
  }

  std::shared_ptr<CudaBuffer> buf_;
  std::vector<size_t> shape_;
};

// ----------------------------------------------------------------------- Linear ---
// y = act(x . W^T + b), W stored [out, in] as FastNN's Linear keeps it; one fused launch instead
// of transpose + matmul + expand + add (+ activation).
class Linear {
 public:
  Linear(Tensor weight, Tensor bias) : w_(std::move(weight)), b_(std::move(bias)) {
    if (w_.ndim() != 2) throw std::invalid_argument("weight must be [out, in]");
    if (b_.ndim() != 0 && (b_.ndim() != 1 || b_.shape()[0] != w_.shape()[0]))
      throw std::invalid_argument("bias must be [out]");
  }
  explicit Linear(Tensor weight) : Linear(std::move(weight), Tensor()) {}

  Tensor forward(const Tensor& x, int act = FASTNN_B200_ACT_NONE) const {
    const size_t in = w_.shape()[1], out = w_.shape()[0];
    if (x.ndim() < 1 || x.shape().back() != in)
      throw std::invalid_argument("Expected input features " + std::to_string(in));
    const size_t rows = x.numel() / (in ? in : 1);
    auto y = std::make_shared<CudaBuffer>(rows * out);
    const float* bias = b_.ndim() == 1 ? b_.data() : nullptr;
    if (api().linear_forward(FASTNN_B200_NT, x.data(), w_.data(), bias, y->ptr(), static_cast<int>(rows),
                             static_cast<int>(in), static_cast<int>(out), act) != 0)
      throw CudaError("CUDA linear_forward failed");
    std::vector<size_t> shape(x.shape().begin(), x.shape().end() - 1);
    shape.push_back(out);
    return Tensor(std::move(y), std::move(shape));
  }

 private:
  Tensor w_, b_;
};

}  // namespace host
}  // namespace fastnn
