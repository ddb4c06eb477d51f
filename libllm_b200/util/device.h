// Device memory, pinned host memory and the element types of the engine.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <utility>

#include "util/error.h"

namespace llm {

// The numbers are the ones the kernel libraries take (libllm_b200/csrc/common.cuh: LlmDtype).
enum class DType : int { F32 = 0, BF16 = 1, I32 = 2 };
inline size_t dtype_size(DType t) { return t == DType::BF16 ? 2 : 4; }
inline const char *dtype_name(DType t) { return t == DType::F32 ? "float32" : t == DType::BF16 ? "bfloat16" : "int32"; }

#define LLM_CUDA(expr)                                                                                         \
  do {                                                                                                         \
    cudaError_t e_ = (expr);                                                                                   \
    if (e_ != cudaSuccess)                                                                                     \
      LLM_THROW(Extension, "%s failed: %s", #expr, cudaGetErrorString(e_));                                    \
  } while (0)

class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t bytes, bool zero = false) { allocate(bytes, zero); }
  ~DeviceBuffer() { release(); }
  DeviceBuffer(DeviceBuffer &&o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
  DeviceBuffer &operator=(DeviceBuffer &&o) noexcept {
    if (this != &o) {
      release();
      ptr_ = o.ptr_;
      bytes_ = o.bytes_;
      o.ptr_ = nullptr;
      o.bytes_ = 0;
    }
    return *this;
  }
  DeviceBuffer(const DeviceBuffer &) = delete;
  DeviceBuffer &operator=(const DeviceBuffer &) = delete;

  void allocate(size_t bytes, bool zero = false) {
    release();
    if (bytes == 0) return;
    const cudaError_t e = cudaMalloc(&ptr_, bytes);
    if (e != cudaSuccess) {
      ptr_ = nullptr;
      cudaGetLastError();
      LLM_THROW(Extension, "cannot allocate %.1f MB of device memory: %s", bytes / 1e6, cudaGetErrorString(e));
    }
    bytes_ = bytes;
    if (zero) LLM_CUDA(cudaMemset(ptr_, 0, bytes));
  }
  void release() {
    if (ptr_) cudaFree(ptr_);
    ptr_ = nullptr;
    bytes_ = 0;
  }
  void *get() const { return ptr_; }
  template <typename T>
  T *as() const { return reinterpret_cast<T *>(ptr_); }
  size_t bytes() const { return bytes_; }
  explicit operator bool() const { return ptr_ != nullptr; }

 private:
  void *ptr_ = nullptr;
  size_t bytes_ = 0;
};

class PinnedBuffer {
 public:
  PinnedBuffer() = default;
  explicit PinnedBuffer(size_t bytes) { allocate(bytes); }
  ~PinnedBuffer() { release(); }
  PinnedBuffer(PinnedBuffer &&o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
  PinnedBuffer &operator=(PinnedBuffer &&o) noexcept {
    if (this != &o) {
      release();
      ptr_ = o.ptr_;
      bytes_ = o.bytes_;
      o.ptr_ = nullptr;
      o.bytes_ = 0;
    }
    return *this;
  }
  PinnedBuffer(const PinnedBuffer &) = delete;
  PinnedBuffer &operator=(const PinnedBuffer &) = delete;
  void allocate(size_t bytes) {
    release();
    if (bytes == 0) return;
    const cudaError_t e = cudaMallocHost(&ptr_, bytes);
    if (e != cudaSuccess) {
      ptr_ = nullptr;
      cudaGetLastError();
      LLM_THROW(Extension, "cannot allocate %zu bytes of pinned host memory: %s", bytes, cudaGetErrorString(e));
    }
    bytes_ = bytes;
  }
  void release() {
    if (ptr_) cudaFreeHost(ptr_);
    ptr_ = nullptr;
    bytes_ = 0;
  }
  void *get() const { return ptr_; }
  template <typename T>
  T *as() const { return reinterpret_cast<T *>(ptr_); }
  size_t bytes() const { return bytes_; }

 private:
  void *ptr_ = nullptr;
  size_t bytes_ = 0;
};

// A view of activations on the device: [rows, cols] with a row stride, or, with parts > 1,
// [parts, rows, cols] partial results (32-bit) that the consumer adds in order.
struct Act {
  void *data = nullptr;
  DType dtype = DType::F32;
  int64_t rows = 0, cols = 0, ld = 0;
  int parts = 1;
  int64_t part_stride = 0;
};

// A weight on the device: [rows, cols] row-major, or a vector (rows = 1).
struct Weight {
  DeviceBuffer buf;
  DType dtype = DType::F32;
  int64_t rows = 0, cols = 0;
  void *data() const { return buf.get(); }
};

}  // namespace llm
