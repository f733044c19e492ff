// A stand-in for the reference's tensor/tensor.h with just what its CPU rotary kernel
// (infMain/source/op/kernels/cpu/rope_kernel.cpp) touches: ptr<T>() and ptr<T>(index) on a
// buffer the caller owns, and the UNUSED macro.  It lets that one file compile unmodified
// without the reference's allocator, logging and linear-algebra dependencies.
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>

#ifndef UNUSED
#define UNUSED(x) (void)(x)
#endif

namespace tensor {
class Tensor {
 public:
  Tensor() = default;
  explicit Tensor(void* data) : data_(data) {}
  template <typename T> T* ptr() { return static_cast<T*>(data_); }
  template <typename T> const T* ptr() const { return static_cast<const T*>(data_); }
  template <typename T> T* ptr(int64_t index) { return static_cast<T*>(data_) + index; }
  template <typename T> const T* ptr(int64_t index) const { return static_cast<const T*>(data_) + index; }

 private:
  void* data_ = nullptr;
};
}  // namespace tensor
