// Shared helpers of the C++ host layer: error translation between the C ABI's status codes and the
// exception types libmolgrid's users catch, and small RAII wrappers for device staging.
#ifndef LMGB200_COMMON_H_
#define LMGB200_COMMON_H_

#include <cuda_runtime.h>

#include <cstddef>
#include <stdexcept>
#include <string>

#include "lmg_b200.h"

#ifdef __CUDACC__
#define CUDA_CALLABLE_MEMBER __host__ __device__
#else
#define CUDA_CALLABLE_MEMBER
#endif

// Same contract as the reference macro of this name (include/libmolgrid/common.h:41-47):
// a failing CUDA runtime call becomes std::runtime_error.
#define LMG_CUDA_CHECK(call)                                                               \
  do {                                                                                     \
    cudaError_t lmg_err_ = (call);                                                         \
    if (lmg_err_ != cudaSuccess)                                                           \
      throw std::runtime_error(std::string("CUDA Error: ") + cudaGetErrorString(lmg_err_)); \
  } while (0)

namespace libmolgrid {

inline std::string itoa(long long v) { return std::to_string(v); }

namespace detail {

// status code of the C ABI -> the exception the reference throws in the same situation
inline void check(int rc) {
  if (rc == LMG_OK) return;
  std::string msg = lmg_last_error();
  if (rc == LMG_ERR_OUT_OF_RANGE) throw std::out_of_range(msg);
  if (rc == LMG_ERR_INVALID_ARGUMENT) throw std::invalid_argument(msg);
  throw std::runtime_error(msg);
}

// Scratch memory handed to the C ABI: one buffer per host thread and device, grown on demand.
inline void* workspace(size_t bytes) {
  struct Slot { void* p = nullptr; size_t cap = 0; };
  thread_local Slot slots[64];
  int dev = 0;
  LMG_CUDA_CHECK(cudaGetDevice(&dev));
  Slot& s = slots[dev & 63];
  if (bytes > s.cap) {
    if (s.p) cudaFree(s.p);
    s.p = nullptr;
    s.cap = 0;
    LMG_CUDA_CHECK(cudaMalloc(&s.p, bytes));
    s.cap = bytes;
  }
  return s.p;
}

// Device copy of a host array for the duration of one call (host-grid overloads compute on the
// GPU as well: there is no CPU implementation of the path in this library).
template <typename T>
class Staged {
 public:
  Staged(T* host, size_t n, bool copy_in, bool copy_out) : host_(host), n_(n), out_(copy_out) {
    if (n_ == 0) return;
    LMG_CUDA_CHECK(cudaMalloc(&dev_, n_ * sizeof(T)));
    if (copy_in) LMG_CUDA_CHECK(cudaMemcpy(dev_, host_, n_ * sizeof(T), cudaMemcpyHostToDevice));
  }
  Staged(const Staged&) = delete;
  Staged& operator=(const Staged&) = delete;
  ~Staged() {
    if (dev_) cudaFree(dev_);
  }
  T* get() const { return dev_; }
  void finish() {
    if (out_ && n_) LMG_CUDA_CHECK(cudaMemcpy(host_, dev_, n_ * sizeof(T), cudaMemcpyDeviceToHost));
  }

 private:
  T* host_;
  T* dev_ = nullptr;
  size_t n_;
  bool out_;
};

}  // namespace detail
}  // namespace libmolgrid

#endif
