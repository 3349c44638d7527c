// Shared host/device helpers for libvbt_b200.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/vbt_b200.h"

namespace vb {

// ---------------------------------------------------------------------------------------
// status plumbing: every extern "C" entry returns a code and leaves the text in a
// thread-local string, the plain-C shape of "throw std::invalid_argument(msg)".
// ---------------------------------------------------------------------------------------
std::string& last_error_ref();
inline vbt_b200_status fail(vbt_b200_status code, const std::string& msg) {
  last_error_ref() = msg;
  return code;
}
#define VB_REQUIRE(cond, code, msg)          \
  do {                                       \
    if (!(cond)) return ::vb::fail((code), (msg)); \
  } while (0)
#define VB_ARG(cond, msg) VB_REQUIRE(cond, VBT_B200_INVALID_ARGUMENT, msg)
#define VB_CUDA(expr)                                                                   \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess)                                                             \
      return ::vb::fail(VBT_B200_CUDA_ERROR,                                            \
                        std::string(#expr) + ": " + cudaGetErrorString(e__));           \
  } while (0)
#define VB_TRY(expr)                         \
  do {                                       \
    vbt_b200_status s__ = (expr);            \
    if (s__ != VBT_B200_OK) return s__;      \
  } while (0)
#define VB_LAUNCH_CHECK() VB_CUDA(cudaGetLastError())

// Makes the device that owns `ptr` current for the scope of one entry point.
class DeviceScope {
 public:
  explicit DeviceScope(const void* ptr) {
    cudaGetDevice(&prev_);
    cudaPointerAttributes attr{};
    if (ptr && cudaPointerGetAttributes(&attr, ptr) == cudaSuccess &&
        (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged)) {
      dev_ = attr.device;
    } else {
      cudaGetLastError();  // clear "invalid value" for host pointers
      dev_ = prev_;
    }
    if (dev_ != prev_) cudaSetDevice(dev_);
  }
  ~DeviceScope() {
    if (dev_ != prev_) cudaSetDevice(prev_);
  }
  int device() const { return dev_; }

 private:
  int prev_{0};
  int dev_{0};
};

int sm_count(int device);

inline int itemsize(int dtype) {
  switch (dtype) {
    case VBT_B200_BOOL: return 1;
    case VBT_B200_I32: return 4;
    case VBT_B200_I64: return 8;
    case VBT_B200_F32: return 4;
    case VBT_B200_F16: return 2;
    case VBT_B200_BF16: return 2;
  }
  return 0;
}
inline bool is_float_dtype(int dtype) {
  return dtype == VBT_B200_F32 || dtype == VBT_B200_F16 || dtype == VBT_B200_BF16;
}
inline int64_t numel(const vbt_b200_tensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.ndim; ++i) n *= t.sizes[i];
  return n;
}
inline bool is_dense_row_major(const vbt_b200_tensor& t) {
  int64_t expect = 1;
  for (int i = t.ndim - 1; i >= 0; --i) {
    if (t.sizes[i] == 0) return true;
    if (t.sizes[i] != 1 && t.strides[i] != expect) return false;
    expect *= t.sizes[i];
  }
  return true;
}
vbt_b200_status validate_tensor(const vbt_b200_tensor* t, const char* what);

// ---------------------------------------------------------------------------------------
// 32-bit division by an invariant (n < 2^31): q = (umulhi(n, m) + n) >> s
// ---------------------------------------------------------------------------------------
struct FastDiv {
  uint32_t d{1}, m{0}, s{0};
  FastDiv() = default;
  explicit FastDiv(uint32_t div) : d(div) {
    if (div <= 1) { d = 1; m = 0; s = 0; return; }
    uint32_t l = 0;
    while ((1ull << l) < div) ++l;
    s = l;
    m = static_cast<uint32_t>(((1ull << 32) * ((1ull << l) - div)) / div + 1);
  }
  __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
    return (__umulhi(n, m) + n) >> s;
#else
    return static_cast<uint32_t>(((static_cast<uint64_t>(n) * m >> 32) + n) >> s);
#endif
  }
  __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};

// ---------------------------------------------------------------------------------------
// device-side element helpers
// ---------------------------------------------------------------------------------------
template <class T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

template <class T> struct is_float_storage { static constexpr bool value = false; };
template <> struct is_float_storage<float> { static constexpr bool value = true; };
template <> struct is_float_storage<__half> { static constexpr bool value = true; };
template <> struct is_float_storage<__nv_bfloat16> { static constexpr bool value = true; };

// Calls fn(T{}) with the storage type of a dtype code; returns false for unknown codes.
#define VB_DISPATCH_FLOAT(dtype, T, ...)                                  \
  [&]() -> bool {                                                         \
    switch (dtype) {                                                      \
      case VBT_B200_F32: { using T = float; __VA_ARGS__; return true; }   \
      case VBT_B200_F16: { using T = __half; __VA_ARGS__; return true; }  \
      case VBT_B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; return true; } \
    }                                                                     \
    return false;                                                         \
  }()

}  // namespace vb
