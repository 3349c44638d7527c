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
// SM count of the device that is current on the calling thread (launchers run under a DeviceScope).
inline int current_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 148;
  }
  return sm_count(dev);
}
// Device that owns `ptr`, or the current device for a pointer CUDA does not know.
inline int device_of(const void* ptr) {
  cudaPointerAttributes attr{};
  if (ptr && cudaPointerGetAttributes(&attr, ptr) == cudaSuccess &&
      (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged))
    return attr.device;
  cudaGetLastError();
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

inline int itemsize(int dtype) {
  switch (dtype) {
    case VBT_B200_BOOL: return 1;
    case VBT_B200_I32: return 4;
    case VBT_B200_I64: return 8;
    case VBT_B200_F32: return 4;
    case VBT_B200_F16: return 2;
    case VBT_B200_BF16: return 2;
    case VBT_B200_C64: return 8;
    case VBT_B200_C128: return 16;
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
// validate_tensor plus: a tensor with elements must have a data pointer (a kernel given a null
// base would fault on the device).
vbt_b200_status validate_data(const vbt_b200_tensor* t, const char* what);

// ---------------------------------------------------------------------------------------
// observability: what the last call on this thread launched, and process-wide launch counts
// (the counterpart of the reference's TensorIterStats / CudaReductionLastStats test hooks)
// ---------------------------------------------------------------------------------------
vbt_b200_launch_info& launch_info_ref();
void count_launches(int family, int n);
inline void note_launch(int family, int kernel, dim3 grid, dim3 block, int vec, int splits, int cluster,
                        int launches, int64_t out_numel, int64_t slice_len, size_t workspace_bytes,
                        const void* stream) {
  vbt_b200_launch_info& li = launch_info_ref();
  li.family = family;
  li.kernel = kernel;
  li.grid[0] = grid.x; li.grid[1] = grid.y; li.grid[2] = grid.z;
  li.block[0] = block.x; li.block[1] = block.y; li.block[2] = block.z;
  li.vec = vec;
  li.splits = splits;
  li.cluster = cluster;
  li.launches = launches;
  li.out_numel = out_numel;
  li.slice_len = slice_len;
  li.workspace_bytes = workspace_bytes;
  li.stream = const_cast<void*>(stream);
  count_launches(family, launches);
}

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
// linear index over a list of dims (last dim fastest) -> element offset; used for the kept /
// reduced dims of a reduction and for the leading dims of an indexed tensor
// ---------------------------------------------------------------------------------------
struct DimList {
  int n;
  FastDiv div[VBT_B200_MAX_NDIM];
  int64_t stride[VBT_B200_MAX_NDIM];
  __device__ __forceinline__ int64_t offset(uint32_t lin) const {
    int64_t off = 0;
    for (int d = n - 1; d >= 0; --d) {
      uint32_t c;
      div[d].divmod(lin, lin, c);
      off += static_cast<int64_t>(c) * stride[d];
    }
    return off;
  }
};
inline void fill_dimlist(DimList& dl, const int64_t* sizes, const int64_t* strides, int n) {
  dl.n = n;
  for (int i = 0; i < n; ++i) {
    dl.div[i] = FastDiv(static_cast<uint32_t>(sizes[i]));
    dl.stride[i] = strides[i];
  }
}

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
