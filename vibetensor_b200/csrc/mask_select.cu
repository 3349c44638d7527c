// Boolean mask -> ascending int64 indices of its true positions (stream compaction).
//
// The reference turns a CUDA bool mask into an index tensor before it runs the ordinary
// advanced-index gather: either CUB (reduce_sum_u8_as_i32, one D2H count, then
// select_indices_from_u8_flags_i64) or, by default, a D2H copy of the whole mask, a host scan
// and an H2D copy of the indices (src/vbt/core/indexing_advanced_cuda.cu:2191-2429).  Here:
// three small launches on the caller's stream and no host pass over the mask --
//   1. per-tile true counts (a tile = 4096 mask bytes),
//   2. one block turns the counts into exclusive offsets and writes the total,
//   3. every tile writes the positions of its true bytes at offset + rank, in mask order.
// The mask is read twice (2 bytes per element) and 8 bytes are written per true element.
#include "common.cuh"

namespace vb {
namespace {

constexpr int kMsThreads = 256;
constexpr int kMsItems = 16;                       // mask bytes per thread
constexpr int kMsTile = kMsThreads * kMsItems;     // 4096

struct MaskParams {
  const uint8_t* mask;
  int64_t n;
  int64_t stride;   // elements (= bytes)
  int vec;          // stride == 1 and 16-byte aligned base: uint4 loads
};

// the thread's 16 flags as a bit set (bit k = mask[first + k] != 0)
__device__ __forceinline__ uint32_t load_flags(const MaskParams& p, int64_t first) {
  uint32_t bits = 0;
  if (p.vec && first + kMsItems <= p.n) {
    const uint4 v = *reinterpret_cast<const uint4*>(p.mask + first);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if ((w[q] >> (8 * b)) & 0xffu) bits |= 1u << (4 * q + b);
  } else {
#pragma unroll
    for (int k = 0; k < kMsItems; ++k) {
      const int64_t i = first + k;
      if (i < p.n && p.mask[i * p.stride] != 0) bits |= 1u << k;
    }
  }
  return bits;
}

__global__ void __launch_bounds__(kMsThreads) mask_count_kernel(const __grid_constant__ MaskParams p,
                                                                unsigned* tile_counts) {
  __shared__ unsigned red[kMsThreads / 32];
  const int t = threadIdx.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kMsTile + static_cast<int64_t>(t) * kMsItems;
  unsigned c = __popc(load_flags(p, first));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
  if ((t & 31) == 0) red[t >> 5] = c;
  __syncthreads();
  if (t == 0) {
    unsigned s = 0;
#pragma unroll
    for (int w = 0; w < kMsThreads / 32; ++w) s += red[w];
    tile_counts[blockIdx.x] = s;
  }
}

// one block: counts -> exclusive offsets (64-bit), total -> *count_out
__global__ void __launch_bounds__(1024) mask_scan_kernel(const unsigned* tile_counts, unsigned long long* tile_offsets,
                                                         int64_t ntiles, unsigned long long* count_out) {
  __shared__ unsigned long long warp_tot[32];
  __shared__ unsigned long long carry_s, chunk_s;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  if (t == 0) carry_s = 0ull;
  __syncthreads();
  for (int64_t base = 0; base < ntiles; base += 1024) {
    const int64_t i = base + t;
    const unsigned long long v = i < ntiles ? tile_counts[i] : 0ull;
    unsigned long long x = v;  // inclusive scan within the warp
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned long long y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_tot[w] = x;
    __syncthreads();
    if (w == 0) {
      const unsigned long long wt = warp_tot[lane];
      unsigned long long sc = wt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long y = __shfl_up_sync(0xffffffffu, sc, d);
        if (lane >= d) sc += y;
      }
      warp_tot[lane] = sc - wt;  // exclusive prefix of the warp totals
      if (lane == 31) chunk_s = sc;
    }
    __syncthreads();
    const unsigned long long carry = carry_s;
    if (i < ntiles) tile_offsets[i] = carry + warp_tot[w] + (x - v);
    __syncthreads();
    if (t == 0) carry_s = carry + chunk_s;
    __syncthreads();
  }
  if (t == 0) *count_out = carry_s;
}

__global__ void __launch_bounds__(kMsThreads) mask_select_kernel(const __grid_constant__ MaskParams p,
                                                                 const unsigned long long* tile_offsets,
                                                                 int64_t* out, int64_t capacity) {
  __shared__ unsigned warp_tot[kMsThreads / 32];
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kMsTile + static_cast<int64_t>(t) * kMsItems;
  uint32_t bits = load_flags(p, first);
  const unsigned c = __popc(bits);
  unsigned x = c;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  if (lane == 31) warp_tot[w] = x;
  __syncthreads();
  unsigned before = x - c;
  for (int ww = 0; ww < w; ++ww) before += warp_tot[ww];
  int64_t o = static_cast<int64_t>(tile_offsets[blockIdx.x]) + before;
  while (bits) {
    const int k = __ffs(bits) - 1;
    bits &= bits - 1;
    if (o < capacity) out[o] = first + k;
    ++o;
  }
}

}  // namespace
}  // namespace vb

extern "C" {

vbt_b200_status vbt_b200_mask_select_workspace_bytes(int64_t n, size_t* bytes) {
  using namespace vb;
  VB_ARG(bytes != nullptr && n >= 0, "mask_select: bad argument");
  const int64_t ntiles = (n + kMsTile - 1) / kMsTile;
  // counts (u32, padded to 8 bytes) then offsets (u64)
  *bytes = static_cast<size_t>((ntiles * 4 + 7) / 8 * 8 + ntiles * 8);
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_mask_select(const vbt_b200_tensor* mask, int64_t* out_indices, int64_t capacity,
                                     uint64_t* count_out, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  using namespace vb;
  VB_ARG(mask != nullptr && count_out != nullptr, "index: null argument");
  VB_TRY(validate_tensor(mask, "index"));
  VB_ARG(mask->dtype == VBT_B200_BOOL, "index: mask must be a bool tensor");
  VB_ARG(mask->ndim == 1, std::string("index: ") + "CUDA advanced indexing does not support boolean mask indices"
                              " of rank other than 1");
  VB_ARG(capacity >= 0 && (capacity == 0 || out_indices != nullptr), "index: bad index buffer");
  const int64_t n = mask->sizes[0];
  const int64_t stride = mask->strides[0];
  const uint8_t* base = static_cast<const uint8_t*>(mask->data);
  DeviceScope scope(count_out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    VB_CUDA(cudaMemsetAsync(count_out, 0, 8, s));
    return VBT_B200_OK;
  }
  VB_ARG(base != nullptr, "index: null mask data");
  VB_ARG(stride >= 0, "index: mask with a negative stride");
  size_t need = 0;
  VB_TRY(vbt_b200_mask_select_workspace_bytes(n, &need));
  VB_ARG(workspace != nullptr && workspace_bytes >= need && reinterpret_cast<uintptr_t>(workspace) % 8 == 0,
         "index: mask workspace too small (see vbt_b200_mask_select_workspace_bytes)");
  const int64_t ntiles = (n + kMsTile - 1) / kMsTile;
  VB_ARG(ntiles <= 0x7fffffff, "advanced indexing too large");
  unsigned* counts = static_cast<unsigned*>(workspace);
  unsigned long long* offsets =
      reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + (ntiles * 4 + 7) / 8 * 8);
  MaskParams p{};
  p.mask = base; p.n = n; p.stride = stride;
  p.vec = (stride == 1 && reinterpret_cast<uintptr_t>(base) % 16 == 0) ? 1 : 0;
  mask_count_kernel<<<static_cast<unsigned>(ntiles), kMsThreads, 0, s>>>(p, counts);
  VB_LAUNCH_CHECK();
  mask_scan_kernel<<<1, 1024, 0, s>>>(counts, offsets, ntiles, reinterpret_cast<unsigned long long*>(count_out));
  VB_LAUNCH_CHECK();
  if (capacity > 0) {
    mask_select_kernel<<<static_cast<unsigned>(ntiles), kMsThreads, 0, s>>>(p, offsets, out_indices, capacity);
    VB_LAUNCH_CHECK();
  }
  return VBT_B200_OK;
}

}  // extern "C"
