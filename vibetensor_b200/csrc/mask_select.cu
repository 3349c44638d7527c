// Boolean mask -> ascending int64 indices of its true positions (stream compaction).
//
// The reference turns a CUDA bool mask into an index tensor before it runs the ordinary
// advanced-index gather: either CUB (reduce_sum_u8_as_i32, one D2H count, then
// select_indices_from_u8_flags_i64) or, by default, a D2H copy of the whole mask, a host scan
// and an H2D copy of the indices (src/vbt/core/indexing_advanced_cuda.cu:2191-2429).  Here:
// three small launches on the caller's stream and no host pass over the mask --
//   1. per-tile true counts (a tile = 16384 mask bytes, four 16-byte loads per thread); every
//      thread also leaves each load's 16 flags as a 16-bit word in the workspace,
//   2. one block turns the counts into exclusive offsets and writes the total,
//   3. every tile reads its flag words back and writes the positions of the set bits at
//      offset + rank, in mask order.
// The mask itself is read once; the flag words add 1/8 byte per element written and read back,
// and 8 bytes are written per true element.  No block waits on another.
#include "common.cuh"

namespace vb {
namespace {

constexpr int kMsThreads = 256;
constexpr int kMsItems = 16;                       // mask bytes per thread and sub-tile (one 16-byte load)
constexpr int kMsSub = 4;                          // sub-tiles a block walks
constexpr int kMsSubTile = kMsThreads * kMsItems;  // 4096 mask bytes
constexpr int kMsTile = kMsSubTile * kMsSub;       // 16384 mask bytes per block

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
    for (int q = 0; q < 4; ++q) {
      // four bytes at a time: bit 7 of every non-zero byte, then the four bits gathered by one multiply
      // (the partial products that are not wanted land on distinct bits below bit 28: no carries)
      const uint32_t nz = (((w[q] & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w[q]) & 0x80808080u;
      bits |= (((nz >> 7) * 0x10204080u) >> 28) << (4 * q);
    }
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
                                                                unsigned* tile_counts, uint16_t* flag_words) {
  __shared__ unsigned red[kMsThreads / 32];
  const int t = threadIdx.x;
  const int64_t tile_first = static_cast<int64_t>(blockIdx.x) * kMsTile;
  uint32_t bits[kMsSub];
#pragma unroll
  for (int q = 0; q < kMsSub; ++q)  // the loads of all sub-tiles are in flight together
    bits[q] = load_flags(p, tile_first + q * kMsSubTile + static_cast<int64_t>(t) * kMsItems);
  unsigned c = 0;
#pragma unroll
  for (int q = 0; q < kMsSub; ++q) {
    flag_words[(static_cast<int64_t>(blockIdx.x) * kMsSub + q) * kMsThreads + t] = static_cast<uint16_t>(bits[q]);
    c += __popc(bits[q]);
  }
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

// one block: counts -> the exclusive offset (64-bit) of every GROUP of kScanItems consecutive tiles,
// total -> *count_out.  A thread sums one group (four 16-byte loads), the block scans the 1024
// sums, and the offsets go out coalesced; the select kernel adds the counts of the earlier tiles
// of its own group.  (One offset per tile, written by a 1024-wide scan in sixteen rounds, took
// 18 us on a 2^28-element mask; sixteen consecutive offsets per thread, 13 us: those stores were
// 128 bytes apart.)
constexpr int kScanItems = 16;
__global__ void __launch_bounds__(1024) mask_scan_kernel(const unsigned* tile_counts, unsigned long long* group_offsets,
                                                         int64_t ntiles, unsigned long long* count_out) {
  __shared__ unsigned long long warp_tot[32];
  __shared__ unsigned long long chunk_s;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  unsigned long long carry = 0ull;
  const int64_t ngroups = (ntiles + kScanItems - 1) / kScanItems;
  for (int64_t gbase = 0; gbase < ngroups; gbase += 1024) {
    const int64_t g = gbase + t;
    const int64_t i0 = g * kScanItems;
    unsigned long long mine = 0ull;
    if (i0 + kScanItems <= ntiles && reinterpret_cast<uintptr_t>(tile_counts) % 16 == 0) {
#pragma unroll
      for (int k = 0; k < kScanItems / 4; ++k) {
        const uint4 q = reinterpret_cast<const uint4*>(tile_counts + i0)[k];
        mine += static_cast<unsigned long long>(q.x) + q.y + q.z + q.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < kScanItems; ++k)
        if (i0 + k < ntiles) mine += tile_counts[i0 + k];
    }
    unsigned long long x = mine;  // inclusive scan within the warp
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned long long y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    __syncthreads();  // warp_tot and chunk_s may still be read from the previous round
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
    if (g < ngroups) group_offsets[g] = carry + warp_tot[w] + (x - mine);
    carry += chunk_s;
  }
  if (t == 0) *count_out = carry;
}

__global__ void __launch_bounds__(kMsThreads) mask_select_kernel(const uint16_t* flag_words, const unsigned* tile_counts,
                                                                 const unsigned long long* group_offsets,
                                                                 int64_t* out, int64_t capacity) {
  __shared__ unsigned warp_tot[kMsSub][kMsThreads / 32];
  __shared__ unsigned long long base_s;
  if (threadIdx.x < 32) {
    // this tile's first output slot: the group's offset + the counts of the group's earlier tiles
    const int64_t g0 = static_cast<int64_t>(blockIdx.x) / kScanItems * kScanItems;
    const int k = threadIdx.x;
    unsigned c0 = (k < kScanItems && g0 + k < static_cast<int64_t>(blockIdx.x)) ? tile_counts[g0 + k] : 0u;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) c0 += __shfl_xor_sync(0xffffffffu, c0, d);
    if (k == 0) base_s = group_offsets[blockIdx.x / kScanItems] + c0;
  }
  __shared__ uint16_t pos[kMsTile];  // tile-relative positions of the set bits, in mask order
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  uint32_t bits[kMsSub];
  unsigned c[kMsSub], x[kMsSub];
#pragma unroll
  for (int q = 0; q < kMsSub; ++q)
    bits[q] = flag_words[(static_cast<int64_t>(blockIdx.x) * kMsSub + q) * kMsThreads + t];
#pragma unroll
  for (int q = 0; q < kMsSub; ++q) {
    c[q] = __popc(bits[q]);
    x[q] = c[q];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned y = __shfl_up_sync(0xffffffffu, x[q], d);
      if (lane >= d) x[q] += y;
    }
    if (lane == 31) warp_tot[q][w] = x[q];
  }
  __syncthreads();
  // rank of this thread's first set bit: earlier sub-tiles, earlier warps of the sub-tile, earlier lanes
  unsigned total = 0;
#pragma unroll
  for (int q = 0; q < kMsSub; ++q) {
    unsigned before = total + x[q] - c[q];
#pragma unroll
    for (int ww = 0; ww < kMsThreads / 32; ++ww) {
      if (ww < w) before += warp_tot[q][ww];
      total += warp_tot[q][ww];
    }
    unsigned o = before;
    uint32_t bq = bits[q];
    while (bq) {
      const int k = __ffs(bq) - 1;
      bq &= bq - 1;
      pos[o++] = static_cast<uint16_t>(q * kMsSubTile + t * kMsItems + k);
    }
  }
  __syncthreads();
  // coalesced 8-byte stores: consecutive threads write consecutive output slots (16-byte stores
  // from the first even slot on measured slower: 193 -> 208 us on 2^28 elements)
  const int64_t tile_first = static_cast<int64_t>(blockIdx.x) * kMsTile;
  const int64_t base = static_cast<int64_t>(base_s);  // written before the first barrier above
  for (unsigned i = t; i < total; i += kMsThreads)
    if (base + i < capacity) out[base + i] = tile_first + pos[i];
}

}  // namespace
}  // namespace vb

extern "C" {

vbt_b200_status vbt_b200_mask_select_workspace_bytes(int64_t n, size_t* bytes) {
  using namespace vb;
  VB_ARG(bytes != nullptr && n >= 0, "mask_select: bad argument");
  const int64_t ntiles = (n + kMsTile - 1) / kMsTile;
  // counts (u32, padded to 8 bytes), offsets (u64), flag words (u16 per 16 mask bytes)
  *bytes = static_cast<size_t>((ntiles * 4 + 7) / 8 * 8 + ntiles * 8 + ntiles * kMsSub * kMsThreads * 2);
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
  uint16_t* flag_words = reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(offsets) + ntiles * 8);
  MaskParams p{};
  p.mask = base; p.n = n; p.stride = stride;
  p.vec = (stride == 1 && reinterpret_cast<uintptr_t>(base) % 16 == 0) ? 1 : 0;
  mask_count_kernel<<<static_cast<unsigned>(ntiles), kMsThreads, 0, s>>>(p, counts, flag_words);
  VB_LAUNCH_CHECK();
  mask_scan_kernel<<<1, 1024, 0, s>>>(counts, offsets, ntiles, reinterpret_cast<unsigned long long*>(count_out));
  VB_LAUNCH_CHECK();
  if (capacity > 0) {
    mask_select_kernel<<<static_cast<unsigned>(ntiles), kMsThreads, 0, s>>>(flag_words, counts, offsets, out_indices, capacity);
    VB_LAUNCH_CHECK();
  }
  note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_MASK_SELECT, dim3(static_cast<unsigned>(ntiles)), dim3(kMsThreads), 16,
              1, 0, capacity > 0 ? 3 : 2, n, n, need, s);
  return VBT_B200_OK;
}

}  // extern "C"
