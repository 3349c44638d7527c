// Boolean mask -> ascending int64 indices of its true positions (stream compaction).
//
// The reference turns a CUDA bool mask into an index tensor before it runs the ordinary
// advanced-index gather: either CUB (reduce_sum_u8_as_i32, one D2H count, then
// select_indices_from_u8_flags_i64) or, by default, a D2H copy of the whole mask, a host scan
// and an H2D copy of the indices (src/vbt/core/indexing_advanced_cuda.cu:2191-2429).  Here:
// three small launches on the caller's stream and no host pass over the mask --
//   1. per-tile true counts (a tile = 16384 mask bytes, four 16-byte loads per thread; a block
//      walks several tiles with the next one's loads in flight); every
//      thread also leaves each load's 16 flags as a 16-bit word in the workspace (the bits of a
//      word in the order that is cheapest to produce, see flag_bit_of),
//   2. one block turns the counts into exclusive offsets and writes the total,
//   3. every tile reads its flag words back as 32-bit words; a warp walks its words in order and
//      lane L writes the position of bit L at offset + rank, in mask order.
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
constexpr int kMsCountBlocksPerSm = 5;             // resident blocks of the count kernel (48 registers)

struct MaskParams {
  const uint8_t* mask;
  int64_t n;
  int64_t stride;   // elements (= bytes)
  int vec;          // stride == 1 and 16-byte aligned base: uint4 loads
};

// Where the flag of element k (0..15) of a 16-byte group sits in the group's 16-bit flag word.
// Not k itself: with bit 7 of byte b of 32-bit word q standing for element 4q + b, the four words
// shifted by 7, 6, 5 and 4 and OR-ed leave element (q, b) at bit 8b + q, and folding the upper half
// onto the lower one (>> 12) packs that into 16 bits with two more instructions -- element 4q + b
// ends at q + 4 * {0, 2, 1, 3}[b].  The select kernel reads the words with the same map.
__host__ __device__ constexpr int flag_bit_of(int k) {
  const int q = k >> 2, b = k & 3;
  return q + 4 * (b == 0 ? 0 : b == 1 ? 2 : b == 2 ? 1 : 3);
}
// the inverse: which element of the group bit f stands for
__host__ __device__ constexpr int element_of_flag_bit(int f) {
  const int q = f & 3, g = f >> 2;
  return 4 * q + (g == 0 ? 0 : g == 1 ? 2 : g == 2 ? 1 : 3);
}

// 16 mask bytes -> their 16 flags (bit flag_bit_of(k) = byte k != 0)
__device__ __forceinline__ uint32_t flags_of(const uint4& v) {
  // bit 7 of every non-zero byte (the low seven bits carry into it, or it is set already)
  auto nz = [](uint32_t w) { return (((w & 0x7f7f7f7fu) + 0x7f7f7f7fu) | w) & 0x80808080u; };
  const uint32_t u = (nz(v.x) >> 7) | (nz(v.y) >> 6) | (nz(v.z) >> 5) | (nz(v.w) >> 4);  // element 4q + b at bit 8b + q
  return (u | (u >> 12)) & 0xffffu;
}

// the thread's 16 flags as a bit set, for any stride, alignment and tail
__device__ __forceinline__ uint32_t load_flags(const MaskParams& p, int64_t first) {
  if (p.vec && first + kMsItems <= p.n) return flags_of(*reinterpret_cast<const uint4*>(p.mask + first));
  uint32_t bits = 0;
#pragma unroll
  for (int k = 0; k < kMsItems; ++k) {
    const int64_t i = first + k;
    if (i < p.n && p.mask[i * p.stride] != 0) bits |= 1u << flag_bit_of(k);
  }
  return bits;
}

// A block walks tiles blockIdx.x, + gridDim.x, ...; the 16-byte loads of its next tile are issued
// before the flags of the current one are worked out, so the block always has loads in flight.
// (One tile per block, loads -> arithmetic -> reduction -> exit, reached 4.7 TB/s.)
__global__ void __launch_bounds__(kMsThreads, kMsCountBlocksPerSm) mask_count_kernel(const __grid_constant__ MaskParams p,
                                                                unsigned* tile_counts, uint16_t* flag_words,
                                                                int64_t ntiles) {
  __shared__ unsigned red[2][kMsThreads / 32];
  const int t = threadIdx.x;
  // whole tiles of a dense, aligned mask are fetched ahead as raw 16-byte words
  auto whole = [&](int64_t tile) { return p.vec && (tile + 1) * kMsTile <= p.n; };
  auto fetch = [&](int64_t tile, uint4 (&raw)[kMsSub]) {
    const uint4* src = reinterpret_cast<const uint4*>(p.mask + tile * kMsTile) + t;
#pragma unroll
    for (int q = 0; q < kMsSub; ++q) raw[q] = src[q * kMsThreads];
  };
  uint4 ahead[kMsSub];
  int64_t tile = blockIdx.x;
  if (tile < ntiles && whole(tile)) fetch(tile, ahead);
  int phase = 0;
  for (; tile < ntiles; tile += gridDim.x) {
    uint32_t bits[kMsSub];
    const int64_t next = tile + gridDim.x;
    if (whole(tile)) {
      uint4 cur[kMsSub];
#pragma unroll
      for (int q = 0; q < kMsSub; ++q) cur[q] = ahead[q];
      if (next < ntiles && whole(next)) fetch(next, ahead);
#pragma unroll
      for (int q = 0; q < kMsSub; ++q) bits[q] = flags_of(cur[q]);
    } else {
#pragma unroll
      for (int q = 0; q < kMsSub; ++q)
        bits[q] = load_flags(p, tile * kMsTile + q * kMsSubTile + static_cast<int64_t>(t) * kMsItems);
    }
    unsigned c = 0;
#pragma unroll
    for (int q = 0; q < kMsSub; ++q) {
      flag_words[(tile * kMsSub + q) * kMsThreads + t] = static_cast<uint16_t>(bits[q]);
      c += __popc(bits[q]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
    if ((t & 31) == 0) red[phase][t >> 5] = c;
    __syncthreads();  // the other half of `red` is written next: one barrier per tile is enough
    if (t == 0) {
      unsigned s = 0;
#pragma unroll
      for (int w = 0; w < kMsThreads / 32; ++w) s += red[phase][w];
      tile_counts[tile] = s;
    }
    phase ^= 1;
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

// The flag words of a tile, read as 32-bit words, cover 32 consecutive mask positions each.  A
// warp owns 64 consecutive words (2048 positions): lane L holds words L and L + 32, the warp walks
// them in order, every word is broadcast and lane L answers for bit L -- its output slot is the
// count of set bits before the word plus the set bits of the word that stand for earlier
// positions.  The lanes with a set bit write consecutive slots, so the stores are already
// compacted and coalesced and nothing is staged in shared memory; slots and positions are 32-bit
// values relative to the warp's first slot and first position, and the store is predicated.
// (History on a 2^28-element mask, half of it set.  Every thread expanding its own 16 flags into
// a shared-memory list, one loop turn per set bit, and the block copying the list out: 193 us,
// issue-bound.  Lane per bit with 64-bit slots and a branch around the store: 20 - 25 instructions
// per word, 192 - 226 us.  This form, ten instructions per word: 182 us; what bounds it now is
// the SM-to-L2 request path, 83 % busy, with 1.19 sectors sent per sector of output because a
// warp's run of slots starts anywhere.  Staging the list in shared memory again to send whole
// aligned sectors cost more instructions than it saved requests: 215 us.)
constexpr int kMsWordsPerWarp = kMsTile / 32 / (kMsThreads / 32);  // 64
static_assert(kMsWordsPerWarp == 64, "a lane holds two words of its warp's share");
__global__ void __launch_bounds__(kMsThreads) mask_select_kernel(const uint32_t* flag_bits, const unsigned* tile_counts,
                                                                 const unsigned long long* group_offsets,
                                                                 int64_t* out, int64_t capacity) {
  __shared__ unsigned warp_tot[kMsThreads / 32];
  __shared__ unsigned long long base_s;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  if (t < 32) {
    // this tile's first output slot: the group's offset + the counts of the group's earlier tiles
    const int64_t g0 = static_cast<int64_t>(blockIdx.x) / kScanItems * kScanItems;
    unsigned c0 = (t < kScanItems && g0 + t < static_cast<int64_t>(blockIdx.x)) ? tile_counts[g0 + t] : 0u;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) c0 += __shfl_xor_sync(0xffffffffu, c0, d);
    if (t == 0) base_s = group_offsets[blockIdx.x / kScanItems] + c0;
  }
  const int64_t word0 = (static_cast<int64_t>(blockIdx.x) * (kMsThreads / 32) + w) * kMsWordsPerWarp;
  const uint32_t wa = flag_bits[word0 + lane], wb = flag_bits[word0 + 32 + lane];
  // set bits in the warp's earlier words, for both of the lane's words by one scan (a half holds
  // at most 1024 set bits: 16 bits each).  The loop below fetches them with a shuffle rather than
  // counting every word twice: the population-count unit runs at 16 lanes per clock.
  const unsigned ca = __popc(wa), cb = __popc(wb);
  unsigned x = ca | (cb << 16);
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  const unsigned both = __shfl_sync(0xffffffffu, x, 31);
  const unsigned pa = (x & 0xffffu) - ca, pb = (both & 0xffffu) + (x >> 16) - cb;
  if (lane == 0) warp_tot[w] = (both & 0xffffu) + (both >> 16);
  // the position within a word that bit L stands for, and the bits that stand for earlier ones
  const int mine_at = 16 * (lane >> 4) + element_of_flag_bit(lane & 15);
  uint32_t earlier = 0;
#pragma unroll
  for (int f = 0; f < 32; ++f)
    if (16 * (f >> 4) + element_of_flag_bit(f & 15) < mine_at) earlier |= 1u << f;
  __syncthreads();
  unsigned before = 0;
#pragma unroll
  for (int ww = 0; ww < kMsThreads / 32; ++ww)
    if (ww < w) before += warp_tot[ww];
  const int64_t first_slot = static_cast<int64_t>(base_s) + before;
  int64_t* const outp = out + first_slot;
  // word0 * 32 is a multiple of 2048 and the warp covers 2048 positions: the low half never carries
  const unsigned long long pos0 = static_cast<unsigned long long>(word0) * 32u;
  const uint32_t pos_hi = static_cast<uint32_t>(pos0 >> 32), pos_lo = static_cast<uint32_t>(pos0) + mine_at;
  const uint32_t my_bit = 1u << lane;
  if (capacity - first_slot >= kMsWordsPerWarp * 32) {
    // every slot of this warp exists (the usual case)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint32_t mine = half ? wb : wa;
      const unsigned mine_before = half ? pb : pa;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const uint32_t word = __shfl_sync(0xffffffffu, mine, i);
        const unsigned slot = __shfl_sync(0xffffffffu, mine_before, i) + __popc(word & earlier);
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .u64 a;\n\t"
            "setp.ne.u32 p, %4, 0;\n\t"
            "mad.wide.u32 a, %1, 8, %0;\n\t"
            "@p st.global.v2.u32 [a], {%2, %3};\n\t}"
            :: "l"(outp), "r"(slot), "r"(pos_lo + (half * 32 + i) * 32), "r"(pos_hi), "r"(word & my_bit)
            : "memory");
      }
    }
  } else {
    // the caller's buffer ends inside this warp's share (or before it): checked stores
    const int64_t room = capacity - first_slot;
    unsigned o = 0;
    for (int i = 0; i < kMsWordsPerWarp; ++i) {
      const uint32_t word = __shfl_sync(0xffffffffu, i < 32 ? wa : wb, i & 31);
      const int64_t slot = o + __popc(word & earlier);
      if ((word & my_bit) && slot < room)
        outp[slot] = static_cast<int64_t>((static_cast<unsigned long long>(pos_hi) << 32) | (pos_lo + i * 32));
      o += __popc(word);
    }
  }
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
  const int64_t count_blocks = std::min<int64_t>(ntiles, int64_t{sm_count(scope.device())} * kMsCountBlocksPerSm);
  mask_count_kernel<<<static_cast<unsigned>(count_blocks), kMsThreads, 0, s>>>(p, counts, flag_words, ntiles);
  VB_LAUNCH_CHECK();
  mask_scan_kernel<<<1, 1024, 0, s>>>(counts, offsets, ntiles, reinterpret_cast<unsigned long long*>(count_out));
  VB_LAUNCH_CHECK();
  if (capacity > 0) {
    mask_select_kernel<<<static_cast<unsigned>(ntiles), kMsThreads, 0, s>>>(reinterpret_cast<const uint32_t*>(flag_words), counts, offsets,
                                                                              out_indices, capacity);
    VB_LAUNCH_CHECK();
  }
  note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_MASK_SELECT, dim3(static_cast<unsigned>(ntiles)), dim3(kMsThreads), 16,
              1, 0, capacity > 0 ? 3 : 2, n, n, need, s);
  return VBT_B200_OK;
}

}  // extern "C"
