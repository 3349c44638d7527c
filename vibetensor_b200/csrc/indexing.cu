// Row gather, row scatter / scatter-add, last-dim index / index_put (sm_100a).
//
// Replaces embedding_gather_f32_kernel / embedding_backward_accum_f32_kernel (one thread
// and one 64-bit division per scalar, grid capped at 65 535 blocks;
// src/vbt/ops/embedding_cuda.cu:47-87), advanced_index_cuda_kernel /
// advanced_index_put_cuda_kernel (per-element coordinate decode;
// src/vbt/core/indexing_advanced_cuda.cu:1325-1453) and the Triton gather / scatter_add
// kernels (vibe_kernels/indexing/kernels.py:13-186).
//
//   gather        the output is a flat run of 16-byte chunks; a thread moves four chunks,
//                 a warp always covers 512 contiguous bytes of one table row.
//   scatter-add   a block takes 256 updates, sorts their (row, position) keys in shared
//                 memory, and each warp walks 32 sorted entries: equal rows are summed in
//                 registers (in update order) and leave the block as ONE vector atomic per
//                 16-byte chunk (red.global.add.v4.f32 / 64-bit integer atomics).  With
//                 Zipf-distributed rows this removes most same-address atomic traffic.
//
// Bad indices never fault: they are skipped and counted in the caller's status block.
#include <climits>
#include <mutex>

#include "bulk_copy.cuh"
#include "common.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;

struct IndexSrc {
  const void* idx;
  int is32;
  __device__ __forceinline__ int64_t get(int64_t i) const {
    return is32 ? static_cast<int64_t>(static_cast<const int32_t*>(idx)[i])
                : static_cast<const int64_t*>(idx)[i];
  }
};

// returns false for an index that must be skipped (and records it)
__device__ __forceinline__ bool normalize(int64_t& v, int64_t V, int policy, unsigned long long* status,
                                          bool record) {
  if (policy == VBT_B200_INDEX_CLAMP) {
    v = v < 0 ? 0 : (v > V - 1 ? V - 1 : v);
    if (V > 0) return true;
  } else {
    const int64_t raw = v;
    if (policy == VBT_B200_INDEX_WRAP && v < 0) v += V;
    if (v >= 0 && v < V) return true;
    v = raw;
  }
  if (record && status) {
    if (atomicAdd(&status[0], 1ull) == 0ull) status[1] = static_cast<unsigned long long>(v);
  }
  return false;
}

// 16-byte chunks per thread.  Measured on 4 M random 1 KiB rows: 1 -> 0.77, 2 -> 0.91 - 0.92, 4 -> 0.86 -
// 0.88, 8 -> 0.75, 16 -> 0.46 of the copy bandwidth (the same order on 256-byte and 4 KiB rows).
#ifndef VB_GATHER_U
#define VB_GATHER_U 2
#endif
constexpr int kGatherU = VB_GATHER_U;
struct GatherParams {
  const char* table;
  char* out;
  IndexSrc idx;
  int64_t N, V;
  int64_t row_stride_bytes;
  uint32_t cpr;       // 16-byte chunks per row
  FastDiv div_cpr;
  int64_t total;      // N * cpr
  int policy;
  unsigned long long* status;
  int scatter;        // 0: out[i] = table[idx[i]]   1: table[idx[i]] = out[i]
};

// chunk-flat row copy, both directions
__global__ void __launch_bounds__(kThreads) rows_copy_kernel(const __grid_constant__ GatherParams p) {
  constexpr int U = kGatherU;
  const int64_t g0 = static_cast<int64_t>(blockIdx.x) * (kThreads * U) + threadIdx.x;
  int4 data[U];
  int64_t dst_off[U];
  bool ok[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t g = g0 + u * kThreads;
    ok[u] = false;
    data[u] = make_int4(0, 0, 0, 0);
    if (g < p.total) {
      // N < 2^31 is guaranteed by the host; the 64-bit division only runs for huge outputs
      uint32_t row, c;
      if (p.total <= 0x7fffffff) {
        p.div_cpr.divmod(static_cast<uint32_t>(g), row, c);
      } else {
        row = static_cast<uint32_t>(g / p.cpr);
        c = static_cast<uint32_t>(g - static_cast<int64_t>(row) * p.cpr);
      }
      int64_t v = p.idx.get(row);
      const bool good = normalize(v, p.V, p.policy, p.status, c == 0);
      const int64_t toff = v * p.row_stride_bytes + static_cast<int64_t>(c) * 16;
      if (!p.scatter) {
        ok[u] = true;
        dst_off[u] = g * 16;
        if (good) data[u] = *reinterpret_cast<const int4*>(p.table + toff);
      } else if (good) {
        ok[u] = true;
        dst_off[u] = toff;
        data[u] = *reinterpret_cast<const int4*>(p.out + g * 16);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (ok[u]) {
      char* dst = p.scatter ? const_cast<char*>(p.table) : p.out;
      *reinterpret_cast<int4*>(dst + dst_off[u]) = data[u];
    }
  }
}

// element-wise fallback: any element size, any strides
struct ElemParams {
  const char* table;
  char* out;
  IndexSrc idx;
  int64_t N, V, D;
  int64_t s0, s1;  // table strides, elements
  int es;
  int policy;
  unsigned long long* status;
  int scatter;
};
__global__ void __launch_bounds__(kThreads) rows_copy_elem_kernel(const __grid_constant__ ElemParams p) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (e >= p.N * p.D) return;
  const int64_t row = e / p.D, j = e - row * p.D;
  int64_t v = p.idx.get(row);
  const bool good = normalize(v, p.V, p.policy, p.status, j == 0);
  const char* t = p.table + (v * p.s0 + j * p.s1) * p.es;
  char* o = p.out + e * p.es;
  if (!p.scatter) {
    for (int b = 0; b < p.es; ++b) o[b] = good ? t[b] : 0;
  } else if (good) {
    char* tw = const_cast<char*>(t);
    for (int b = 0; b < p.es; ++b) tw[b] = o[b];
  }
}

// ------------------------------------------------------------------------------------
// scatter-add with in-block duplicate aggregation
// ------------------------------------------------------------------------------------
constexpr uint64_t kSkipKey = ~0ull;

struct ScatterParams {
  char* table;
  const char* values;
  IndexSrc idx;
  int64_t N, V;
  uint32_t cpr;  // 16-byte chunks per row
  int policy;
  unsigned long long* status;
  int use_padding;
  int64_t padding_idx;
  const unsigned* counts;  // float tables only: scale every row's sum by 1 / counts[row] (may be null)
};

template <class T> struct AddVec;
template <> struct AddVec<float> {
  using acc_t = float4;
  __device__ static acc_t zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ static void add(acc_t& a, const int4& raw) {
    a.x += __int_as_float(raw.x); a.y += __int_as_float(raw.y);
    a.z += __int_as_float(raw.z); a.w += __int_as_float(raw.w);
  }
  __device__ static void flush(char* dst, const acc_t& a) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a.x), "f"(a.y),
                 "f"(a.z), "f"(a.w) : "memory");
  }
};
template <> struct AddVec<int64_t> {
  struct acc_t { unsigned long long a, b; };
  __device__ static acc_t zero() { return acc_t{0ull, 0ull}; }
  __device__ static void add(acc_t& a, const int4& raw) {
    a.a += (static_cast<unsigned long long>(static_cast<unsigned>(raw.y)) << 32) | static_cast<unsigned>(raw.x);
    a.b += (static_cast<unsigned long long>(static_cast<unsigned>(raw.w)) << 32) | static_cast<unsigned>(raw.z);
  }
  __device__ static void flush(char* dst, const acc_t& a) {
    atomicAdd(reinterpret_cast<unsigned long long*>(dst), a.a);
    atomicAdd(reinterpret_cast<unsigned long long*>(dst) + 1, a.b);
  }
};
template <> struct AddVec<int32_t> {
  using acc_t = uint4;
  __device__ static acc_t zero() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ static void add(acc_t& a, const int4& raw) {
    a.x += static_cast<unsigned>(raw.x); a.y += static_cast<unsigned>(raw.y);
    a.z += static_cast<unsigned>(raw.z); a.w += static_cast<unsigned>(raw.w);
  }
  __device__ static void flush(char* dst, const acc_t& a) {
    unsigned* d = reinterpret_cast<unsigned*>(dst);
    atomicAdd(d, a.x); atomicAdd(d + 1, a.y); atomicAdd(d + 2, a.z); atomicAdd(d + 3, a.w);
  }
};

// Block-local aggregation in front of the atomics.  A block takes kRingBatch consecutive updates,
// sorts their (row, position) keys in shared memory so that equal rows are adjacent and in update
// order, and every warp then walks its share of the sorted keys: it adds up runs of equal rows in
// registers and sends one vector atomic per run and 16-byte chunk.  With 1024 updates per block
// the Zipf(1.1) workload issues 0.53 atomics per update (256 per block: 0.65; 4096: 0.43, but
// the sort and the lower occupancy cost more than that saves).
// The value rows come in by asynchronous copies: every warp owns a ring of row slots in shared
// memory (8 KiB: eight rows of 1 KiB) and keeps that many rows in flight while it adds up the oldest one.  A lane reads
// back only the 16-byte chunks it copied itself, so the ring needs no barrier:
// cp.async.wait_group orders a lane's own copies.  K = 16-byte chunks per lane and row pass.
#ifndef VB_SCATTER_RING_DEPTH
#define VB_SCATTER_RING_DEPTH 8
#endif
constexpr int kRingBytesPerWarp = VB_SCATTER_RING_DEPTH * 1024;  // 8 rows of 1 KiB in flight per warp; fewer, wider slots for wider rows
#ifndef VB_SCATTER_BATCH
#define VB_SCATTER_BATCH 1024
#endif
constexpr int kRingBatch = VB_SCATTER_BATCH;  // updates per block: the larger, the more duplicates meet before the atomics
constexpr int kPosBits = 12;                  // kRingBatch <= 4096
template <class T, int K>
__global__ void __launch_bounds__(kThreads) scatter_add_ring_kernel(const __grid_constant__ ScatterParams p) {
  using AV = AddVec<T>;
  using acc_t = typename AV::acc_t;
  constexpr int kRing = kRingBytesPerWarp / (K * 512) > 8 ? 8 : kRingBytesPerWarp / (K * 512);
  extern __shared__ __align__(16) unsigned char ring_raw[];  // [sorted keys][warp][slot][K * 32 lanes] 16-byte chunks
  uint64_t* const keys = reinterpret_cast<uint64_t*>(ring_raw);  // (row << kPosBits) | position, sorted
  unsigned char* const ring0 = ring_raw + kRingBatch * 8;
  const int t = threadIdx.x;
  const int64_t b0 = static_cast<int64_t>(blockIdx.x) * kRingBatch;
#pragma unroll
  for (int u = 0; u < kRingBatch / kThreads; ++u) {
    uint64_t key = kSkipKey;
    const int pos = u * kThreads + t;
    const int64_t i = b0 + pos;
    if (i < p.N) {
      int64_t v = p.idx.get(i);
      if (!(p.use_padding && v == p.padding_idx)) {
        if (normalize(v, p.V, p.policy, p.status, true))
          key = (static_cast<uint64_t>(v) << kPosBits) | static_cast<uint64_t>(pos);
      }
    }
    keys[pos] = key;
  }
  __syncthreads();
  // bitonic sort of the block's keys; equal rows end up adjacent and in update order
  for (int k = 2; k <= kRingBatch; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
      for (int u = 0; u < kRingBatch / kThreads / 2; ++u) {
        // the u-th pair of this thread: i has bit j clear
        const int h = u * kThreads + t;
        const int i = ((h & ~(j - 1)) << 1) | (h & (j - 1));
        const uint64_t a = keys[i], b = keys[i | j];
        const bool up = (i & k) == 0;
        if ((a > b) == up) { keys[i] = b; keys[i | j] = a; }
      }
      __syncthreads();
    }
  }
  constexpr int kPerWarp = kRingBatch / (kThreads / 32);
  const int lane = t & 31, w = t >> 5;
  const int e_begin = w * kPerWarp;
  const int64_t row_bytes = static_cast<int64_t>(p.cpr) * 16;
  constexpr uint32_t kSlotBytes = K * 32 * 16;
  const uint32_t my_ring = smem_addr(ring0) + static_cast<uint32_t>(w) * (kRing * kSlotBytes) + static_cast<uint32_t>(lane) * 16u;
  for (uint32_t cb = 0; cb < p.cpr; cb += 32 * K) {  // column block of 32*K chunks
    acc_t acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = AV::zero();
    uint64_t cur = kSkipKey;  // current row (key >> 8), kSkipKey = none
    auto flush = [&](uint64_t row) {
      char* dst = p.table + static_cast<int64_t>(row) * row_bytes;
      if constexpr (std::is_same_v<T, float>) {
        if (p.counts != nullptr) {  // scale_grad_by_freq: this block's share of the row, over the row's count
          const float sc = 1.0f / static_cast<float>(p.counts[row]);
#pragma unroll
          for (int k = 0; k < K; ++k) { acc[k].x *= sc; acc[k].y *= sc; acc[k].z *= sc; acc[k].w *= sc; }
        }
      }
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const uint32_t c = cb + k * 32 + lane;
        if (c < p.cpr) AV::flush(dst + static_cast<int64_t>(c) * 16, acc[k]);
        acc[k] = AV::zero();
      }
    };
    // entry e of this warp -> ring slot e % kRing; one commit group per entry, empty for skipped ones
    auto issue = [&](int e) {
      if (e < kPerWarp) {
        const uint64_t key = keys[e_begin + e];
        if (key != kSkipKey) {
          const char* src = p.values + (b0 + static_cast<int64_t>(key & ((1u << kPosBits) - 1u))) * row_bytes;
#pragma unroll
          for (int k = 0; k < K; ++k) {
            const uint32_t c = cb + k * 32 + lane;
            if (c < p.cpr)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(my_ring + (e % kRing) * kSlotBytes + k * 512u),
                           "l"(src + static_cast<int64_t>(c) * 16)
                           : "memory");
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int e = 0; e < kRing; ++e) issue(e);
#pragma unroll 1
    for (int e0 = 0; e0 < kPerWarp; e0 += kRing) {
#pragma unroll
      for (int r = 0; r < kRing; ++r) {
        const int e = e0 + r;
        asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");
        const uint64_t key = keys[e_begin + e];
        if (key != kSkipKey) {  // skipped entries sort to the end
          const uint64_t row = key >> kPosBits;
          if (row != cur) {
            if (cur != kSkipKey) flush(cur);
            cur = row;
          }
#pragma unroll
          for (int k = 0; k < K; ++k) {
            const uint32_t c = cb + k * 32 + lane;
            if (c < p.cpr) {
              int4 raw;
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                           : "r"(my_ring + r * kSlotBytes + k * 512u));
              AV::add(acc[k], raw);
            }
          }
        }
        issue(e + kRing);  // the slot just read is free again (same lane wrote and read it)
      }
    }
    if (cur != kSkipKey) flush(cur);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
}

// element-wise atomic fallback (rows that are not whole aligned 16-byte chunks)
struct ScatterElemParams {
  char* table;
  const char* values;
  IndexSrc idx;
  int64_t N, V, D;
  int policy;
  unsigned long long* status;
  int use_padding;
  int64_t padding_idx;
  const unsigned* counts;  // as ScatterParams::counts
};
template <class T>
__device__ __forceinline__ void atomic_add_elem(T* dst, T v);
template <> __device__ __forceinline__ void atomic_add_elem<float>(float* d, float v) { atomicAdd(d, v); }
template <> __device__ __forceinline__ void atomic_add_elem<int64_t>(int64_t* d, int64_t v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(d), static_cast<unsigned long long>(v));
}
template <> __device__ __forceinline__ void atomic_add_elem<int32_t>(int32_t* d, int32_t v) { atomicAdd(d, v); }

template <class T>
__global__ void __launch_bounds__(kThreads) scatter_add_elem_kernel(const __grid_constant__ ScatterElemParams p) {
  const int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (e >= p.N * p.D) return;
  const int64_t row = e / p.D, j = e - row * p.D;
  int64_t v = p.idx.get(row);
  if (p.use_padding && v == p.padding_idx) return;
  if (!normalize(v, p.V, p.policy, p.status, j == 0)) return;
  T val = reinterpret_cast<const T*>(p.values)[e];
  if constexpr (std::is_same_v<T, float>) {
    if (p.counts != nullptr) val *= 1.0f / static_cast<float>(p.counts[v]);
  }
  atomic_add_elem<T>(reinterpret_cast<T*>(p.table) + v * p.D + j, val);
}

// occurrences of every in-range, non-padding row (embedding_count_by_freq_i64_kernel,
// src/vbt/ops/embedding_cuda.cu:89-103); bad indices are reported by the accumulate pass
__global__ void __launch_bounds__(kThreads) count_rows_kernel(IndexSrc idx, int64_t N, int64_t V, int policy,
                                                              int use_padding, int64_t padding_idx,
                                                              unsigned* counts) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < N;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    int64_t v = idx.get(i);
    if (use_padding && v == padding_idx) continue;
    if (!normalize(v, V, policy, nullptr, false)) continue;
    atomicAdd(&counts[v], 1u);
  }
}

// ------------------------------------------------------------------------------------
// sorted scatter-add: radix-sort (row, position) pairs, then accumulate runs
//
// The block-local aggregation above still sends one atomic per distinct row PER BLOCK; with
// 64-bit integer rows (256 scalar atomics per 2 KiB row) the L2 atomic units, not HBM, set
// the pace.  Sorting ALL updates by destination row first makes every row one contiguous
// run: a warp walks 32 sorted entries, sums each run in update order in registers, and a
// run that lies wholly inside the warp's slice is the ONLY writer of its row, so it starts
// from the row's old contents and ends with a plain store.  Only runs that cross a slice
// boundary (rows with more updates than a slice holds) use atomics.  Results are exact for
// integers; for fp32 every row updated from a single slice is old + u1 + u2 + ... in update
// order -- bit-identical to a sequential loop -- and independent of scheduling.
//
// Sort: LSD radix, 8 bits per pass over just the bits the row range needs; per pass a
// block histogram, one exclusive scan, and a stable scatter (ranks from per-bit ballots).
// ------------------------------------------------------------------------------------
constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;                            // per thread
constexpr int kSortTile = kSortThreads * kSortItems;      // 4096 items per block
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kWarpChunk = kSortTile / kSortWarps;        // 512 consecutive items per warp

struct KeyParams {
  IndexSrc idx;
  int64_t N, V;
  int policy;
  unsigned long long* status;
  int use_padding;
  int64_t padding_idx;
  uint32_t* keys;
  uint32_t* vals;
};
// Least-significant-digit radix sort of (key = destination row, value = update position), RB bits
// per pass: 8, or 11 for tables of 257 .. 2047 rows (one pass instead of two).
// Every pass is three launches -- per-block digit counts, a scan over (digit, block), a stable
// scatter -- and the first pass's count kernel also makes the keys from the index tensor
// (key = V for an update that must be skipped: it sorts last).

// Lanes of the warp that hold the same digit as this lane (this lane included); lanes with
// valid == false match nobody.  One ballot per digit bit: the hardware's match.any measured slower
// the more lanes agree -- the pass over the skewed high digit took twice the time of the others.
template <int BITS>
__device__ __forceinline__ unsigned same_digit_lanes(uint32_t digit, bool valid) {
  unsigned peers = __ballot_sync(0xffffffffu, valid);
#pragma unroll
  for (int b = 0; b < BITS; ++b) {
    const bool bit = (digit >> b) & 1u;
    const unsigned m = __ballot_sync(0xffffffffu, bit);
    peers &= bit ? m : ~m;
  }
  return valid ? peers : 0u;
}

// hist[d * nblocks + b] = number of items of block b whose digit is d
// and totals[d] += the same counts (totals is zero on entry)
template <int RB, bool FIRST>
__global__ void __launch_bounds__(kSortThreads) radix_hist_kernel(const __grid_constant__ KeyParams kp, const uint32_t* keys,
                                                                  int64_t n, uint32_t mul, int shift, uint32_t* hist,
                                                                  int nblocks, uint32_t* totals) {
  constexpr int NB = 1 << RB;
  __shared__ uint32_t h[NB];
  for (int d = threadIdx.x; d < NB; d += kSortThreads) h[d] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSortTile;
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t i = base + k * kSortThreads + threadIdx.x;
    uint32_t digit = 0;
    if (i < n) {
      uint32_t key;
      if constexpr (FIRST) {
        int64_t v = kp.idx.get(i);
        key = static_cast<uint32_t>(kp.V);
        if (!(kp.use_padding && v == kp.padding_idx)) {
          if (normalize(v, kp.V, kp.policy, kp.status, true)) key = static_cast<uint32_t>(v);
        }
        kp.keys[i] = key;
        kp.vals[i] = static_cast<uint32_t>(i);
      } else {
        key = keys[i];
      }
      digit = ((key * mul) >> shift) & (NB - 1);
    }
    // one shared-memory atomic per distinct digit of the warp: a hot row puts many equal digits in a warp
    const unsigned peers = same_digit_lanes<RB>(digit, i < n);
    if (peers && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&h[digit], static_cast<uint32_t>(__popc(peers)));
  }
  __syncthreads();
  for (int d = threadIdx.x; d < NB; d += kSortThreads) {
    hist[static_cast<int64_t>(d) * nblocks + blockIdx.x] = h[d];
    if (h[d]) atomicAdd(&totals[d], h[d]);
  }
}

// block d turns row d of hist ([2^RB][nblocks], counts) into output start offsets:
// (items with a smaller digit) + (items with digit d in earlier blocks)
template <int RB>
__global__ void __launch_bounds__(1024) radix_scan_kernel(uint32_t* hist, int nblocks, const uint32_t* totals) {
  constexpr int NB = 1 << RB;
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t base_s;
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const int d = blockIdx.x;
  auto block_inclusive = [&](uint32_t v) {  // inclusive scan over the 1024 threads
#pragma unroll
    for (int k = 1; k < 32; k <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, v, k);
      if (lane >= k) v += y;
    }
    __syncthreads();  // warp_sums may still be read from the previous use
    if (lane == 31) warp_sums[w] = v;
    __syncthreads();
    if (w == 0) {
      uint32_t s = warp_sums[lane], si = s;
#pragma unroll
      for (int k = 1; k < 32; k <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, si, k);
        if (lane >= k) si += y;
      }
      warp_sums[lane] = si - s;
    }
    __syncthreads();
    return v + warp_sums[w];
  };
  uint32_t mine = 0;
  for (int tt = t; tt < NB; tt += 1024)
    if (tt < d) mine += totals[tt];
  const uint32_t below = block_inclusive(mine);  // thread 1023 holds the full sum
  if (t == 1023) base_s = below;
  __syncthreads();
  uint32_t carry = base_s;
  uint32_t* row = hist + static_cast<int64_t>(d) * nblocks;
  for (int b0 = 0; b0 < nblocks; b0 += 1024) {
    const int b = b0 + t;
    const uint32_t c = b < nblocks ? row[b] : 0u;
    const uint32_t incl = block_inclusive(c);
    if (b < nblocks) row[b] = carry + incl - c;
    __syncthreads();
    if (t == 1023) base_s = carry + incl;
    __syncthreads();
    carry = base_s;
  }
}

// Stable scatter of one 4096-item tile by the current digit.  The tile is first put in digit order
// in shared memory (rank within the warp's run by per-bit ballots, then warp and digit prefixes), and
// only then written out: consecutive threads write consecutive addresses of a digit's run.  (The
// first form wrote every item straight to its final place -- 32 lanes, up to 32 sectors per store
// -- and took 43 us per pass on 4 M items where the traffic is worth 11 us.)
template <int RB>
__global__ void __launch_bounds__(kSortThreads, 3) radix_scatter_kernel(const uint32_t* keys_in, const uint32_t* vals_in,
                                                                     uint32_t* keys_out, uint32_t* vals_out,
                                                                     int64_t n, uint32_t mul, int shift,
                                                                     const uint32_t* hist, int nblocks) {
  constexpr int NB = 1 << RB;
  extern __shared__ uint32_t scat_raw[];  // [kSortWarps][NB] counts, [NB] tile starts, [NB] output bases, keys, values
  uint32_t* const cnt_raw = scat_raw;
  uint32_t* const tstart = cnt_raw + kSortWarps * NB;
  uint32_t* const gbase = tstart + NB;
  uint32_t* const sk = gbase + NB;
  uint32_t* const sv = sk + kSortTile;
  __shared__ uint32_t scan_warp[kSortWarps];
  auto cnt = [&](int ww, uint32_t d) -> uint32_t& { return cnt_raw[ww * NB + d]; };
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  for (int i = t; i < kSortWarps * NB; i += kSortThreads) cnt_raw[i] = 0;
  __syncthreads();
  // a warp owns 512 CONSECUTIVE items and takes them 32 at a time, so "earlier in the
  // array" == (earlier warp) or (same warp, earlier round) or (same round, lower lane)
  const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kSortTile;
  const int64_t wbase = tile0 + w * kWarpChunk;
  uint32_t key[kSortItems], val[kSortItems], rank[kSortItems];
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    const bool valid = i < n;
    key[r] = valid ? keys_in[i] : 0u;
    val[r] = valid ? vals_in[i] : 0u;
  }
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    const bool valid = i < n;
    const uint32_t d = ((key[r] * mul) >> shift) & (NB - 1);
    const unsigned peers = same_digit_lanes<RB>(d, valid);
    const uint32_t before = __popc(peers & ((1u << lane) - 1u));
    rank[r] = valid ? cnt(w, d) + before : 0u;
    __syncwarp();
    if (valid && before == 0) cnt(w, d) += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  // per digit: the warps' counts become their exclusive prefix, the sum is the tile's count
  constexpr int DPT = NB / kSortThreads;  // digits per thread (consecutive): 1 or 8
  uint32_t mine[DPT], run = 0;
#pragma unroll
  for (int k = 0; k < DPT; ++k) {
    const int d = t * DPT + k;
    uint32_t tot = 0;
#pragma unroll
    for (int ww = 0; ww < kSortWarps; ++ww) {
      const uint32_t c = cnt(ww, d);
      cnt(ww, d) = tot;
      tot += c;
    }
    mine[k] = tot;
    run += tot;
  }
  // exclusive scan of the tile's digit counts over the block
  uint32_t x = run;
#pragma unroll
  for (int dd = 1; dd < 32; dd <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, dd);
    if (lane >= dd) x += y;
  }
  if (lane == 31) scan_warp[w] = x;
  __syncthreads();
  uint32_t before_me = x - run;
#pragma unroll
  for (int ww = 0; ww < kSortWarps; ++ww)
    if (ww < w) before_me += scan_warp[ww];
#pragma unroll
  for (int k = 0; k < DPT; ++k) {
    const int d = t * DPT + k;
    tstart[d] = before_me;
    // where digit d's run of this tile starts in the output, minus its start inside the tile
    gbase[d] = hist[static_cast<int64_t>(d) * nblocks + blockIdx.x] - before_me;
    before_me += mine[k];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    if (i < n) {
      const uint32_t d = ((key[r] * mul) >> shift) & (NB - 1);
      const uint32_t pos = tstart[d] + cnt(w, d) + rank[r];
      sk[pos] = key[r];
      sv[pos] = val[r];
    }
  }
  __syncthreads();
  const int64_t left = n - tile0;
  const uint32_t tile_n = static_cast<uint32_t>(left < kSortTile ? left : kSortTile);
  for (uint32_t i = t; i < tile_n; i += kSortThreads) {
    const uint32_t k = sk[i];
    const uint32_t dst = gbase[((k * mul) >> shift) & (NB - 1)] + i;
    keys_out[dst] = k;
    vals_out[dst] = sv[i];
  }
}

struct SortedScatterParams {
  char* table;
  const char* values;
  const uint32_t* keys;   // sorted rows; V = skip
  const uint32_t* vals;   // original update positions
  int64_t N, V;
  uint32_t cpr;
};

// One warp per slice of kSortedPerWarp consecutive sorted entries.  The warp walks the slice in
// order, adds up every run of equal rows in registers (in update order) and adds the run's sum
// to the row once, with the same vector atomics as the other engine -- exact for the integer
// tables this engine is the default for; a float row receives `row + (u1 + u2 + ...)`.  A run
// that spills into the next slice is finished by that slice's warp with an add of its own: with
// 256 entries per slice the hottest row of the Zipf(1.1) workload (13 % of all updates) takes
// 2 000 atomic adds per element instead of the 17 000 that 32-entry slices sent to one address.
// The value rows arrive through the warp's ring of kSortedRing shared-memory slots filled by
// asynchronous copies, so kSortedRing rows are in flight per warp at all times.
constexpr int kSortedRing = 8;
constexpr int kSortedPerWarp = 256;
template <class T, int K>
__global__ void __launch_bounds__(kThreads) scatter_add_sorted_kernel(const __grid_constant__ SortedScatterParams p) {
  using AV = AddVec<T>;
  using acc_t = typename AV::acc_t;
  extern __shared__ __align__(16) unsigned char ring_raw[];  // [warp][slot][K * 32 lanes] 16-byte chunks, then keys, positions
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t slice = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + w;
  const int64_t s0 = slice * kSortedPerWarp;
  if (s0 >= p.N) return;
  const uint32_t skip = static_cast<uint32_t>(p.V);
  constexpr uint32_t kSlotBytes = K * 32 * 16;
  uint32_t* const my_keys = reinterpret_cast<uint32_t*>(ring_raw + (kThreads / 32) * kSortedRing * kSlotBytes) + w * (2 * kSortedPerWarp);
  uint32_t* const my_pos = my_keys + kSortedPerWarp;
#pragma unroll
  for (int u = 0; u < kSortedPerWarp / 32; ++u) {
    const int64_t me = s0 + u * 32 + lane;
    my_keys[u * 32 + lane] = me < p.N ? p.keys[me] : skip;
    my_pos[u * 32 + lane] = me < p.N ? p.vals[me] : 0u;
  }
  __syncwarp();
  const int64_t row_bytes = static_cast<int64_t>(p.cpr) * 16;
  const uint32_t my_ring = smem_addr(ring_raw) + static_cast<uint32_t>(w) * (kSortedRing * kSlotBytes) + static_cast<uint32_t>(lane) * 16u;
  for (uint32_t cb = 0; cb < p.cpr; cb += 32 * K) {
    acc_t acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = AV::zero();
    uint32_t cur = skip;  // row of the open run (skip = none)
    auto flush = [&](uint32_t row) {
      char* dst = p.table + static_cast<int64_t>(row) * row_bytes;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const uint32_t c = cb + k * 32 + lane;
        if (c < p.cpr) AV::flush(dst + static_cast<int64_t>(c) * 16, acc[k]);
        acc[k] = AV::zero();
      }
    };
    // entry e -> ring slot e % kSortedRing; one commit group per entry, empty for skipped ones
    auto issue = [&](int e) {
      if (e < kSortedPerWarp) {
        const uint32_t key = my_keys[e];
        if (key != skip) {
          const char* src = p.values + static_cast<int64_t>(my_pos[e]) * row_bytes;
#pragma unroll
          for (int k = 0; k < K; ++k) {
            const uint32_t c = cb + k * 32 + lane;
            if (c < p.cpr)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(my_ring + (e % kSortedRing) * kSlotBytes + k * 512u),
                           "l"(src + static_cast<int64_t>(c) * 16)
                           : "memory");
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int e = 0; e < kSortedRing; ++e) issue(e);
#pragma unroll 1
    for (int e0 = 0; e0 < kSortedPerWarp; e0 += kSortedRing) {
#pragma unroll
      for (int r = 0; r < kSortedRing; ++r) {
        const int e = e0 + r;
        asm volatile("cp.async.wait_group %0;" ::"n"(kSortedRing - 1) : "memory");
        const uint32_t key = my_keys[e];
        if (key != skip) {  // skipped updates sort to the very end
          if (key != cur) {
            if (cur != skip) flush(cur);
            cur = key;
          }
#pragma unroll
          for (int k = 0; k < K; ++k) {
            const uint32_t c = cb + k * 32 + lane;
            if (c < p.cpr) {
              int4 raw;
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                           : "r"(my_ring + r * kSlotBytes + k * 512u));
              AV::add(acc[k], raw);
            }
          }
        }
        issue(e + kSortedRing);  // the slot just read is free again (same lane wrote and read it)
      }
    }
    if (cur != skip) flush(cur);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
}

// ------------------------------------------------------------------------------------
// last-dim index / index_put: out[r, k] = src[r, idx[k]], r running over the leading dims
// ------------------------------------------------------------------------------------
struct LastDimParams {
  char* self;       // [leading dims..., K0]: row r starts rows.offset(r) elements in, column stride sk
  char* other;      // dense [B, K]
  IndexSrc idx;
  int64_t B, K0, K, sk;
  DimList rows;     // the leading dims of self (any strides), collapsed where they merge
  int es;
  int policy;
  unsigned long long* status;
  int mode;  // 0 gather, 1 put overwrite, 2 put accumulate
  int dtype;
};
// A thread owns one index position k and walks kLdRows rows: the index is read and normalised
// once, writes (gather) / reads (put) of the dense operand are coalesced along k, and the
// kLdRows strided accesses to `self` are independent loads in flight.  E is an unsigned integer
// of the element size; accumulate uses the typed atomics.
constexpr int kLdRows = 8;
template <class E>
__global__ void __launch_bounds__(kThreads) lastdim_kernel(const __grid_constant__ LastDimParams p) {
  const int64_t k = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (k >= p.K) return;
  int64_t v = p.idx.get(k);
  const bool good = normalize(v, p.K0, p.policy, p.status, blockIdx.y == 0);
  E* self = reinterpret_cast<E*>(p.self) + v * p.sk;
  E* other = reinterpret_cast<E*>(p.other) + k;
  for (int64_t b0 = static_cast<int64_t>(blockIdx.y) * kLdRows; b0 < p.B;
       b0 += static_cast<int64_t>(gridDim.y) * kLdRows) {
    E val[kLdRows];
    int64_t off[kLdRows];
#pragma unroll
    for (int r = 0; r < kLdRows; ++r) off[r] = b0 + r < p.B ? p.rows.offset(static_cast<uint32_t>(b0 + r)) : 0;
    if (p.mode == 0) {
#pragma unroll
      for (int r = 0; r < kLdRows; ++r) val[r] = (good && b0 + r < p.B) ? self[off[r]] : E(0);
#pragma unroll
      for (int r = 0; r < kLdRows; ++r)
        if (b0 + r < p.B) other[(b0 + r) * p.K] = val[r];
    } else if (good) {
#pragma unroll
      for (int r = 0; r < kLdRows; ++r) val[r] = b0 + r < p.B ? other[(b0 + r) * p.K] : E(0);
#pragma unroll
      for (int r = 0; r < kLdRows; ++r) {
        if (b0 + r >= p.B) continue;
        E* d = self + off[r];
        if (p.mode == 1) {
          *d = val[r];
        } else if constexpr (sizeof(E) == 4) {
          if (p.dtype == VBT_B200_F32) atomicAdd(reinterpret_cast<float*>(d), __uint_as_float(val[r]));
          else atomicAdd(reinterpret_cast<unsigned*>(d), static_cast<unsigned>(val[r]));
        } else if constexpr (sizeof(E) == 8) {
          atomicAdd(reinterpret_cast<unsigned long long*>(d), static_cast<unsigned long long>(val[r]));
        }
      }
    }
  }
}

// Gather form for long rows.  The kernel above sends one 32-byte sector request through L1 per
// element (random positions): eight times the useful bytes on the L2 -> SM path, which
// saturates at about a third of HBM speed.  Here the index list -- the same for every row --
// is read ONCE per block and kept in registers (EPT entries per thread, position
// k = chunk start + j * blockDim + t), and the block then walks its rows: each row is brought
// into shared memory piece by piece with bulk asynchronous copies (two stages, so the next
// piece loads while the current one is served), every thread moves those of its entries that
// fall inside the piece from the staged piece into an OUTPUT tile that also lives in shared
// memory, and after the row's last piece the tile goes out with full 16-byte stores.  Global
// memory therefore sees only whole-sector traffic: the row read once per index chunk
// (coalesced) and every output sector written exactly once -- partial-sector writes, which
// cost a read-modify-write under ECC, never leave the SM.  Index lists longer than one block's
// tile are split over blockIdx.y (each such block stages the rows again; they come from L2).
// shared-memory accesses by 32-bit shared-space address: the inner loop below is issue-bound, and
// a generic pointer costs it an address conversion per access
__device__ __forceinline__ void sts(uint32_t a, uint8_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(static_cast<uint32_t>(v)) : "memory");
}
__device__ __forceinline__ void sts(uint32_t a, uint16_t v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"(v) : "memory"); }
__device__ __forceinline__ void sts(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts(uint32_t a, uint64_t v) {
  asm volatile("st.shared.u64 [%0], %1;" ::"r"(a), "l"(static_cast<unsigned long long>(v)) : "memory");
}

// v = shared[addr] if d < n (else v keeps its value) and shared[addr] = v if d < n, each as ONE
// predicated instruction: a branch around the access costs a divergence-stack round trip per
// entry, several times the access itself
__device__ __forceinline__ void lds_if_below(uint8_t& v, uint32_t d, uint32_t n, uint32_t addr) {
  uint32_t w = v;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p ld.shared.u8 %0, [%3];\n\t}" : "+r"(w) : "r"(d), "r"(n), "r"(addr));
  v = static_cast<uint8_t>(w);
}
__device__ __forceinline__ void lds_if_below(uint16_t& v, uint32_t d, uint32_t n, uint32_t addr) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p ld.shared.u16 %0, [%3];\n\t}" : "+h"(v) : "r"(d), "r"(n), "r"(addr));
}
__device__ __forceinline__ void lds_if_below(uint32_t& v, uint32_t d, uint32_t n, uint32_t addr) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p ld.shared.u32 %0, [%3];\n\t}" : "+r"(v) : "r"(d), "r"(n), "r"(addr));
}
__device__ __forceinline__ void lds_if_below(uint64_t& v, uint32_t d, uint32_t n, uint32_t addr) {
  unsigned long long w = v;
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %1, %2;\n\t@p ld.shared.u64 %0, [%3];\n\t}" : "+l"(w) : "r"(d), "r"(n), "r"(addr));
  v = w;
}
__device__ __forceinline__ void sts_if_below(uint32_t addr, uint8_t v, uint32_t d, uint32_t n) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %2, %3;\n\t@p st.shared.u8 [%0], %1;\n\t}" ::"r"(addr), "r"(static_cast<uint32_t>(v)), "r"(d), "r"(n) : "memory");
}
__device__ __forceinline__ void sts_if_below(uint32_t addr, uint16_t v, uint32_t d, uint32_t n) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %2, %3;\n\t@p st.shared.u16 [%0], %1;\n\t}" ::"r"(addr), "h"(v), "r"(d), "r"(n) : "memory");
}
__device__ __forceinline__ void sts_if_below(uint32_t addr, uint32_t v, uint32_t d, uint32_t n) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %2, %3;\n\t@p st.shared.u32 [%0], %1;\n\t}" ::"r"(addr), "r"(v), "r"(d), "r"(n) : "memory");
}
__device__ __forceinline__ void sts_if_below(uint32_t addr, uint64_t v, uint32_t d, uint32_t n) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %2, %3;\n\t@p st.shared.u64 [%0], %1;\n\t}" ::"r"(addr), "l"(static_cast<unsigned long long>(v)), "r"(d), "r"(n) : "memory");
}

constexpr int kStThreads = 1024;
constexpr int kStagedSmemMax = 220 * 1024;  // dynamic shared memory the staged kernel may ask for
static __device__ unsigned vb_index_fault;  // a bounded wait on a staged copy gave up

constexpr int kStMaxPieces = 30;
constexpr int kStMaxStages = 4;  // row pieces in flight + the one being served

// GROUPED (rows of several pieces): before the first row the block regroups its index entries by
// the piece their source position falls in -- a counting sort through shared memory, done once
// -- so that a warp's 32 * EPT entries are consecutive in that order and belong to one piece,
// sometimes two.  A warp then skips, with one uniform branch, every (row, piece) step that holds
// none of its entries: an entry is touched once per row instead of once per row and piece, which
// is what the issue slots and the shared-memory pipe were spent on.  A regrouped entry is one
// 32-bit word: source position in the high bits, output slot of the tile in the low KBITS.
template <class E, int EPT, bool GROUPED>
__global__ void __launch_bounds__(kStThreads, 1) lastdim_staged_kernel(const __grid_constant__ LastDimParams p,
                                                                       const int piece, const int npieces,
                                                                       const int use_bulk, const int nstages) {
  extern __shared__ __align__(128) unsigned char st_raw[];
  __shared__ __align__(8) uint64_t bars[kStMaxStages];
  __shared__ uint32_t bstart[kStMaxPieces + 2];  // GROUPED: first regrouped entry of every piece (+ dead, + end)
  __shared__ uint32_t cursor[kStMaxPieces + 1];
  constexpr int KBITS = EPT == 32 ? 15 : (EPT == 16 ? 14 : 13);  // bits of a tile slot (EPT * 1024 slots)
  constexpr uint32_t KMASK = (1u << KBITS) - 1u;
  constexpr uint32_t DEADV = (1u << (32 - KBITS)) - 1u;  // GROUPED: source field of an entry without a source
  const int t = threadIdx.x, lane = t & 31, w = t >> 5;
  const size_t stage_bytes = (static_cast<size_t>(piece) * sizeof(E) + 127) / 128 * 128;
  E* const obuf = reinterpret_cast<E*>(st_raw + nstages * stage_bytes);  // [EPT * kStThreads] output tile
  auto stage_ptr = [&](int st) { return reinterpret_cast<E*>(st_raw + st * stage_bytes); };
  const int64_t kc0 = static_cast<int64_t>(blockIdx.y) * (kStThreads * EPT);
  const int64_t left = p.K - kc0;
  const uint32_t ntile = static_cast<uint32_t>(left < kStThreads * EPT ? left : kStThreads * EPT);  // outputs of this block per row
  const uint32_t upiece = static_cast<uint32_t>(piece);
  const uint32_t k0 = static_cast<uint32_t>(p.K0);
  // this block's index entries.  Plain form: source position, 0xffffffff (in no piece) to skip.
  uint32_t v[EPT];
  uint32_t bad = 0;  // plain form: positions whose index is out of range (the gathered value is zero)
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const uint32_t slot = static_cast<uint32_t>(j) * kStThreads + t;
    v[j] = GROUPED ? ((DEADV << KBITS) | slot) : 0xffffffffu;
    if (slot < ntile) {
      int64_t x = p.idx.get(kc0 + slot);
      if (normalize(x, p.K0, p.policy, p.status, blockIdx.x == 0))
        v[j] = GROUPED ? ((static_cast<uint32_t>(x) << KBITS) | slot) : static_cast<uint32_t>(x);
      else
        bad |= 1u << j;
    }
  }
  if constexpr (GROUPED) {
    // counting sort of the block's entries by piece (dead entries -- bad index, or past the end of
    // the list -- form one more group at the end), through the shared memory the pipeline uses later
    uint32_t* scratch = reinterpret_cast<uint32_t*>(st_raw);
    for (int i = t; i <= npieces; i += kStThreads) cursor[i] = 0;
    __syncthreads();
    auto group_of = [&](uint32_t entry) {
      const uint32_t src = entry >> KBITS;
      return src == DEADV ? static_cast<uint32_t>(npieces) : src / upiece;
    };
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
      const uint32_t g = group_of(v[j]);
      const unsigned peers = __match_any_sync(0xffffffffu, g);
      if (lane == __ffs(peers) - 1) atomicAdd(&cursor[g], static_cast<uint32_t>(__popc(peers)));
    }
    __syncthreads();
    if (t == 0) {
      uint32_t run = 0;
      for (int i = 0; i <= npieces; ++i) {
        const uint32_t c = cursor[i];
        bstart[i] = run;
        cursor[i] = run;
        run += c;
      }
      bstart[npieces + 1] = run;  // == EPT * kStThreads
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
      const uint32_t g = group_of(v[j]);
      const unsigned peers = __match_any_sync(0xffffffffu, g);
      const int leader = __ffs(peers) - 1;
      uint32_t base = 0;
      if (lane == leader) base = atomicAdd(&cursor[g], static_cast<uint32_t>(__popc(peers)));
      base = __shfl_sync(0xffffffffu, base, leader);
      scratch[base + __popc(peers & ((1u << lane) - 1u))] = v[j];
    }
    __syncthreads();
    // a warp takes 32 * EPT consecutive regrouped entries
#pragma unroll
    for (int j = 0; j < EPT; ++j) v[j] = scratch[static_cast<uint32_t>(w) * (32 * EPT) + j * 32 + lane];
    __syncthreads();  // scratch is free again before the first row piece lands in it
  }
  if (use_bulk && t == 0) {
    for (int st = 0; st < nstages; ++st) mbar_init(&bars[st], 1);
    mbar_init_fence();
  }
  __syncthreads();
  constexpr int VE = 16 / sizeof(E);
  const bool vec_out = (reinterpret_cast<uintptr_t>(p.other) % 16 == 0) && (p.K % VE == 0) && (ntile % VE == 0);
  // (row, piece) pairs in the order this block visits them; `nb, nq` run nstages - 1 pairs ahead
  auto advance = [&](uint32_t& bb, int& qq) {
    if (++qq == npieces) {
      qq = 0;
      bb += gridDim.x;
    }
  };
  auto issue = [&](uint32_t bb, int qq, int stage) {  // thread 0 only; the stage's previous readers are past a barrier
    const uint32_t c0 = static_cast<uint32_t>(qq) * upiece;
    const uint32_t n = min(upiece, k0 - c0);
    const E* src = reinterpret_cast<const E*>(p.self) + p.rows.offset(bb) + c0;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const uint32_t bytes = n * static_cast<uint32_t>(sizeof(E));
    mbar_arrive_expect_tx(&bars[stage], bytes);
    bulk_copy_g2s(stage_ptr(stage), src, bytes, &bars[stage]);
  };
  // GROUPED: the regrouped entries this warp holds are [wr0, wr1)
  const uint32_t wr0 = static_cast<uint32_t>(w) * (32 * EPT), wr1 = wr0 + 32 * EPT;
  uint32_t b = blockIdx.x, nb = blockIdx.x;  // B < 2^31 (checked by the host)
  int q = 0, nq = 0;
  for (int st = 0; st + 1 < nstages; ++st) {  // fill the pipeline
    if (use_bulk && t == 0 && nb < p.B) issue(nb, nq, st);
    advance(nb, nq);
  }
  int stage = 0, ahead = nstages - 1;  // ahead: the stage the next copy goes to (consumed in the last iteration)
  uint32_t phase = 0;                   // parity of this stage's current use
  for (; b < p.B;) {
    const uint32_t c0 = static_cast<uint32_t>(q) * upiece;
    const uint32_t n = min(upiece, k0 - c0);
    E* const tl = stage_ptr(stage);
    if (use_bulk) {
      const bool ok = mbar_wait_bounded(&bars[stage], phase);
      if (__syncthreads_or(!ok)) {
        // give up: note the fault, let the copies that may still be in flight land, and leave
        if (t == 0) {
          atomicExch(&vb_index_fault, 1u);
          mbar_wait_bounded(&bars[stage], phase);
        }
        __syncthreads();
        return;
      }
      if (t == 0 && nb < p.B) issue(nb, nq, ahead);
    } else {
      __syncthreads();  // readers of the previous piece, and of the output tile, are done
      const E* src = reinterpret_cast<const E*>(p.self) + p.rows.offset(b) + c0;
      for (uint32_t i = t; i < n; i += kStThreads) tl[i] = src[i];
      __syncthreads();
    }
    advance(nb, nq);
    const uint32_t tl_s = smem_addr(tl);
    constexpr uint32_t ES = static_cast<uint32_t>(sizeof(E));
    constexpr int kBatch = 8;
    if constexpr (GROUPED) {
      const uint32_t ob_s = smem_addr(obuf);
      if (bstart[q] < wr1 && bstart[q + 1] > wr0) {  // this warp holds entries of piece q
        // batches of kBatch loads, then their stores: a store right behind its load would make
        // every entry wait out the shared-memory latency (the next load may not pass the store)
#pragma unroll
        for (int j0 = 0; j0 < EPT; j0 += kBatch) {
          E val[kBatch];
#pragma unroll
          for (int u = 0; u < kBatch; ++u) {
            const uint32_t d = (v[j0 + u] >> KBITS) - c0;
            val[u] = E(0);
            lds_if_below(val[u], d, n, tl_s + d * ES);
          }
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            sts_if_below(ob_s + (v[j0 + u] & KMASK) * ES, val[u], (v[j0 + u] >> KBITS) - c0, n);
        }
      }
      if (q == 0 && bstart[npieces] < wr1 && bstart[npieces + 1] > wr0) {  // ... or dead entries
#pragma unroll
        for (int j = 0; j < EPT; ++j)
          if ((v[j] >> KBITS) == DEADV && (v[j] & KMASK) < ntile) sts(ob_s + (v[j] & KMASK) * ES, E(0));
      }
    } else {
      // entry j of this thread lands in tile slot j * kStThreads + t
      const uint32_t ob_s = smem_addr(obuf) + static_cast<uint32_t>(t) * ES;
#pragma unroll
      for (int j0 = 0; j0 < EPT; j0 += kBatch) {
        E val[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const uint32_t d = v[j0 + u] - c0;
          val[u] = E(0);
          lds_if_below(val[u], d, n, tl_s + d * ES);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) sts_if_below(ob_s + (j0 + u) * kStThreads * ES, val[u], v[j0 + u] - c0, n);
      }
      if (bad != 0 && q == 0) {  // rare: an out-of-range index gathers zero
#pragma unroll
        for (int j = 0; j < EPT; ++j)
          if ((bad >> j) & 1u) sts(ob_s + j * kStThreads * ES, E(0));
      }
    }
    if (q == npieces - 1) {
      __syncthreads();  // the tile is complete
      E* out = reinterpret_cast<E*>(p.other) + static_cast<int64_t>(b) * p.K + kc0;
      if (vec_out) {
        const int4* s4 = reinterpret_cast<const int4*>(obuf);
        int4* d4 = reinterpret_cast<int4*>(out);
        for (uint32_t i = t; i < ntile / VE; i += kStThreads) d4[i] = s4[i];
      } else {
        for (uint32_t i = t; i < ntile; i += kStThreads) out[i] = obuf[i];
      }
      // the next writes into the tile come after the barrier at the top of the next iteration
    }
    advance(b, q);
    ahead = stage;
    if (++stage == nstages) {
      stage = 0;
      phase ^= 1u;
    }
  }
}

// Rows of 4-byte elements too long for the tile form above (the row AND an output tile do not fit
// one SM's shared memory together) but at most 65 536 elements: the outputs stay in REGISTERS.  A
// block of 1024 threads owns up to 32 768 consecutive output positions -- 32 per thread, in groups
// of four consecutive positions so that they leave as 16-byte stores.  Their source positions fit
// 16 bits each: half of them live in 8 registers, the other half in 32 KiB of shared memory (read
// back with conflict-free 16-byte loads once per staged piece), which leaves the registers to the
// outputs and lets a full complement of 32 warps hide the latencies.  The rest of the shared
// memory belongs to the row: two or three stages filled by bulk asynchronous copies.  For every
// staged piece a thread tests its entries (subtract, compare, predicated shared load -- a branch
// around the load measured four times slower): no output tile, no second trip through shared
// memory, one block-wide barrier per piece.  An index list longer than 32 768 is cut into EQUAL
// chunks (blockIdx.y); the blocks of one row set visit the same rows at the same pace, so the
// second and later readers of a row find it in L2.
constexpr int kWdThreads = 1024;
constexpr int kWdEpt = 32;
#ifndef VB_WIDE_REG_WORDS
#define VB_WIDE_REG_WORDS 2
#endif
constexpr int kWdRegWords = VB_WIDE_REG_WORDS;  // 16-byte words of entries (8 entries each) a thread keeps in registers
constexpr int kWdEntryBytes = kWdThreads * (kWdEpt / 8 - kWdRegWords) * 16;  // the rest: shared memory
constexpr int kWdSmemMax = 227 * 1024 - 1024;
constexpr int kWdMaxStages = 4;
#ifndef VB_LASTDIM_WIDE
#define VB_LASTDIM_WIDE 1
#endif
#ifndef VB_WIDE_STAGES
#define VB_WIDE_STAGES 2
#endif
#ifndef VB_WIDE_STAGE_MAX
#define VB_WIDE_STAGE_MAX (96 * 1024)
#endif
template <bool NOBAR>
__global__ void __launch_bounds__(kWdThreads, 1) lastdim_wide_kernel(const __grid_constant__ LastDimParams p,
                                                                     const int piece, const int npieces,
                                                                     const int nstages, const int kchunk) {
  extern __shared__ __align__(128) unsigned char st_raw[];  // [entries: words x 1024 x 16 bytes][stages]
  __shared__ __align__(8) uint64_t bars[kWdMaxStages];
  __shared__ unsigned served[kWdMaxStages];  // warps that are done with the stage's current piece
  using E = uint32_t;
  const int t = threadIdx.x;
  unsigned char* const stages = st_raw + kWdEntryBytes;
  const uint32_t stage_bytes = (static_cast<uint32_t>(piece) * 4u + 127u) / 128u * 128u;
  // the index list is cut into equal chunks of kchunk <= 32 768 positions (a multiple of 4), one per blockIdx.y
  const int64_t kc0 = static_cast<int64_t>(blockIdx.y) * kchunk;
  const int64_t left = p.K - kc0;
  const uint32_t ntile = static_cast<uint32_t>(left < kchunk ? left : kchunk);
  const uint32_t upiece = static_cast<uint32_t>(piece);
  const uint32_t k0 = static_cast<uint32_t>(p.K0);
  // 16-byte words of entries that hold any live slot (word k covers slots from k * 8192 on): the
  // same for every thread, so skipping the rest is a uniform branch
  const int nwords = static_cast<int>((ntile + 2 * kWdThreads * 4 - 1) / (2 * kWdThreads * 4));
  // entry e of this thread is output slot (e / 4) * 4096 + t * 4 + e % 4 of the block's tile; the
  // thread's k-th 16-byte word of entries (e = 8k .. 8k + 7) sits at [k][t], so a warp reads 512
  // consecutive bytes.  Only this thread reads what it writes here: no barrier in between.
  bool bad = false;  // some slot's index is out of range (it gathers zero)
  const uint32_t ent_s = smem_addr(st_raw) + static_cast<uint32_t>(t) * 16u;
  uint32_t er[kWdRegWords > 0 ? kWdRegWords : 1][4];
#pragma unroll
  for (int k = 0; k < kWdEpt / 8; ++k) {
    uint32_t w[4];
#pragma unroll
    for (int h = 0; h < 8; ++h) {
      const int e = k * 8 + h;
      const uint32_t slot = static_cast<uint32_t>(e >> 2) * (kWdThreads * 4) + static_cast<uint32_t>(t) * 4u + (e & 3);
      uint32_t src = 0;
      if (slot < ntile) {
        int64_t x = p.idx.get(kc0 + slot);
        if (normalize(x, p.K0, p.policy, p.status, blockIdx.x == 0)) src = static_cast<uint32_t>(x);
        else bad = true;
      }
      if (h & 1) w[h >> 1] |= src << 16;
      else w[h >> 1] = src;
    }
    if (k < kWdRegWords) {
#pragma unroll
      for (int h = 0; h < 4; ++h) er[k < kWdRegWords ? k : 0][h] = w[h];
    } else {
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(ent_s + (k - kWdRegWords) * (kWdThreads * 16)),
                   "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                   : "memory");
    }
  }
  if (t == 0) {
    for (int st = 0; st < nstages; ++st) {
      mbar_init(&bars[st], 1);
      served[st] = 0;
    }
    mbar_init_fence();
  }
  __syncthreads();
  const bool vec_out = (reinterpret_cast<uintptr_t>(p.other) % 16 == 0) && (p.K % 4 == 0);
  auto advance = [&](uint32_t& bb, int& qq) {
    if (++qq == npieces) {
      qq = 0;
      bb += gridDim.x;
    }
  };
  auto issue = [&](uint32_t bb, int qq, int stage) {  // one thread; the stage's previous readers are done with it
    const uint32_t c0 = static_cast<uint32_t>(qq) * upiece;
    const uint32_t n = min(upiece, k0 - c0);
    const E* src = reinterpret_cast<const E*>(p.self) + p.rows.offset(bb) + c0;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive_expect_tx(&bars[stage], n * 4u);
    bulk_copy_g2s(stages + stage * stage_bytes, src, n * 4u, &bars[stage]);
  };
  uint32_t b = blockIdx.x, nb = blockIdx.x;
  int q = 0, nq = 0;
  // NOBAR: no block-wide barrier in the loop.  A warp that has served a piece counts itself off
  // on the piece's stage, and the warp that counts off last refills the stage (with the piece
  // nstages steps ahead), so (nb, nq) run nstages steps ahead of (b, q).  Otherwise the block
  // meets at a barrier per piece and thread 0 refills the stage served one step earlier; (nb, nq)
  // run nstages - 1 steps ahead.  Measured: the barrier form is a few percent faster when a row
  // has one reader, the other when several chunk blocks share the rows.
  for (int st = 0; st + (NOBAR ? 0 : 1) < nstages; ++st) {  // fill the pipeline
    if (t == 0 && nb < p.B) issue(nb, nq, st);
    advance(nb, nq);
  }
  int stage = 0, ahead = nstages - 1;
  uint32_t phase = 0;
  uint32_t o[kWdEpt];
#pragma unroll
  for (int e = 0; e < kWdEpt; ++e) o[e] = 0;
  for (; b < p.B;) {
    const uint32_t c0 = static_cast<uint32_t>(q) * upiece;
    const uint32_t n = min(upiece, k0 - c0);
    const bool ok = mbar_wait_bounded(&bars[stage], phase);
    if constexpr (NOBAR) {
      if (!ok) {
        // give up: note the fault, let the copies that may still be in flight land, and leave (the
        // other warps run into the same limit: no refill comes once a warp has left)
        atomicExch(&vb_index_fault, 1u);
        for (int st = 0; st < nstages; ++st) mbar_wait_bounded(&bars[st], st < stage ? phase ^ 1u : phase);
        return;
      }
    } else {
      if (__syncthreads_or(!ok)) {
        // give up: note the fault, let the copies that may still be in flight land, and leave
        if (t == 0) {
          atomicExch(&vb_index_fault, 1u);
          for (int st = 0; st < nstages; ++st) mbar_wait_bounded(&bars[st], st < stage ? phase ^ 1u : phase);
        }
        __syncthreads();
        return;
      }
      if (t == 0 && nb < p.B) issue(nb, nq, ahead);
      advance(nb, nq);
    }
    const uint32_t tl_s = smem_addr(stages + stage * stage_bytes) - c0 * 4u;  // address of source position 0
#pragma unroll
    for (int k = 0; k < kWdEpt / 8; ++k) {
      if (k >= nwords) break;
      uint32_t w[4];
      if (k < kWdRegWords) {
#pragma unroll
        for (int h = 0; h < 4; ++h) w[h] = er[k < kWdRegWords ? k : 0][h];
      } else {
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                     : "r"(ent_s + (k - kWdRegWords) * (kWdThreads * 16)));
      }
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const uint32_t s0 = w[h] & 0xffffu, s1 = w[h] >> 16;
        lds_if_below(o[k * 8 + 2 * h], s0 - c0, n, tl_s + s0 * 4u);
        lds_if_below(o[k * 8 + 2 * h + 1], s1 - c0, n, tl_s + s1 * 4u);
      }
    }
    if (q == npieces - 1) {
      if (bad) {  // rare: find the slots again from the index list
#pragma unroll
        for (int e = 0; e < kWdEpt; ++e) {
          const uint32_t slot = static_cast<uint32_t>(e >> 2) * (kWdThreads * 4) + static_cast<uint32_t>(t) * 4u + (e & 3);
          if (slot < ntile) {
            int64_t x = p.idx.get(kc0 + slot);
            if (!normalize(x, p.K0, p.policy, nullptr, false)) o[e] = 0;
          }
        }
      }
      E* out = reinterpret_cast<E*>(p.other) + static_cast<int64_t>(b) * p.K + kc0;
#pragma unroll
      for (int g = 0; g < kWdEpt / 4; ++g) {
        if (g >= 2 * nwords) break;
        const uint32_t slot = static_cast<uint32_t>(g) * (kWdThreads * 4) + static_cast<uint32_t>(t) * 4u;
        if (vec_out && slot + 3 < ntile) {
          *reinterpret_cast<uint4*>(out + slot) = make_uint4(o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]);
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (slot + u < ntile) out[slot + u] = o[4 * g + u];
        }
      }
    }
    if constexpr (NOBAR) {
      __syncwarp();
      if ((t & 31) == 0) {
        __threadfence_block();  // this warp's reads of the stage come before its count
        if (atomicAdd(&served[stage], 1u) == kWdThreads / 32 - 1) {
          __threadfence_block();  // the other warps' counts (and the reads in front of them) come before the refill
          served[stage] = 0;      // next touched after the refill below has landed
          if (nb < p.B) issue(nb, nq, stage);
        }
      }
      advance(nb, nq);
    }
    advance(b, q);
    ahead = stage;
    if (++stage == nstages) {
      stage = 0;
      phase ^= 1u;
    }
  }
}

// ------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------
vbt_b200_status check_idx(const vbt_b200_tensor* idx, const char* name, IndexSrc* src, int64_t* n) {
  VB_TRY(validate_data(idx, name));
  VB_ARG(idx->dtype == VBT_B200_I64 || idx->dtype == VBT_B200_I32,
         std::string(name) + ": only Int32 and Int64 index tensors are supported");
  VB_ARG(is_dense_row_major(*idx), std::string(name) + ": index tensor must be contiguous");
  *n = numel(*idx);
  VB_ARG(*n <= 0x7fffffff, std::string(name) + ": too many indices for one call");
  src->idx = idx->data;
  src->is32 = idx->dtype == VBT_B200_I32;
  return VBT_B200_OK;
}

vbt_b200_status rows_copy(const char* name, const vbt_b200_tensor* dense, const vbt_b200_tensor* table,
                          const vbt_b200_tensor* idx, int policy, void* status, cudaStream_t s,
                          int scatter) {
  VB_TRY(validate_data(dense, name));
  VB_TRY(validate_data(table, name));
  VB_ARG(table->ndim == 2, std::string(name) + ": table must be rank 2");
  VB_ARG(dense->dtype == table->dtype, std::string(name) + ": dtype mismatch");
  VB_ARG(policy >= 0 && policy <= 2, std::string(name) + ": unknown index policy");
  IndexSrc is{};
  int64_t N = 0;
  VB_TRY(check_idx(idx, name, &is, &N));
  const int64_t V = table->sizes[0], D = table->sizes[1];
  VB_ARG(is_dense_row_major(*dense) && numel(*dense) == N * D,
         std::string(name) + ": dense operand must be contiguous [N, D]");
  if (scatter) VB_ARG(table->strides[1] == 1 || D <= 1, std::string(name) + ": table rows must be contiguous");
  if (N == 0 || D == 0) return VBT_B200_OK;
  VB_ARG(V > 0 || policy != VBT_B200_INDEX_CLAMP, std::string(name) + ": empty table");
  const int es = itemsize(table->dtype);
  const int64_t s0 = table->strides[0], s1 = D > 1 ? table->strides[1] : 1;
  DeviceScope scope(dense->data);
  const bool chunked = s1 == 1 && (D * es) % 16 == 0 && (s0 * es) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(table->data) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(dense->data) % 16 == 0 && s0 >= 0 &&
                       D * es / 16 <= 0x7fffffff;
  if (chunked) {
    GatherParams p{};
    p.table = static_cast<const char*>(table->data);
    p.out = static_cast<char*>(dense->data);
    p.idx = is;
    p.N = N;
    p.V = V;
    p.row_stride_bytes = s0 * es;
    p.cpr = static_cast<uint32_t>(D * es / 16);
    p.div_cpr = FastDiv(p.cpr);
    p.total = N * p.cpr;
    p.policy = policy;
    p.status = static_cast<unsigned long long*>(status);
    p.scatter = scatter;
    const int64_t blocks = (p.total + kThreads * kGatherU - 1) / (kThreads * kGatherU);
    VB_ARG(blocks <= 0x7fffffff, std::string(name) + ": too large for one call");
    rows_copy_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(p);
    note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_ROWS_COPY, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 16 / es,
                1, 0, 1, N * D, N, 0, s);
  } else {
    ElemParams p{};
    p.table = static_cast<const char*>(table->data);
    p.out = static_cast<char*>(dense->data);
    p.idx = is;
    p.N = N; p.V = V; p.D = D; p.s0 = s0; p.s1 = s1; p.es = es;
    p.policy = policy;
    p.status = static_cast<unsigned long long*>(status);
    p.scatter = scatter;
    const int64_t blocks = (N * D + kThreads - 1) / kThreads;
    VB_ARG(blocks <= 0x7fffffff, std::string(name) + ": too large for one call");
    rows_copy_elem_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(p);
    note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_ROWS_COPY_ELEM, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 1,
                1, 0, 1, N * D, N, 0, s);
  }
  VB_LAUNCH_CHECK();
  return VBT_B200_OK;
}

template <class T>
vbt_b200_status scatter_add_typed(const ScatterParams& p, const ScatterElemParams& pe, bool chunked,
                                  cudaStream_t s) {
  if (chunked) {
    const unsigned g = static_cast<unsigned>((p.N + kRingBatch - 1) / kRingBatch);
    // sorted keys + a ring of row slots per warp; more than 48 KiB needs the per-function opt-in
    auto go = [&](auto kern, int K) -> vbt_b200_status {
      const int ring = std::min(8, kRingBytesPerWarp / (K * 512));
      const size_t smem = static_cast<size_t>(kRingBatch) * 8 + static_cast<size_t>(kThreads / 32) * ring * K * 512;
      static std::mutex mu;
      static bool done[3][64] = {};
      int dev = 0;
      VB_CUDA(cudaGetDevice(&dev));
      {
        std::lock_guard<std::mutex> lk(mu);
        bool& d = done[K == 1 ? 0 : (K == 2 ? 1 : 2)][dev >= 0 && dev < 64 ? dev : 0];
        if (dev < 0 || dev >= 64 || !d) {
          VB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
          d = true;
        }
      }
      kern<<<g, kThreads, smem, s>>>(p);
      return VBT_B200_OK;
    };
    if (p.cpr <= 32) VB_TRY(go(scatter_add_ring_kernel<T, 1>, 1));
    else if (p.cpr <= 64) VB_TRY(go(scatter_add_ring_kernel<T, 2>, 2));
    else VB_TRY(go(scatter_add_ring_kernel<T, 4>, 4));
    note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_SCATTER_ADD, dim3(g), dim3(kThreads), 16 / static_cast<int>(sizeof(T)),
                1, 0, 1 + (p.counts ? 2 : 0), p.N * p.cpr * (16 / static_cast<int64_t>(sizeof(T))), p.N, 0, s);
  } else {
    const int64_t blocks = (pe.N * pe.D + kThreads - 1) / kThreads;
    VB_ARG(blocks <= 0x7fffffff, "index_put_: too large for one call");
    scatter_add_elem_kernel<T><<<static_cast<unsigned>(blocks), kThreads, 0, s>>>(pe);
    note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_SCATTER_ADD_ELEM, dim3(static_cast<unsigned>(blocks)), dim3(kThreads),
                1, 1, 0, 1 + (pe.counts ? 2 : 0), pe.N * pe.D, pe.N, 0, s);
  }
  VB_LAUNCH_CHECK();
  return VBT_B200_OK;
}

vbt_b200_status scatter_add_rows(const char* name, const vbt_b200_tensor* table, const vbt_b200_tensor* idx,
                                 const vbt_b200_tensor* values, int policy, void* status, int use_padding,
                                 int64_t padding_idx, cudaStream_t s, unsigned* counts = nullptr) {
  VB_TRY(validate_data(table, name));
  VB_TRY(validate_data(values, name));
  VB_ARG(table->ndim == 2, std::string(name) + ": table must be rank 2");
  VB_ARG(values->dtype == table->dtype, std::string(name) + ": dtype mismatch");
  VB_ARG(policy >= 0 && policy <= 2, std::string(name) + ": unknown index policy");
  const int dt = table->dtype;
  VB_ARG(dt == VBT_B200_F32 || dt == VBT_B200_I64 || dt == VBT_B200_I32,
         std::string(name) + ": accumulate supports float32, int32 and int64");
  IndexSrc is{};
  int64_t N = 0;
  VB_TRY(check_idx(idx, name, &is, &N));
  const int64_t V = table->sizes[0], D = table->sizes[1];
  VB_ARG(is_dense_row_major(*table), std::string(name) + ": table must be contiguous");
  VB_ARG(is_dense_row_major(*values) && numel(*values) == N * D,
         std::string(name) + ": values must be contiguous [N, D]");
  if (N == 0 || D == 0) return VBT_B200_OK;
  const int es = itemsize(dt);
  DeviceScope scope(table->data);
  const bool chunked = (D * es) % 16 == 0 && reinterpret_cast<uintptr_t>(table->data) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(values->data) % 16 == 0 && V < (int64_t{1} << 55);
  ScatterParams p{};
  p.table = static_cast<char*>(table->data);
  p.values = static_cast<const char*>(values->data);
  p.idx = is;
  p.N = N; p.V = V;
  p.cpr = static_cast<uint32_t>(D * es / 16);
  p.policy = policy;
  p.status = static_cast<unsigned long long*>(status);
  p.use_padding = use_padding;
  p.padding_idx = padding_idx;
  p.counts = counts;
  ScatterElemParams pe{};
  pe.table = p.table; pe.values = p.values; pe.idx = is; pe.N = N; pe.V = V; pe.D = D;
  pe.policy = policy; pe.status = p.status; pe.use_padding = use_padding; pe.padding_idx = padding_idx;
  pe.counts = counts;
  if (counts != nullptr) {
    VB_ARG(dt == VBT_B200_F32, std::string(name) + ": scale_grad_by_freq needs a float32 table");
    VB_CUDA(cudaMemsetAsync(counts, 0, static_cast<size_t>(V) * 4, s));
    const unsigned g = static_cast<unsigned>(
        std::min<int64_t>((N + kThreads - 1) / kThreads, int64_t{sm_count(scope.device())} * 8));
    count_rows_kernel<<<g, kThreads, 0, s>>>(is, N, V, policy, use_padding, padding_idx, counts);
    VB_LAUNCH_CHECK();
  }
  switch (dt) {
    case VBT_B200_F32: return scatter_add_typed<float>(p, pe, chunked, s);
    case VBT_B200_I64: return scatter_add_typed<int64_t>(p, pe, chunked, s);
    default: return scatter_add_typed<int32_t>(p, pe, chunked, s);
  }
}

constexpr int kMaxRadixBins = 1 << 11;
size_t sorted_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  const int64_t nblocks = (n + kSortTile - 1) / kSortTile;
  const size_t arrays = 4 * ((static_cast<size_t>(n) * 4 + 255) / 256 * 256);
  return arrays + static_cast<size_t>(nblocks) * kMaxRadixBins * 4 + 4 * kMaxRadixBins * 4;  // + per-pass digit totals
}

// one pass of the sort; FIRST also makes the keys
template <int RB>
vbt_b200_status radix_pass(const KeyParams& kp, bool first, uint32_t* const keys[2], uint32_t* const vals[2], int cur,
                           int64_t N, uint32_t mul, int shift, uint32_t* hist, int nblocks, uint32_t* tot,
                           cudaStream_t s) {
  constexpr int NB = 1 << RB;
  constexpr int kScatterSmem = (kSortWarps * NB + 2 * NB + 2 * kSortTile) * 4;
  if (first) radix_hist_kernel<RB, true><<<nblocks, kSortThreads, 0, s>>>(kp, keys[cur], N, mul, shift, hist, nblocks, tot);
  else radix_hist_kernel<RB, false><<<nblocks, kSortThreads, 0, s>>>(kp, keys[cur], N, mul, shift, hist, nblocks, tot);
  radix_scan_kernel<RB><<<NB, 1024, 0, s>>>(hist, nblocks, tot);
  if (kScatterSmem > 48 * 1024) {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      VB_CUDA(cudaFuncSetAttribute(radix_scatter_kernel<RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, kScatterSmem));
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  radix_scatter_kernel<RB><<<nblocks, kSortThreads, kScatterSmem, s>>>(keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1],
                                                                       N, mul, shift, hist, nblocks);
  return VBT_B200_OK;
}

template <class T>
void launch_sorted(const SortedScatterParams& p, cudaStream_t s) {
  const int64_t slices = (p.N + kSortedPerWarp - 1) / kSortedPerWarp;
  const unsigned g = static_cast<unsigned>((slices + kThreads / 32 - 1) / (kThreads / 32));
  // per warp: a ring of kSortedRing row slots plus its keys and positions; K = 2 needs the opt-in
  constexpr int kMeta = (kThreads / 32) * kSortedPerWarp * 8;
  if (p.cpr <= 32) {
    scatter_add_sorted_kernel<T, 1><<<g, kThreads, (kThreads / 32) * kSortedRing * 512 + kMeta, s>>>(p);
  } else {
    constexpr int kSmem = (kThreads / 32) * kSortedRing * 1024 + kMeta;
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    {
      std::lock_guard<std::mutex> lk(mu);
      if (dev < 0 || dev >= 64 || !done[dev]) {
        cudaFuncSetAttribute(scatter_add_sorted_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (dev >= 0 && dev < 64) done[dev] = true;
      }
    }
    scatter_add_sorted_kernel<T, 2><<<g, kThreads, kSmem, s>>>(p);
  }
}

vbt_b200_status scatter_add_rows_sorted(const char* name, const vbt_b200_tensor* table,
                                        const vbt_b200_tensor* idx, const vbt_b200_tensor* values, int policy,
                                        void* status, int use_padding, int64_t padding_idx, void* ws,
                                        size_t ws_bytes, cudaStream_t s) {
  VB_TRY(validate_data(table, name));
  VB_TRY(validate_data(values, name));
  VB_ARG(table->ndim == 2, std::string(name) + ": table must be rank 2");
  const int dt = table->dtype;
  const int64_t V = table->sizes[0], D = table->sizes[1];
  const int es = itemsize(dt);
  IndexSrc is{};
  int64_t N = 0;
  VB_TRY(check_idx(idx, name, &is, &N));
  const bool chunked = (D * es) % 16 == 0 && D > 0 && reinterpret_cast<uintptr_t>(table->data) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(values->data) % 16 == 0 && V < (int64_t{1} << 31);
  const bool typed = dt == VBT_B200_F32 || dt == VBT_B200_I64 || dt == VBT_B200_I32;
  if (!chunked || !typed || N == 0)  // shapes the sorted kernels do not take: same result, atomic path
    return scatter_add_rows(name, table, idx, values, policy, status, use_padding, padding_idx, s);
  VB_ARG(values->dtype == dt, std::string(name) + ": dtype mismatch");
  VB_ARG(policy >= 0 && policy <= 2, std::string(name) + ": unknown index policy");
  VB_ARG(is_dense_row_major(*table), std::string(name) + ": table must be contiguous");
  VB_ARG(is_dense_row_major(*values) && numel(*values) == N * D,
         std::string(name) + ": values must be contiguous [N, D]");
  const size_t need = sorted_workspace_bytes(N);
  VB_ARG(ws != nullptr && ws_bytes >= need,
         std::string(name) + ": workspace too small (see vbt_b200_index_put_rows_sorted_workspace_bytes)");
  VB_ARG(reinterpret_cast<uintptr_t>(ws) % 16 == 0, std::string(name) + ": workspace must be 16-byte aligned");
  DeviceScope scope(table->data);
  const size_t arr = (static_cast<size_t>(N) * 4 + 255) / 256 * 256;
  char* w = static_cast<char*>(ws);
  uint32_t* keys[2] = {reinterpret_cast<uint32_t*>(w), reinterpret_cast<uint32_t*>(w + 2 * arr)};
  uint32_t* vals[2] = {reinterpret_cast<uint32_t*>(w + arr), reinterpret_cast<uint32_t*>(w + 3 * arr)};
  uint32_t* hist = reinterpret_cast<uint32_t*>(w + 4 * arr);
  const int nblocks = static_cast<int>((N + kSortTile - 1) / kSortTile);
  uint32_t* totals = hist + static_cast<size_t>(nblocks) * kMaxRadixBins;  // [4 passes][bins]
  VB_CUDA(cudaMemsetAsync(totals, 0, 4 * kMaxRadixBins * 4, s));
  KeyParams kp{};
  kp.idx = is; kp.N = N; kp.V = V; kp.policy = policy;
  kp.status = static_cast<unsigned long long*>(status);
  kp.use_padding = use_padding; kp.padding_idx = padding_idx;
  kp.keys = keys[0]; kp.vals = vals[0];
  int bits = 1;
  while ((int64_t{1} << bits) <= V) ++bits;  // keys run 0..V (V = skip)
  // 11-bit digits only where one pass then does (at most 2048 rows).  Two 11-bit passes instead of
  // three 8-bit ones measured SLOWER on 2^20 rows and 4 M updates (0.97 against 0.94 ms for the
  // whole scatter-add): per-block counts and offsets grow with bins x blocks, and their
  // digit-major layout makes those accesses uncoalesced.
  const int rb = bits <= 11 && bits > 8 ? 11 : 8;
  // The accumulating kernel needs equal rows NEXT TO each other, not the rows in order.  Rows that
  // take more than 16 bits are therefore grouped by the top 16 bits of a multiplicative hash of the
  // row -- two passes whatever the table's height.  The rows of a hash bucket stay in update
  // order, so another row of the same bucket can cut a run in two: that costs one more add to the
  // row, nothing else (a strided set of rows, which would fill a bucket of the plain low bits,
  // is spread by the multiply).  Measured on 2^20 rows, 4 M Zipf(1.1) updates: fp32 0.924 -> 0.876 ms
  // (sort 176 -> 125 us, accumulation 745 -> 757 us); int64 rows, whose adds go out as two 8-byte
  // atomics per 16 bytes, lost in the accumulation what the sort gained and keep the full sort.
  const bool hashed = bits > 16 && es == 4;
  const int passes = hashed ? 2 : (bits + rb - 1) / rb;
  const uint32_t mul = hashed ? 0x9E3779B1u : 1u;
  int cur = 0;
  for (int ps = 0; ps < passes; ++ps) {
    uint32_t* tot = totals + ps * kMaxRadixBins;
    const int shift = hashed ? 16 + 8 * ps : ps * rb;
    if (rb == 11) VB_TRY(radix_pass<11>(kp, ps == 0, keys, vals, cur, N, mul, shift, hist, nblocks, tot, s));
    else VB_TRY(radix_pass<8>(kp, ps == 0, keys, vals, cur, N, mul, shift, hist, nblocks, tot, s));
    cur ^= 1;
  }
  SortedScatterParams sp{};
  sp.table = static_cast<char*>(table->data);
  sp.values = static_cast<const char*>(values->data);
  sp.keys = keys[cur]; sp.vals = vals[cur];
  sp.N = N; sp.V = V;
  sp.cpr = static_cast<uint32_t>(D * es / 16);
  switch (dt) {
    case VBT_B200_F32: launch_sorted<float>(sp, s); break;
    case VBT_B200_I64: launch_sorted<int64_t>(sp, s); break;
    default: launch_sorted<int32_t>(sp, s); break;
  }
  VB_LAUNCH_CHECK();
  note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_SCATTER_ADD_SORTED, dim3(static_cast<unsigned>((N + 255) / 256)),
              dim3(kThreads), 16 / es, 1, 0, 2 + 3 * passes, N * D, N, need, s);
  return VBT_B200_OK;
}

template <class E, int EPT, bool GROUPED>
vbt_b200_status launch_staged_ept(const LastDimParams& p, int piece, int npieces, int use_bulk, int nstages, dim3 grid,
                                  size_t smem, cudaStream_t s) {
  // the opt-in to more than 48 KiB of dynamic shared memory is per function and per device
  static std::mutex mu;
  static bool done[64] = {};
  int dev = 0;
  VB_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      VB_CUDA(cudaFuncSetAttribute(lastdim_staged_kernel<E, EPT, GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kStagedSmemMax));
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  lastdim_staged_kernel<E, EPT, GROUPED><<<grid, kStThreads, smem, s>>>(p, piece, npieces, use_bulk, nstages);
  return VBT_B200_OK;
}
template <class E, int EPT>
vbt_b200_status launch_staged_grp(const LastDimParams& p, int piece, int npieces, int use_bulk, int nstages, dim3 grid,
                                  size_t smem, cudaStream_t s) {
  // regroup the entries by piece when there are several pieces, the packed entry can hold every
  // source position, and the sort's scratch (4 bytes per entry) fits the shared memory asked for
  constexpr int KBITS = EPT == 32 ? 15 : (EPT == 16 ? 14 : 13);
  const bool grouped = npieces > 1 && npieces <= kStMaxPieces && p.K0 < (int64_t{1} << (32 - KBITS)) - 1 &&
                       static_cast<size_t>(EPT) * kStThreads * 4 <= smem;
  return grouped ? launch_staged_ept<E, EPT, true>(p, piece, npieces, use_bulk, nstages, grid, smem, s)
                 : launch_staged_ept<E, EPT, false>(p, piece, npieces, use_bulk, nstages, grid, smem, s);
}
template <class E>
vbt_b200_status launch_staged(const LastDimParams& p, int ept, int piece, int npieces, int use_bulk, int nstages,
                              dim3 grid, size_t smem, cudaStream_t s) {
  constexpr int kCap = sizeof(E) == 8 ? 16 : 32;  // the output tile stays <= 128 KiB
  if constexpr (kCap >= 32) {
    if (ept == 32) return launch_staged_grp<E, 32>(p, piece, npieces, use_bulk, nstages, grid, smem, s);
  }
  if (ept == 16) return launch_staged_grp<E, 16>(p, piece, npieces, use_bulk, nstages, grid, smem, s);
  return launch_staged_grp<E, 8>(p, piece, npieces, use_bulk, nstages, grid, smem, s);
}

// self: rank >= 1, any strides; the index applies to its LAST dim.  other: dense
// [leading dims of self..., index shape...] (only its element count and density are checked).
vbt_b200_status lastdim(const char* name, const vbt_b200_tensor* self, const vbt_b200_tensor* idx,
                        const vbt_b200_tensor* other, int mode, int policy, void* status, cudaStream_t s) {
  VB_TRY(validate_data(self, name));
  VB_TRY(validate_data(other, name));
  VB_ARG(self->ndim >= 1,
         std::string(name) + ": advanced indexing is not supported for 0-d tensors on CUDA");
  VB_ARG(self->ndim <= VBT_B200_MAX_NDIM, std::string(name) + ": rank too large");
  VB_ARG(other->dtype == self->dtype, std::string(name) + ": dtype mismatch");
  VB_ARG(policy >= 0 && policy <= 2, std::string(name) + ": unknown index policy");
  IndexSrc is{};
  int64_t K = 0;
  VB_TRY(check_idx(idx, name, &is, &K));
  const int nd = self->ndim;
  int64_t B = 1;
  for (int d = 0; d + 1 < nd; ++d) B *= self->sizes[d];
  VB_ARG(is_dense_row_major(*other) && numel(*other) == B * K,
         std::string(name) + ": dense operand must be contiguous [leading dims..., index shape...]");
  if (mode == 2)
    VB_ARG(self->dtype == VBT_B200_F32 || self->dtype == VBT_B200_I64 || self->dtype == VBT_B200_I32,
           std::string(name) + ": accumulate supports float32, int32 and int64");
  if (B * K == 0) return VBT_B200_OK;
  VB_ARG(B <= 0x7fffffff, std::string(name) + ": too many rows for one call");
  DeviceScope scope(other->data);
  LastDimParams p{};
  p.self = static_cast<char*>(self->data);
  p.other = static_cast<char*>(other->data);
  p.idx = is;
  p.B = B; p.K0 = self->sizes[nd - 1]; p.K = K; p.sk = self->strides[nd - 1];
  // leading dims: drop size 1, merge neighbours that one stride walks
  int64_t lsz[VBT_B200_MAX_NDIM], lst[VBT_B200_MAX_NDIM];
  int nl = 0;
  for (int d = 0; d + 1 < nd; ++d) {
    const int64_t size = self->sizes[d], stride = self->strides[d];
    if (size == 1) continue;
    if (nl > 0 && lst[nl - 1] == stride * size) {
      lsz[nl - 1] *= size;
      lst[nl - 1] = stride;
    } else {
      lsz[nl] = size;
      lst[nl] = stride;
      ++nl;
    }
  }
  fill_dimlist(p.rows, lsz, lst, nl);
  p.es = itemsize(self->dtype);
  p.policy = policy;
  p.status = static_cast<unsigned long long*>(status);
  p.mode = mode;
  p.dtype = self->dtype;
  // Long rows and many indices: serve the gather from shared memory.  Staging reads the whole
  // row once per index chunk; the direct kernel pays a 32-byte sector per element.
  const int64_t row_bytes = p.K0 * p.es;
  // entries per thread: the fewest index chunks first (every chunk stages the rows again), then
  // the smallest output tile (which leaves the most shared memory for the row pieces)
  const int ept_cap = p.es == 8 ? 16 : 32;  // output tile of a block: <= 128 KiB
  int ept = 8;
  int64_t nchunks = (K + int64_t{kStThreads} * 8 - 1) / (int64_t{kStThreads} * 8);
  for (int e = 16; e <= ept_cap; e *= 2) {
    const int64_t c = (K + int64_t{kStThreads} * e - 1) / (int64_t{kStThreads} * e);
    if (c < nchunks) {
      nchunks = c;
      ept = e;
    }
  }
  // bulk copies need 16-byte aligned sources and sizes: every row start and every piece boundary
  bool bulk = reinterpret_cast<uintptr_t>(self->data) % 16 == 0 && row_bytes % 16 == 0;
  for (int i = 0; i < nl; ++i) bulk = bulk && (lst[i] * p.es) % 16 == 0;
  const bool staged_ok = mode == 0 && p.sk == 1 && K >= 4096 && B >= 32 && row_bytes >= 32 * 1024 &&
                         p.K0 <= 0x7fffffff && nchunks * row_bytes * 2 <= K * 32 && nchunks <= 65535;
  // rows of 4-byte elements that the tile form would have to cut into pieces, and whose positions
  // fit 16 bits: outputs in registers, the whole shared memory for the row
  const size_t tile_bytes0 = static_cast<size_t>(ept) * kStThreads * p.es;
  const int64_t wide_chunks = (K + int64_t{kWdThreads} * kWdEpt - 1) / (int64_t{kWdThreads} * kWdEpt);
  const int wide_kchunk = static_cast<int>(((K + wide_chunks - 1) / wide_chunks + 3) / 4 * 4);  // equal shares
  if (VB_LASTDIM_WIDE && staged_ok && bulk && p.es == 4 && p.K0 <= 65536 &&
      row_bytes > (kStagedSmemMax - static_cast<int64_t>(tile_bytes0)) / 2 / 1024 * 1024 &&
      wide_chunks * row_bytes * 2 <= K * 32) {
    // as many stages as fit beside the entries, each a whole piece of <= 64 KiB
    const int64_t room = kWdSmemMax - kWdEntryBytes;
    int nstages = VB_WIDE_STAGES;
    const int64_t stage_max = std::min<int64_t>(room / nstages / 1024 * 1024, VB_WIDE_STAGE_MAX);
    const int npieces = static_cast<int>((row_bytes + stage_max - 1) / stage_max);
    const int64_t per = (p.K0 + npieces - 1) / npieces;
    const int piece = static_cast<int>((per + 31) / 32 * 32);  // whole 128-byte lines
    const size_t stage = static_cast<size_t>(piece) * 4;
    nstages = static_cast<int>(std::min<int64_t>(nstages, room / static_cast<int64_t>(stage)));
    const int sms = sm_count(scope.device());
    const unsigned gx = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(B, sms / wide_chunks)));
    const dim3 grid(gx, static_cast<unsigned>(wide_chunks));
    const size_t smem = kWdEntryBytes + nstages * stage;
    static std::mutex mu;
    static bool done[64] = {};
    {
      std::lock_guard<std::mutex> lk(mu);
      const int dev = scope.device();
      if (dev < 0 || dev >= 64 || !done[dev]) {
        VB_CUDA(cudaFuncSetAttribute(lastdim_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kWdSmemMax));
        VB_CUDA(cudaFuncSetAttribute(lastdim_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kWdSmemMax));
        if (dev >= 0 && dev < 64) done[dev] = true;
      }
    }
    if (wide_chunks > 1) lastdim_wide_kernel<true><<<grid, kWdThreads, smem, s>>>(p, piece, npieces, nstages, wide_kchunk);
    else lastdim_wide_kernel<false><<<grid, kWdThreads, smem, s>>>(p, piece, npieces, nstages, wide_kchunk);
    VB_LAUNCH_CHECK();
    note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_LASTDIM_WIDE, grid, dim3(kWdThreads), kWdEpt, npieces, 0, 1, B * K,
                K, 0, s);
    return VBT_B200_OK;
  }
  if (staged_ok) {
    const size_t tile_bytes = static_cast<size_t>(ept) * kStThreads * p.es;
    // two stages: the next piece (or row) loads while this one is served.  Deeper pipelines of
    // smaller pieces measured slower: every piece costs a block-wide barrier, and with twelve
    // pieces per row the barriers, not the copies, set the pace.
    const int64_t avail = kStagedSmemMax - static_cast<int64_t>(tile_bytes);
    const int nstages = 2;
    const int64_t stage_max = avail / nstages / 1024 * 1024;
    const int npieces = static_cast<int>((row_bytes + stage_max - 1) / stage_max);
    const int64_t per = (p.K0 + npieces - 1) / npieces;
    const int piece = static_cast<int>((per + 15) / 16 * 16);  // whole 16-byte units for every element size
    const size_t stage = (static_cast<size_t>(piece) * p.es + 127) / 128 * 128;
    const int sms = sm_count(scope.device());
    const unsigned gx = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(B, sms / nchunks)));
    const dim3 grid(gx, static_cast<unsigned>(nchunks));
    const size_t smem = nstages * stage + tile_bytes;
    vbt_b200_status st;
    switch (p.es) {
      case 1: st = launch_staged<uint8_t>(p, ept, piece, npieces, bulk, nstages, grid, smem, s); break;
      case 2: st = launch_staged<uint16_t>(p, ept, piece, npieces, bulk, nstages, grid, smem, s); break;
      case 4: st = launch_staged<uint32_t>(p, ept, piece, npieces, bulk, nstages, grid, smem, s); break;
      default: st = launch_staged<uint64_t>(p, ept, piece, npieces, bulk, nstages, grid, smem, s); break;
    }
    VB_TRY(st);
    VB_LAUNCH_CHECK();
    note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_LASTDIM_STAGED, grid, dim3(kStThreads), ept, npieces, 0, 1, B * K,
                K, 0, s);
    return VBT_B200_OK;
  }
  const int64_t gx = (K + kThreads - 1) / kThreads, gy = (B + kLdRows - 1) / kLdRows;
  const dim3 g(static_cast<unsigned>(gx), static_cast<unsigned>(std::min<int64_t>(gy, 65535)));
  switch (p.es) {
    case 1: lastdim_kernel<uint8_t><<<g, kThreads, 0, s>>>(p); break;
    case 2: lastdim_kernel<uint16_t><<<g, kThreads, 0, s>>>(p); break;
    case 4: lastdim_kernel<uint32_t><<<g, kThreads, 0, s>>>(p); break;
    default: lastdim_kernel<uint64_t><<<g, kThreads, 0, s>>>(p); break;
  }
  VB_LAUNCH_CHECK();
  note_launch(VBT_B200_FAMILY_INDEX, VBT_B200_IK_LASTDIM, g, dim3(kThreads), 1, 1, 0, 1, B * K, K, 0, s);
  return VBT_B200_OK;
}

}  // namespace
}  // namespace vb

extern "C" {

vbt_b200_status vbt_b200_index_rows(const vbt_b200_tensor* out, const vbt_b200_tensor* table,
                                    const vbt_b200_tensor* idx, int32_t policy, void* index_status,
                                    void* stream) {
  return vb::rows_copy("index", out, table, idx, policy, index_status, static_cast<cudaStream_t>(stream), 0);
}

vbt_b200_status vbt_b200_index_put_rows(const vbt_b200_tensor* table, const vbt_b200_tensor* idx,
                                        const vbt_b200_tensor* values, int32_t accumulate, int32_t policy,
                                        void* index_status, void* stream) {
  if (accumulate)
    return vb::scatter_add_rows("index_put_", table, idx, values, policy, index_status, 0, 0,
                                static_cast<cudaStream_t>(stream));
  return vb::rows_copy("index_put_", values, table, idx, policy, index_status,
                       static_cast<cudaStream_t>(stream), 1);
}

size_t vbt_b200_index_put_rows_sorted_workspace_bytes(int64_t num_indices) {
  return vb::sorted_workspace_bytes(num_indices);
}

vbt_b200_status vbt_b200_index_put_rows_sorted(const vbt_b200_tensor* table, const vbt_b200_tensor* idx,
                                               const vbt_b200_tensor* values, int32_t policy, void* index_status,
                                               void* workspace, size_t workspace_bytes, void* stream) {
  return vb::scatter_add_rows_sorted("index_put_", table, idx, values, policy, index_status, 0, 0, workspace,
                                     workspace_bytes, static_cast<cudaStream_t>(stream));
}

vbt_b200_status vbt_b200_index_lastdim(const vbt_b200_tensor* out, const vbt_b200_tensor* src,
                                       const vbt_b200_tensor* idx, int32_t policy, void* index_status,
                                       void* stream) {
  return vb::lastdim("index", src, idx, out, 0, policy, index_status, static_cast<cudaStream_t>(stream));
}

vbt_b200_status vbt_b200_index_put_lastdim(const vbt_b200_tensor* self, const vbt_b200_tensor* idx,
                                           const vbt_b200_tensor* values, int32_t accumulate, int32_t policy,
                                           void* index_status, void* stream) {
  return vb::lastdim("index_put_", self, idx, values, accumulate ? 2 : 1, policy, index_status,
                     static_cast<cudaStream_t>(stream));
}

vbt_b200_status vbt_b200_embedding(const vbt_b200_tensor* out, const vbt_b200_tensor* weight,
                                   const vbt_b200_tensor* idx, void* index_status, void* stream) {
  using namespace vb;
  const char* name = "vt::embedding";
  VB_ARG(weight && idx && out, std::string(name) + ": null tensor descriptor");
  VB_ARG(weight->dtype == VBT_B200_F32, std::string(name) + ": weight must be float32");
  VB_ARG(weight->ndim == 2, std::string(name) + ": weight must be rank 2");
  VB_ARG(weight->strides[0] >= 0 && weight->strides[1] >= 0,
         std::string(name) + ": weight strides must be non-negative");
  VB_ARG(idx->dtype == VBT_B200_I64, std::string(name) + ": indices must be int64");
  return rows_copy(name, out, weight, idx, VBT_B200_INDEX_STRICT, index_status,
                   static_cast<cudaStream_t>(stream), 0);
}

vbt_b200_status vbt_b200_embedding_backward(const vbt_b200_tensor* grad_weight, const vbt_b200_tensor* idx,
                                            const vbt_b200_tensor* grad_out, int64_t padding_idx,
                                            void* index_status, void* stream) {
  return vb::scatter_add_rows("vt::embedding", grad_weight, idx, grad_out, VBT_B200_INDEX_STRICT,
                              index_status, 1, padding_idx, static_cast<cudaStream_t>(stream));
}

vbt_b200_status vbt_b200_embedding_backward_by_freq(const vbt_b200_tensor* grad_weight,
                                                    const vbt_b200_tensor* idx, const vbt_b200_tensor* grad_out,
                                                    int64_t padding_idx, void* counts, size_t counts_bytes,
                                                    void* index_status, void* stream) {
  using namespace vb;
  VB_ARG(grad_weight != nullptr && grad_weight->ndim == 2, "vt::embedding: grad_weight must be rank 2");
  VB_ARG(counts != nullptr && counts_bytes >= static_cast<size_t>(grad_weight->sizes[0]) * 4,
         "vt::embedding: scale_grad_by_freq needs 4 bytes of count scratch per weight row");
  return scatter_add_rows("vt::embedding", grad_weight, idx, grad_out, VBT_B200_INDEX_STRICT, index_status, 1,
                          padding_idx, static_cast<cudaStream_t>(stream), static_cast<unsigned*>(counts));
}

vbt_b200_status vbt_b200_index_status_check(void* index_status, const char* what, int64_t dim_size,
                                            void* stream) {
  using namespace vb;
  VB_ARG(index_status != nullptr, "index_status_check: null status block");
  DeviceScope scope(index_status);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned long long h[2] = {0, 0};
  unsigned fault = 0;
  VB_CUDA(cudaMemcpyAsync(h, index_status, sizeof(h), cudaMemcpyDeviceToHost, s));
  VB_CUDA(cudaMemcpyFromSymbolAsync(&fault, vb_index_fault, sizeof(fault), 0, cudaMemcpyDeviceToHost, s));
  VB_CUDA(cudaStreamSynchronize(s));
  if (fault != 0) {
    const unsigned zero = 0;
    VB_CUDA(cudaMemcpyToSymbolAsync(vb_index_fault, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s));
    VB_CUDA(cudaStreamSynchronize(s));
    return fail(VBT_B200_CUDA_ERROR, std::string(what ? what : "index") +
                                         ": a staged row copy did not complete in time; the output of an "
                                         "earlier last-dim index call on this device is incomplete");
  }
  if (h[0] == 0) return VBT_B200_OK;
  VB_CUDA(cudaMemsetAsync(index_status, 0, sizeof(h), s));
  return fail(VBT_B200_OUT_OF_RANGE,
              std::string(what ? what : "index") + ": index " + std::to_string(static_cast<long long>(h[1])) +
                  " is out of range for dimension with size " + std::to_string(dim_size) + " (" +
                  std::to_string(h[0]) + " bad indices)");
}

}  // extern "C"
