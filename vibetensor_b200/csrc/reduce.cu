// Dim reductions: sum / mean / max / min / prod / argmax / argmin (sm_100a).
//
// Replaces cuda_reduce_dispatch and the K1 (one atomic per input element), K2 and K3
// kernels of the reference (src/vbt/ops/cuda_reduction.cu:254-416, :907-2034).  Every
// reduction is brought to one of three shapes on the host:
//
//   ROW      the reduced dims are one run with stride 1: each output owns a contiguous
//            slice.  Short slices: one warp per output.  Long slices: `splits` blocks per
//            output sweep the slice together, block b taking the 16 KiB pieces b, b + splits,
//            b + 2*splits, ... so that at any moment the resident blocks read one compact
//            window of memory; block partials go to the workspace and the block that
//            arrives last folds them in block order.
//   COL      memory is [A, R, B] with B contiguous and R reduced: a warp reads whole
//            16-byte-per-lane rows (coalesced), the 8 warps of a block split R, blocks
//            split R further through the same workspace + last-arriver fold.
//   GENERIC  anything else: one warp per output walks the reduced index space through a
//            multiply-shift offset decoder.
//
// No floating-point atomics anywhere: for a given shape the order of additions is fixed,
// so results repeat bit for bit from run to run.  There are no spin waits either -- the
// cross-block fold is done by whichever block draws the last ticket, and that block puts the
// ticket counter back to zero, so a workspace whose ticket area was zero before a call is zero
// again after it.
//
// Workspace layout: [kTicketBytes of uint32 ticket counters][partials, 16-byte aligned].
#include <cooperative_groups.h>

#include <cfloat>
#include <climits>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace vb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxDims = VBT_B200_MAX_NDIM;
constexpr size_t kTicketBytes = 4096;  // fixed ticket area at the start of every workspace
// 16-byte loads a thread of the long-slice ROW kernel keeps in flight
#ifndef VB_ROW_U
#define VB_ROW_U 4
#endif
constexpr int kRowU = VB_ROW_U;
#ifndef VB_COL_CLUSTER
#define VB_COL_CLUSTER 1
#endif
// blocks per SM the long-slice ROW kernel is split into when few outputs share the GPU
#ifndef VB_ROW_BLOCKS_PER_SM
#define VB_ROW_BLOCKS_PER_SM 4
#endif
// 1 = the blocks of a slice each read one contiguous run instead of sweeping it together
// (kept for A/B measurements of the two assignments; the library is built with 0)
#ifndef VB_ROW_CONTIGUOUS
#define VB_ROW_CONTIGUOUS 0
#endif

// ------------------------------------------------------------------------------------
// reducers
// ------------------------------------------------------------------------------------
template <class A, class I>
struct Pair {
  A v;
  I i;
};

template <class A> __device__ __forceinline__ A lowest();
template <> __device__ __forceinline__ float lowest<float>() { return -INFINITY; }
template <> __device__ __forceinline__ int64_t lowest<int64_t>() { return LLONG_MIN; }
template <class A> __device__ __forceinline__ A highest();
template <> __device__ __forceinline__ float highest<float>() { return INFINITY; }
template <> __device__ __forceinline__ int64_t highest<int64_t>() { return LLONG_MAX; }

__device__ __forceinline__ float shfl_down(float v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
__device__ __forceinline__ int64_t shfl_down(int64_t v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
__device__ __forceinline__ int32_t shfl_down(int32_t v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
template <class A, class I>
__device__ __forceinline__ Pair<A, I> shfl_down(Pair<A, I> p, int d) {
  return Pair<A, I>{shfl_down(p.v, d), shfl_down(p.i, d)};
}

template <class A>
struct SumR {
  using acc_t = A;
  using idx_t = int32_t;  // unused
  static constexpr bool kIndexed = false;
  __device__ static acc_t init() { return A(0); }
  __device__ static void accum(acc_t& a, A v, idx_t) {
    if constexpr (sizeof(A) == 8) a = static_cast<A>(static_cast<uint64_t>(a) + static_cast<uint64_t>(v));
    else a += v;
  }
  __device__ static acc_t combine(acc_t a, acc_t b) {
    if constexpr (sizeof(A) == 8) return static_cast<A>(static_cast<uint64_t>(a) + static_cast<uint64_t>(b));
    else return a + b;
  }
};
template <class A>
struct ProdR {
  using acc_t = A;
  using idx_t = int32_t;  // unused
  static constexpr bool kIndexed = false;
  __device__ static acc_t init() { return A(1); }
  __device__ static void accum(acc_t& a, A v, idx_t) { a = combine(a, v); }
  __device__ static acc_t combine(acc_t a, acc_t b) {
    if constexpr (sizeof(A) == 8) return static_cast<A>(static_cast<uint64_t>(a) * static_cast<uint64_t>(b));
    else return a * b;
  }
};
// max / min: NaN never wins here (comparisons are false); "NaN at position 0 wins" of the
// reference's scan (src/vbt/python/tensor_bindings.cc:361-379) is applied at finalize.
template <class A, bool MAX>
struct ExtR {
  using acc_t = A;
  using idx_t = int32_t;  // unused
  static constexpr bool kIndexed = false;
  __device__ static acc_t init() { return MAX ? lowest<A>() : highest<A>(); }
  __device__ static void accum(acc_t& a, A v, idx_t) { a = (MAX ? (v > a) : (v < a)) ? v : a; }
  __device__ static acc_t combine(acc_t a, acc_t b) { return (MAX ? (b > a) : (b < a)) ? b : a; }
};
// argmax / argmin: first extremum wins (tensor_bindings.cc:630-682).  I is the index type
// carried through the reduction: 32-bit whenever the reduced extent allows it (index
// arithmetic, selects and shuffles are then half the work).
template <class A, bool MAX, class I>
struct ArgR {
  using acc_t = Pair<A, I>;
  using idx_t = I;
  static constexpr bool kIndexed = true;
  static constexpr I kNone = sizeof(I) == 4 ? static_cast<I>(INT_MAX) : static_cast<I>(LLONG_MAX);
  __device__ static acc_t init() { return acc_t{MAX ? lowest<A>() : highest<A>(), kNone}; }
  // Every kernel feeds one accumulator indices in increasing order, so an equal value never
  // displaces the one already held: the tie-break is only needed when partials meet (combine).
  __device__ static void accum(acc_t& a, A v, idx_t i) {
    // branch-free: one compare feeding two selects
    const bool take = MAX ? (v > a.v) : (v < a.v);
    a.v = take ? v : a.v;
    a.i = take ? i : a.i;
  }
  __device__ static acc_t combine(acc_t a, acc_t b) {
    return ((MAX ? (b.v > a.v) : (b.v < a.v)) || (b.v == a.v && b.i < a.i)) ? b : a;
  }
};

template <class T> struct Widen { using type = float; };
template <> struct Widen<int64_t> { using type = int64_t; };
__device__ __forceinline__ float widen(float x) { return x; }
__device__ __forceinline__ float widen(__half x) { return __half2float(x); }
__device__ __forceinline__ float widen(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ int64_t widen(int64_t x) { return x; }

__device__ __forceinline__ float ld_cg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ int64_t ld_cg(const int64_t* p) {
  return static_cast<int64_t>(__ldcg(reinterpret_cast<const long long*>(p)));
}
__device__ __forceinline__ int32_t ld_cg(const int32_t* p) { return __ldcg(p); }
template <class A, class I>
__device__ __forceinline__ Pair<A, I> ld_cg(const Pair<A, I>* p) {
  return Pair<A, I>{ld_cg(&p->v), ld_cg(&p->i)};
}

template <class R>
__device__ __forceinline__ typename R::acc_t warp_reduce(typename R::acc_t a) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) a = R::combine(a, shfl_down(a, d));
  return a;
}
// all threads call; result valid in thread 0
template <class R>
__device__ __forceinline__ typename R::acc_t block_reduce(typename R::acc_t a, typename R::acc_t* smem) {
  a = warp_reduce<R>(a);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) smem[w] = a;
  __syncthreads();
  if (w == 0) {
    a = lane < kWarps ? smem[lane] : R::init();
    a = warp_reduce<R>(a);
  }
  return a;
}

// ------------------------------------------------------------------------------------
// finalize: acc -> output element(s)
// ------------------------------------------------------------------------------------
enum { OP_SUM = 0, OP_MEAN, OP_MAX, OP_MIN, OP_PROD, OP_ARGMAX, OP_ARGMIN };

// Cross-GPU combine of the local results (sharded reductions, one process per GPU).  The block
// that holds a tile's final local values writes each of them, as ONE 8-byte word holding the value
// and the call's epoch, into slot [rank] of EVERY rank's exchange buffer with plain peer stores
// over NVLink; the same thread then reads the `world` words of its value from its own buffer until
// every one carries the epoch (a bounded wait), and folds them in rank order -- the same order on
// every rank, so all ranks end with bit-identical results -- before scaling, casting and storing.
// An aligned 8-byte store lands whole, so value and epoch need no fence and no separate flag: the
// exchange costs one one-way trip over the link plus the poll, not a store / fence / flag / poll
// chain.  Buffers alternate between two halves by the epoch's parity, so a rank that is already
// one call ahead never overwrites words a slower rank is still reading.  world == 0: no exchange.
constexpr int kXchgMaxRanks = VBT_B200_FABRIC_MAX_RANKS;
constexpr int kXchgTiles = 1024;                              // most tiles one call may exchange
constexpr unsigned long long kXchgTimeoutNs = 5000000000ull;  // a peer that never arrives: give up after 5 s
struct Xchg {
  int world;
  int rank;
  int owner;        // rank whose shard holds global position 0 (the NaN rule of max / min)
  unsigned epoch;
  int slot_floats;  // values per rank in a slot area
  float scale;      // applied to the folded value (1 / global count for a mean)
  unsigned long long* slots[kXchgMaxRanks];  // rank r's slot area of this call's half: [world][slot_floats] words
  unsigned* status;                          // this rank's error word
};

struct OutSpec {
  void* out;        // values (may be null for arg ops)
  int64_t* out_idx; // indices (arg ops)
  int out_dtype;
  int op;
  float inv_count_n;  // reduce count as float, for MEAN
  int nan_first;      // MAX / MIN: a NaN at position 0 of the slice wins (off for the shards of a
                      // sharded reduction that do not hold the global position 0)
  Xchg x;
};

__device__ __forceinline__ void store_value(const OutSpec& o, int64_t i, float v) {
  switch (o.out_dtype) {
    case VBT_B200_F32: static_cast<float*>(o.out)[i] = v; break;
    case VBT_B200_F16: static_cast<__half*>(o.out)[i] = __float2half_rn(v); break;
    case VBT_B200_BF16: static_cast<__nv_bfloat16*>(o.out)[i] = __float2bfloat16_rn(v); break;
  }
}
__device__ __forceinline__ void store_value(const OutSpec& o, int64_t i, int64_t v) {
  static_cast<int64_t*>(o.out)[i] = v;
}
__device__ __forceinline__ bool is_nan(float v) { return v != v; }
__device__ __forceinline__ bool is_nan(int64_t) { return false; }

// first: the slice's element 0 (widened), needed for the NaN-at-0 rule
template <class R, class A>
__device__ __forceinline__ void finalize(const OutSpec& o, int64_t i, typename R::acc_t acc, A first) {
  if constexpr (R::kIndexed) {
    if (is_nan(first)) { acc.v = first; acc.i = 0; }
    // nothing beat the identity: every element is the identity value (or NaN), the CPU scan
    // keeps its first element
    if (acc.i == R::kNone) acc.i = 0;
    if (o.out) store_value(o, i, acc.v);
    if (o.out_idx) o.out_idx[i] = static_cast<int64_t>(acc.i);
  } else {
    if ((o.op == OP_MAX || o.op == OP_MIN) && o.nan_first) {
      if (is_nan(first)) acc = first;
    }
    if constexpr (sizeof(A) == 4) {
      if (o.op == OP_MEAN) acc = acc / o.inv_count_n;
    }
    store_value(o, i, acc);
  }
}

__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Every thread of the block that holds the final LOCAL values of `tile` calls this; `has` marks
// the threads that own one (value v, slot e of the tile's vals_per_tile, output element out_i).
// first: the thread's slice element 0 (for the owner rank's NaN rule).
template <class R>
__device__ void exchange_finalize(const OutSpec& o, int tile, int vals_per_tile, int e, bool has, float v,
                                  int64_t out_i, float first) {
  if (!has) return;
  const Xchg& x = o.x;
  const int slot = tile * vals_per_tile + e;
  if ((o.op == OP_MAX || o.op == OP_MIN) && o.nan_first && first != first) v = first;
  const unsigned long long word = (static_cast<unsigned long long>(x.epoch) << 32) | __float_as_uint(v);
  for (int r = 0; r < x.world; ++r) st_relaxed_sys(x.slots[r] + x.rank * x.slot_floats + slot, word);
  const unsigned long long* mine = x.slots[x.rank] + slot;
  float acc = R::init(), fo = 0.f;
  const unsigned long long t0 = global_timer_ns();
  for (int r = 0; r < x.world; ++r) {
    unsigned long long w = ld_relaxed_sys(mine + r * x.slot_floats);
    for (unsigned tries = 0; static_cast<unsigned>(w >> 32) != x.epoch; ++tries) {
      if ((tries & 15u) == 15u) {
        if (global_timer_ns() - t0 > kXchgTimeoutNs) {
          atomicExch(x.status, 1u);  // the host reads this word; the output stays unwritten
          return;
        }
        __nanosleep(100);
      }
      w = ld_relaxed_sys(mine + r * x.slot_floats);
    }
    const float vr = __uint_as_float(static_cast<unsigned>(w));
    acc = R::combine(acc, vr);
    if (r == x.owner) fo = vr;
  }
  if (o.op == OP_MAX || o.op == OP_MIN) {
    if (fo != fo) acc = fo;  // only the owner of global position 0 can have published a NaN
  }
  store_value(o, out_i, acc * x.scale);
}

template <class R>
constexpr bool kCanExchange = !R::kIndexed && std::is_same_v<typename R::acc_t, float>;

// ------------------------------------------------------------------------------------
// ROW kernels
// ------------------------------------------------------------------------------------
template <class T, int V>
__device__ __forceinline__ void load_widen(const T* p, typename Widen<T>::type (&w)[V]) {
  if constexpr (V == 1) {
    w[0] = widen(*p);
  } else {
    const Vec<T, V> v = *reinterpret_cast<const Vec<T, V>*>(p);
#pragma unroll
    for (int j = 0; j < V; ++j) w[j] = widen(v.v[j]);
  }
}

struct RowParams {
  const void* x;
  int64_t n;          // slice length
  int64_t rows;
  DimList kept;       // row index -> slice base offset
  int splits;         // blocks that share one slice
  void* ws_partials;
  unsigned* ws_counters;
  OutSpec o;
};

// One warp per slice: short slices, and -- for argmax / argmin -- slices of up to 32 KiB when
// there are enough of them to fill the GPU.  A block per 16 KiB slice spends most of its
// instructions on the reduction tree (eight warp trees, a shared-memory stage, two barriers for
// sixteen elements per thread: the ncu capture of argmax on the C1 shape showed 77 % of the
// issue slots busy); a warp that walks the whole slice pays one tree.  U vectors in flight per
// lane, four accumulators; every accumulator sees its indices in increasing order.
template <class T, class R, int V>
__global__ void __launch_bounds__(kThreads) row_warp_kernel(const __grid_constant__ RowParams p) {
  using A = typename Widen<T>::type;
  using acc_t = typename R::acc_t;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int lane = threadIdx.x & 31;
  const T* x = static_cast<const T*>(p.x) + p.kept.offset(static_cast<uint32_t>(row));
  constexpr int U = V >= 8 ? 4 : 8;
  acc_t acc[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) acc[u] = R::init();
  const int64_t nvec = p.n / V;
  using idx_t = typename R::idx_t;
  int64_t i = lane;
  for (; i + (U - 1) * 32 < nvec; i += U * 32) {
    A w[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) load_widen<T, V>(x + (i + u * 32) * V, w[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const idx_t base = static_cast<idx_t>(i + u * 32) * V;
#pragma unroll
      for (int j = 0; j < V; ++j) R::accum(acc[u & 3], w[u][j], base + j);
    }
  }
  for (; i < nvec; i += 32) {
    A w[V];
    load_widen<T, V>(x + i * V, w);
    const idx_t base = static_cast<idx_t>(i) * V;
#pragma unroll
    for (int j = 0; j < V; ++j) R::accum(acc[0], w[j], base + j);
  }
  if constexpr (V > 1) {
    const int64_t t = nvec * V + lane;
    if (t < p.n) R::accum(acc[0], widen(x[t]), static_cast<idx_t>(t));
  }
  acc_t a = R::combine(R::combine(acc[0], acc[1]), R::combine(acc[2], acc[3]));
  a = warp_reduce<R>(a);
  if (lane == 0) finalize<R, A>(p.o, row, a, widen(x[0]));
}

// A block per slice that one unrolled pass covers (at most 256 threads x 4 vectors): no loop, no
// sweep arithmetic, 32-bit indices, and the slice's first element taken from the vector thread 0
// holds anyway.  The general kernel below executes about 200 warp instructions per warp for the
// twenty that load and add a 16 KiB slice's share (ncu on the C1 shapes: 6.4 M warp instructions,
// issue slots 55 % busy), and its run time follows the instruction count -- sum 11.3 us, max
// 12.9 us, argmax 15.3 us on the same 64 MiB -- so the fixed part is what this kernel cuts:
// straight-line code, and half the warps for slices of 512 vectors and less (measured on
// [4096,4096] fp32: max 12.5 -> 11.0 us, mean 11.7 -> 11.3 us; bf16 sum 10.4 -> 6.8 us).
#ifndef VB_ROW_ONCE
#define VB_ROW_ONCE 1
#endif
constexpr int kOnceU = 4;  // vectors per thread: 256 threads for slices of more than 512 vectors, else 128
template <class T, class R, int V, int kOnceThreads>
__global__ void __launch_bounds__(kOnceThreads) row_once_kernel(const __grid_constant__ RowParams p) {
  using A = typename Widen<T>::type;
  using acc_t = typename R::acc_t;
  using idx_t = typename R::idx_t;
  constexpr int U = kOnceU;
  constexpr int kOnceWarps = kOnceThreads / 32;
  __shared__ acc_t smem[kOnceWarps];
  const uint32_t row = blockIdx.x;
  const int t = threadIdx.x;
  const T* x = static_cast<const T*>(p.x) + (p.kept.n == 1 ? static_cast<int64_t>(row) * p.kept.stride[0] : p.kept.offset(row));
  const uint32_t n = static_cast<uint32_t>(p.n), nvec = n / V;
  A w[U][V];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t iv = static_cast<uint32_t>(u) * kOnceThreads + t;
    if (iv < nvec) {
      load_widen<T, V>(x + iv * V, w[u]);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) w[u][j] = A(0);
    }
  }
  acc_t acc[2] = {R::init(), R::init()};
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t iv = static_cast<uint32_t>(u) * kOnceThreads + t;
    if (iv < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) R::accum(acc[u & 1], w[u][j], static_cast<idx_t>(iv * V + j));
    }
  }
  A first = w[0][0];  // thread 0: element 0 of the slice, when the slice has a whole vector
  if constexpr (V > 1) {
    const uint32_t te = nvec * V + t;  // elements after the last whole vector
    if (te < n) {
      const A v = widen(x[te]);
      R::accum(acc[1], v, static_cast<idx_t>(te));
      if (nvec == 0) first = v;
    }
  }
  acc_t a = R::combine(acc[0], acc[1]);
  a = warp_reduce<R>(a);
  const int lane = t & 31, wi = t >> 5;
  if (lane == 0) smem[wi] = a;
  __syncthreads();
  if (t == 0) {
#pragma unroll
    for (int k = 1; k < kOnceWarps; ++k) a = R::combine(a, smem[k]);
    finalize<R, A>(p.o, row, a, first);
  }
}

// `splits` blocks per slice (grid = rows x splits).  One sweep of a slice's blocks covers
// splits * U * kThreads consecutive vectors: block b reads the b-th run of U * kThreads
// vectors of every sweep.  All blocks of the grid therefore work inside one window of
// splits * 16 KiB that slides over the slice, instead of `splits` far-apart streams.
template <class T, class R, int V, int U>
__global__ void __launch_bounds__(kThreads) row_block_kernel(const __grid_constant__ RowParams p) {
  using A = typename Widen<T>::type;
  using acc_t = typename R::acc_t;
  using idx_t = typename R::idx_t;
  __shared__ acc_t smem[kWarps];
  __shared__ bool is_last;
  const int64_t row = blockIdx.x;
  const int split = blockIdx.y;
  const T* x = static_cast<const T*>(p.x) + p.kept.offset(static_cast<uint32_t>(row));
  acc_t acc[U];
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = R::init();
  const int64_t nvec = p.n / V;
#if VB_ROW_CONTIGUOUS
  // measurement build only: each block reads one contiguous run of the slice
  const int64_t per = ((nvec + p.splits - 1) / p.splits + U * kThreads - 1) / (U * kThreads) * (U * kThreads);
  const int64_t end = min(nvec, (static_cast<int64_t>(split) + 1) * per);
  const int64_t sweep = U * kThreads;
  int64_t i = static_cast<int64_t>(split) * per + threadIdx.x;
#else
  const int64_t end = nvec;
  const int64_t sweep = static_cast<int64_t>(p.splits) * (U * kThreads);
  int64_t i = static_cast<int64_t>(split) * (U * kThreads) + threadIdx.x;
#endif
  for (; i + (U - 1) * kThreads < end; i += sweep) {
    A w[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) load_widen<T, V>(x + (i + u * kThreads) * V, w[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const idx_t base = static_cast<idx_t>(i + u * kThreads) * V;
#pragma unroll
      for (int j = 0; j < V; ++j) R::accum(acc[u], w[u][j], base + j);
    }
  }
  // the sweep that runs off the end of the slice
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t iv = i + u * kThreads;
    if (iv < end) {
      A w[V];
      load_widen<T, V>(x + iv * V, w);
      const idx_t base = static_cast<idx_t>(iv) * V;
#pragma unroll
      for (int j = 0; j < V; ++j) R::accum(acc[u], w[j], base + j);
    }
  }
  if constexpr (V > 1) {
    const int64_t t = nvec * V + threadIdx.x;  // elements after the last whole vector
    if (split == 0 && t < p.n) R::accum(acc[U - 1], widen(x[t]), static_cast<idx_t>(t));
  }
#pragma unroll
  for (int d = 1; d < U; d <<= 1)
#pragma unroll
    for (int u = 0; u + d < U; u += 2 * d) acc[u] = R::combine(acc[u], acc[u + d]);
  acc_t a = block_reduce<R>(acc[0], smem);
  if (p.splits == 1) {
    if constexpr (kCanExchange<R>) {
      if (p.o.x.world > 0) {
        exchange_finalize<R>(p.o, static_cast<int>(row), 1, 0, threadIdx.x == 0, a, row, widen(x[0]));
        return;
      }
    }
    if (threadIdx.x == 0) finalize<R, A>(p.o, row, a, widen(x[0]));
    return;
  }
  acc_t* part = static_cast<acc_t*>(p.ws_partials) + row * p.splits;
  if (threadIdx.x == 0) {
    part[split] = a;
    __threadfence();
    const unsigned t = atomicAdd(&p.ws_counters[row], 1u);
    is_last = (t == static_cast<unsigned>(p.splits) - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // fold the block partials in block order: thread t takes blocks t, t+256, ... in order,
  // then the fixed shuffle tree -- the same order on every run
  acc_t f = R::init();
  for (int s = threadIdx.x; s < p.splits; s += kThreads) f = R::combine(f, ld_cg(part + s));
  __syncthreads();
  f = block_reduce<R>(f, smem);
  if (threadIdx.x == 0) p.ws_counters[row] = 0u;  // every block of this slice has drawn its ticket: leave the counter as found
  if constexpr (kCanExchange<R>) {
    if (p.o.x.world > 0) {
      exchange_finalize<R>(p.o, static_cast<int>(row), 1, 0, threadIdx.x == 0, f, row, widen(x[0]));
      return;
    }
  }
  if (threadIdx.x == 0) finalize<R, A>(p.o, row, f, widen(x[0]));
}

// ------------------------------------------------------------------------------------
// COL kernel: memory [A, Rn, B], B contiguous, reduce Rn
// ------------------------------------------------------------------------------------
struct ColParams {
  const void* x;
  int64_t B, Rn, S;   // S = stride of the reduced dim (elements)
  DimList outer;      // a -> base offset
  int64_t A;
  int splits;
  int64_t chunk;      // reduced rows per split
  void* ws_partials;
  unsigned* ws_counters;
  int ctiles;
  OutSpec o;
};

template <class T, class R, int V>
__global__ void __launch_bounds__(kThreads) col_kernel(const __grid_constant__ ColParams p) {
  using A = typename Widen<T>::type;
  using acc_t = typename R::acc_t;
  __shared__ acc_t smem[kWarps][32 * V + 1];
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int ct = blockIdx.x, split = blockIdx.y;
  const int64_t a = blockIdx.z;
  const int64_t col = (static_cast<int64_t>(ct) * 32 + lane) * V;
  const bool active = col < p.B;  // B % V == 0 in vector mode
  const T* x = static_cast<const T*>(p.x) + p.outer.offset(static_cast<uint32_t>(a)) + col;
  const int64_t r0 = static_cast<int64_t>(split) * p.chunk;
  const int64_t r1 = min(p.Rn, r0 + p.chunk);
  acc_t acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = R::init();
  if (active) {
    constexpr int U = 4;
    int64_t r = r0 + w;
    for (; r + (U - 1) * kWarps < r1; r += U * kWarps) {
      A v[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) load_widen<T, V>(x + (r + u * kWarps) * p.S, v[u]);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) R::accum(acc[j], v[u][j], static_cast<typename R::idx_t>(r + u * kWarps));
    }
    for (; r < r1; r += kWarps) {
      A v[V];
      load_widen<T, V>(x + r * p.S, v);
#pragma unroll
      for (int j = 0; j < V; ++j) R::accum(acc[j], v[j], static_cast<typename R::idx_t>(r));
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) smem[w][lane * V + j] = acc[j];
  __syncthreads();
  // threads 0 .. 32V-1 each own one column of the tile: fold the 8 warps in warp order
  const int ncols = 32 * V;
  acc_t colacc = R::init();
  const int c = threadIdx.x;
  const int64_t gcol = static_cast<int64_t>(ct) * ncols + c;
  const bool owner = c < ncols && gcol < p.B;
  if (owner) {
#pragma unroll
    for (int ww = 0; ww < kWarps; ++ww) colacc = R::combine(colacc, smem[ww][c]);
  }
  const int64_t out_i = a * p.B + gcol;
  const T* first_p = static_cast<const T*>(p.x) + p.outer.offset(static_cast<uint32_t>(a)) + gcol;
  if (p.splits == 1) {
    if constexpr (kCanExchange<R>) {
      if (p.o.x.world > 0) {
        exchange_finalize<R>(p.o, static_cast<int>(a * p.ctiles + ct), ncols, c, owner, colacc, out_i,
                             owner ? widen(*first_p) : 0.f);
        return;
      }
    }
    if (owner) finalize<R, A>(p.o, out_i, colacc, widen(*first_p));
    return;
  }
  acc_t* part = static_cast<acc_t*>(p.ws_partials) +
                ((a * p.ctiles + ct) * p.splits) * ncols;  // [split][col]
  if (owner) part[static_cast<int64_t>(split) * ncols + c] = colacc;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(&p.ws_counters[a * p.ctiles + ct], 1u);
    is_last = (t == static_cast<unsigned>(p.splits) - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (threadIdx.x == 0) p.ws_counters[a * p.ctiles + ct] = 0u;  // all tickets drawn: leave the counter as found
  acc_t f = R::init();
  if (owner) {
    // chunk order, kFoldBatch independent loads in flight at a time (a loop of load-then-combine
    // would pay one L2 round trip per chunk; the usual 37 chunks take three trips)
    constexpr int kFoldBatch = sizeof(acc_t) <= 8 ? 16 : 8;
    for (int s0 = 0; s0 < p.splits; s0 += kFoldBatch) {
      acc_t t[kFoldBatch];
#pragma unroll
      for (int u = 0; u < kFoldBatch; ++u)
        t[u] = s0 + u < p.splits ? ld_cg(part + static_cast<int64_t>(s0 + u) * ncols + c) : R::init();
#pragma unroll
      for (int u = 0; u < kFoldBatch; ++u) f = R::combine(f, t[u]);
    }
  }
  if constexpr (kCanExchange<R>) {
    if (p.o.x.world > 0) {
      exchange_finalize<R>(p.o, static_cast<int>(a * p.ctiles + ct), ncols, c, owner, f, out_i,
                           owner ? widen(*first_p) : 0.f);
      return;
    }
  }
  if (owner) finalize<R, A>(p.o, out_i, f, widen(*first_p));
}

// COL through a thread-block cluster: the blocks that split R for one column tile form a
// cluster (2..16 blocks along grid.y) and fold their partials through distributed shared
// memory -- no workspace, no ticket, no memset in front of the kernel.  Used for small
// problems, where those few microseconds are a large part of the run time.
template <class T, class R, int V>
__global__ void __launch_bounds__(kThreads) col_cluster_kernel(const __grid_constant__ ColParams p) {
  namespace cg = cooperative_groups;
  using A = typename Widen<T>::type;
  using acc_t = typename R::acc_t;
  __shared__ acc_t smem[kWarps][32 * V + 1];
  __shared__ acc_t part_s[32 * V];
  constexpr unsigned kMaxCluster = 16;
  // pushed partials: where they fit beside `smem`, and not for (value, index) pairs, whose launch
  // measured slower that way (argmax over the strided dim of [4096,4096]: 17.2 against 15.9 us; sum,
  // mean and amax: 12.2 - 12.7 against 12.9 - 13.3 us)
  constexpr bool kPushPartials = !R::kIndexed && sizeof(acc_t) * 32 * V * kMaxCluster <= 16 * 1024;
  __shared__ acc_t pushed[kPushPartials ? kMaxCluster : 1][kPushPartials ? 32 * V : 1];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int ct = blockIdx.x, split = blockIdx.y;
  const int64_t a = blockIdx.z;
  const int64_t col = (static_cast<int64_t>(ct) * 32 + lane) * V;
  const bool active = col < p.B;
  const T* x = static_cast<const T*>(p.x) + p.outer.offset(static_cast<uint32_t>(a)) + col;
  const int64_t r0 = static_cast<int64_t>(split) * p.chunk;
  const int64_t r1 = min(p.Rn, r0 + p.chunk);
  acc_t acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = R::init();
  if (active) {
    int64_t r = r0 + w;
    // UU rows in flight per thread, while that many are left
    auto batches = [&](auto uu) {
      constexpr int UU = decltype(uu)::value;
      for (; r + (UU - 1) * kWarps < r1; r += UU * kWarps) {
        A v[UU][V];
#pragma unroll
        for (int u = 0; u < UU; ++u) load_widen<T, V>(x + (r + u * kWarps) * p.S, v[u]);
#pragma unroll
        for (int u = 0; u < UU; ++u)
#pragma unroll
          for (int j = 0; j < V; ++j) R::accum(acc[j], v[u][j], static_cast<typename R::idx_t>(r + u * kWarps));
      }
    };
    // (value, index) reducers: written sixteen deep, the compiler keeps about eight loads in
    // flight under the compare-select chains; written eight deep, about four
    if constexpr (R::kIndexed) batches(std::integral_constant<int, 16>{});
    batches(std::integral_constant<int, 8>{});
    batches(std::integral_constant<int, 2>{});
    for (; r < r1; r += kWarps) {
      A v[V];
      load_widen<T, V>(x + r * p.S, v);
#pragma unroll
      for (int j = 0; j < V; ++j) R::accum(acc[j], v[j], static_cast<typename R::idx_t>(r));
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) smem[w][lane * V + j] = acc[j];
  __syncthreads();
  const int ncols = 32 * V;
  const int c = threadIdx.x;
  const int64_t gcol = static_cast<int64_t>(ct) * ncols + c;
  const bool owner = c < ncols && gcol < p.B;
  if (c < ncols) {
    acc_t colacc = R::init();
    if (owner) {
#pragma unroll
      for (int ww = 0; ww < kWarps; ++ww) colacc = R::combine(colacc, smem[ww][c]);
    }
    part_s[c] = colacc;
  }
  cg::cluster_group cluster = cg::this_cluster();
  if constexpr (kPushPartials) {
    // every block stores its partials into block 0's shared memory (remote stores do not wait),
    // one cluster barrier, block 0 folds from its own memory in chunk order and the others leave:
    // no chain of remote loads and no second barrier to keep the readers' sources alive
    if (c < ncols) cluster.map_shared_rank(&pushed[0][0], 0)[cluster.block_rank() * (32 * V) + c] = part_s[c];
    cluster.sync();
    if (cluster.block_rank() == 0 && owner) {
      acc_t f = R::init();
      const unsigned nb = cluster.num_blocks();
#pragma unroll
      for (unsigned r = 0; r < kMaxCluster; ++r)
        if (r < nb) f = R::combine(f, pushed[r][c]);  // chunk order
      const T* first_p = static_cast<const T*>(p.x) + p.outer.offset(static_cast<uint32_t>(a)) + gcol;
      finalize<R, A>(p.o, a * p.B + gcol, f, widen(*first_p));
    }
  } else {
    cluster.sync();  // every block's part_s is complete and visible cluster-wide
    if (cluster.block_rank() == 0 && owner) {
      acc_t f = R::init();
      const unsigned nb = cluster.num_blocks();
      for (unsigned r = 0; r < nb; ++r) f = R::combine(f, cluster.map_shared_rank(part_s, r)[c]);  // chunk order
      const T* first_p = static_cast<const T*>(p.x) + p.outer.offset(static_cast<uint32_t>(a)) + gcol;
      finalize<R, A>(p.o, a * p.B + gcol, f, widen(*first_p));
    }
    cluster.sync();  // nobody leaves while block 0 may still read its shared memory
  }
}

// ------------------------------------------------------------------------------------
// GENERIC kernel: one warp per output
// ------------------------------------------------------------------------------------
struct GenParams {
  const void* x;
  DimList kept;
  DimList red;
  int64_t nout;
  uint32_t nred;
  OutSpec o;
};

template <class T, class R>
__global__ void __launch_bounds__(kThreads) generic_kernel(const __grid_constant__ GenParams p) {
  using A = typename Widen<T>::type;
  const int64_t oi = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (oi >= p.nout) return;
  const int lane = threadIdx.x & 31;
  const T* x = static_cast<const T*>(p.x) + p.kept.offset(static_cast<uint32_t>(oi));
  typename R::acc_t acc = R::init();
  for (uint32_t j = lane; j < p.nred; j += 32)
    R::accum(acc, widen(x[p.red.offset(j)]), static_cast<typename R::idx_t>(j));
  acc = warp_reduce<R>(acc);
  if (lane == 0) finalize<R, A>(p.o, oi, acc, widen(x[0]));
}

// fills an output with a constant (empty reduction domains)
template <class T>
__global__ void fill_kernel(T* out, int64_t n, T v) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = v;
}

// ------------------------------------------------------------------------------------
// host plan
// ------------------------------------------------------------------------------------
enum Shape { kRowWarp, kRowBlock, kCol, kGeneric, kEmptyDomain, kNoOutput };

struct Plan {
  Shape shape{kGeneric};
  int64_t nout{1}, nred{1};
  // kept / reduced dims after dropping size-1 dims and merging, outermost first
  int nk{0}, nr{0};
  int64_t ksize[kMaxDims]{}, kstride[kMaxDims]{}, rsize[kMaxDims]{}, rstride[kMaxDims]{};
  int splits{1};
  int64_t chunk{0};
  int ctiles{0};
  int cluster{0};  // COL: > 1 = fold R-chunks inside a thread-block cluster of this many blocks
  int V{1};
  size_t ws_partial_bytes{0}, ws_counter_bytes{0};
  int64_t out_sizes[kMaxDims]{};
  int out_ndim{0};
};

const char* op_name(int op) {
  static const char* const n[] = {"sum", "mean", "amax", "amin", "prod", "argmax", "argmin"};
  return (op >= 0 && op < VBT_B200_R_COUNT) ? n[op] : "reduce";
}

vbt_b200_status normalize_dims(const vbt_b200_tensor& self, const int64_t* dims, int ndims,
                               const char* name, bool* reduced /*[ndim]*/) {
  const int nd = self.ndim;
  for (int d = 0; d < nd; ++d) reduced[d] = ndims == 0;
  for (int i = 0; i < ndims; ++i) {
    int64_t d = dims[i];
    if (d < 0) d += nd;
    VB_ARG(d >= 0 && d < nd, std::string(name) + ": dim out of range");
    reduced[d] = true;
  }
  return VBT_B200_OK;
}

size_t acc_bytes(int op, int dtype) {
  const size_t a = dtype == VBT_B200_I64 ? 8 : 4;
  return (op == OP_ARGMAX || op == OP_ARGMIN) ? 16 : a;
}

// sms: SM count of the device the call runs on (grid sizing only; any value gives a correct plan)
vbt_b200_status make_plan(int op, const vbt_b200_tensor& self, const int64_t* dims, int ndims,
                          bool keepdim, int sms, Plan* pl) {
  const char* name = op_name(op);
  VB_ARG(self.ndim <= kMaxDims, std::string(name) + ": rank too large");
  bool reduced[kMaxDims + 1];
  VB_TRY(normalize_dims(self, dims, ndims, name, reduced));
  const int nd = self.ndim;
  pl->out_ndim = 0;
  pl->nout = 1;
  pl->nred = 1;
  for (int d = 0; d < nd; ++d) {
    if (reduced[d]) {
      pl->nred *= self.sizes[d];
      if (keepdim) pl->out_sizes[pl->out_ndim++] = 1;
    } else {
      pl->nout *= self.sizes[d];
      pl->out_sizes[pl->out_ndim++] = self.sizes[d];
    }
  }
  if (pl->nout == 0) { pl->shape = kNoOutput; return VBT_B200_OK; }
  if (pl->nred == 0) { pl->shape = kEmptyDomain; return VBT_B200_OK; }
  // split into kept / reduced lists (outermost first), drop size-1, merge neighbours
  auto push = [](int& n, int64_t* sz, int64_t* st, int64_t size, int64_t stride) {
    if (size == 1) return;
    if (n > 0 && st[n - 1] == stride * size) {  // previous (outer) dim continues this one
      sz[n - 1] *= size;
      st[n - 1] = stride;
      return;
    }
    sz[n] = size;
    st[n] = stride;
    ++n;
  };
  pl->nk = pl->nr = 0;
  for (int d = 0; d < nd; ++d) {
    if (reduced[d]) push(pl->nr, pl->rsize, pl->rstride, self.sizes[d], self.strides[d]);
    else push(pl->nk, pl->ksize, pl->kstride, self.sizes[d], self.strides[d]);
  }
  VB_ARG(pl->nout <= 0x7fffffff, std::string(name) + ": too many outputs for one call");
  const int es = itemsize(self.dtype);
  const int vmax = 16 / es;
  const uintptr_t base = reinterpret_cast<uintptr_t>(self.data);
  auto all_multiple = [&](const int64_t* st, int n, int v) {
    for (int i = 0; i < n; ++i)
      if (st[i] % v) return false;
    return true;
  };
  const size_t ab = acc_bytes(op, self.dtype);
  if (pl->nr == 1 && pl->rstride[0] == 1) {
    // ROW
    const int64_t n = pl->rsize[0];
    pl->V = (base % 16 == 0 && all_multiple(pl->kstride, pl->nk, vmax)) ? vmax : 1;
    // argmax / argmin also take it for slices of up to 32 KiB when there are enough of them: their
    // (value, index) reduction tree is what a block per 16 KiB slice spends its time on (15.3 us
    // against 12.7 us on [4096,4096] fp32); sum and max are faster with a block per slice there
    // (11.3 against 12.3 us: a block asks for its 16 KiB at once)
    const bool indexed = op == OP_ARGMAX || op == OP_ARGMIN;
    if ((n * es <= 4096 && pl->nout >= 64) || (indexed && n * es <= 32768 && pl->nout >= int64_t{sms} * 16)) {
      pl->shape = kRowWarp;
      return VBT_B200_OK;
    }
    pl->shape = kRowBlock;
    const int64_t per_block_min = int64_t{kThreads} * vmax * kRowU;  // one unrolled pass
    int64_t splits = 1;
    if (pl->nout < 2 * sms) {
      splits = std::min<int64_t>((n + per_block_min - 1) / per_block_min,
                                 (int64_t{sms} * VB_ROW_BLOCKS_PER_SM + pl->nout - 1) / pl->nout);
      splits = std::max<int64_t>(splits, 1);
    }
    pl->splits = static_cast<int>(std::min<int64_t>(splits, 65535));
    pl->chunk = 0;
    if (static_cast<size_t>(pl->nout) * 4 > kTicketBytes) pl->splits = 1;  // more slices than tickets
    if (pl->splits > 1) {
      pl->ws_partial_bytes = static_cast<size_t>(pl->nout) * pl->splits * ab;
      pl->ws_counter_bytes = static_cast<size_t>(pl->nout) * 4;
    }
    return VBT_B200_OK;
  }
  if (pl->nr == 1 && pl->nk >= 1 && pl->kstride[pl->nk - 1] == 1) {
    // COL: last kept dim contiguous
    const int64_t B = pl->ksize[pl->nk - 1];
    const int64_t Rn = pl->rsize[0];
    int64_t A = 1;
    for (int i = 0; i + 1 < pl->nk; ++i) A *= pl->ksize[i];
    if (A <= 65535) {
      bool vec = base % 16 == 0 && B % vmax == 0 && pl->rstride[0] % vmax == 0 &&
                 all_multiple(pl->kstride, pl->nk - 1, vmax);
      pl->V = vec ? vmax : 1;
      // 16-byte lanes only pay off when a tile of 32 lanes is mostly inside B
      if (vec && B < 32 * vmax / 2) pl->V = 1;
      pl->shape = kCol;
      const int ncols = 32 * pl->V;
      pl->ctiles = static_cast<int>((B + ncols - 1) / ncols);
      // about one resident wave of blocks (4 per SM): a second, partial wave only adds a tail
      int64_t want = (int64_t{sms} * 4) / (pl->ctiles * A);
      if (static_cast<size_t>(A) * pl->ctiles * 4 > kTicketBytes) want = 1;  // more tiles than tickets
      int64_t splits = std::max<int64_t>(1, std::min<int64_t>(want, (Rn + 31) / 32));
      splits = std::min<int64_t>(splits, 65535);
      int64_t chunk = (Rn + splits - 1) / splits;
      splits = (Rn + chunk - 1) / chunk;
      pl->splits = static_cast<int>(splits);
      pl->chunk = chunk;
      if (splits > 1) {
        pl->ws_partial_bytes = static_cast<size_t>(A) * pl->ctiles * splits * ncols * ab;
        pl->ws_counter_bytes = static_cast<size_t>(A) * pl->ctiles * 4;
        // up to 256 MiB of input and enough column tiles to fill the GPU with clusters of
        // <= 16 blocks: take the cluster path (the workspace stays sized as the fallback)
        const int64_t bytes = pl->nout * Rn * es;
        if (VB_COL_CLUSTER && bytes <= (int64_t{256} << 20) && Rn >= 512) {
          int cl = 16;
          while (cl > 2 && static_cast<int64_t>(pl->ctiles) * A * cl > int64_t{sms} * 5) cl >>= 1;
          if (static_cast<int64_t>(pl->ctiles) * A * cl >= sms) pl->cluster = cl;
        }
      }
      return VBT_B200_OK;
    }
  }
  pl->shape = kGeneric;
  VB_ARG(pl->nred <= 0x7fffffff, std::string(name) + ": reduced extent too large for this layout");
  return VBT_B200_OK;
}

// Whether this device can co-schedule clusters of `cluster` blocks of `kern`; asked once per
// (kernel, cluster size, device) -- the query and the attribute call cost several microseconds
// of host time, which matters on the small problems the cluster path exists for.
bool cluster_launch_ok(const void* kern, int cluster, const cudaLaunchConfig_t& cfg) {
  static std::mutex mu;
  static std::map<std::tuple<const void*, int, int>, bool> known;
  int dev = 0;
  cudaGetDevice(&dev);
  const auto key = std::make_tuple(kern, cluster, dev);
  std::lock_guard<std::mutex> lk(mu);
  auto it = known.find(key);
  if (it != known.end()) return it->second;
  bool ok = true;
  if (cluster > 8)
    ok = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
  int max_clusters = 0;
  ok = ok && cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) == cudaSuccess && max_clusters > 0;
  if (!ok) cudaGetLastError();
  known[key] = ok;
  return ok;
}

// ws: [kTicketBytes tickets][partials].  tickets_zeroed: the caller guarantees the ticket area
// is zero (it was zeroed once and only this library has written to it since).
template <class T, class R>
vbt_b200_status launch(const Plan& pl, const vbt_b200_tensor& self, const OutSpec& o, void* ws,
                       bool tickets_zeroed, cudaStream_t s) {
  constexpr int VMAX = 16 / sizeof(T);
  unsigned* tickets = static_cast<unsigned*>(ws);
  void* partials = ws ? static_cast<char*>(ws) + kTicketBytes : nullptr;
  const size_t ws_used = pl.ws_partial_bytes ? kTicketBytes + pl.ws_partial_bytes : 0;
  if (pl.shape == kRowWarp || pl.shape == kRowBlock) {
    RowParams p{};
    p.x = self.data;
    p.n = pl.rsize[0];
    p.rows = pl.nout;
    fill_dimlist(p.kept, pl.ksize, pl.kstride, pl.nk);
    p.splits = pl.splits;
    p.o = o;
    if (pl.shape == kRowWarp) {
      const unsigned g = static_cast<unsigned>((pl.nout + kWarps - 1) / kWarps);
      if (pl.V > 1) row_warp_kernel<T, R, VMAX><<<g, kThreads, 0, s>>>(p);
      else row_warp_kernel<T, R, 1><<<g, kThreads, 0, s>>>(p);
      VB_LAUNCH_CHECK();
      note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_ROW_WARP, dim3(g), dim3(kThreads), pl.V, 1, 0, 1, pl.nout,
                  pl.nred, 0, s);
    } else {
      int launches = 1;
      if (pl.splits > 1) {
        p.ws_partials = partials;
        p.ws_counters = tickets;
        if (!tickets_zeroed) {
          VB_CUDA(cudaMemsetAsync(tickets, 0, pl.ws_counter_bytes, s));
          ++launches;
        }
      }
      dim3 g(static_cast<unsigned>(pl.nout), static_cast<unsigned>(pl.splits));
      if (VB_ROW_ONCE && pl.splits == 1 && pl.V > 1 && o.x.world == 0 && pl.nred <= int64_t{256} * kOnceU * VMAX &&
          pl.nout >= 64) {
        const bool wide = pl.nred > int64_t{128} * kOnceU * VMAX;
        if (wide) row_once_kernel<T, R, VMAX, 256><<<g.x, 256, 0, s>>>(p);
        else row_once_kernel<T, R, VMAX, 128><<<g.x, 128, 0, s>>>(p);
        VB_LAUNCH_CHECK();
        note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_ROW_ONCE, dim3(g.x), dim3(wide ? 256 : 128), pl.V, 1, 0, 1, pl.nout,
                    pl.nred, 0, s);
        return VBT_B200_OK;
      }
      if (pl.V > 1) row_block_kernel<T, R, VMAX, kRowU><<<g, kThreads, 0, s>>>(p);
      else row_block_kernel<T, R, 1, kRowU><<<g, kThreads, 0, s>>>(p);
      VB_LAUNCH_CHECK();
      note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_ROW_BLOCK, g, dim3(kThreads), pl.V, pl.splits, 0, launches,
                  pl.nout, pl.nred, ws_used, s);
    }
    return VBT_B200_OK;
  }
  if (pl.shape == kCol) {
    ColParams p{};
    p.x = self.data;
    p.B = pl.ksize[pl.nk - 1];
    p.Rn = pl.rsize[0];
    p.S = pl.rstride[0];
    fill_dimlist(p.outer, pl.ksize, pl.kstride, pl.nk - 1);
    p.A = pl.nout / p.B;
    p.splits = pl.splits;
    p.chunk = pl.chunk;
    p.ctiles = pl.ctiles;
    p.o = o;
    if (pl.cluster > 1) {
      // small problem: fold the R-chunks inside a cluster instead of through the workspace
      p.splits = pl.cluster;
      p.chunk = (p.Rn + pl.cluster - 1) / pl.cluster;
      auto kern = pl.V > 1 ? col_cluster_kernel<T, R, VMAX> : col_cluster_kernel<T, R, 1>;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(static_cast<unsigned>(pl.ctiles), static_cast<unsigned>(pl.cluster), static_cast<unsigned>(p.A));
      cfg.blockDim = dim3(kThreads);
      cfg.stream = s;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = static_cast<unsigned>(pl.cluster);
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      if (cluster_launch_ok(reinterpret_cast<const void*>(kern), pl.cluster, cfg)) {
        VB_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
        note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_COL_CLUSTER, cfg.gridDim, cfg.blockDim, pl.V, pl.cluster,
                    pl.cluster, 1, pl.nout, pl.nred, 0, s);
        return VBT_B200_OK;
      }
      // this device cannot co-schedule such a cluster: use the workspace path
      p.splits = pl.splits;
      p.chunk = pl.chunk;
    }
    int launches = 1;
    if (pl.splits > 1) {
      p.ws_partials = partials;
      p.ws_counters = tickets;
      if (!tickets_zeroed) {
        VB_CUDA(cudaMemsetAsync(tickets, 0, pl.ws_counter_bytes, s));
        ++launches;
      }
    }
    dim3 g(static_cast<unsigned>(pl.ctiles), static_cast<unsigned>(pl.splits), static_cast<unsigned>(p.A));
    if (pl.V > 1) col_kernel<T, R, VMAX><<<g, kThreads, 0, s>>>(p);
    else col_kernel<T, R, 1><<<g, kThreads, 0, s>>>(p);
    VB_LAUNCH_CHECK();
    note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_COL, g, dim3(kThreads), pl.V, pl.splits, 0, launches, pl.nout,
                pl.nred, ws_used, s);
    return VBT_B200_OK;
  }
  GenParams p{};
  p.x = self.data;
  fill_dimlist(p.kept, pl.ksize, pl.kstride, pl.nk);
  fill_dimlist(p.red, pl.rsize, pl.rstride, pl.nr);
  p.nout = pl.nout;
  p.nred = static_cast<uint32_t>(pl.nred);
  p.o = o;
  const unsigned g = static_cast<unsigned>((pl.nout + kWarps - 1) / kWarps);
  generic_kernel<T, R><<<g, kThreads, 0, s>>>(p);
  VB_LAUNCH_CHECK();
  note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_GENERIC, dim3(g), dim3(kThreads), 1, 1, 0, 1, pl.nout, pl.nred, 0, s);
  return VBT_B200_OK;
}

template <class T>
vbt_b200_status launch_op(int op, const Plan& pl, const vbt_b200_tensor& self, const OutSpec& o,
                          void* ws, bool tz, cudaStream_t s) {
  using A = typename Widen<T>::type;
  switch (op) {
    case OP_SUM:
    case OP_MEAN: return launch<T, SumR<A>>(pl, self, o, ws, tz, s);
    case OP_PROD: return launch<T, ProdR<A>>(pl, self, o, ws, tz, s);
    case OP_MAX: return launch<T, ExtR<A, true>>(pl, self, o, ws, tz, s);
    case OP_MIN: return launch<T, ExtR<A, false>>(pl, self, o, ws, tz, s);
    case OP_ARGMAX:
      return pl.nred < 0x7fffffff ? launch<T, ArgR<A, true, int32_t>>(pl, self, o, ws, tz, s)
                                  : launch<T, ArgR<A, true, int64_t>>(pl, self, o, ws, tz, s);
    case OP_ARGMIN:
      return pl.nred < 0x7fffffff ? launch<T, ArgR<A, false, int32_t>>(pl, self, o, ws, tz, s)
                                  : launch<T, ArgR<A, false, int64_t>>(pl, self, o, ws, tz, s);
  }
  return fail(VBT_B200_INVALID_ARGUMENT, "reduce: unknown op code");
}

vbt_b200_status check_dtypes(int op, const vbt_b200_tensor& self, const vbt_b200_tensor* out,
                             const vbt_b200_tensor* out_index) {
  const char* name = op_name(op);
  const int dt = self.dtype;
  if (op == OP_MEAN)
    VB_ARG(is_float_dtype(dt), "mean: expected dtype=float32");
  else
    VB_ARG(dt == VBT_B200_I64 || is_float_dtype(dt), std::string(name) + ": unsupported dtype");
  const bool arg = op == OP_ARGMAX || op == OP_ARGMIN;
  if (arg) VB_ARG(out_index && out_index->dtype == VBT_B200_I64, std::string(name) + ": index output must be int64");
  else VB_ARG(out != nullptr, std::string(name) + ": null output");
  if (out)
    VB_ARG(out->dtype == dt || (out->dtype == VBT_B200_F32 && is_float_dtype(dt)),
           std::string(name) + ": output dtype mismatch");
  return VBT_B200_OK;
}

vbt_b200_status check_out_shape(const Plan& pl, const vbt_b200_tensor* t, const char* name) {
  if (!t) return VBT_B200_OK;
  bool ok = t->ndim == pl.out_ndim;
  for (int d = 0; ok && d < pl.out_ndim; ++d) ok = t->sizes[d] == pl.out_sizes[d];
  VB_ARG(ok, std::string(name) + ": output has the wrong shape");
  VB_ARG(is_dense_row_major(*t), std::string(name) + ": output must be dense");
  return VBT_B200_OK;
}

}  // namespace
}  // namespace vb

namespace vb {
namespace {

size_t plan_workspace_bytes(const Plan& pl) {
  if (pl.ws_partial_bytes == 0) return 0;
  return kTicketBytes + (pl.ws_partial_bytes + 15) / 16 * 16;
}

vbt_b200_status reduce_impl(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* out_index,
                            const vbt_b200_tensor* self, const int64_t* dims, int32_t ndims, int32_t keepdim,
                            void* workspace, size_t workspace_bytes, bool tickets_zeroed, bool nan_first,
                            void* stream, const Xchg* xchg = nullptr) {
  VB_ARG(op >= 0 && op < VBT_B200_R_COUNT, "reduce: unknown op code");
  const char* name = op_name(op);
  VB_TRY(validate_data(self, name));
  if (out) VB_TRY(validate_data(out, name));
  if (out_index) VB_TRY(validate_data(out_index, name));
  VB_TRY(check_dtypes(op, *self, out, out_index));
  const void* anchor = out ? out->data : out_index->data;
  DeviceScope scope(anchor);
  Plan pl;
  VB_TRY(make_plan(op, *self, dims, ndims, keepdim != 0, sm_count(scope.device()), &pl));
  if (xchg != nullptr) {
    // the exchange lives in the ticket kernels' epilogue: no cluster fold, and only the layouts
    // whose final values sit in one block per tile
    pl.cluster = 0;
    const bool row_ok = pl.shape == kRowBlock && pl.nout == 1;
    const bool col_ok = pl.shape == kCol;
    VB_ARG(row_ok || col_ok, std::string(name) + ": this layout has no fused exchange (use the partial + all-reduce path)");
    if (col_ok) {
      const int64_t tiles = (pl.nout / pl.ksize[pl.nk - 1]) * pl.ctiles;
      VB_ARG(tiles <= kXchgTiles && tiles * 32 * pl.V <= xchg->slot_floats,
             std::string(name) + ": too many outputs for the exchange buffer");
    }
  }
  VB_TRY(check_out_shape(pl, out, name));
  VB_TRY(check_out_shape(pl, out_index, name));
  if (pl.shape == kNoOutput) return VBT_B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pl.shape == kEmptyDomain) {
    // cuda_reduction.cu:1176-1216
    if (op == OP_MAX || op == OP_ARGMAX) return fail(VBT_B200_RUNTIME_ERROR, "amax: empty");
    if (op == OP_MIN || op == OP_ARGMIN) return fail(VBT_B200_RUNTIME_ERROR, "amin: empty");
    const double v = op == OP_SUM ? 0.0 : (op == OP_PROD ? 1.0 : NAN);
    const unsigned g = static_cast<unsigned>((pl.nout + 255) / 256);
    switch (out->dtype) {
      case VBT_B200_F32: fill_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(out->data), pl.nout, static_cast<float>(v)); break;
      case VBT_B200_F16: fill_kernel<__half><<<g, 256, 0, s>>>(static_cast<__half*>(out->data), pl.nout, __float2half_rn(static_cast<float>(v))); break;
      case VBT_B200_BF16: fill_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out->data), pl.nout, __float2bfloat16_rn(static_cast<float>(v))); break;
      case VBT_B200_I64: fill_kernel<int64_t><<<g, 256, 0, s>>>(static_cast<int64_t*>(out->data), pl.nout, static_cast<int64_t>(op == OP_PROD ? 1 : 0)); break;
    }
    VB_LAUNCH_CHECK();
    note_launch(VBT_B200_FAMILY_REDUCE, VBT_B200_RK_FILL, dim3(g), dim3(256), 1, 1, 0, 1, pl.nout, 0, 0, s);
    return VBT_B200_OK;
  }
  const size_t need = plan_workspace_bytes(pl);
  if (need > 0) {
    VB_ARG(workspace != nullptr && workspace_bytes >= need,
           std::string(name) + ": workspace too small (see vbt_b200_reduce_workspace_bytes)");
    VB_ARG(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, std::string(name) + ": workspace must be 16-byte aligned");
  }
  OutSpec o{};
  o.out = out ? out->data : nullptr;
  o.out_idx = out_index ? static_cast<int64_t*>(out_index->data) : nullptr;
  o.out_dtype = out ? out->dtype : self->dtype;
  o.op = op;
  o.inv_count_n = static_cast<float>(pl.nred);
  o.nan_first = nan_first ? 1 : 0;
  if (xchg != nullptr) o.x = *xchg;
  switch (self->dtype) {
    case VBT_B200_F32: return launch_op<float>(op, pl, *self, o, workspace, tickets_zeroed, s);
    case VBT_B200_F16: return launch_op<__half>(op, pl, *self, o, workspace, tickets_zeroed, s);
    case VBT_B200_BF16: return launch_op<__nv_bfloat16>(op, pl, *self, o, workspace, tickets_zeroed, s);
    case VBT_B200_I64: return launch_op<int64_t>(op, pl, *self, o, workspace, tickets_zeroed, s);
  }
  return fail(VBT_B200_INVALID_ARGUMENT, std::string(name) + ": unsupported dtype");
}

}  // namespace
}  // namespace vb

extern "C" {

size_t vbt_b200_reduce_workspace_bytes(int32_t op, const vbt_b200_tensor* self, const int64_t* dims,
                                       int32_t ndims) {
  using namespace vb;
  if (!self || validate_tensor(self, "reduce") != VBT_B200_OK) return 0;
  Plan pl;
  if (make_plan(op, *self, dims, ndims, false, sm_count(device_of(self->data)), &pl) != VBT_B200_OK) return 0;
  return plan_workspace_bytes(pl);
}

vbt_b200_status vbt_b200_reduce_shape(const vbt_b200_tensor* self, const int64_t* dims, int32_t ndims,
                                      int32_t keepdim, int64_t* out_sizes, int32_t* out_ndim) {
  using namespace vb;
  VB_TRY(validate_tensor(self, "reduce"));
  VB_ARG(self->ndim <= kMaxDims, "reduce: rank too large");
  bool reduced[kMaxDims + 1];
  VB_TRY(normalize_dims(*self, dims, ndims, "reduce", reduced));
  int n = 0;
  for (int d = 0; d < self->ndim; ++d) {
    if (!reduced[d]) out_sizes[n++] = self->sizes[d];
    else if (keepdim) out_sizes[n++] = 1;
  }
  *out_ndim = n;
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_reduce(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* out_index,
                                const vbt_b200_tensor* self, const int64_t* dims, int32_t ndims,
                                int32_t keepdim, void* workspace, size_t workspace_bytes, void* stream) {
  return vb::reduce_impl(op, out, out_index, self, dims, ndims, keepdim, workspace, workspace_bytes, false, true,
                         stream);
}

vbt_b200_status vbt_b200_reduce_zeroed_ws(int32_t op, const vbt_b200_tensor* out,
                                          const vbt_b200_tensor* out_index, const vbt_b200_tensor* self,
                                          const int64_t* dims, int32_t ndims, int32_t keepdim, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  return vb::reduce_impl(op, out, out_index, self, dims, ndims, keepdim, workspace, workspace_bytes, true, true,
                         stream);
}

vbt_b200_status vbt_b200_reduce_partial(int32_t op, const vbt_b200_tensor* partial,
                                        const vbt_b200_tensor* shard, const int64_t* dims, int32_t ndims,
                                        int32_t keepdim, void* workspace, size_t workspace_bytes,
                                        int32_t flags, void* stream) {
  using namespace vb;
  VB_ARG(op == VBT_B200_R_SUM || op == VBT_B200_R_MAX || op == VBT_B200_R_MIN,
         "reduce_partial: only sum / max / min combine across shards");
  VB_ARG(partial && shard, "reduce_partial: null tensor descriptor");
  VB_ARG(partial->dtype == VBT_B200_F32 || partial->dtype == VBT_B200_I64,
         "reduce_partial: partials are float32 or int64");
  return reduce_impl(op, partial, nullptr, shard, dims, ndims, keepdim, workspace, workspace_bytes,
                     (flags & VBT_B200_PARTIAL_WS_ZEROED) != 0, (flags & VBT_B200_PARTIAL_NOT_FIRST) == 0, stream);
}

}  // extern "C"

// =====================================================================================
// Fabric exchange: the buffers behind the fused sharded reductions (one process per GPU, or
// several GPUs in one process), and vbt_b200_reduce_exchange.
//
// Every rank owns one device buffer: two halves (call parity) of [world][slot_floats] 8-byte
// words (value, epoch) and an error word.  Ranks exchange a handle to it
// (an IPC memory handle plus, for ranks of the same process, the raw pointer) and map each
// other's buffer; after that a sharded reduction is ONE kernel launch per rank -- no
// collective library call, no scale-and-cast launch behind it.
// =====================================================================================
#include <unistd.h>

struct vbt_b200_fabric_comm {
  int device{0}, rank{0}, world{0};
  size_t slot_floats{0};
  char* local{nullptr};                          // this rank's buffer (cudaMalloc)
  char* base[VBT_B200_FABRIC_MAX_RANKS]{};       // every rank's buffer as seen from this device
  bool opened[VBT_B200_FABRIC_MAX_RANKS]{};      // mapped through cudaIpcOpenMemHandle
  bool connected{false};
  unsigned epoch{0};
};

namespace vb {
namespace {
struct CommHandle {  // what ranks exchange; VBT_B200_FABRIC_HANDLE_BYTES covers it
  cudaIpcMemHandle_t ipc;
  int64_t pid;
  uint64_t ptr;
  int32_t device;
  int32_t world;
  uint64_t slot_floats;
};
static_assert(sizeof(CommHandle) <= VBT_B200_FABRIC_HANDLE_BYTES, "handle size");

size_t comm_slot_bytes(const vbt_b200_fabric_comm& c) { return static_cast<size_t>(c.world) * c.slot_floats * 8; }
size_t comm_total_bytes(const vbt_b200_fabric_comm& c) { return 2 * comm_slot_bytes(c) + 256; }
}  // namespace
}  // namespace vb

extern "C" {

vbt_b200_status vbt_b200_fabric_comm_create(int32_t device, int32_t rank, int32_t world, size_t slot_floats,
                                            vbt_b200_fabric_comm** out) {
  using namespace vb;
  VB_ARG(out != nullptr, "fabric_comm_create: null argument");
  VB_ARG(world >= 1 && world <= VBT_B200_FABRIC_MAX_RANKS, "[Fabric] comm: world size must be 1..8");
  VB_ARG(rank >= 0 && rank < world, "[Fabric] comm: rank out of range");
  VB_ARG(slot_floats >= 1 && slot_floats <= (size_t{1} << 24), "[Fabric] comm: slot size out of range");
  int prev = 0;
  VB_CUDA(cudaGetDevice(&prev));
  VB_CUDA(cudaSetDevice(device));
  auto* c = new vbt_b200_fabric_comm();
  c->device = device; c->rank = rank; c->world = world; c->slot_floats = slot_floats;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, comm_total_bytes(*c));
  if (e == cudaSuccess) e = cudaMemset(p, 0, comm_total_bytes(*c));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    delete c;
    return fail(VBT_B200_CUDA_ERROR, std::string("[Fabric] comm: allocating the exchange buffer: ") + cudaGetErrorString(e));
  }
  c->local = static_cast<char*>(p);
  c->base[rank] = c->local;
  *out = c;
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_fabric_comm_handle(const vbt_b200_fabric_comm* c, void* handle_out) {
  using namespace vb;
  VB_ARG(c != nullptr && handle_out != nullptr, "fabric_comm_handle: null argument");
  CommHandle h{};
  int prev = 0;
  VB_CUDA(cudaGetDevice(&prev));
  VB_CUDA(cudaSetDevice(c->device));
  const cudaError_t e = cudaIpcGetMemHandle(&h.ipc, c->local);
  cudaSetDevice(prev);
  if (e != cudaSuccess) cudaGetLastError();  // same-process peers need only the pointer below
  h.pid = static_cast<int64_t>(getpid());
  h.ptr = reinterpret_cast<uint64_t>(c->local);
  h.device = c->device;
  h.world = c->world;
  h.slot_floats = c->slot_floats;
  std::memset(handle_out, 0, VBT_B200_FABRIC_HANDLE_BYTES);
  std::memcpy(handle_out, &h, sizeof(h));
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_fabric_comm_connect(vbt_b200_fabric_comm* c, const void* handles) {
  using namespace vb;
  VB_ARG(c != nullptr && handles != nullptr, "fabric_comm_connect: null argument");
  VB_ARG(!c->connected, "[Fabric] comm: already connected");
  int prev = 0;
  VB_CUDA(cudaGetDevice(&prev));
  VB_CUDA(cudaSetDevice(c->device));
  vbt_b200_status st = VBT_B200_OK;
  for (int r = 0; r < c->world && st == VBT_B200_OK; ++r) {
    if (r == c->rank) continue;
    CommHandle h{};
    std::memcpy(&h, static_cast<const char*>(handles) + static_cast<size_t>(r) * VBT_B200_FABRIC_HANDLE_BYTES, sizeof(h));
    if (h.world != c->world || h.slot_floats != c->slot_floats) {
      st = fail(VBT_B200_INVALID_ARGUMENT, "[Fabric] comm: ranks disagree on world size or slot size");
      break;
    }
    if (h.pid == static_cast<int64_t>(getpid())) {
      // another GPU of this process: plain peer access to its buffer
      int can = 0;
      cudaError_t e = cudaDeviceCanAccessPeer(&can, c->device, h.device);
      if (e == cudaSuccess && can) {
        e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
      }
      if (e != cudaSuccess || !can) {
        cudaGetLastError();
        st = fail(VBT_B200_RUNTIME_ERROR, "[Fabric] comm: device " + std::to_string(c->device) +
                                              " cannot access device " + std::to_string(h.device) + " memory (no P2P path)");
        break;
      }
      c->base[r] = reinterpret_cast<char*>(h.ptr);
    } else {
      void* p = nullptr;
      const cudaError_t e = cudaIpcOpenMemHandle(&p, h.ipc, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        cudaGetLastError();
        st = fail(VBT_B200_RUNTIME_ERROR, std::string("[Fabric] comm: mapping rank ") + std::to_string(r) +
                                              "'s exchange buffer: " + cudaGetErrorString(e));
        break;
      }
      c->base[r] = static_cast<char*>(p);
      c->opened[r] = true;
    }
  }
  cudaSetDevice(prev);
  if (st == VBT_B200_OK) c->connected = true;
  return st;
}

vbt_b200_status vbt_b200_fabric_comm_status(vbt_b200_fabric_comm* c, void* stream) {
  using namespace vb;
  VB_ARG(c != nullptr, "fabric_comm_status: null argument");
  int prev = 0;
  VB_CUDA(cudaGetDevice(&prev));
  VB_CUDA(cudaSetDevice(c->device));
  unsigned word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* status = c->local + 2 * comm_slot_bytes(*c);
  cudaError_t e = cudaMemcpyAsync(&word, status, 4, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && word != 0) e = cudaMemsetAsync(status, 0, 4, s);
  cudaSetDevice(prev);
  VB_CUDA(e);
  VB_REQUIRE(word == 0, VBT_B200_RUNTIME_ERROR,
             "[Fabric] exchange: a rank did not arrive within the time limit; the results of that call are missing");
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_fabric_comm_destroy(vbt_b200_fabric_comm* c) {
  if (c == nullptr) return VBT_B200_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(c->device);
  for (int r = 0; r < c->world; ++r)
    if (c->opened[r]) cudaIpcCloseMemHandle(c->base[r]);
  if (c->local) cudaFree(c->local);
  cudaSetDevice(prev);
  cudaGetLastError();
  delete c;
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_reduce_exchange(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* shard,
                                         const int64_t* dims, int32_t ndims, int32_t keepdim, void* workspace,
                                         size_t workspace_bytes, int32_t flags, vbt_b200_fabric_comm* comm,
                                         int32_t first_owner_rank, float scale, void* stream) {
  using namespace vb;
  VB_ARG(op == VBT_B200_R_SUM || op == VBT_B200_R_MAX || op == VBT_B200_R_MIN,
         "reduce_exchange: only sum / max / min combine across shards");
  VB_ARG(out && shard && comm, "reduce_exchange: null argument");
  VB_ARG(comm->connected || comm->world == 1, "[Fabric] comm: not connected");
  VB_ARG(is_float_dtype(shard->dtype) && is_float_dtype(out->dtype),
         "reduce_exchange: floating shards and outputs only");
  VB_ARG(first_owner_rank >= 0 && first_owner_rank < comm->world, "reduce_exchange: owner rank out of range");
  VB_ARG(device_of(out->data) == comm->device, "[Fabric] comm: the output lives on another device than the exchange buffer");
  Xchg x{};
  x.world = comm->world;
  x.rank = comm->rank;
  x.owner = first_owner_rank;
  x.epoch = comm->epoch + 1;
  x.slot_floats = static_cast<int>(comm->slot_floats);
  x.scale = scale;
  const size_t half = x.epoch & 1u;
  for (int r = 0; r < comm->world; ++r) {
    x.slots[r] = reinterpret_cast<unsigned long long*>(comm->base[r] + half * comm_slot_bytes(*comm));
  }
  x.status = reinterpret_cast<unsigned*>(comm->local + 2 * comm_slot_bytes(*comm));
  const vbt_b200_status st =
      reduce_impl(op, out, nullptr, shard, dims, ndims, keepdim, workspace, workspace_bytes,
                  (flags & VBT_B200_PARTIAL_WS_ZEROED) != 0, comm->rank == first_owner_rank, stream, &x);
  if (st == VBT_B200_OK) comm->epoch = x.epoch;  // the epoch only advances with a launch: ranks stay in step
  return st;
}

}  // extern "C"

// =====================================================================================
// vbt_b200_reduce_noalloc: the same reduction for callers that cannot hand over scratch.
//
// Some hosts of this library have no way to obtain device memory at call time: a plugin
// kernel running under a host whose allocator API only hands out "dense like" outputs, a
// callback that runs while the allocator's lock is held, or an embedder that forbids
// cudaMalloc after start-up.  For them the split reductions' scratch (chunk partials and
// ticket counters) lives in the fixed device array below instead of a caller workspace.
//
//  * The array is part of the loaded module: every GPU that loads the library holds
//    VBT_B200_NOALLOC_SCRATCH_BYTES of it until the process exits.
//  * Host code must not pass the array's name to a kernel -- in host code that name is only
//    a stand-in for the symbol, not a device address.  The device address is looked up with
//    cudaGetSymbolAddress once per device, with that device current, and cached.  That
//    look-up happens on the FIRST call on a device, so make that first call outside any
//    stream capture.
//  * Nothing is allocated or freed here, by this library or by anything it calls.
//  * All calls on a device share the one array, and it keeps whatever the previous call
//    left in it.  The only part that has to start at zero -- the ticket counters -- is
//    cleared on the stream at the start of every call.  Two calls whose kernels can overlap
//    on the GPU (different streams, no dependency) would race on the array: callers must
//    order them.
//  * Shapes whose scratch need exceeds the array are rejected with INVALID_ARGUMENT.
// =====================================================================================
static __device__ __align__(256) unsigned char vb_noalloc_scratch[VBT_B200_NOALLOC_SCRATCH_BYTES];

namespace vb {
namespace {
// device address of vb_noalloc_scratch per device ordinal; looked up under the mutex
vbt_b200_status noalloc_scratch_ptr(int device, void** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* cached[kMaxDevices] = {};
  VB_ARG(device >= 0 && device < kMaxDevices, "reduce_noalloc: device ordinal out of range");
  std::lock_guard<std::mutex> lk(mu);
  if (cached[device] == nullptr) {
    void* p = nullptr;
    // `device` is current here (DeviceScope in the caller), so this resolves that device's copy
    VB_CUDA(cudaGetSymbolAddress(&p, vb_noalloc_scratch));
    VB_REQUIRE(p != nullptr, VBT_B200_CUDA_ERROR, "reduce_noalloc: symbol address is null");
    cached[device] = p;
  }
  *out = cached[device];
  return VBT_B200_OK;
}
}  // namespace
}  // namespace vb

extern "C" vbt_b200_status vbt_b200_reduce_noalloc(int32_t op, const vbt_b200_tensor* out,
                                                   const vbt_b200_tensor* out_index,
                                                   const vbt_b200_tensor* self, const int64_t* dims,
                                                   int32_t ndims, int32_t keepdim, void* stream) {
  using namespace vb;
  VB_ARG(op >= 0 && op < VBT_B200_R_COUNT, "reduce_noalloc: unknown op code");
  VB_TRY(validate_tensor(self, "reduce_noalloc"));
  VB_ARG(out != nullptr || out_index != nullptr, "reduce_noalloc: null output");
  const size_t need = vbt_b200_reduce_workspace_bytes(op, self, dims, ndims);
  if (need > VBT_B200_NOALLOC_SCRATCH_BYTES)
    return fail(VBT_B200_INVALID_ARGUMENT,
                std::string(op_name(op)) + ": this shape needs " + std::to_string(need) +
                    " bytes of scratch, more than the fixed " +
                    std::to_string(static_cast<size_t>(VBT_B200_NOALLOC_SCRATCH_BYTES)) +
                    " bytes of vbt_b200_reduce_noalloc; use vbt_b200_reduce with a workspace");
  void* scratch = nullptr;
  if (need > 0) {
    const void* anchor = out ? out->data : out_index->data;
    DeviceScope scope(anchor);
    VB_TRY(noalloc_scratch_ptr(scope.device(), &scratch));
  }
  return vbt_b200_reduce(op, out, out_index, self, dims, ndims, keepdim, scratch, need, stream);
}
