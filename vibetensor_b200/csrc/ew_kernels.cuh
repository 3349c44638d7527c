// Elementwise kernels over a TiPlan (sm_100a).
//
// Two kernels replace the reference's dense / *_ti_strided_kernel family
// (src/vbt/ops/cuda_elementwise.cu:1409-1663, :2216-2246, :2534-2569, :2645-2662):
//
//   ew_flat_kernel   every operand is contiguous or a single broadcast value: 16-byte
//                    vectors, several per thread in flight.
//   ew_tiled_kernel  general broadcast / strided case.  Dim 0 is the dim the OUTPUT is
//                    contiguous in; a thread owns one 16-byte output vector along dim 0 and
//                    walks dim 1, so stores stay coalesced whatever the inputs look like.
//                    Offsets of the outer dims are decoded ONCE per block with 32-bit
//                    multiply-shift division; inside the loop there is only pointer
//                    stepping.  Operands that do not vary along dim 1 are loaded once and
//                    stay in registers (a broadcast operand, or a "transposed" operand whose
//                    rows have to be gathered element-wise, costs nothing per output row).
//
// The reference decodes every element's offset with up to 2*ndim 64-bit divisions per
// operand (include/vbt/core/tensor_iterator/cuda.h:25-42).
#pragma once
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "ti_plan.h"

namespace vb {

constexpr int kMaxOuter = VBT_B200_MAX_NDIM - 2;
constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;

template <int NOPS>
struct TiledParams {
  char* ptr[NOPS];
  int64_t s0[NOPS];
  int64_t s1[NOPS];
  int64_t so[NOPS][kMaxOuter];
  FastDiv odiv[kMaxOuter];
  FastDiv div_t0, div_t1;
  int n_outer;
  uint32_t n0v;   // vectors along dim 0
  int64_t size1;
  int log2_w0;    // threads along dim 0 = 1 << log2_w0
  int L;          // dim-1 passes per block
};

template <int NOPS>
struct FlatParams {
  char* ptr[NOPS];
  int s[NOPS];  // 0 or 1
  int64_t n;    // elements
};

// SPLAT: the operand is known at compile time to be broadcast along dim 0 (stride 0): one
// scalar load, and every lane of the vector is the SAME value to the compiler, so per-lane
// work on it (conversion, comparison) is done once.
template <class T, int V, bool SPLAT = false>
__device__ __forceinline__ Vec<T, V> load_vec(const T* p, int64_t s0) {
  Vec<T, V> r;
  if constexpr (V == 1) {
    r.v[0] = *p;
  } else if constexpr (SPLAT) {
    const T x = *p;
#pragma unroll
    for (int j = 0; j < V; ++j) r.v[j] = x;
  } else {
    if (s0 == 1) {
      r = *reinterpret_cast<const Vec<T, V>*>(p);
    } else if (s0 == 0) {
      const T x = *p;
#pragma unroll
      for (int j = 0; j < V; ++j) r.v[j] = x;
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) r.v[j] = p[j * s0];
    }
  }
  return r;
}

// stride 0 or 1 only (no gather): the form the deep-unrolled loops use
template <class T, int V>
__device__ __forceinline__ Vec<T, V> load_vec01(const T* p, bool unit) {
  Vec<T, V> r;
  if constexpr (V == 1) {
    r.v[0] = *p;
  } else {
    if (unit) {
      r = *reinterpret_cast<const Vec<T, V>*>(p);
    } else {
      const T x = *p;
#pragma unroll
      for (int j = 0; j < V; ++j) r.v[j] = x;
    }
  }
  return r;
}

// two floats -> two 16-bit storage values with ONE conversion instruction
__device__ __forceinline__ uint32_t pack2(float lo, float hi, __nv_bfloat16) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi, __half) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <class F, class = void>
struct has_split : std::false_type {};
template <class F>
struct has_split<F, std::void_t<decltype(F::kSplit)>> : std::bool_constant<F::kSplit> {};

template <class F, class = void>
struct has_packed2 : std::false_type {};
template <class F>
struct has_packed2<F, std::void_t<decltype(F::kPacked2)>> : std::bool_constant<F::kPacked2> {};

template <class F, class = void>
struct has_float_fn : std::false_type {};
template <class F>
struct has_float_fn<F, std::void_t<decltype(F::kFloatMath)>> : std::bool_constant<F::kFloatMath> {};

template <class F, class TO, class T1, class T2, class T3, int NIN, int V>
__device__ __forceinline__ Vec<TO, V> apply_vec(const F& f, const Vec<T1, V>& a,
                                                const Vec<T2, V>& b, const Vec<T3, V>& c) {
  Vec<TO, V> o;
  if constexpr (has_packed2<F>::value && sizeof(TO) == 2 && sizeof(T1) == 2 && sizeof(T2) == 2 && V % 2 == 0) {
    const uint32_t* wa = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* wb = reinterpret_cast<const uint32_t*>(&b);
    uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < V / 2; ++j) w[j] = f.pair(wa[j], wb[j]);
  } else if constexpr (has_float_fn<F>::value && sizeof(TO) == 2 && V % 2 == 0) {
    // 16-bit float outputs: compute in float, round and pack two lanes per instruction
    uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < V; j += 2) {
      const float lo = f.fn(to_f(a.v[j]), to_f(b.v[j]), to_f(c.v[j]));
      const float hi = f.fn(to_f(a.v[j + 1]), to_f(b.v[j + 1]), to_f(c.v[j + 1]));
      w[j / 2] = pack2(lo, hi, TO{});
    }
  } else {
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = f(a.v[j], b.v[j], c.v[j]);
  }
  return o;
}

// INV: bitmask of inputs known at compile time not to vary along dim 1 (bit 0 = first
// input); -1 = decide at run time from the strides (loads are hoisted, arithmetic is not).
// BC0: bitmask of inputs known at compile time to be broadcast along dim 0 (only used
// together with INV >= 0).
// Register budget: 4 resident blocks per SM for one- and two-input ops (64 registers); below
// that the kernel cannot cover HBM latency.  Three-input ops are left to the compiler (the
// write-dominated fused chains run best with the registers they ask for).
template <class F, class TO, class T1, class T2, class T3, int NIN, int V, int INV, int BC0 = 0>
__global__ void __launch_bounds__(kEwThreads, NIN >= 3 ? 1 : 4)
ew_tiled_kernel(const __grid_constant__ TiledParams<NIN + 1> p, const F f) {
  // rows in flight per thread: fewer when two or three inputs of eight 16-bit lanes each are
  // widened to float (register budget)
  constexpr int UNR = (V >= 8 && INV < 0 && (NIN >= 3 || (NIN == 2 && !has_packed2<F>::value))) ? 2 : kEwUnroll;
  uint32_t b = blockIdx.x, t0, t1;
  p.div_t0.divmod(b, b, t0);
  p.div_t1.divmod(b, b, t1);
  int64_t base[NIN + 1];
#pragma unroll
  for (int k = 0; k <= NIN; ++k) base[k] = 0;
  for (int d = 0; d < p.n_outer; ++d) {
    uint32_t c;
    p.odiv[d].divmod(b, b, c);
#pragma unroll
    for (int k = 0; k <= NIN; ++k) base[k] += static_cast<int64_t>(c) * p.so[k][d];
  }
  const uint32_t w0 = 1u << p.log2_w0;
  const uint32_t tx = threadIdx.x & (w0 - 1), ty = threadIdx.x >> p.log2_w0;
  const int R = kEwThreads >> p.log2_w0;
  const uint32_t v = t0 * w0 + tx;
  if (v >= p.n0v) return;
  const int64_t row0 = static_cast<int64_t>(t1) * (static_cast<int64_t>(R) * p.L) + ty;
  if (row0 >= p.size1) return;
  const int64_t rows_left = (p.size1 - row0 + R - 1) / R;
  const int n = rows_left < p.L ? static_cast<int>(rows_left) : p.L;
#pragma unroll
  for (int k = 0; k <= NIN; ++k) base[k] += static_cast<int64_t>(v) * V * p.s0[k] + row0 * p.s1[k];

  TO* po = reinterpret_cast<TO*>(p.ptr[0]) + base[0];
  const T1* p1 = reinterpret_cast<const T1*>(p.ptr[1]) + base[1];
  const T2* p2 = NIN >= 2 ? reinterpret_cast<const T2*>(p.ptr[NIN >= 2 ? 2 : 0]) + base[NIN >= 2 ? 2 : 0] : nullptr;
  const T3* p3 = NIN >= 3 ? reinterpret_cast<const T3*>(p.ptr[NIN >= 3 ? 3 : 0]) + base[NIN >= 3 ? 3 : 0] : nullptr;
  const int64_t so_ = R * p.s1[0];
  const int64_t st1 = R * p.s1[1];
  const int64_t st2 = NIN >= 2 ? R * p.s1[NIN >= 2 ? 2 : 0] : 0;
  const int64_t st3 = NIN >= 3 ? R * p.s1[NIN >= 3 ? 3 : 0] : 0;
  const int64_t s01 = p.s0[1];
  const int64_t s02 = NIN >= 2 ? p.s0[NIN >= 2 ? 2 : 0] : 0;
  const int64_t s03 = NIN >= 3 ? p.s0[NIN >= 3 ? 3 : 0] : 0;
  const bool inv1 = INV >= 0 ? ((INV >> 0) & 1) : (st1 == 0);
  const bool inv2 = NIN >= 2 && (INV >= 0 ? ((INV >> 1) & 1) : (st2 == 0));
  const bool inv3 = NIN >= 3 && (INV >= 0 ? ((INV >> 2) & 1) : (st3 == 0));

  Vec<T1, V> a0{};
  Vec<T2, V> b0{};
  Vec<T3, V> c0{};
  constexpr bool sp1 = INV >= 0 && (BC0 & 1), sp2 = INV >= 0 && (BC0 & 2), sp3 = INV >= 0 && (BC0 & 4);
  if (inv1) a0 = load_vec<T1, V, sp1>(p1, s01);
  if constexpr (NIN >= 2) { if (inv2) b0 = load_vec<T2, V, sp2>(p2, s02); }
  if constexpr (NIN >= 3) { if (inv3) c0 = load_vec<T3, V, sp3>(p3, s03); }

  if constexpr (INV == 6 && NIN == 3 && has_split<F>::value && sizeof(TO) == 2 && V % 2 == 0) {
    // inputs 2 and 3 are constant along the rows: their part of the expression is computed
    // once, the loop only loads input 1, finishes the expression, rounds in pairs and stores
    float t[V];
#pragma unroll
    for (int j = 0; j < V; ++j) t[j] = f.pre(to_f(b0.v[j]), to_f(c0.v[j]));
    auto finish = [&](const Vec<T1, V>& av, int l) {
      Vec<TO, V> o;
      uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < V; j += 2)
        w[j / 2] = pack2(f.fin(to_f(av.v[j]), t[j]), f.fin(to_f(av.v[j + 1]), t[j + 1]), TO{});
      *reinterpret_cast<Vec<TO, V>*>(po + l * so_) = o;
    };
    int l = 0;
    for (; l + 8 <= n; l += 8) {  // eight rows' loads in flight, then eight stores
      Vec<T1, V> av[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) av[u] = load_vec<T1, V, sp1>(p1 + (l + u) * st1, s01);
#pragma unroll
      for (int u = 0; u < 8; ++u) finish(av[u], l + u);
    }
    for (; l < n; ++l) finish(load_vec<T1, V, sp1>(p1 + l * st1, s01), l);
    return;
  }
  if constexpr (NIN <= 2 && INV < 0) {
    // exactly one input varies along the rows (a unary op, or a binary op whose other operand
    // is constant along them): DEEP rows in flight per thread (eight; four when 16-bit
    // values are widened to float lane by lane, which would not fit the register budget
    // eight deep).  Two separate loops so that only one buffer is live at a time.
    constexpr int DEEP = ((sizeof(T1) == 2 || sizeof(T2) == 2) && !has_packed2<F>::value) ? 4 : 8;
    auto emit = [&](const Vec<T1, V>& av, const Vec<T2, V>& bv, int l) {
      const Vec<TO, V> o = apply_vec<F, TO, T1, T2, T3, NIN, V>(f, av, bv, c0);
      if constexpr (V == 1) po[l * so_] = o.v[0];
      else *reinterpret_cast<Vec<TO, V>*>(po + l * so_) = o;
    };
    if (!inv1 && (NIN == 1 || inv2) && (V == 1 || s01 == 0 || s01 == 1)) {
      const bool unit = s01 == 1;
      int l = 0;
      for (; l + DEEP <= n; l += DEEP) {
        Vec<T1, V> av[DEEP];
#pragma unroll
        for (int u = 0; u < DEEP; ++u) av[u] = load_vec01<T1, V>(p1 + (l + u) * st1, unit);
#pragma unroll
        for (int u = 0; u < DEEP; ++u) emit(av[u], b0, l + u);
      }
      for (; l < n; ++l) emit(load_vec01<T1, V>(p1 + l * st1, unit), b0, l);
      return;
    }
    if constexpr (NIN == 2) {
      if (inv1 && !inv2 && (V == 1 || s02 == 0 || s02 == 1)) {
        const bool unit = s02 == 1;
        int l = 0;
        for (; l + DEEP <= n; l += DEEP) {
          Vec<T2, V> bv[DEEP];
#pragma unroll
          for (int u = 0; u < DEEP; ++u) bv[u] = load_vec01<T2, V>(p2 + (l + u) * st2, unit);
#pragma unroll
          for (int u = 0; u < DEEP; ++u) emit(a0, bv[u], l + u);
        }
        for (; l < n; ++l) emit(a0, load_vec01<T2, V>(p2 + l * st2, unit), l);
        return;
      }
    }
  }
  // General case.  When no input needs a gather along dim 0 (every stride there is 0 or 1) the
  // loads are the two-way load_vec01 and UNR rows are in flight; the gather form (V scalar loads
  // per input) is kept out of that loop -- with it inside, the 16-bit kernels spill -- and
  // runs one row at a time.
  const bool u1 = s01 == 1, u2 = s02 == 1, u3 = s03 == 1;
  const bool nogather = V == 1 || ((inv1 || s01 == 0 || u1) && (NIN < 2 || inv2 || s02 == 0 || u2) &&
                                   (NIN < 3 || inv3 || s03 == 0 || u3));
  int l = 0;
  if (nogather) {
    // invariant inputs sit in every slot of the row buffers once, so that the loop body has no
    // select between two vectors (which the compiler would do through local memory)
    Vec<T1, V> a[UNR];
    Vec<T2, V> bb[NIN >= 2 ? UNR : 1];
    Vec<T3, V> c[NIN >= 3 ? UNR : 1];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      a[u] = a0;
      if constexpr (NIN >= 2) bb[u] = b0; else bb[0] = b0;
      if constexpr (NIN >= 3) c[u] = c0; else c[0] = c0;
    }
    for (; l + UNR <= n; l += UNR) {
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (!inv1) a[u] = load_vec01<T1, V>(p1 + (l + u) * st1, u1);
        if constexpr (NIN >= 2) { if (!inv2) bb[u] = load_vec01<T2, V>(p2 + (l + u) * st2, u2); }
        if constexpr (NIN >= 3) { if (!inv3) c[u] = load_vec01<T3, V>(p3 + (l + u) * st3, u3); }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const Vec<TO, V> o = apply_vec<F, TO, T1, T2, T3, NIN, V>(f, a[u], bb[NIN >= 2 ? u : 0], c[NIN >= 3 ? u : 0]);
        if constexpr (V == 1) po[(l + u) * so_] = o.v[0];
        else *reinterpret_cast<Vec<TO, V>*>(po + (l + u) * so_) = o;
      }
    }
    for (; l < n; ++l) {
      if (!inv1) a[0] = load_vec01<T1, V>(p1 + l * st1, u1);
      if constexpr (NIN >= 2) { if (!inv2) bb[0] = load_vec01<T2, V>(p2 + l * st2, u2); }
      if constexpr (NIN >= 3) { if (!inv3) c[0] = load_vec01<T3, V>(p3 + l * st3, u3); }
      const Vec<TO, V> o = apply_vec<F, TO, T1, T2, T3, NIN, V>(f, a[0], bb[0], c[0]);
      if constexpr (V == 1) po[l * so_] = o.v[0];
      else *reinterpret_cast<Vec<TO, V>*>(po + l * so_) = o;
    }
    return;
  }
  for (; l < n; ++l) {
    const Vec<T1, V> a = inv1 ? a0 : load_vec<T1, V, sp1>(p1 + l * st1, s01);
    Vec<T2, V> bb = b0;
    Vec<T3, V> c = c0;
    if constexpr (NIN >= 2) { if (!inv2) bb = load_vec<T2, V, sp2>(p2 + l * st2, s02); }
    if constexpr (NIN >= 3) { if (!inv3) c = load_vec<T3, V, sp3>(p3 + l * st3, s03); }
    const Vec<TO, V> o = apply_vec<F, TO, T1, T2, T3, NIN, V>(f, a, bb, c);
    if constexpr (V == 1) po[l * so_] = o.v[0];
    else *reinterpret_cast<Vec<TO, V>*>(po + l * so_) = o;
  }
}

template <class F, class TO, class T1, class T2, class T3, int NIN, int V>
__global__ void __launch_bounds__(kEwThreads)
ew_flat_kernel(const __grid_constant__ FlatParams<NIN + 1> p, const F f) {
  const int64_t nvec = p.n / V;
  TO* po = reinterpret_cast<TO*>(p.ptr[0]);
  const T1* p1 = reinterpret_cast<const T1*>(p.ptr[1]);
  const T2* p2 = reinterpret_cast<const T2*>(p.ptr[NIN >= 2 ? 2 : 0]);
  const T3* p3 = reinterpret_cast<const T3*>(p.ptr[NIN >= 3 ? 3 : 0]);
  const int s1 = p.s[1], s2 = NIN >= 2 ? p.s[NIN >= 2 ? 2 : 0] : 0, s3 = NIN >= 3 ? p.s[NIN >= 3 ? 3 : 0] : 0;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * (kEwThreads * kEwUnroll) + threadIdx.x;
  Vec<T1, V> a[kEwUnroll];
  Vec<T2, V> bb[kEwUnroll];
  Vec<T3, V> c[kEwUnroll];
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const int64_t i = first + u * kEwThreads;
    bb[u] = Vec<T2, V>{};
    c[u] = Vec<T3, V>{};
    if (i < nvec) {
      a[u] = load_vec<T1, V>(p1 + i * V * s1, s1);
      if constexpr (NIN >= 2) bb[u] = load_vec<T2, V>(p2 + i * V * s2, s2);
      if constexpr (NIN >= 3) c[u] = load_vec<T3, V>(p3 + i * V * s3, s3);
    } else {
      a[u] = Vec<T1, V>{};
    }
  }
#pragma unroll
  for (int u = 0; u < kEwUnroll; ++u) {
    const int64_t i = first + u * kEwThreads;
    if (i < nvec) {
      const Vec<TO, V> o = apply_vec<F, TO, T1, T2, T3, NIN, V>(f, a[u], bb[u], c[u]);
      *reinterpret_cast<Vec<TO, V>*>(po + i * V) = o;
    }
  }
  if constexpr (V > 1) {  // ragged tail, at most V-1 elements
    if (blockIdx.x == 0) {
      const int64_t i = nvec * V + threadIdx.x;
      if (i < p.n) {
        T2 bv{};
        T3 cv{};
        if constexpr (NIN >= 2) bv = p2[i * s2];
        if constexpr (NIN >= 3) cv = p3[i * s3];
        po[i] = f(p1[i * s1], bv, cv);
      }
    }
  }
}

// Transposing variant: some inputs are contiguous along ANOTHER iteration dim than the output
// (a transposed view copied to dense, an op between a tensor and its transpose, ...).  Read
// straight from global memory they cost one 32-byte sector per element.  Here a block owns a
// (32P x 32P) tile over (dim 0, dim 1 := the inputs' contiguous dim): up to two such inputs
// are loaded along THEIR contiguous dim, P elements per lane, into shared memory; the block
// synchronises; every warp then reads the tile transposed while it writes 32P consecutive
// outputs along dim 0, P per lane.  P = 2 when every staged operand and the output allow
// aligned element pairs, else 1.  Inputs not in `tmask` are read directly with their strides.
constexpr int kTrMaxStaged = 2;
template <class F, class TO, class T1, class T2, class T3, int NIN, int P>
__global__ void __launch_bounds__(kEwThreads)
ew_transpose_kernel(const __grid_constant__ TiledParams<NIN + 1> p, const F f, const int tmask) {
  constexpr int TILE = 32 * P;
  constexpr int PITCH = TILE + 2;  // even, so element pairs stay aligned
  constexpr int kMaxEs = sizeof(T1) > sizeof(T2) ? (sizeof(T1) > sizeof(T3) ? sizeof(T1) : sizeof(T3))
                                                 : (sizeof(T2) > sizeof(T3) ? sizeof(T2) : sizeof(T3));
  __shared__ __align__(16) unsigned char sm[kTrMaxStaged][TILE * PITCH * kMaxEs];
  uint32_t b = blockIdx.x, t0, t1;
  p.div_t0.divmod(b, b, t0);
  p.div_t1.divmod(b, b, t1);
  int64_t base[NIN + 1];
#pragma unroll
  for (int k = 0; k <= NIN; ++k) base[k] = 0;
  for (int d = 0; d < p.n_outer; ++d) {
    uint32_t c;
    p.odiv[d].divmod(b, b, c);
#pragma unroll
    for (int k = 0; k <= NIN; ++k) base[k] += static_cast<int64_t>(c) * p.so[k][d];
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t i0 = static_cast<int64_t>(t0) * TILE, j0 = static_cast<int64_t>(t1) * TILE;
  const int64_t size0 = p.n0v;  // elements along dim 0
  // shared-memory slot of each staged input (first staged -> slot 0, second -> slot 1)
  const int slot1 = 0, slot2 = (tmask & 1) ? 1 : 0, slot3 = ((tmask & 1) ? 1 : 0) + ((tmask & 2) ? 1 : 0);
  T1* s1 = reinterpret_cast<T1*>(sm[slot1]);
  T2* s2 = reinterpret_cast<T2*>(sm[slot2 < kTrMaxStaged ? slot2 : 0]);
  T3* s3 = reinterpret_cast<T3*>(sm[slot3 < kTrMaxStaged ? slot3 : 0]);
  const T1* g1 = reinterpret_cast<const T1*>(p.ptr[1]) + base[1];
  const T2* g2 = reinterpret_cast<const T2*>(p.ptr[NIN >= 2 ? 2 : 0]) + base[NIN >= 2 ? 2 : 0];
  const T3* g3 = reinterpret_cast<const T3*>(p.ptr[NIN >= 3 ? 3 : 0]) + base[NIN >= 3 ? 3 : 0];
  const int64_t a0 = p.s0[1], a1 = p.s1[1];
  const int64_t b0 = p.s0[NIN >= 2 ? 2 : 0], b1 = p.s1[NIN >= 2 ? 2 : 0];
  const int64_t c0 = p.s0[NIN >= 3 ? 3 : 0], c1 = p.s1[NIN >= 3 ? 3 : 0];
  // stage: a warp reads 32P consecutive elements along dim 1 (stride 1 for staged inputs)
#pragma unroll
  for (int r = 0; r < TILE / 8; ++r) {
    const int il = w + 8 * r;
    const int64_t i = i0 + il, j = j0 + lane * P;
    if (i < size0 && j < p.size1) {  // size1 % P == 0 when P == 2
      if (tmask & 1)
        *reinterpret_cast<Vec<T1, P>*>(s1 + il * PITCH + lane * P) = *reinterpret_cast<const Vec<T1, P>*>(g1 + i * a0 + j);
      if constexpr (NIN >= 2) {
        if (tmask & 2)
          *reinterpret_cast<Vec<T2, P>*>(s2 + il * PITCH + lane * P) = *reinterpret_cast<const Vec<T2, P>*>(g2 + i * b0 + j);
      }
      if constexpr (NIN >= 3) {
        if (tmask & 4)
          *reinterpret_cast<Vec<T3, P>*>(s3 + il * PITCH + lane * P) = *reinterpret_cast<const Vec<T3, P>*>(g3 + i * c0 + j);
      }
    }
  }
  __syncthreads();
  // direct inputs that are constant over the whole tile (a broadcast mask, a scalar) are
  // read once per thread instead of once per element
  const bool k1 = !(tmask & 1) && a0 == 0 && a1 == 0;
  const bool k2 = NIN >= 2 && !(tmask & 2) && b0 == 0 && b1 == 0;
  const bool k3 = NIN >= 3 && !(tmask & 4) && c0 == 0 && c1 == 0;
  T1 ka{};
  T2 kb{};
  T3 kc{};
  if (k1) ka = g1[0];
  if constexpr (NIN >= 2) { if (k2) kb = g2[0]; }
  if constexpr (NIN >= 3) { if (k3) kc = g3[0]; }
  // compute and store: a warp writes 32P consecutive elements along dim 0, P per lane
  TO* go = reinterpret_cast<TO*>(p.ptr[0]) + base[0];
#pragma unroll
  for (int r = 0; r < TILE / 8; ++r) {
    const int jl = w + 8 * r;
    const int64_t i = i0 + lane * P, j = j0 + jl;
    if (i < size0 && j < p.size1) {  // size0 % P == 0 when P == 2
      Vec<TO, P> o;
#pragma unroll
      for (int e = 0; e < P; ++e) {
        const int il = lane * P + e;
        const T1 a = (tmask & 1) ? s1[il * PITCH + jl] : (k1 ? ka : g1[(i + e) * a0 + j * a1]);
        T2 bb{};
        T3 c{};
        if constexpr (NIN >= 2) bb = (tmask & 2) ? s2[il * PITCH + jl] : (k2 ? kb : g2[(i + e) * b0 + j * b1]);
        if constexpr (NIN >= 3) c = (tmask & 4) ? s3[il * PITCH + jl] : (k3 ? kc : g3[(i + e) * c0 + j * c1]);
        o.v[e] = f(a, bb, c);
      }
      *reinterpret_cast<Vec<TO, P>*>(go + i * p.s0[0] + j * p.s1[0]) = o;  // s0[0] == 1 when P == 2
    }
  }
}

// Transposing variant for 16- and 32-bit outputs and staged inputs of up to 32 bits (a bool mask,
// a bf16 or fp32 operand): a (64 x 64) tile, but every lane moves FOUR elements per access
// instead of two (8 or 16 bytes), so a warp instruction covers two rows of 16 lanes.  Staged inputs are written to shared memory
// already transposed (tile[j][i], one store per element) with the 4-element groups of a row
// XOR-swizzled by the row's group index: the 16 lanes of a half-warp then hit 16 different banks
// on the store, and the vector reads along i are conflict-free.  Needs sizes, strides and bases
// that keep groups of four aligned; the host checks.
// LIE: one more input lies like the output (unit stride along dim 0, groups of four aligned; bits
// 4..6 of `tmask` say which) and is brought into the staging slot that the transposed inputs leave
// free.  A separate instantiation: with the extra paths compiled into the one kernel, the where()
// of the four-launch chain -- which cannot use them -- ran 14 % slower.
// one-input ops (copies, unary ops on a transposed view) walk four tiles per block; with more
// operands in play that order measured slower than one tile per block
template <int NIN> constexpr int kTr4TilesPerBlock = NIN == 1 ? 4 : 1;

template <class F, class TO, class T1, class T2, class T3, int NIN, bool LIE = false>
__global__ void __launch_bounds__(kEwThreads)
ew_transpose4_kernel(const __grid_constant__ TiledParams<NIN + 1> p, const F f, const int tmask) {
  constexpr int TILE = 64;
  constexpr int kStageEs = (sizeof(T1) == 4 || (NIN >= 2 && sizeof(T2) == 4) || (NIN >= 3 && sizeof(T3) == 4)) ? 4 : 2;
  __shared__ __align__(16) unsigned char sm[kTrMaxStaged][TILE * TILE * kStageEs];
  uint32_t b = blockIdx.x, t0, t1;
  p.div_t0.divmod(b, b, t0);
  p.div_t1.divmod(b, b, t1);
  int64_t base[NIN + 1];
#pragma unroll
  for (int k = 0; k <= NIN; ++k) base[k] = 0;
  for (int d = 0; d < p.n_outer; ++d) {
    uint32_t c;
    p.odiv[d].divmod(b, b, c);
#pragma unroll
    for (int k = 0; k <= NIN; ++k) base[k] += static_cast<int64_t>(c) * p.so[k][d];
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int h = lane >> 4, q = lane & 15;
  const int64_t i0 = static_cast<int64_t>(t0) * TILE;
  const int64_t size0 = p.n0v;
  const int slot2 = (tmask & 1) ? 1 : 0, slot3 = ((tmask & 1) ? 1 : 0) + ((tmask & 2) ? 1 : 0);
  T1* s1 = reinterpret_cast<T1*>(sm[0]);
  T2* s2 = reinterpret_cast<T2*>(sm[slot2 < kTrMaxStaged ? slot2 : 0]);
  T3* s3 = reinterpret_cast<T3*>(sm[slot3 < kTrMaxStaged ? slot3 : 0]);
  const T1* g1 = reinterpret_cast<const T1*>(p.ptr[1]) + base[1];
  const T2* g2 = reinterpret_cast<const T2*>(p.ptr[NIN >= 2 ? 2 : 0]) + base[NIN >= 2 ? 2 : 0];
  const T3* g3 = reinterpret_cast<const T3*>(p.ptr[NIN >= 3 ? 3 : 0]) + base[NIN >= 3 ? 3 : 0];
  const int64_t a0 = p.s0[1], a1 = p.s1[1];
  const int64_t b0 = p.s0[NIN >= 2 ? 2 : 0], b1 = p.s1[NIN >= 2 ? 2 : 0];
  const int64_t c0 = p.s0[NIN >= 3 ? 3 : 0], c1 = p.s1[NIN >= 3 ? 3 : 0];
  // a block walks kTiles consecutive tiles along dim 1: the offset decoding above is paid once
  constexpr int kTiles = kTr4TilesPerBlock<NIN>;
  if constexpr (NIN == 1 && sizeof(T1) <= 4) {
    // One transposed input (a copy or a unary op on a transposed view): the tiles alternate
    // between the two staging slots, and the loads of tile t + 1 are in flight -- in registers --
    // while tile t is written out.  One barrier per tile.  Same shared-memory layout as below.
    constexpr int kRounds = sizeof(T1) == 2 ? TILE / 32 : TILE / 16;
    constexpr int kWordsPerRound = sizeof(T1) == 1 ? 1 : 4;
    uint32_t raw[kRounds * kWordsPerRound];
    auto load_tile = [&](int64_t j0) {
      const int64_t j = j0 + q * 4;
      if (j >= p.size1) return;
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        if constexpr (sizeof(T1) == 2) {
          const int64_t i = i0 + 2 * (w * 2 + h + 16 * r);
          if (i >= size0) continue;  // size0 is a multiple of four: the odd row exists too
          const uint2 ve = *reinterpret_cast<const uint2*>(g1 + i * a0 + j);
          const uint2 vo = *reinterpret_cast<const uint2*>(g1 + (i + 1) * a0 + j);
          raw[4 * r] = ve.x; raw[4 * r + 1] = ve.y; raw[4 * r + 2] = vo.x; raw[4 * r + 3] = vo.y;
        } else if constexpr (sizeof(T1) == 4) {
          const int64_t i = i0 + w * 2 + h + 16 * r;
          if (i >= size0) continue;
          const uint4 v = *reinterpret_cast<const uint4*>(g1 + i * a0 + j);
          raw[4 * r] = v.x; raw[4 * r + 1] = v.y; raw[4 * r + 2] = v.z; raw[4 * r + 3] = v.w;
        } else {
          const int64_t i = i0 + w * 2 + h + 16 * r;
          if (i >= size0) continue;
          raw[r] = *reinterpret_cast<const uint32_t*>(g1 + i * a0 + j);
        }
      }
    };
    auto put_tile = [&](unsigned char* slot, int64_t j0) {
      if (j0 + q * 4 >= p.size1) return;
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        if constexpr (sizeof(T1) == 2) {
          const int pi = w * 2 + h + 16 * r;
          if (i0 + 2 * pi >= size0) continue;
          uint32_t* d = reinterpret_cast<uint32_t*>(slot) + (q * 4) * (TILE / 2);
          const int wi = pi ^ (2 * q);
          d[0 * (TILE / 2) + wi] = __byte_perm(raw[4 * r], raw[4 * r + 2], 0x5410);
          d[1 * (TILE / 2) + wi] = __byte_perm(raw[4 * r], raw[4 * r + 2], 0x7632);
          d[2 * (TILE / 2) + wi] = __byte_perm(raw[4 * r + 1], raw[4 * r + 3], 0x5410);
          d[3 * (TILE / 2) + wi] = __byte_perm(raw[4 * r + 1], raw[4 * r + 3], 0x7632);
        } else {
          const int il = w * 2 + h + 16 * r;
          if (i0 + il >= size0) continue;
          const int col = (((il >> 2) ^ q) << 2) + (il & 3);
          if constexpr (sizeof(T1) == 4) {
            uint32_t* d = reinterpret_cast<uint32_t*>(slot) + (q * 4) * TILE + col;
#pragma unroll
            for (int e = 0; e < 4; ++e) d[e * TILE] = raw[4 * r + e];
          } else {
            uint8_t* d = reinterpret_cast<uint8_t*>(slot) + (q * 4) * TILE + col;
#pragma unroll
            for (int e = 0; e < 4; ++e) d[e * TILE] = static_cast<uint8_t>(raw[r] >> (8 * e));
          }
        }
      }
    };
    TO* const go = reinterpret_cast<TO*>(p.ptr[0]) + base[0];
    const int64_t first_j0 = static_cast<int64_t>(t1) * kTiles * TILE;
    if (first_j0 < p.size1) load_tile(first_j0);
#pragma unroll 1
    for (int tt = 0; tt < kTiles; ++tt) {
      const int64_t j0 = first_j0 + static_cast<int64_t>(tt) * TILE;
      if (j0 >= p.size1) break;
      unsigned char* const slot = sm[tt & 1];
      put_tile(slot, j0);
      __syncthreads();  // also: every thread has left the tile that used this slot two turns ago
      if (tt + 1 < kTiles && j0 + TILE < p.size1) load_tile(j0 + TILE);
      const T1* const st = reinterpret_cast<const T1*>(slot);
#pragma unroll
      for (int r = 0; r < TILE / 16; ++r) {
        const int jl = w * 2 + h + 16 * r;
        const int64_t i = i0 + q * 4, j = j0 + jl;
        if (i < size0 && j < p.size1) {
          const Vec<T1, 4> va = *reinterpret_cast<const Vec<T1, 4>*>(st + jl * TILE + ((q ^ ((jl >> 2) & 15)) << 2));
          const Vec<TO, 4> o = apply_vec<F, TO, T1, T2, T3, NIN, 4>(f, va, Vec<T2, 4>{}, Vec<T3, 4>{});
          *reinterpret_cast<Vec<TO, 4>*>(go + i + j * p.s1[0]) = o;
        }
      }
    }
    return;
  }
#pragma unroll 1
  for (int tt = 0; tt < kTiles; ++tt) {
  const int64_t j0 = (static_cast<int64_t>(t1) * kTiles + tt) * TILE;
  if (j0 >= p.size1) break;
  if (tt > 0) __syncthreads();  // readers of the previous tile are done
  // 8- and 32-bit inputs: a lane takes four elements of ONE row and stores them one by one.
  // 16-bit inputs: a lane takes four elements of TWO adjacent rows and stores, per column, the
  // (even row, odd row) pair as one 32-bit word -- half the shared-memory stores per element.
  // Both produce the same layout: tile[j][i] with the groups of four along i XOR-swizzled by j / 4.
  auto stage = [&](auto* sdst, const auto* gsrc, int64_t st0) {
    using E = std::remove_cv_t<std::remove_pointer_t<decltype(gsrc)>>;
    const int64_t j = j0 + q * 4;
    if (j >= p.size1) return;
    if constexpr (sizeof(E) == 2) {
      uint32_t* d = reinterpret_cast<uint32_t*>(sdst) + (q * 4) * (TILE / 2);
#pragma unroll
      for (int r = 0; r < TILE / 32; ++r) {
        const int pi = w * 2 + h + 16 * r;  // row pair within the tile
        const int64_t i = i0 + 2 * pi;
        if (i >= size0) continue;           // size0 is a multiple of four: the odd row exists too
        const uint2 ve = *reinterpret_cast<const uint2*>(gsrc + i * st0 + j);
        const uint2 vo = *reinterpret_cast<const uint2*>(gsrc + (i + 1) * st0 + j);
        const int wi = pi ^ (2 * q);
        d[0 * (TILE / 2) + wi] = __byte_perm(ve.x, vo.x, 0x5410);
        d[1 * (TILE / 2) + wi] = __byte_perm(ve.x, vo.x, 0x7632);
        d[2 * (TILE / 2) + wi] = __byte_perm(ve.y, vo.y, 0x5410);
        d[3 * (TILE / 2) + wi] = __byte_perm(ve.y, vo.y, 0x7632);
      }
    } else {
      using R = std::conditional_t<sizeof(E) == 1, uint8_t, uint32_t>;
#pragma unroll
      for (int r = 0; r < TILE / 16; ++r) {
        const int il = w * 2 + h + 16 * r;
        const int64_t i = i0 + il;
        if (i >= size0) continue;
        const Vec<R, 4> v = *reinterpret_cast<const Vec<R, 4>*>(gsrc + i * st0 + j);
        const int col = (((il >> 2) ^ q) << 2) + (il & 3);  // swizzled position of row-element il
        R* d = reinterpret_cast<R*>(sdst) + (q * 4) * TILE + col;
#pragma unroll
        for (int e = 0; e < 4; ++e) d[e * TILE] = v.v[e];
      }
    }
  };
  // an input that is read as it lies (bits 4..6 of tmask: unit stride along dim 0, groups of four
  // aligned) goes into the free staging slot by asynchronous copies issued BEFORE the transposed
  // input is staged, so that a tile costs one round trip to memory, not two; every thread reads
  // back only what it copied itself
  unsigned char* const lie = sm[kTrMaxStaged - 1];
  auto copy_as_it_lies = [&](const auto* gsrc, int64_t st1) {
    using E = std::remove_cv_t<std::remove_pointer_t<decltype(gsrc)>>;
#pragma unroll
    for (int r = 0; r < TILE / 16; ++r) {
      const int jl = w * 2 + h + 16 * r;
      const int64_t i = i0 + q * 4, j = j0 + jl;
      if (i < size0 && j < p.size1)
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(lie)) + static_cast<uint32_t>((jl * TILE + q * 4) * sizeof(E))),
                     "l"(gsrc + i + j * st1), "n"(4 * sizeof(E))
                     : "memory");
    }
  };
  if constexpr (LIE && sizeof(T1) <= 4) { if (tmask & 16) copy_as_it_lies(g1, a1); }
  if constexpr (LIE && NIN >= 2 && sizeof(T2) <= 4) { if (tmask & 32) copy_as_it_lies(g2, b1); }
  if constexpr (LIE && NIN >= 3 && sizeof(T3) <= 4) { if (tmask & 64) copy_as_it_lies(g3, c1); }
  if constexpr (sizeof(T1) <= 4) { if (tmask & 1) stage(s1, g1, a0); }
  if constexpr (NIN >= 2 && sizeof(T2) <= 4) { if (tmask & 2) stage(s2, g2, b0); }
  if constexpr (NIN >= 3 && sizeof(T3) <= 4) { if (tmask & 4) stage(s3, g3, c0); }
  if constexpr (LIE) asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();
  const bool k1 = !(tmask & 1) && a0 == 0 && a1 == 0;
  const bool k2 = NIN >= 2 && !(tmask & 2) && b0 == 0 && b1 == 0;
  const bool k3 = NIN >= 3 && !(tmask & 4) && c0 == 0 && c1 == 0;
  T1 ka{};
  T2 kb{};
  T3 kc{};
  if (k1) ka = g1[0];
  if constexpr (NIN >= 2) { if (k2) kb = g2[0]; }
  if constexpr (NIN >= 3) { if (k3) kc = g3[0]; }
  TO* go = reinterpret_cast<TO*>(p.ptr[0]) + base[0];
#pragma unroll
  for (int r = 0; r < TILE / 16; ++r) {
    const int jl = w * 2 + h + 16 * r;
    const int64_t i = i0 + q * 4, j = j0 + jl;
    if (i < size0 && j < p.size1) {
      const int so = jl * TILE + ((q ^ ((jl >> 2) & 15)) << 2);
      Vec<T1, 4> va;
      Vec<T2, 4> vb{};
      Vec<T3, 4> vc{};
      if constexpr (sizeof(T1) <= 4) {
        if (tmask & 1) va = *reinterpret_cast<const Vec<T1, 4>*>(s1 + so);
      }
      if (LIE && sizeof(T1) <= 4 && (tmask & 16)) {
        va = *reinterpret_cast<const Vec<T1, 4>*>(lie + (jl * TILE + q * 4) * sizeof(T1));
      } else if (!(tmask & 1) || sizeof(T1) > 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) va.v[e] = k1 ? ka : g1[(i + e) * a0 + j * a1];
      }
      if constexpr (NIN >= 2) {
        if constexpr (sizeof(T2) <= 4) {
          if (tmask & 2) vb = *reinterpret_cast<const Vec<T2, 4>*>(s2 + so);
        }
        if (LIE && sizeof(T2) <= 4 && (tmask & 32)) {
          vb = *reinterpret_cast<const Vec<T2, 4>*>(lie + (jl * TILE + q * 4) * sizeof(T2));
        } else if (!(tmask & 2) || sizeof(T2) > 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) vb.v[e] = k2 ? kb : g2[(i + e) * b0 + j * b1];
        }
      }
      if constexpr (NIN >= 3) {
        if constexpr (sizeof(T3) <= 4) {
          if (tmask & 4) vc = *reinterpret_cast<const Vec<T3, 4>*>(s3 + so);
        }
        if (LIE && sizeof(T3) <= 4 && (tmask & 64)) {
          vc = *reinterpret_cast<const Vec<T3, 4>*>(lie + (jl * TILE + q * 4) * sizeof(T3));
        } else if (!(tmask & 4) || sizeof(T3) > 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) vc.v[e] = k3 ? kc : g3[(i + e) * c0 + j * c1];
        }
      }
      const Vec<TO, 4> o = apply_vec<F, TO, T1, T2, T3, NIN, 4>(f, va, vb, vc);
      *reinterpret_cast<Vec<TO, 4>*>(go + i + j * p.s1[0]) = o;
    }
  }
  }
}

// Host: picks the kernel for the plan and launches it.  INV_SPECIAL >= 0 additionally
// instantiates the tiled vector kernel for that compile-time invariance mask and uses it
// when the plan's strides match it.
// LEAN leaves out the transposing kernels (used for the long tail of ops, to bound the size of
// the library): such plans run on the tiled kernel, which takes any strides.
template <class F, class TO, class T1, class T2, class T3, int NIN, int INV_SPECIAL = -1, int BC0_SPECIAL = 0,
          bool LEAN = false>
vbt_b200_status launch_ew(const TiPlan& plan, const F& f, cudaStream_t stream) {
  if (plan.numel == 0) return VBT_B200_OK;
  auto note = [&](int kind, unsigned grid, int vec) {
    note_launch(VBT_B200_FAMILY_ELEMENTWISE, kind, dim3(grid), dim3(kEwThreads), vec, 1, 0, 1, plan.numel, 0, 0, stream);
  };
  constexpr int kMaxEs = static_cast<int>(std::max({sizeof(TO), sizeof(T1), NIN >= 2 ? sizeof(T2) : size_t{1},
                                                    NIN >= 3 ? sizeof(T3) : size_t{1}}));
  constexpr int V = 16 / kMaxEs > 8 ? 8 : 16 / kMaxEs;  // 1-byte types: 8 lanes keep the register count sane
  bool flat_vec = false;
  const TiKernel kind = choose_ti_kernel(plan, V, &flat_vec);
  if (kind == kTiFlat) {
    FlatParams<NIN + 1> fp{};
    for (int k = 0; k <= NIN; ++k) {
      fp.ptr[k] = plan.ptr[k];
      fp.s[k] = static_cast<int>(plan.stride[k][0]);
    }
    fp.n = plan.numel;
    if (flat_vec) {
      const int64_t nvec = plan.numel / V;
      const int64_t blocks = std::max<int64_t>(1, (nvec + kEwThreads * kEwUnroll - 1) / (kEwThreads * kEwUnroll));
      VB_ARG(blocks <= 0x7fffffff, "elementwise: tensor too large for one launch");
      ew_flat_kernel<F, TO, T1, T2, T3, NIN, V><<<static_cast<unsigned>(blocks), kEwThreads, 0, stream>>>(fp, f);
      note(0, static_cast<unsigned>(blocks), V);
    } else {
      const int64_t blocks = (plan.numel + kEwThreads * kEwUnroll - 1) / (kEwThreads * kEwUnroll);
      VB_ARG(blocks <= 0x7fffffff, "elementwise: tensor too large for one launch");
      ew_flat_kernel<F, TO, T1, T2, T3, NIN, 1><<<static_cast<unsigned>(blocks), kEwThreads, 0, stream>>>(fp, f);
      note(0, static_cast<unsigned>(blocks), 1);
    }
    VB_LAUNCH_CHECK();
    return VBT_B200_OK;
  }

  if constexpr (!LEAN) {
    int dimj = -1;
    const int tmask = transpose_candidates(plan, &dimj);
    if (tmask != 0) {
      TiPlan tpl = plan;  // make the partner dim dim 1
      if (dimj != 1) {
        std::swap(tpl.shape[1], tpl.shape[dimj]);
        for (int k = 0; k <= NIN; ++k) std::swap(tpl.stride[k][1], tpl.stride[k][dimj]);
      }
      TiledParams<NIN + 1> tp{};
      const int nd = tpl.ndim;
      int64_t outer = 1;
      for (int k = 0; k <= NIN; ++k) {
        tp.ptr[k] = tpl.ptr[k];
        tp.s0[k] = tpl.stride[k][0];
        tp.s1[k] = tpl.stride[k][1];
        for (int d = 2; d < nd; ++d) tp.so[k][d - 2] = tpl.stride[k][d];
      }
      tp.n_outer = nd - 2;
      for (int d = 2; d < nd; ++d) {
        VB_ARG(tpl.shape[d] <= 0x7fffffff, "elementwise: dim too large");
        tp.odiv[d - 2] = FastDiv(static_cast<uint32_t>(tpl.shape[d]));
        outer *= tpl.shape[d];
      }
      // element pairs: every staged input and the output must keep pairs aligned
      auto group_ok = [&](int k, bool along1, int g) {
        const int es = tpl.esize[k];
        if (es > 4) return false;
        if (reinterpret_cast<uintptr_t>(tpl.ptr[k]) % (g * es)) return false;
        for (int d = 0; d < nd; ++d) {
          const bool unit = along1 ? d == 1 : d == 0;
          if (unit ? tpl.stride[k][d] != 1 : (tpl.stride[k][d] % g != 0)) return false;
        }
        return true;
      };
      auto pair_ok = [&](int k, bool along1) { return group_ok(k, along1, 2); };
      bool pairs = sizeof(TO) <= 4 && sizeof(T1) <= 4 && (NIN < 2 || sizeof(T2) <= 4) && (NIN < 3 || sizeof(T3) <= 4) &&
                   tpl.shape[0] % 2 == 0 && tpl.shape[1] % 2 == 0 && pair_ok(0, false);
      bool quads = (sizeof(TO) == 2 || sizeof(TO) == 4) && tpl.shape[0] % 4 == 0 && tpl.shape[1] % 4 == 0 && group_ok(0, false, 4);
      int staged = 0, use_mask = 0;
      for (int k = 1; k <= NIN; ++k)
        if ((tmask >> (k - 1)) & 1) {
          if (staged == kTrMaxStaged) continue;  // a third transposed input is read directly
          ++staged;
          use_mask |= 1 << (k - 1);
          pairs = pairs && pair_ok(k, true);
          quads = quads && tpl.esize[k] <= 4 && group_ok(k, true, 4);
        }
      if constexpr (sizeof(TO) == 2 || sizeof(TO) == 4) {
        constexpr int kTilesPerBlock = kTr4TilesPerBlock<NIN>;
        const int64_t q0 = (tpl.shape[0] + 63) / 64, q1 = ((tpl.shape[1] + 63) / 64 + kTilesPerBlock - 1) / kTilesPerBlock;
        if (quads && q0 * q1 * outer <= 0x7fffffff && tpl.shape[0] <= 0x7fffffff) {
          tp.div_t0 = FastDiv(static_cast<uint32_t>(q0));
          tp.div_t1 = FastDiv(static_cast<uint32_t>(q1));
          tp.n0v = static_cast<uint32_t>(tpl.shape[0]);
          tp.size1 = tpl.shape[1];
          // one input that lies like the output may use the staging slot the transposed ones leave free
          int lies = 0;
          if (staged < kTrMaxStaged)
            for (int k = 1; k <= NIN && !lies; ++k)
              if (!((use_mask >> (k - 1)) & 1) && tpl.esize[k] <= 4 && group_ok(k, false, 4)) lies = 16 << (k - 1);
          if constexpr (NIN >= 2) {
            if (lies) {
              ew_transpose4_kernel<F, TO, T1, T2, T3, NIN, true><<<static_cast<unsigned>(q0 * q1 * outer), kEwThreads, 0, stream>>>(tp, f, use_mask | lies);
              VB_LAUNCH_CHECK();
              note(3, static_cast<unsigned>(q0 * q1 * outer), 4);
              return VBT_B200_OK;
            }
          }
          ew_transpose4_kernel<F, TO, T1, T2, T3, NIN><<<static_cast<unsigned>(q0 * q1 * outer), kEwThreads, 0, stream>>>(tp, f, use_mask);
          VB_LAUNCH_CHECK();
          note(3, static_cast<unsigned>(q0 * q1 * outer), 4);
          return VBT_B200_OK;
        }
      }
      const int tile = pairs ? 64 : 32;
      const int64_t tiles0 = (tpl.shape[0] + tile - 1) / tile;
      const int64_t tiles1 = (tpl.shape[1] + tile - 1) / tile;
      const int64_t blocks = tiles0 * tiles1 * outer;
      if (blocks <= 0x7fffffff && tpl.shape[0] <= 0x7fffffff) {
        constexpr bool kPairTypes = sizeof(TO) <= 4 && sizeof(T1) <= 4 && (NIN < 2 || sizeof(T2) <= 4) &&
                                    (NIN < 3 || sizeof(T3) <= 4);
        if constexpr (kPairTypes) if (pairs) {
          tp.div_t0 = FastDiv(static_cast<uint32_t>(tiles0));
          tp.div_t1 = FastDiv(static_cast<uint32_t>(tiles1));
          tp.n0v = static_cast<uint32_t>(tpl.shape[0]);
          tp.size1 = tpl.shape[1];
          ew_transpose_kernel<F, TO, T1, T2, T3, NIN, 2><<<static_cast<unsigned>(blocks), kEwThreads, 0, stream>>>(tp, f, use_mask);
          VB_LAUNCH_CHECK();
          note(3, static_cast<unsigned>(blocks), 2);
          return VBT_B200_OK;
        }
        tp.div_t0 = FastDiv(static_cast<uint32_t>(tiles0));
        tp.div_t1 = FastDiv(static_cast<uint32_t>(tiles1));
        tp.n0v = static_cast<uint32_t>(tpl.shape[0]);
        tp.size1 = tpl.shape[1];
        ew_transpose_kernel<F, TO, T1, T2, T3, NIN, 1><<<static_cast<unsigned>(blocks), kEwThreads, 0, stream>>>(tp, f, use_mask);
        VB_LAUNCH_CHECK();
        note(3, static_cast<unsigned>(blocks), 1);
        return VBT_B200_OK;
      }
    }
  }
  const bool vec = kind == kTiTiledVec;
  const int v = vec ? V : 1;
  TiledParams<NIN + 1> tp{};
  const int nd = plan.ndim;
  const int64_t size0 = plan.shape[0];
  const int64_t size1 = nd >= 2 ? plan.shape[1] : 1;
  const int64_t n0v = size0 / v;
  VB_ARG(n0v <= 0x7fffffff && size1 <= (int64_t{1} << 40), "elementwise: dim too large");
  for (int k = 0; k <= NIN; ++k) {
    tp.ptr[k] = plan.ptr[k];
    tp.s0[k] = plan.stride[k][0];
    tp.s1[k] = nd >= 2 ? plan.stride[k][1] : 0;
    for (int d = 2; d < nd; ++d) tp.so[k][d - 2] = plan.stride[k][d];
  }
  tp.n_outer = std::max(0, nd - 2);
  int64_t outer = 1;
  for (int d = 2; d < nd; ++d) {
    VB_ARG(plan.shape[d] <= 0x7fffffff, "elementwise: dim too large");
    tp.odiv[d - 2] = FastDiv(static_cast<uint32_t>(plan.shape[d]));
    outer *= plan.shape[d];
  }
  int log2_w0 = 0;
  while ((int64_t{1} << log2_w0) < n0v && (1 << log2_w0) < kEwThreads) ++log2_w0;
  const int w0 = 1 << log2_w0;
  const int R = kEwThreads / w0;
  const int64_t tiles0 = (n0v + w0 - 1) / w0;
  // rows per block: long enough to amortise the per-block offset decode and to reuse
  // hoisted operands, short enough to leave >= ~16 blocks per SM when the tensor allows
  // rows per thread.  Long walks (32) pay when an operand that has to be GATHERED along dim 0
  // is constant along dim 1: it is fetched once and reused for every row.
  const int want_rows = 32;
  int L = static_cast<int>(std::min<int64_t>(want_rows, (size1 + R - 1) / R));
  const int sms = current_sm_count();
  while (L > 4 && tiles0 * ((size1 + int64_t{R} * L - 1) / (int64_t{R} * L)) * outer < int64_t{sms} * 16) L /= 2;
  L = std::max(L, 1);
  const int64_t tiles1 = (size1 + int64_t{R} * L - 1) / (int64_t{R} * L);
  const int64_t blocks = tiles0 * tiles1 * outer;
  VB_ARG(blocks <= 0x7fffffff && tiles0 <= 0x7fffffff && tiles1 <= 0x7fffffff,
         "elementwise: tensor too large for one launch");
  tp.div_t0 = FastDiv(static_cast<uint32_t>(tiles0));
  tp.div_t1 = FastDiv(static_cast<uint32_t>(tiles1));
  tp.n0v = static_cast<uint32_t>(n0v);
  tp.size1 = size1;
  tp.log2_w0 = log2_w0;
  tp.L = L;
  const unsigned g = static_cast<unsigned>(blocks);
  note(vec ? 1 : 2, g, v);
  if (vec) {
    if constexpr (INV_SPECIAL >= 0) {
      int mask = 0;
      for (int k = 1; k <= NIN; ++k)
        if (tp.s1[k] == 0) mask |= 1 << (k - 1);
      if (mask == INV_SPECIAL) {
        if constexpr (BC0_SPECIAL != 0) {
          int bc = 0;
          for (int k = 1; k <= NIN; ++k)
            if (tp.s0[k] == 0) bc |= 1 << (k - 1);
          if (bc == BC0_SPECIAL) {
            ew_tiled_kernel<F, TO, T1, T2, T3, NIN, V, INV_SPECIAL, BC0_SPECIAL><<<g, kEwThreads, 0, stream>>>(tp, f);
            VB_LAUNCH_CHECK();
            return VBT_B200_OK;
          }
        }
        ew_tiled_kernel<F, TO, T1, T2, T3, NIN, V, INV_SPECIAL><<<g, kEwThreads, 0, stream>>>(tp, f);
        VB_LAUNCH_CHECK();
        return VBT_B200_OK;
      }
    }
    ew_tiled_kernel<F, TO, T1, T2, T3, NIN, V, -1><<<g, kEwThreads, 0, stream>>>(tp, f);
  } else {
    ew_tiled_kernel<F, TO, T1, T2, T3, NIN, 1, -1><<<g, kEwThreads, 0, stream>>>(tp, f);
  }
  VB_LAUNCH_CHECK();
  return VBT_B200_OK;
}

}  // namespace vb
