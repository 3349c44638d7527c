// Row-wise softmax / log_softmax / RMSNorm (sm_100a).
//
// Plain CUDA replacements for the Triton kernels the reference compiles at run time
// (vibe_kernels/softmax/vbt_native.py:39-97, vibe_kernels/rmsnorm/vbt_native.py:55-103).
// Those read each row from global memory three (softmax) or two (RMSNorm) times; here a
// row is read ONCE into registers with 16-byte loads, reduced with warp shuffles (plus one
// shared-memory hop when a whole block shares a row) and written once.
//
//   group kernel   rows up to 128 vectors: G = 8/16/32 lanes own a row, several rows per
//                  warp in flight; persistent over rows so RMSNorm's gamma stays in
//                  registers.
//   block kernel   rows up to 2048 vectors: 128 or 256 threads own a row.
//   stream kernel  anything longer or not 16-byte aligned: block per row, two passes
//                  (online max/sum, then write); the second pass is served by L2.
//
// Math is FP32 whatever the storage type.
//   softmax:  m = max x;  e = exp(x - m) = 2^((x - m) * log2 e);  s = max(sum e, 1e-20);  y = e / s
//             (the reference evaluates exp(x - (log s + m)), the same value; log_softmax is
//              x - m - log s)
//   rmsnorm:  r = rsqrt(sum x^2 / n + eps);  y = x * r * gamma
#include <cfloat>

#include "common.cuh"

namespace vb {
namespace {

enum { K_SOFTMAX = 0, K_LOG_SOFTMAX = 1, K_RMSNORM = 2 };

struct RowParams {
  const void* x;
  void* out;
  const float* gamma;
  float* inv_rms;
  int64_t rows;
  int64_t cols;
  int64_t x_row_stride;  // elements
  float eps;
  int gamma_smem;  // block kernel: gamma staged in dynamic shared memory (cols floats)
};

// 2^x on the special-function unit.  exp(d) is taken as 2^(d * log2 e), the form Triton's tl.exp
// lowers to in the reference's softmax kernel (2 ulp, far inside every tolerance of this path);
// the multiply is done on float pairs by the caller.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int G>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int d = G / 2; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int d = G / 2; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// per-thread slice of a row held in registers: VPL vectors of V elements
template <class T, int VPL>
struct RowRegs {
  static constexpr int V = 16 / sizeof(T);
  float v[VPL][V];
};

// the three row computations on a register-resident slice; reduce_max / reduce_sum fold a
// scalar across the threads that share the row
template <class T, int KIND, int VPL, class RMax, class RSum>
__device__ __forceinline__ void row_math(float (&v)[VPL][16 / sizeof(T)], const bool (&valid)[VPL],
                                         const float (&g)[VPL][16 / sizeof(T)], const RowParams& p,
                                         RMax reduce_max, RSum reduce_sum, float* inv_out) {
  constexpr int V = 16 / sizeof(T);
  // Arithmetic on float pairs with the packed fp32 instructions of sm_100 (__fmul2_rn,
  // __fadd2_rn, __ffma2_rn): one issue slot per two lanes; these kernels keep the issue slots
  // about half busy, so instruction count matters next to bytes.
  if constexpr (KIND == K_RMSNORM) {
    float2 ss2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (valid[k])
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const float2 x2 = make_float2(v[k][j], v[k][j + 1]);
          ss2 = __ffma2_rn(x2, x2, ss2);
        }
    const float ss = reduce_sum(ss2.x + ss2.y);
    const float inv = rsqrtf(ss / static_cast<float>(p.cols) + p.eps);
    *inv_out = inv;
    const float2 inv2 = make_float2(inv, inv);
#pragma unroll
    for (int k = 0; k < VPL; ++k)
#pragma unroll
      for (int j = 0; j < V; j += 2) {
        const float2 r2 = __fmul2_rn(__fmul2_rn(make_float2(v[k][j], v[k][j + 1]), inv2),
                                     make_float2(g[k][j], g[k][j + 1]));
        v[k][j] = r2.x;
        v[k][j + 1] = r2.y;
      }
  } else {
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (valid[k])
#pragma unroll
        for (int j = 0; j < V; ++j) m = fmaxf(m, v[k][j]);
    m = reduce_max(m);
    float2 s2 = make_float2(0.f, 0.f);
    const float2 nm2 = make_float2(-m, -m);
#pragma unroll
    for (int k = 0; k < VPL; ++k)
      if (valid[k])
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const float2 d2 = __fadd2_rn(make_float2(v[k][j], v[k][j + 1]), nm2);
          const float2 t2 = __fmul2_rn(d2, make_float2(1.4426950408889634f, 1.4426950408889634f));
          const float2 e2 = make_float2(ex2_approx(t2.x), ex2_approx(t2.y));
          s2 = __fadd2_rn(s2, e2);
          v[k][j] = KIND == K_SOFTMAX ? e2.x : d2.x;
          v[k][j + 1] = KIND == K_SOFTMAX ? e2.y : d2.y;
        }
    float s = reduce_sum(s2.x + s2.y);
    s = fmaxf(s, 1e-20f);
    if constexpr (KIND == K_SOFTMAX) {
      const float r = 1.0f / s;
      const float2 r2 = make_float2(r, r);
#pragma unroll
      for (int k = 0; k < VPL; ++k)
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const float2 y2 = __fmul2_rn(make_float2(v[k][j], v[k][j + 1]), r2);
          v[k][j] = y2.x;
          v[k][j + 1] = y2.y;
        }
    } else {
      const float ls = logf(s);
      const float2 nls2 = make_float2(-ls, -ls);
#pragma unroll
      for (int k = 0; k < VPL; ++k)
#pragma unroll
        for (int j = 0; j < V; j += 2) {
          const float2 y2 = __fadd2_rn(make_float2(v[k][j], v[k][j + 1]), nls2);
          v[k][j] = y2.x;
          v[k][j + 1] = y2.y;
        }
    }
  }
}

template <class T, int VPL>
__device__ __forceinline__ void load_row(const T* xr, int first_vec, int vec_step, int nvec,
                                         float (&v)[VPL][16 / sizeof(T)], bool (&valid)[VPL]) {
  constexpr int V = 16 / sizeof(T);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int j = first_vec + k * vec_step;
    valid[k] = j < nvec;
    if (valid[k]) {
      const Vec<T, V> raw = *reinterpret_cast<const Vec<T, V>*>(xr + static_cast<int64_t>(j) * V);
#pragma unroll
      for (int e = 0; e < V; ++e) v[k][e] = to_f(raw.v[e]);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) v[k][e] = 0.f;
    }
  }
}
template <class T, int VPL>
__device__ __forceinline__ void store_row(T* orow, int first_vec, int vec_step,
                                          const float (&v)[VPL][16 / sizeof(T)], const bool (&valid)[VPL]) {
  constexpr int V = 16 / sizeof(T);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    if (!valid[k]) continue;
    Vec<T, V> raw;
#pragma unroll
    for (int e = 0; e < V; ++e) raw.v[e] = from_f<T>(v[k][e]);
    *reinterpret_cast<Vec<T, V>*>(orow + static_cast<int64_t>(first_vec + k * vec_step) * V) = raw;
  }
}
template <class T, int VPL>
__device__ __forceinline__ void load_gamma(const float* gamma, int first_vec, int vec_step, int nvec,
                                           float (&g)[VPL][16 / sizeof(T)]) {
  constexpr int V = 16 / sizeof(T);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int j = first_vec + k * vec_step;
#pragma unroll
    for (int e = 0; e < V; ++e) g[k][e] = (gamma && j < nvec) ? gamma[static_cast<int64_t>(j) * V + e] : 1.0f;
  }
}

// G lanes per row; a warp keeps RPG rows per group in flight (RPG * 32 / G rows per warp
// iteration) so that short rows still put enough bytes on the wire; persistent over rows
template <class T, int KIND, int G, int VPL, int RPG>
__global__ void __launch_bounds__(256) rowop_group_kernel(const __grid_constant__ RowParams p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int kGroupsPerWarp = 32 / G;
  constexpr int kRowsPerWarp = kGroupsPerWarp * RPG;
  constexpr int kRowsPerBlock = 8 * kRowsPerWarp;
  const int lane = threadIdx.x % G;
  const int gw = (threadIdx.x % 32) / G;  // group within the warp
  const int nvec = static_cast<int>(p.cols / V);
  float g[VPL][V];
  load_gamma<T, VPL>(KIND == K_RMSNORM ? p.gamma : nullptr, lane, G, nvec, g);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRowsPerBlock;
  // every lane of a warp runs the same number of iterations (shuffles are warp-wide)
  const int64_t base_row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + (threadIdx.x / 32) * kRowsPerWarp;
  for (int64_t r0 = base_row; r0 < p.rows; r0 += stride) {
    float v[RPG][VPL][V];
    bool valid[RPG][VPL];
    bool live[RPG];
#pragma unroll
    for (int r = 0; r < RPG; ++r) {
      const int64_t row = r0 + r * kGroupsPerWarp + gw;
      live[r] = row < p.rows;
      const T* xr = static_cast<const T*>(p.x) + (live[r] ? row : 0) * p.x_row_stride;
      load_row<T, VPL>(xr, lane, G, live[r] ? nvec : 0, v[r], valid[r]);
    }
#pragma unroll
    for (int r = 0; r < RPG; ++r) {
      const int64_t row = r0 + r * kGroupsPerWarp + gw;
      float inv = 0.f;
      row_math<T, KIND, VPL>(v[r], valid[r], g, p, [](float a) { return group_max<G>(a); },
                             [](float a) { return group_sum<G>(a); }, &inv);
      if (live[r]) {
        store_row<T, VPL>(static_cast<T*>(p.out) + row * p.cols, lane, G, v[r], valid[r]);
        if (KIND == K_RMSNORM && p.inv_rms && lane == 0) p.inv_rms[row] = inv;
      }
    }
  }
}

// THREADS threads per row, persistent over rows.  gamma is staged once per block in shared
// memory (pinned in registers, 32 values per thread would halve the occupancy; re-read from
// L1/L2 per row it puts a global-load latency into every row's epilogue).
template <class T, int KIND, int THREADS, int VPL>
__global__ void __launch_bounds__(THREADS) rowop_block_kernel(const __grid_constant__ RowParams p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int kWarps = THREADS / 32;
  __shared__ float red[2][kWarps];
  extern __shared__ __align__(16) float gamma_s[];
  const int t = threadIdx.x;
  const int nvec = static_cast<int>(p.cols / V);
  if (KIND == K_RMSNORM && p.gamma_smem) {
    for (int64_t j = t; j < p.cols; j += THREADS) gamma_s[j] = p.gamma[j];
    __syncthreads();
  }
  float ones[VPL][V];
#pragma unroll
  for (int k = 0; k < VPL; ++k)
#pragma unroll
    for (int e = 0; e < V; ++e) ones[k][e] = 1.0f;
  int phase = 0;
  auto block_fold = [&](float a, bool is_max) {
    a = is_max ? group_max<32>(a) : group_sum<32>(a);
    if ((t & 31) == 0) red[phase][t >> 5] = a;
    __syncthreads();
    float r = red[phase][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) r = is_max ? fmaxf(r, red[phase][w]) : r + red[phase][w];
    phase ^= 1;
    return r;
  };
  // 32-bit rows: the block's next row is fetched (raw, 16 bytes per vector) before the current one
  // is worked on, so its loads are in flight through the row's barriers and stores ([32768,4096]
  // fp32: softmax 0.946 -> 0.955, RMSNorm 0.914 -> 0.956 of the measured bandwidth).  16-bit rows
  // hold twice the floats per vector; with the extra registers they fell from 0.98 to 0.76.
  constexpr bool kAhead = sizeof(T) == 4;
  Vec<T, V> ahead[kAhead ? VPL : 1];
  auto fetch = [&](int64_t row) {
    const T* xr = static_cast<const T*>(p.x) + row * p.x_row_stride;
#pragma unroll
    for (int k = 0; k < (kAhead ? VPL : 0); ++k) {
      const int j = t + k * THREADS;
      if (j < nvec) ahead[k] = *reinterpret_cast<const Vec<T, V>*>(xr + static_cast<int64_t>(j) * V);
    }
  };
  if (kAhead && static_cast<int64_t>(blockIdx.x) < p.rows) fetch(blockIdx.x);
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float v[VPL][V];
    bool valid[VPL];
    if constexpr (kAhead) {
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        valid[k] = t + k * THREADS < nvec;
#pragma unroll
        for (int e = 0; e < V; ++e) v[k][e] = valid[k] ? to_f(ahead[k].v[e]) : 0.f;
      }
      if (row + gridDim.x < p.rows) fetch(row + gridDim.x);
    } else {
      load_row<T, VPL>(static_cast<const T*>(p.x) + row * p.x_row_stride, t, THREADS, nvec, v, valid);
    }
    float inv = 0.f;
    row_math<T, KIND, VPL>(v, valid, ones, p, [&](float a) { return block_fold(a, true); },
                           [&](float a) { return block_fold(a, false); }, &inv);
    if constexpr (KIND == K_RMSNORM) {
      if (p.gamma) {
        const float* gsrc = p.gamma_smem ? gamma_s : p.gamma;
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
          if (!valid[k]) continue;
          const float4* gp = reinterpret_cast<const float4*>(gsrc + static_cast<int64_t>(t + k * THREADS) * V);
#pragma unroll
          for (int q = 0; q < V / 4; ++q) {
            const float4 gq = gp[q];
            if constexpr (V == 4) {  // packed multiply; with eight lanes it costs registers, hence blocks per SM
              const float2 lo = __fmul2_rn(make_float2(v[k][0], v[k][1]), make_float2(gq.x, gq.y));
              const float2 hi = __fmul2_rn(make_float2(v[k][2], v[k][3]), make_float2(gq.z, gq.w));
              v[k][0] = lo.x; v[k][1] = lo.y; v[k][2] = hi.x; v[k][3] = hi.y;
            } else {
              v[k][4 * q + 0] *= gq.x; v[k][4 * q + 1] *= gq.y;
              v[k][4 * q + 2] *= gq.z; v[k][4 * q + 3] *= gq.w;
            }
          }
        }
      }
    }
    store_row<T, VPL>(static_cast<T*>(p.out) + row * p.cols, t, THREADS, v, valid);
    if (KIND == K_RMSNORM && p.inv_rms && t == 0) p.inv_rms[row] = inv;
  }
}

// any length / alignment: block per row, scalar loads, two passes
template <class T, int KIND>
__global__ void __launch_bounds__(256) rowop_stream_kernel(const __grid_constant__ RowParams p) {
  __shared__ float red[2][8];
  __shared__ float red2[2][8];
  const int t = threadIdx.x;
  int phase = 0;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* xr = static_cast<const T*>(p.x) + row * p.x_row_stride;
    T* orow = static_cast<T*>(p.out) + row * p.cols;
    // pass 1: online (max, sum) or sum of squares
    float m = -INFINITY, s = 0.f;
    for (int64_t j = t; j < p.cols; j += 256) {
      const float x = to_f(xr[j]);
      if constexpr (KIND == K_RMSNORM) {
        s = fmaf(x, x, s);
      } else {
        const float nm = fmaxf(m, x);
        s = s * (m == nm ? 1.f : expf(m - nm)) + (x == -INFINITY ? 0.f : expf(x - nm));
        m = nm;
      }
    }
    // fold (m, s) pairs across the block
    float wm = group_max<32>(m);
    if constexpr (KIND != K_RMSNORM) s = (m == -INFINITY && wm == -INFINITY) ? s : s * expf(m - wm);
    float ws = group_sum<32>(s);
    if ((t & 31) == 0) { red[phase][t >> 5] = wm; red2[phase][t >> 5] = ws; }
    __syncthreads();
    float bm = red[phase][0];
#pragma unroll
    for (int w = 1; w < 8; ++w) bm = fmaxf(bm, red[phase][w]);
    float bs = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if constexpr (KIND == K_RMSNORM) bs += red2[phase][w];
      else bs += (red[phase][w] == -INFINITY && bm == -INFINITY) ? red2[phase][w]
                                                                 : red2[phase][w] * expf(red[phase][w] - bm);
    }
    phase ^= 1;
    if constexpr (KIND == K_RMSNORM) {
      const float inv = rsqrtf(bs / static_cast<float>(p.cols) + p.eps);
      if (p.inv_rms && t == 0) p.inv_rms[row] = inv;
      for (int64_t j = t; j < p.cols; j += 256)
        orow[j] = from_f<T>(to_f(xr[j]) * inv * (p.gamma ? p.gamma[j] : 1.0f));
    } else {
      bs = fmaxf(bs, 1e-20f);
      const float r = 1.0f / bs, ls = logf(bs);
      for (int64_t j = t; j < p.cols; j += 256) {
        const float d = to_f(xr[j]) - bm;
        orow[j] = from_f<T>(KIND == K_SOFTMAX ? expf(d) * r : d - ls);
      }
    }
  }
}

template <class T, int KIND>
vbt_b200_status launch_rowop(const RowParams& p, cudaStream_t s, int device) {
  constexpr int V = 16 / sizeof(T);
  const int sms = sm_count(device);
  const bool aligned = p.cols % V == 0 && (p.x_row_stride * sizeof(T)) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(p.x) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(p.out) % 16 == 0 &&
                       (KIND != K_RMSNORM || p.gamma == nullptr || reinterpret_cast<uintptr_t>(p.gamma) % 16 == 0);
  const int64_t nvec = aligned ? p.cols / V : (int64_t{1} << 40);
  auto grid = [&](int64_t units, int per_sm) {
    return static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(units, int64_t{sms} * per_sm)));
  };
#define VB_GROUP(G, VPL, RPG)                                                                 \
  rowop_group_kernel<T, KIND, G, VPL, RPG>                                                    \
      <<<grid((p.rows + (256 / G) * RPG - 1) / ((256 / G) * RPG), 8), 256, 0, s>>>(p)
#define VB_BLOCK(TH, VPL, PER_SM) rowop_block_kernel<T, KIND, TH, VPL><<<grid(p.rows, PER_SM), TH, gsmem, s>>>(pp)
  // rmsnorm's gamma goes to shared memory in the block kernels when it fits the default 48 KB
  RowParams pp = p;
  size_t gsmem = 0;
  if (KIND == K_RMSNORM && p.gamma != nullptr && p.cols * 4 <= 40 * 1024) {
    pp.gamma_smem = 1;
    gsmem = static_cast<size_t>(p.cols) * 4;
  }
  // short rows: a few lanes per row with several vectors each keep the shuffle trees short;
  // the register budget (vectors per lane x rows in flight) is set per element width
  if constexpr (V == 4) {
    if (nvec <= 8) VB_GROUP(2, 4, 2);
    else if (nvec <= 16) VB_GROUP(4, 4, 2);
    else if (nvec <= 32) VB_GROUP(8, 4, 2);
    else if (nvec <= 64) VB_GROUP(16, 4, 2);
    else if (nvec <= 128) VB_GROUP(32, 4, 1);
  } else {
    if (nvec <= 8) VB_GROUP(4, 2, 2);
    else if (nvec <= 16) VB_GROUP(8, 2, 2);
    else if (nvec <= 32) VB_GROUP(16, 2, 2);
    else if (nvec <= 64) VB_GROUP(32, 2, 2);
    else if (nvec <= 128) VB_GROUP(32, 4, 1);
  }
  if (nvec <= 128) {
  } else if (nvec <= 256) VB_BLOCK(128, 2, 16);
  else if (nvec <= 512) VB_BLOCK(128, 4, 16);
  else if (nvec <= 1024) VB_BLOCK(256, 4, 8);
  else if (nvec <= 2048) VB_BLOCK(256, 8, 8);
  else rowop_stream_kernel<T, KIND><<<grid(p.rows, 8), 256, 0, s>>>(p);
#undef VB_GROUP
#undef VB_BLOCK
  VB_LAUNCH_CHECK();
  return VBT_B200_OK;
}

template <int KIND>
vbt_b200_status dispatch_rowop(int dtype, const RowParams& p, cudaStream_t s, int device, const char* name) {
  switch (dtype) {
    case VBT_B200_F32: return launch_rowop<float, KIND>(p, s, device);
    case VBT_B200_F16: return launch_rowop<__half, KIND>(p, s, device);
    case VBT_B200_BF16: return launch_rowop<__nv_bfloat16, KIND>(p, s, device);
  }
  return fail(VBT_B200_INVALID_ARGUMENT, std::string(name) + ": expected a floating dtype");
}

template <class T>
__global__ void scale_cast_kernel(T* out, const float* in, int64_t n, float scale) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f<T>(in[i] * scale);
}

}  // namespace
}  // namespace vb

extern "C" {

vbt_b200_status vbt_b200_softmax(void* out, const void* x, int32_t dtype, int64_t rows, int64_t cols,
                                 int64_t x_row_stride, int32_t log_softmax, void* stream) {
  using namespace vb;
  const char* name = log_softmax ? "log_softmax" : "softmax";
  VB_ARG(rows >= 0 && cols >= 0, std::string(name) + ": negative size");
  if (rows == 0 || cols == 0) return VBT_B200_OK;  // empty output, as the reference
  VB_ARG(out && x, std::string(name) + ": null pointer");
  VB_ARG(x_row_stride >= 0, std::string(name) + ": negative row stride");
  DeviceScope scope(out);
  RowParams p{};
  p.x = x; p.out = out; p.rows = rows; p.cols = cols; p.x_row_stride = x_row_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return log_softmax ? dispatch_rowop<K_LOG_SOFTMAX>(dtype, p, s, scope.device(), name)
                     : dispatch_rowop<K_SOFTMAX>(dtype, p, s, scope.device(), name);
}

vbt_b200_status vbt_b200_rmsnorm(void* out, float* inv_rms, const void* x, const float* gamma, int32_t dtype,
                                 int64_t rows, int64_t cols, int64_t x_row_stride, float eps, void* stream) {
  using namespace vb;
  const char* name = "rmsnorm";
  VB_ARG(rows >= 0 && cols >= 0, std::string(name) + ": negative size");
  if (rows == 0 || cols == 0) return VBT_B200_OK;
  VB_ARG(out && x, std::string(name) + ": null pointer");
  VB_ARG(x_row_stride >= 0, std::string(name) + ": negative row stride");
  DeviceScope scope(out);
  RowParams p{};
  p.x = x; p.out = out; p.gamma = gamma; p.inv_rms = inv_rms;
  p.rows = rows; p.cols = cols; p.x_row_stride = x_row_stride; p.eps = eps;
  return dispatch_rowop<K_RMSNORM>(dtype, p, static_cast<cudaStream_t>(stream), scope.device(), name);
}

vbt_b200_status vbt_b200_scale_cast(void* out, int32_t out_dtype, const float* partial, int64_t n, float scale,
                                    void* stream) {
  using namespace vb;
  VB_ARG(n >= 0, "scale_cast: negative size");
  if (n == 0) return VBT_B200_OK;
  VB_ARG(out && partial, "scale_cast: null pointer");
  DeviceScope scope(out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned g = static_cast<unsigned>((n + 255) / 256);
  switch (out_dtype) {
    case VBT_B200_F32: scale_cast_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(out), partial, n, scale); break;
    case VBT_B200_F16: scale_cast_kernel<__half><<<g, 256, 0, s>>>(static_cast<__half*>(out), partial, n, scale); break;
    case VBT_B200_BF16: scale_cast_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), partial, n, scale); break;
    default: return fail(VBT_B200_INVALID_ARGUMENT, "scale_cast: expected a floating dtype");
  }
  VB_LAUNCH_CHECK();
  return VBT_B200_OK;
}

}  // extern "C"
