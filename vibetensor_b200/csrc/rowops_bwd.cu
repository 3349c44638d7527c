// Backward of the row ops (sm_100a): softmax, log_softmax, RMSNorm.
//
//   softmax      dx = y * (dy - sum(dy * y))
//   log_softmax  dx = dy - exp(y) * sum(dy)                    (y holds log-probabilities)
//     (vibe_kernels/softmax/impl/cutedsl_softmax/softmax.py:405-423, :809-828)
//   rmsnorm      n = x * r;  dx = r * (dy*gamma - n * mean(dy*gamma*n));  dgamma = sum_rows dy*n
//     (Triton _rmsnorm_bwd_kernel, vibe_kernels/rmsnorm/vbt_native.py:110-176)
//
// The reference's RMSNorm kernel reads x and dy twice and adds every row's dy*n into dgamma
// with float atomics (order undefined).  Here both rows are read once into registers; each
// persistent block keeps its share of dgamma in registers over all the rows it walks, writes
// one partial row to the caller's workspace, and a second small kernel folds the partial rows
// in a fixed order: no atomics, results reproducible run to run.
//
// One kernel shape serves every row length up to 512 vectors per 256 threads: TPR threads per
// row (8 .. 256), VPL 16-byte vectors per thread, 256 / TPR rows per block iteration.
#include <cfloat>

#include "common.cuh"

namespace vb {
namespace {

enum { B_SOFTMAX = 0, B_LOG_SOFTMAX = 1, B_RMSNORM = 2 };
constexpr int kBwdThreads = 256;

struct BwdParams {
  const void* dy;
  const void* b;         // y (softmax kinds) or x (rmsnorm)
  void* dx;
  const float* gamma;    // rmsnorm, may be null
  const float* inv_rms;  // rmsnorm
  float* ws;             // rmsnorm with dgamma: [gridDim.x][cols] partial sums
  int64_t rows, cols;
  int64_t dy_row_stride, b_row_stride;  // elements
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
template <int G>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int d = G / 2; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// two adjacent storage values <-> float2; the RMSNorm path does its arithmetic on float pairs with
// the packed fp32 instructions of sm_100 (__fmul2_rn / __ffma2_rn: one issue slot per two lanes)
__device__ __forceinline__ float2 pair_f(const float* p) { return make_float2(p[0], p[1]); }
__device__ __forceinline__ float2 pair_f(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ float2 pair_f(const __half* p) {
  return __half22float2(*reinterpret_cast<const __half2*>(p));
}
__device__ __forceinline__ void store_pair(float* p, float2 v) { p[0] = v.x; p[1] = v.y; }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float2 v) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v);
}
__device__ __forceinline__ void store_pair(__half* p, float2 v) {
  *reinterpret_cast<__half2*>(p) = __float22half2_rn(v);
}

template <class T, int VPL>
__device__ __forceinline__ void load_raw(const T* row, int first, int step, int nvec,
                                         Vec<T, 16 / sizeof(T)> (&v)[VPL]) {
  constexpr int V = 16 / sizeof(T);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int j = first + k * step;
    if (j < nvec) {
      v[k] = *reinterpret_cast<const Vec<T, V>*>(row + static_cast<int64_t>(j) * V);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) v[k].v[e] = from_f<T>(0.f);
    }
  }
}

// TPR threads per row, VPL vectors per thread, RIF rows in flight per row slot.  Rows stay in
// registers in their storage type (16-bit rows cost half the registers of their float form,
// which pays for the second row in flight) and are widened where they are used.
template <class T, int KIND, int TPR, int VPL, int RIF>
__global__ void __launch_bounds__(kBwdThreads, VPL * (16 / sizeof(T)) <= 16 ? 2 : 1) rowop_bwd_kernel(const __grid_constant__ BwdParams p) {
  constexpr int V = 16 / sizeof(T);
  constexpr int R = kBwdThreads / TPR;           // row slots per block
  constexpr int kWarpsPerRow = TPR > 32 ? TPR / 32 : 1;
  constexpr bool kGammaRegs = VPL * V <= 16;     // else gamma is re-read per row (L1 / L2 hits)
  __shared__ float red[2][RIF][kBwdThreads / 32];
  const int t = threadIdx.x;
  const int rl = t / TPR;                        // row slot within the block
  const int tl = t % TPR;                        // position within the row
  const int nvec = static_cast<int>(p.cols / V);
  const bool want_dgamma = KIND == B_RMSNORM && p.ws != nullptr;

  constexpr bool kGammaInRegs = kGammaRegs;
  float g[kGammaInRegs ? VPL : 1][V];
  float gg[KIND == B_RMSNORM ? VPL : 1][V];
  if constexpr (KIND == B_RMSNORM) {
#pragma unroll
    for (int k = 0; k < VPL; ++k)
#pragma unroll
      for (int e = 0; e < V; ++e) gg[k][e] = 0.f;
    if constexpr (kGammaInRegs) {
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int j = tl + k * TPR;
#pragma unroll
        for (int e = 0; e < V; ++e) g[k][e] = (p.gamma && j < nvec) ? p.gamma[static_cast<int64_t>(j) * V + e] : 1.0f;
      }
    }
  }
  // gamma of the thread's k-th vector
  auto gamma_vec = [&](int k, float (&gk)[V]) {
    if constexpr (KIND != B_RMSNORM) {
#pragma unroll
      for (int e = 0; e < V; ++e) gk[e] = 1.0f;
    } else if constexpr (kGammaInRegs) {
#pragma unroll
      for (int e = 0; e < V; ++e) gk[e] = g[k][e];
    } else {
      const int j = tl + k * TPR;
#pragma unroll
      for (int e = 0; e < V; ++e) gk[e] = (p.gamma && j < nvec) ? __ldg(p.gamma + static_cast<int64_t>(j) * V + e) : 1.0f;
    }
  };
  int phase = 0;
  // sums s[0..RIF) over the threads of each row, one barrier for all RIF values
  auto row_sums = [&](float (&s)[RIF]) {
    if constexpr (TPR <= 32) {
#pragma unroll
      for (int i = 0; i < RIF; ++i) s[i] = lanes_sum<TPR>(s[i]);
    } else {
#pragma unroll
      for (int i = 0; i < RIF; ++i) {
        s[i] = warp_sum(s[i]);
        if ((t & 31) == 0) red[phase][i][t >> 5] = s[i];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < RIF; ++i) {
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerRow; ++w) r += red[phase][i][rl * kWarpsPerRow + w];
        s[i] = r;
      }
      phase ^= 1;
    }
  };

  // every thread of the block runs the same number of iterations (block-wide barriers inside)
  constexpr int kRowsPerIter = R * RIF;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * kRowsPerIter; r0 < p.rows;
       r0 += static_cast<int64_t>(gridDim.x) * kRowsPerIter) {
    Vec<T, V> a[RIF][VPL], b[RIF][VPL];
    bool live[RIF];
    float inv[RIF];
#pragma unroll
    for (int i = 0; i < RIF; ++i) {
      const int64_t row = r0 + i * R + rl;
      live[i] = row < p.rows;
      const int64_t rr = live[i] ? row : 0;
      load_raw<T, VPL>(static_cast<const T*>(p.dy) + rr * p.dy_row_stride, tl, TPR, live[i] ? nvec : 0, a[i]);
      load_raw<T, VPL>(static_cast<const T*>(p.b) + rr * p.b_row_stride, tl, TPR, live[i] ? nvec : 0, b[i]);
      inv[i] = (KIND == B_RMSNORM && live[i]) ? p.inv_rms[row] : 0.f;
    }
    float s[RIF];
#pragma unroll
    for (int i = 0; i < RIF; ++i) s[i] = 0.f;
    if constexpr (KIND == B_RMSNORM) {
      float2 s2[RIF];
#pragma unroll
      for (int i = 0; i < RIF; ++i) s2[i] = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        float gk[V];
        gamma_vec(k, gk);
#pragma unroll
        for (int e = 0; e < V; e += 2) {
          const float2 g2 = make_float2(gk[e], gk[e + 1]);
          float2 gacc = make_float2(gg[k][e], gg[k][e + 1]);
#pragma unroll
          for (int i = 0; i < RIF; ++i) {
            // dy * x once; 1/rms enters dgamma through the fma and the row sum after the loop
            const float2 dyx = __fmul2_rn(pair_f(&a[i][k].v[e]), pair_f(&b[i][k].v[e]));
            gacc = __ffma2_rn(dyx, make_float2(inv[i], inv[i]), gacc);
            s2[i] = __ffma2_rn(dyx, g2, s2[i]);
          }
          gg[k][e] = gacc.x;
          gg[k][e + 1] = gacc.y;
        }
      }
#pragma unroll
      for (int i = 0; i < RIF; ++i) s[i] = s2[i].x + s2[i].y;
    } else {
#pragma unroll
      for (int k = 0; k < VPL; ++k)
#pragma unroll
        for (int i = 0; i < RIF; ++i)
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const float av = to_f(a[i][k].v[e]), bv = to_f(b[i][k].v[e]);
            if constexpr (KIND == B_SOFTMAX) s[i] = fmaf(av, bv, s[i]);
            else s[i] += av;
          }
    }
    row_sums(s);
#pragma unroll
    for (int i = 0; i < RIF; ++i) {
      if (!live[i]) continue;
      const int64_t row = r0 + i * R + rl;
      T* orow = static_cast<T*>(p.dx) + row * p.cols;
      // rmsnorm: s = sum(dy*gamma*x); dx = r*dy*gamma - x * r^3 * s / cols
      const float c2 = inv[i] * inv[i] * (s[i] * inv[i] / static_cast<float>(p.cols));
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int j = tl + k * TPR;
        if (j >= nvec) continue;
        Vec<T, V> raw;
        if constexpr (KIND == B_RMSNORM) {
          float gk[V];
          gamma_vec(k, gk);
          const float2 inv2 = make_float2(inv[i], inv[i]), nc2 = make_float2(-c2, -c2);
#pragma unroll
          for (int e = 0; e < V; e += 2) {
            const float2 t2 = __fmul2_rn(pair_f(&a[i][k].v[e]), make_float2(gk[e], gk[e + 1]));
            const float2 u2 = __fmul2_rn(pair_f(&b[i][k].v[e]), nc2);
            store_pair(&raw.v[e], __ffma2_rn(t2, inv2, u2));
          }
        } else {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const float av = to_f(a[i][k].v[e]), bv = to_f(b[i][k].v[e]);
            raw.v[e] = from_f<T>(KIND == B_SOFTMAX ? bv * (av - s[i]) : av - expf(bv) * s[i]);
          }
        }
        *reinterpret_cast<Vec<T, V>*>(orow + static_cast<int64_t>(j) * V) = raw;
      }
    }
  }

  if constexpr (KIND == B_RMSNORM) {
    if (!want_dgamma) return;
    float* wrow = p.ws + static_cast<int64_t>(blockIdx.x) * p.cols;
    if constexpr (R == 1) {
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int j = tl + k * TPR;
        if (j >= nvec) continue;
#pragma unroll
        for (int q = 0; q < V / 4; ++q)
          *reinterpret_cast<float4*>(wrow + static_cast<int64_t>(j) * V + 4 * q) =
              make_float4(gg[k][4 * q], gg[k][4 * q + 1], gg[k][4 * q + 2], gg[k][4 * q + 3]);
      }
    } else {
      // fold the R row slots of this block in slot order, then one partial row per block.
      // fold[item][thread] with the item rows padded by TPR words: the threads' stores and the
      // folding loads (consecutive lanes = consecutive positions in the row, then the next item)
      // both spread over the banks
      constexpr int kPer = VPL * V;  // floats per thread; only reached with kPer <= 16
      constexpr int kPitch = kBwdThreads + TPR;
      __shared__ float fold[(VPL * V <= 16 ? VPL * V : 1) * kPitch];
      __syncthreads();
#pragma unroll
      for (int k = 0; k < VPL; ++k)
#pragma unroll
        for (int e = 0; e < V; ++e) fold[(k * V + e) * kPitch + t] = gg[k][e];
      __syncthreads();
      for (int m = t; m < TPR * kPer; m += kBwdThreads) {
        const int pos = m % TPR, item = m / TPR;
        const int j = pos + (item / V) * TPR;
        if (j >= nvec) continue;
        float sum = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) sum += fold[item * kPitch + r * TPR + pos];
        wrow[static_cast<int64_t>(j) * V + item % V] = sum;
      }
    }
  }
}

// any length / alignment: one block per row at a time, scalar accesses, inputs read twice
// (the second read is served by L2).  dgamma partials are accumulated in place in the
// block's own workspace row: column j is always handled by the same thread.
template <class T, int KIND>
__global__ void __launch_bounds__(kBwdThreads) rowop_bwd_stream_kernel(const __grid_constant__ BwdParams p) {
  __shared__ float red[2][kBwdThreads / 32];
  const int t = threadIdx.x;
  int phase = 0;
  float* wrow = (KIND == B_RMSNORM && p.ws) ? p.ws + static_cast<int64_t>(blockIdx.x) * p.cols : nullptr;
  if (wrow)
    for (int64_t j = t; j < p.cols; j += kBwdThreads) wrow[j] = 0.f;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* dy = static_cast<const T*>(p.dy) + row * p.dy_row_stride;
    const T* b = static_cast<const T*>(p.b) + row * p.b_row_stride;
    T* dx = static_cast<T*>(p.dx) + row * p.cols;
    const float inv = KIND == B_RMSNORM ? p.inv_rms[row] : 0.f;
    float s = 0.f;
    for (int64_t j = t; j < p.cols; j += kBwdThreads) {
      const float a = to_f(dy[j]), v = to_f(b[j]);
      if constexpr (KIND == B_SOFTMAX) s = fmaf(a, v, s);
      else if constexpr (KIND == B_LOG_SOFTMAX) s += a;
      else {
        const float n = v * inv;
        if (wrow) wrow[j] = fmaf(a, n, wrow[j]);
        s = fmaf(a * (p.gamma ? p.gamma[j] : 1.0f), n, s);
      }
    }
    s = warp_sum(s);
    if ((t & 31) == 0) red[phase][t >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kBwdThreads / 32; ++w) tot += red[phase][w];
    phase ^= 1;
    const float dm = tot / static_cast<float>(p.cols);
    for (int64_t j = t; j < p.cols; j += kBwdThreads) {
      const float a = to_f(dy[j]), v = to_f(b[j]);
      float r;
      if constexpr (KIND == B_SOFTMAX) r = v * (a - tot);
      else if constexpr (KIND == B_LOG_SOFTMAX) r = a - expf(v) * tot;
      else r = inv * (a * (p.gamma ? p.gamma[j] : 1.0f) - v * inv * dm);
      dx[j] = from_f<T>(r);
    }
  }
}

// dgamma[c] = sum over the partial rows, in a fixed order.  A block owns a strip of 8 columns
// (one 32-byte sector per partial row): lane & 7 is the column, the four lane groups of the 32
// warps take 128 rows per step, so the ~600 partial rows of a launch are five loads per thread,
// all in flight at once.  Lane groups are then folded by shuffles and the warps in warp order.
// (The first form -- 32 columns per block, 8 warps -- ran 4 blocks for 128 columns and took
// 10 us of a 42 us backward pass.)
constexpr int kFoldThreads = 1024;
__global__ void __launch_bounds__(kFoldThreads) dgamma_fold_kernel(float* dgamma, const float* ws, int nparts, int64_t cols) {
  __shared__ float sm[kFoldThreads / 32][8];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 8 + (lane & 7);
  float acc = 0.f;
  if (c < cols) {
    for (int r = w * 4 + (lane >> 3); r < nparts; r += 8 * 128) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int rr = r + 128 * u;
        v[u] = rr < nparts ? __ldcg(ws + static_cast<int64_t>(rr) * cols + c) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) acc += v[u];
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 8);
  acc += __shfl_xor_sync(0xffffffffu, acc, 16);
  if (lane < 8) sm[w][lane] = acc;
  __syncthreads();
  if (w == 0 && lane < 8 && c < cols) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kFoldThreads / 32; ++k) s += sm[k][lane];
    dgamma[c] = s;
  }
}

// kernel shape for a row of nvec vectors: threads per row, vectors per thread; tpr == 0 -> stream
struct BwdShape {
  int tpr, vpl;
};
inline BwdShape pick_shape(int64_t nvec, int vbase) {
  for (int tpr = 8; tpr <= 256; tpr *= 2)
    if (nvec <= int64_t{tpr} * vbase) return {tpr, vbase};
  if (nvec <= int64_t{256} * 2 * vbase) return {256, 2 * vbase};
  return {0, 0};
}
inline unsigned bwd_grid(int64_t rows, int tpr, int rif, int sms) {
  const int rpb = tpr ? (kBwdThreads / tpr) * rif : 1;
  const int64_t units = (rows + rpb - 1) / rpb;
  return static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(units, int64_t{sms} * 4)));
}

template <class T>
bool bwd_aligned(const BwdParams& p) {
  constexpr int V = 16 / sizeof(T);
  auto a16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  return p.cols % V == 0 && (p.dy_row_stride * sizeof(T)) % 16 == 0 && (p.b_row_stride * sizeof(T)) % 16 == 0 &&
         a16(p.dy) && a16(p.b) && a16(p.dx) && (p.ws == nullptr || a16(p.ws)) && (p.cols * 4) % 16 == 0;
}

template <class T, int KIND>
vbt_b200_status launch_bwd(const BwdParams& p, cudaStream_t s, int device, unsigned* grid_out) {
  constexpr int V = 16 / sizeof(T);
  constexpr int VB = V == 4 ? 4 : 2;  // vectors per thread: 16 values in registers per operand
  const int sms = sm_count(device);
  const BwdShape sh = bwd_aligned<T>(p) ? pick_shape(p.cols / V, VB) : BwdShape{0, 0};
  // 16-bit rows: two rows in flight per row slot, so a thread has as many bytes on the wire
  // as with 32-bit rows
  constexpr int RIF = (KIND == B_RMSNORM && sizeof(T) == 2) ? 2 : 1;
  const unsigned g = bwd_grid(p.rows, sh.tpr, RIF, sms);
  if (grid_out) *grid_out = g;
#define VB_BWD(TPR, VPL) rowop_bwd_kernel<T, KIND, TPR, VPL, RIF><<<g, kBwdThreads, 0, s>>>(p)
  if (sh.tpr == 0) rowop_bwd_stream_kernel<T, KIND><<<g, kBwdThreads, 0, s>>>(p);
  else if (sh.vpl == 2 * VB) VB_BWD(256, 2 * VB);
  else if (sh.tpr == 8) VB_BWD(8, VB);
  else if (sh.tpr == 16) VB_BWD(16, VB);
  else if (sh.tpr == 32) VB_BWD(32, VB);
  else if (sh.tpr == 64) VB_BWD(64, VB);
  else if (sh.tpr == 128) VB_BWD(128, VB);
  else VB_BWD(256, VB);
#undef VB_BWD
  VB_LAUNCH_CHECK();
  return VBT_B200_OK;
}

template <int KIND>
vbt_b200_status dispatch_bwd(int dtype, const BwdParams& p, cudaStream_t s, int device, const char* name,
                             unsigned* grid_out) {
  switch (dtype) {
    case VBT_B200_F32: return launch_bwd<float, KIND>(p, s, device, grid_out);
    case VBT_B200_F16: return launch_bwd<__half, KIND>(p, s, device, grid_out);
    case VBT_B200_BF16: return launch_bwd<__nv_bfloat16, KIND>(p, s, device, grid_out);
  }
  return fail(VBT_B200_INVALID_ARGUMENT, std::string(name) + ": expected a floating dtype");
}

// number of partial rows the rmsnorm backward writes for this problem on this device
unsigned rms_bwd_parts(int dtype, int64_t rows, int64_t cols, int device) {
  const int V = dtype == VBT_B200_F32 ? 4 : 8;
  const BwdShape sh = cols % V == 0 ? pick_shape(cols / V, V == 4 ? 4 : 2) : BwdShape{0, 0};
  return bwd_grid(rows, sh.tpr, V == 4 ? 1 : 2, sm_count(device));
}

}  // namespace
}  // namespace vb

extern "C" {

vbt_b200_status vbt_b200_softmax_backward(void* dx, const void* dy, const void* y, int32_t dtype, int64_t rows,
                                          int64_t cols, int64_t dy_row_stride, int64_t y_row_stride,
                                          int32_t log_softmax, void* stream) {
  using namespace vb;
  const char* name = log_softmax ? "log_softmax_backward" : "softmax_backward";
  VB_ARG(rows >= 0 && cols >= 0, std::string(name) + ": negative size");
  if (rows == 0 || cols == 0) return VBT_B200_OK;
  VB_ARG(dx && dy && y, std::string(name) + ": null pointer");
  VB_ARG(dy_row_stride >= 0 && y_row_stride >= 0, std::string(name) + ": negative row stride");
  DeviceScope scope(dx);
  BwdParams p{};
  p.dy = dy; p.b = y; p.dx = dx; p.rows = rows; p.cols = cols;
  p.dy_row_stride = dy_row_stride; p.b_row_stride = y_row_stride;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return log_softmax ? dispatch_bwd<B_LOG_SOFTMAX>(dtype, p, s, scope.device(), name, nullptr)
                     : dispatch_bwd<B_SOFTMAX>(dtype, p, s, scope.device(), name, nullptr);
}

vbt_b200_status vbt_b200_rmsnorm_backward_workspace_bytes(int64_t rows, int64_t cols, int32_t dtype,
                                                          int32_t device, size_t* bytes) {
  using namespace vb;
  VB_ARG(bytes != nullptr, "rmsnorm_backward: null output");
  VB_ARG(rows >= 0 && cols >= 0, "rmsnorm_backward: negative size");
  VB_ARG(is_float_dtype(dtype), "rmsnorm_backward: expected a floating dtype");
  // the stream kernel (unaligned pointers) may be chosen at call time: size for the larger grid
  const unsigned a = rms_bwd_parts(dtype, rows, cols, device);
  const unsigned b = bwd_grid(rows, 0, 1, sm_count(device));
  *bytes = static_cast<size_t>(std::max(a, b)) * static_cast<size_t>(cols) * 4;
  return VBT_B200_OK;
}

vbt_b200_status vbt_b200_rmsnorm_backward(void* dx, float* dgamma, const void* dy, const void* x,
                                          const float* inv_rms, const float* gamma, int32_t dtype, int64_t rows,
                                          int64_t cols, int64_t dy_row_stride, int64_t x_row_stride,
                                          void* workspace, size_t workspace_bytes, void* stream) {
  using namespace vb;
  const char* name = "rmsnorm_backward";
  VB_ARG(rows >= 0 && cols >= 0, std::string(name) + ": negative size");
  VB_ARG(is_float_dtype(dtype), std::string(name) + ": expected a floating dtype");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cols == 0) return VBT_B200_OK;
  if (rows == 0) {
    if (dgamma) {
      DeviceScope scope(dgamma);
      VB_CUDA(cudaMemsetAsync(dgamma, 0, static_cast<size_t>(cols) * 4, s));
    }
    return VBT_B200_OK;
  }
  VB_ARG(dx && dy && x && inv_rms, std::string(name) + ": null pointer");
  VB_ARG(dy_row_stride >= 0 && x_row_stride >= 0, std::string(name) + ": negative row stride");
  DeviceScope scope(dx);
  BwdParams p{};
  p.dy = dy; p.b = x; p.dx = dx; p.gamma = gamma; p.inv_rms = inv_rms;
  p.rows = rows; p.cols = cols; p.dy_row_stride = dy_row_stride; p.b_row_stride = x_row_stride;
  if (dgamma) {
    size_t need = 0;
    VB_TRY(vbt_b200_rmsnorm_backward_workspace_bytes(rows, cols, dtype, scope.device(), &need));
    VB_ARG(workspace != nullptr && workspace_bytes >= need,
           std::string(name) + ": workspace too small (see vbt_b200_rmsnorm_backward_workspace_bytes)");
    p.ws = static_cast<float*>(workspace);
  }
  unsigned parts = 0;
  VB_TRY(dispatch_bwd<B_RMSNORM>(dtype, p, s, scope.device(), name, &parts));
  if (dgamma) {
    dgamma_fold_kernel<<<static_cast<unsigned>((cols + 7) / 8), kFoldThreads, 0, s>>>(dgamma, p.ws, static_cast<int>(parts), cols);
    VB_LAUNCH_CHECK();
  }
  return VBT_B200_OK;
}

}  // extern "C"
