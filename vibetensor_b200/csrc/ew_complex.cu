// Complex64 / Complex128 vt::add and vt::mul, and vt::polygamma: the tail of the reference's
// elementwise table (src/vbt/ops/cuda_elementwise.cu:162-190, :3169-3188, :1288-1330, :3853-3876).
#include "ew_functors.cuh"
#include "ew_kernels.cuh"

namespace vb {
namespace {
struct alignas(8) c64 { float re, im; };
struct alignas(16) c128 { double re, im; };

// OP: VBT_B200_B_ADD or VBT_B200_B_MUL.  The products and the difference / sum are separate
// roundings, as a CPU evaluation of (a.re * b.re - a.im * b.im) without contraction gives.
template <int OP, class C>
struct ComplexF {
  __device__ __forceinline__ C operator()(C a, C b, C) const {
    if constexpr (OP == VBT_B200_B_ADD) {
      return C{a.re + b.re, a.im + b.im};
    } else if constexpr (sizeof(C) == 8) {
      return C{__fsub_rn(__fmul_rn(a.re, b.re), __fmul_rn(a.im, b.im)),
               __fadd_rn(__fmul_rn(a.re, b.im), __fmul_rn(a.im, b.re))};
    } else {
      return C{__dsub_rn(__dmul_rn(a.re, b.re), __dmul_rn(a.im, b.im)),
               __dadd_rn(__dmul_rn(a.re, b.im), __dmul_rn(a.im, b.re))};
    }
  }
};

// psi''(x), the one order the reference computes (see the header).
template <class T>
struct PolygammaF {
  __device__ __forceinline__ T operator()(T n_in, T x_in, T) const {
    const float nf = to_float(n_in);
    if (!(nf == 2.0f)) return from_float<T>(__int_as_float(0x7fc00000));
    double x = static_cast<double>(to_float(x_in));
    if ((x <= 0.0 && x == floor(x)) || x < -1e6) return from_float<T>(__int_as_float(0x7fc00000));
    double sum = 0.0;
    for (int it = 0; it < 100 && x < 10.0; ++it) {
      sum -= 2.0 / (x * x * x);
      x += 1.0;
    }
    const double i1 = 1.0 / x, i2 = i1 * i1, i3 = i2 * i1, i4 = i3 * i1;
    return from_float<T>(static_cast<float>(sum + (-i2 - i3 - 0.5 * i4)));
  }
  __device__ static float to_float(float v) { return v; }
  __device__ static float to_float(__half v) { return __half2float(v); }
  __device__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  template <class U> __device__ static U from_float(float v) {
    if constexpr (std::is_same_v<U, float>) return v;
    else if constexpr (std::is_same_v<U, __half>) return __float2half_rn(v);
    else return __float2bfloat16_rn(v);
  }
};
}  // namespace

// vt::add / vt::mul on complex tensors; every other op code rejects them as the reference does
vbt_b200_status complex_binary(int32_t op, const char* name, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                               const vbt_b200_tensor* b, void* stream) {
  VB_ARG(op == VBT_B200_B_ADD || op == VBT_B200_B_MUL, std::string(name) + ": unsupported dtype");
  VB_ARG(a->dtype == b->dtype, std::string(name) + ": dtype mismatch");
  VB_ARG(out->dtype == a->dtype, std::string(name) + ": output dtype mismatch");
  const vbt_b200_tensor* ops[3] = {out, a, b};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 3, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->dtype == VBT_B200_C64) {
    if (op == VBT_B200_B_ADD) return launch_ew<ComplexF<VBT_B200_B_ADD, c64>, c64, c64, c64, c64, 2, -1, 0, true>(plan, {}, s);
    return launch_ew<ComplexF<VBT_B200_B_MUL, c64>, c64, c64, c64, c64, 2, -1, 0, true>(plan, {}, s);
  }
  if (op == VBT_B200_B_ADD) return launch_ew<ComplexF<VBT_B200_B_ADD, c128>, c128, c128, c128, c128, 2, -1, 0, true>(plan, {}, s);
  return launch_ew<ComplexF<VBT_B200_B_MUL, c128>, c128, c128, c128, c128, 2, -1, 0, true>(plan, {}, s);
}

// strided copy of 16-byte elements (Complex128)
vbt_b200_status copy16(const TiPlan& plan, cudaStream_t s) {
  return launch_ew<CopyF<c128>, c128, c128, c128, c128, 1, -1, 0, true>(plan, {}, s);
}
}  // namespace vb

extern "C" vbt_b200_status vbt_b200_polygamma(const vbt_b200_tensor* out, const vbt_b200_tensor* n,
                                              const vbt_b200_tensor* x, void* stream) {
  using namespace vb;
  const char* name = "vt::polygamma";
  VB_ARG(out && n && x, std::string(name) + ": null tensor descriptor");
  VB_TRY(validate_tensor(n, name));
  VB_ARG(numel(*n) == 1, std::string(name) + ": expected n to be a scalar tensor");
  VB_ARG(is_float_dtype(n->dtype), std::string(name) + ": expected n to have floating dtype");
  VB_ARG(n->dtype == x->dtype, std::string(name) + ": dtype mismatch");
  VB_ARG(out->dtype == x->dtype, std::string(name) + ": output dtype mismatch");
  // n broadcasts over x: the same element for every output
  int64_t zeros[VBT_B200_MAX_NDIM] = {};
  vbt_b200_tensor nb = *n;
  nb.ndim = x->ndim;
  nb.sizes = x->sizes;
  nb.strides = zeros;
  const vbt_b200_tensor* ops[3] = {out, &nb, x};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 3, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  VB_DISPATCH_FLOAT(x->dtype, T, (st = launch_ew<PolygammaF<T>, T, T, T, T, 2, -1, 0, true>(plan, {}, s)));
  return st;
}
