// In-tree binding of libvbt_b200.so: the translation unit a VibeTensor build compiles in place
// of src/vbt/ops/cuda_elementwise.cu and src/vbt/ops/cuda_reduction.cu.
//
// It defines, with the reference's own names and C++ types, the symbols the rest of the core
// links against --
//   TensorImpl vbt_cuda_<op>_impl(const TensorImpl&, ...)   (cuda_elementwise.cu:3348-3939)
//   void vbt_register_cuda_elementwise_kernels()            (cuda_elementwise.cu:3941-4280)
//   TensorImpl vbt_cuda_{sum,prod,min,max,mean}_impl(self, dims, keepdim)
//                                                           (cuda_reduction.cu:2048-2070)
// -- and forwards each to the C ABI of include/vbt_b200.h: outputs and scratch come from the
// stream-ordered caching allocator (vbt::cuda::new_cuda_storage), launches go to
// vbt::cuda::getCurrentStream, every touched storage is recorded on that stream
// (record_stream, include/vbt/cuda/storage.h:20-24), and status codes become the exception
// classes the reference throws.  The reference headers are taken from the checkout the build
// script is pointed at; this file holds none of their code.
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "vbt/core/tensor.h"
#include "vbt/cuda/guard.h"
#include "vbt/cuda/storage.h"
#include "vbt/cuda/stream.h"
#include "vbt/dispatch/dispatcher.h"

#include "vbt_b200.h"

using vbt::core::ScalarType;
using vbt::core::TensorImpl;

namespace {

// The library's dtype codes are the ordinals of vbt::core::ScalarType for the types it serves.
static_assert(static_cast<int>(ScalarType::Bool) == VBT_B200_BOOL, "dtype ordinal");
static_assert(static_cast<int>(ScalarType::Int32) == VBT_B200_I32, "dtype ordinal");
static_assert(static_cast<int>(ScalarType::Int64) == VBT_B200_I64, "dtype ordinal");
static_assert(static_cast<int>(ScalarType::Float32) == VBT_B200_F32, "dtype ordinal");
static_assert(static_cast<int>(ScalarType::Float16) == VBT_B200_F16, "dtype ordinal");
static_assert(static_cast<int>(ScalarType::BFloat16) == VBT_B200_BF16, "dtype ordinal");

vbt_b200_tensor view_of(const TensorImpl& t) {  // borrowed for the duration of the call
  vbt_b200_tensor d;
  d.data = const_cast<void*>(static_cast<const void*>(t.data()));
  d.dtype = static_cast<int32_t>(t.dtype());
  d.ndim = static_cast<int32_t>(t.sizes().size());
  d.sizes = t.sizes().data();
  d.strides = t.strides().data();
  return d;
}

[[noreturn]] void rethrow(vbt_b200_status s) {
  const std::string m = vbt_b200_last_error();
  switch (s) {
    case VBT_B200_INVALID_ARGUMENT: throw std::invalid_argument(m);
    case VBT_B200_OUT_OF_RANGE: throw std::out_of_range(m);
    default: throw std::runtime_error(m);
  }
}
inline void check(vbt_b200_status s) {
  if (s != VBT_B200_OK) rethrow(s);
}

// dense row-major CUDA tensor from the caching allocator (make_cuda_dense_out, cuda_elementwise.cu:96-110)
TensorImpl dense_out(const std::vector<int64_t>& sizes, ScalarType dtype, vbt::core::Device device) {
  int64_t n = 1;
  for (int64_t s : sizes) n *= s;
  std::vector<int64_t> strides(sizes.size());
  int64_t st = 1;
  for (std::size_t i = sizes.size(); i-- > 0;) {
    strides[i] = st;
    st *= sizes[i] == 0 ? 1 : sizes[i];
  }
  auto storage = vbt::cuda::new_cuda_storage(static_cast<std::size_t>(n) * vbt::core::itemsize(dtype), device.index);
  return TensorImpl(storage, sizes, std::move(strides), /*storage_offset=*/0, dtype, device);
}

void require_cuda(const TensorImpl& t, const char* name) {
  if (t.device().type != kDLCUDA) throw std::runtime_error(std::string(name) + ": expected CUDA tensor");
}

std::vector<int64_t> broadcast_of(const vbt_b200_tensor* const* in, int n) {
  int64_t shape[VBT_B200_MAX_NDIM];
  int32_t nd = 0;
  check(vbt_b200_broadcast_shape(in, n, shape, &nd));
  return std::vector<int64_t>(shape, shape + nd);
}

struct Launch {  // device guard + current stream of the device the first operand lives on
  explicit Launch(const TensorImpl& t)
      : guard(t.device().index), stream(vbt::cuda::getCurrentStream(t.device().index)) {}
  void* handle() const { return reinterpret_cast<void*>(stream.handle()); }
  void record(const TensorImpl& t) const { vbt::cuda::record_stream(t.storage(), stream); }
  vbt::cuda::DeviceGuard guard;
  vbt::cuda::Stream stream;
};

TensorImpl unary(int32_t op, const char* name, const TensorImpl& a, ScalarType out_dtype) {
  require_cuda(a, name);
  const vbt_b200_tensor da = view_of(a);
  TensorImpl out = dense_out(a.sizes(), out_dtype, a.device());
  if (out.numel() == 0) return out;
  const Launch l(a);
  const vbt_b200_tensor dout = view_of(out);
  check(vbt_b200_unary(op, &dout, &da, l.handle()));
  l.record(out);
  l.record(a);
  return out;
}

// A CPU 0-d tensor on either side is the reference's scalar operand (cuda_elementwise.cu:2893-2961).
bool is_cpu_scalar(const TensorImpl& t) { return t.device().type == kDLCPU && t.sizes().empty(); }

TensorImpl binary(int32_t op, const char* name, const TensorImpl& a, const TensorImpl& b, bool to_bool) {
  if (is_cpu_scalar(a) != is_cpu_scalar(b)) {
    const bool left = is_cpu_scalar(a);
    const TensorImpl& t = left ? b : a;
    const TensorImpl& s = left ? a : b;
    require_cuda(t, name);
    if (s.dtype() != t.dtype()) throw std::invalid_argument(std::string(name) + ": dtype mismatch");
    TensorImpl out = dense_out(t.sizes(), to_bool ? ScalarType::Bool : t.dtype(), t.device());
    if (out.numel() == 0) return out;
    const Launch l(t);
    const vbt_b200_tensor dt = view_of(t), dout = view_of(out);
    check(vbt_b200_binary_scalar(op, &dout, &dt, s.data(), left ? 1 : 0, l.handle()));
    l.record(out);
    l.record(t);
    return out;
  }
  require_cuda(a, name);
  require_cuda(b, name);
  const vbt_b200_tensor da = view_of(a), db = view_of(b);
  const vbt_b200_tensor* in[2] = {&da, &db};
  TensorImpl out = dense_out(broadcast_of(in, 2), to_bool ? ScalarType::Bool : a.dtype(), a.device());
  if (out.numel() == 0) return out;
  const Launch l(a);
  const vbt_b200_tensor dout = view_of(out);
  check(vbt_b200_binary(op, &dout, &da, &db, l.handle()));
  l.record(out);
  l.record(a);
  l.record(b);
  return out;
}

TensorImpl ternary(int32_t op, const char* name, const TensorImpl& a, const TensorImpl& b, const TensorImpl& c) {
  require_cuda(a, name);
  const vbt_b200_tensor da = view_of(a), db = view_of(b), dc = view_of(c);
  const vbt_b200_tensor* in[3] = {&da, &db, &dc};
  TensorImpl out = dense_out(broadcast_of(in, 3), a.dtype(), a.device());
  if (out.numel() == 0) return out;
  const Launch l(a);
  const vbt_b200_tensor dout = view_of(out);
  check(vbt_b200_ternary(op, &dout, &da, &db, &dc, l.handle()));
  l.record(out);
  l.record(a);
  l.record(b);
  l.record(c);
  return out;
}

TensorImpl where(const TensorImpl& cond, const TensorImpl& x, const TensorImpl& y) {
  require_cuda(x, "vt::where");
  const vbt_b200_tensor dc = view_of(cond), dx = view_of(x), dy = view_of(y);
  const vbt_b200_tensor* in[3] = {&dc, &dx, &dy};
  TensorImpl out = dense_out(broadcast_of(in, 3), x.dtype(), x.device());
  if (out.numel() == 0) return out;
  const Launch l(x);
  const vbt_b200_tensor dout = view_of(out);
  check(vbt_b200_where(&dout, &dc, &dx, &dy, l.handle()));
  l.record(out);
  l.record(cond);
  l.record(x);
  l.record(y);
  return out;
}

TensorImpl reduce(int32_t op, const char* name, const TensorImpl& self, const std::vector<int64_t>& dims,
                  bool keepdim) {
  require_cuda(self, name);
  const vbt_b200_tensor dx = view_of(self);
  int64_t shape[VBT_B200_MAX_NDIM];
  int32_t nd = 0;
  check(vbt_b200_reduce_shape(&dx, dims.data(), static_cast<int32_t>(dims.size()), keepdim ? 1 : 0, shape, &nd));
  TensorImpl out = dense_out(std::vector<int64_t>(shape, shape + nd), self.dtype(), self.device());
  const Launch l(self);
  const std::size_t ws_bytes =
      vbt_b200_reduce_workspace_bytes(op, &dx, dims.data(), static_cast<int32_t>(dims.size()));
  vbt::core::StoragePtr ws;
  if (ws_bytes) ws = vbt::cuda::new_cuda_storage(ws_bytes, self.device().index);
  const vbt_b200_tensor dout = view_of(out);
  check(vbt_b200_reduce(op, &dout, nullptr, &dx, dims.data(), static_cast<int32_t>(dims.size()), keepdim ? 1 : 0,
                        ws ? ws->data() : nullptr, ws_bytes, l.handle()));
  if (ws) vbt::cuda::record_stream(ws, l.stream);
  l.record(out);
  l.record(self);
  return out;
}

}  // namespace

// ---- the op table: name, library op code; one definition and one registration per entry ----
#define VBT_B200_UNARY_SAME(X)                                                                        \
  X(relu, RELU) X(neg, NEG) X(abs, ABS) X(square, SQUARE) X(exp, EXP) X(log, LOG) X(sqrt, SQRT)         \
  X(rsqrt, RSQRT) X(sin, SIN) X(cos, COS) X(tanh, TANH) X(sigmoid, SIGMOID) X(silu, SILU) X(gelu, GELU) \
  X(reciprocal, RECIPROCAL) X(sign, SIGN) X(floor, FLOOR) X(ceil, CEIL) X(trunc, TRUNC)                 \
  X(round, ROUND) X(expm1, EXPM1) X(log1p, LOG1P) X(softplus, SOFTPLUS) X(relu6, RELU6)                 \
  X(hardtanh, HARDTANH) X(exp2, EXP2) X(log2, LOG2) X(log10, LOG10) X(sinh, SINH) X(cosh, COSH)         \
  X(asinh, ASINH) X(acosh, ACOSH) X(atanh, ATANH) X(tan, TAN) X(asin, ASIN) X(acos, ACOS)               \
  X(atan, ATAN) X(erf, ERF) X(erfc, ERFC) X(lgamma, LGAMMA) X(sinc, SINC) X(frac, FRAC)                 \
  X(deg2rad, DEG2RAD) X(rad2deg, RAD2DEG) X(mish, MISH) X(selu, SELU) X(elu, ELU) X(celu, ELU)          \
  X(hardsigmoid, HARDSIGMOID) X(hardshrink, HARDSHRINK) X(softshrink, SOFTSHRINK) X(logit, LOGIT)       \
  X(angle, ANGLE) X(positive, POSITIVE) X(conj_physical, POSITIVE) X(sgn, SGN)                          \
  X(nan_to_num, NAN_TO_NUM) X(bitwise_not, BITWISE_NOT)
#define VBT_B200_UNARY_BOOL(X)                                                                        \
  X(isfinite, ISFINITE) X(isinf, ISINF) X(isnan, ISNAN) X(isneginf, ISNEGINF) X(isposinf, ISPOSINF)     \
  X(signbit, SIGNBIT) X(logical_not, LOGICAL_NOT)
#define VBT_B200_BINARY_SAME(X)                                                                       \
  X(add, ADD) X(sub, SUB) X(mul, MUL) X(div, DIV) X(true_divide, DIV) X(maximum, MAXIMUM)               \
  X(minimum, MINIMUM) X(clamp_min, MAXIMUM) X(clamp_max, MINIMUM) X(fmax, FMAX) X(fmin, FMIN)           \
  X(pow, POW) X(float_power, POW) X(fmod, FMOD) X(remainder, REMAINDER) X(atan2, ATAN2)                 \
  X(copysign, COPYSIGN) X(hypot, HYPOT) X(xlogy, XLOGY) X(xlog1py, XLOG1PY)                             \
  X(special_xlog1py, XLOG1PY) X(logaddexp, LOGADDEXP) X(logaddexp2, LOGADDEXP2)                         \
  X(nextafter, NEXTAFTER) X(heaviside, HEAVISIDE) X(rsub, RSUB) X(tanh_backward, TANH_BACKWARD)         \
  X(sigmoid_backward, SIGMOID_BACKWARD) X(silu_backward, SILU_BACKWARD)                                 \
  X(logit_backward, LOGIT_BACKWARD) X(mse_loss, MSE_LOSS) X(ldexp, LDEXP) X(bitwise_and, BITWISE_AND)   \
  X(bitwise_or, BITWISE_OR) X(bitwise_xor, BITWISE_XOR) X(bitwise_left_shift, LSHIFT)                   \
  X(bitwise_right_shift, RSHIFT) X(gcd, GCD) X(lcm, LCM)
#define VBT_B200_BINARY_BOOL(X)                                                                       \
  X(eq, EQ) X(ne, NE) X(lt, LT) X(gt, GT) X(le, LE) X(ge, GE) X(logical_and, LOGICAL_AND)               \
  X(logical_or, LOGICAL_OR) X(logical_xor, LOGICAL_XOR)
#define VBT_B200_TERNARY(X)                                                                           \
  X(clamp, CLAMP) X(clip, CLAMP) X(lerp, LERP) X(threshold, THRESHOLD) X(addcmul, ADDCMUL)              \
  X(addcdiv, ADDCDIV) X(huber_loss, HUBER_LOSS) X(smooth_l1_loss, SMOOTH_L1_LOSS)

extern "C" {

#define DEF_U_SAME(name, CODE) \
  TensorImpl vbt_cuda_##name##_impl(const TensorImpl& a) { return unary(VBT_B200_U_##CODE, "vt::" #name, a, a.dtype()); }
#define DEF_U_BOOL(name, CODE) \
  TensorImpl vbt_cuda_##name##_impl(const TensorImpl& a) { return unary(VBT_B200_U_##CODE, "vt::" #name, a, ScalarType::Bool); }
#define DEF_B_SAME(name, CODE)                                                   \
  TensorImpl vbt_cuda_##name##_impl(const TensorImpl& a, const TensorImpl& b) {  \
    return binary(VBT_B200_B_##CODE, "vt::" #name, a, b, false);                 \
  }
#define DEF_B_BOOL(name, CODE)                                                   \
  TensorImpl vbt_cuda_##name##_impl(const TensorImpl& a, const TensorImpl& b) {  \
    return binary(VBT_B200_B_##CODE, "vt::" #name, a, b, true);                  \
  }
#define DEF_T(name, CODE)                                                                             \
  TensorImpl vbt_cuda_##name##_impl(const TensorImpl& a, const TensorImpl& b, const TensorImpl& c) {  \
    return ternary(VBT_B200_T_##CODE, "vt::" #name, a, b, c);                                         \
  }
VBT_B200_UNARY_SAME(DEF_U_SAME)
VBT_B200_UNARY_BOOL(DEF_U_BOOL)
VBT_B200_BINARY_SAME(DEF_B_SAME)
VBT_B200_BINARY_BOOL(DEF_B_BOOL)
VBT_B200_TERNARY(DEF_T)

TensorImpl vbt_cuda_where_impl(const TensorImpl& cond, const TensorImpl& x, const TensorImpl& y) {
  return where(cond, x, y);
}
// masked_fill(self, mask, value) = where(mask, value, self) (cuda_elementwise.cu:3924-3926)
TensorImpl vbt_cuda_masked_fill_impl(const TensorImpl& self, const TensorImpl& mask, const TensorImpl& value) {
  return where(mask, value, self);
}

// vt::polygamma(n, x): n a one-element tensor on x's device (cuda_elementwise.cu:3853-3876)
TensorImpl vbt_cuda_polygamma_impl(const TensorImpl& n, const TensorImpl& a) {
  require_cuda(a, "vt::polygamma");
  require_cuda(n, "vt::polygamma");
  if (n.device().index != a.device().index) throw std::invalid_argument("vt::polygamma: device mismatch");
  const vbt_b200_tensor dn = view_of(n), da = view_of(a);
  TensorImpl out = dense_out(std::vector<int64_t>(a.sizes().begin(), a.sizes().end()), a.dtype(), a.device());
  const Launch l(a);
  const vbt_b200_tensor dout = view_of(out);
  check(vbt_b200_polygamma(&dout, &dn, &da, l.handle()));  // scalar / dtype rules and their messages: the library's
  l.record(out);
  l.record(n);
  l.record(a);
  return out;
}

TensorImpl vbt_cuda_sum_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim) {
  return reduce(VBT_B200_R_SUM, "vt::sum", self, dims, keepdim);
}
TensorImpl vbt_cuda_prod_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim) {
  return reduce(VBT_B200_R_PROD, "vt::prod", self, dims, keepdim);
}
TensorImpl vbt_cuda_min_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim) {
  return reduce(VBT_B200_R_MIN, "vt::min", self, dims, keepdim);
}
TensorImpl vbt_cuda_max_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim) {
  return reduce(VBT_B200_R_MAX, "vt::max", self, dims, keepdim);
}
TensorImpl vbt_cuda_mean_impl(const TensorImpl& self, std::vector<int64_t> dims, bool keepdim) {
  return reduce(VBT_B200_R_MEAN, "vt::mean", self, dims, keepdim);
}

// Registers every kernel above whose op the dispatcher has a schema for, once
// (cuda_elementwise.cu:3941-4280 does the same with the reference's own kernels).
void vbt_register_cuda_elementwise_kernels() {
  static std::once_flag once;
  std::call_once(once, []() {
    auto& D = vbt::dispatch::Dispatcher::instance();
#define REG(name, CODE) \
  if (D.has("vt::" #name)) D.registerCudaKernel("vt::" #name, &vbt_cuda_##name##_impl);
    VBT_B200_UNARY_SAME(REG)
    VBT_B200_UNARY_BOOL(REG)
    VBT_B200_BINARY_SAME(REG)
    VBT_B200_BINARY_BOOL(REG)
    VBT_B200_TERNARY(REG)
    REG(where, 0)
    REG(masked_fill, 0)
    REG(polygamma, 0)
#undef REG
  });
}

}  // extern "C"
