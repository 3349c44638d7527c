// The long tail of vbt_b200_binary / vbt_b200_binary_scalar: pow, fmod, remainder, atan2, ...,
// the *_backward forms and ldexp.  Reached for op codes in [VBT_B200_B_POW, VBT_B200_B_LDEXP];
// the integer and logical ops live in ew_int_ext.cu.
#include "ew_functors_ext.cuh"
#include "ew_kernels.cuh"

namespace vb {
const char* binary_ext_name(int op) {
  static const char* const names[VBT_B200_B_COUNT - kBinaryCore] = {
      "vt::pow", "vt::fmod", "vt::remainder", "vt::atan2", "vt::copysign", "vt::hypot", "vt::xlogy",
      "vt::xlog1py", "vt::logaddexp", "vt::logaddexp2", "vt::nextafter", "vt::heaviside", "vt::rsub",
      "vt::tanh_backward", "vt::sigmoid_backward", "vt::silu_backward", "vt::logit_backward",
      "vt::mse_loss", "vt::ldexp", "vt::bitwise_and", "vt::bitwise_or", "vt::bitwise_xor", "vt::lshift",
      "vt::rshift", "vt::gcd", "vt::lcm", "vt::logical_and", "vt::logical_or", "vt::logical_xor"};
  return names[op - kBinaryCore];
}
vbt_b200_status binary_int_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                               const vbt_b200_tensor* b, void* stream);  // ew_int_ext.cu

static vbt_b200_status check_float_ext(int32_t op, const std::string& name, const vbt_b200_tensor* out,
                                       const vbt_b200_tensor* a, int b_dtype) {
  VB_ARG(out && a, name + ": null tensor descriptor");
  VB_ARG(a->dtype == b_dtype, name + ": dtype mismatch");
  VB_ARG(out->dtype == a->dtype, name + ": output dtype mismatch");
  const int dt = a->dtype;
  if (dt == VBT_B200_BOOL && (op == VBT_B200_B_FMOD || op == VBT_B200_B_REMAINDER || op == VBT_B200_B_RSUB))
    return fail(VBT_B200_INVALID_ARGUMENT, name + ": boolean not supported");
  if (!is_float_dtype(dt))
    VB_ARG(dt == VBT_B200_I64 && binary_ext_int_ok(op),
           name + (dt == VBT_B200_I64 ? ": floating tensor expected" : ": unsupported dtype"));
  return VBT_B200_OK;
}

vbt_b200_status binary_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                           const vbt_b200_tensor* b, void* stream) {
  if (!binary_ext_is_float_op(op)) return binary_int_ext(op, out, a, b, stream);
  const std::string name = binary_ext_name(op);
  VB_TRY(check_float_ext(op, name, out, a, b->dtype));
  const int dt = a->dtype;
  const vbt_b200_tensor* ops[3] = {out, a, b};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 3, name.c_str(), &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<VBT_B200_B_POW, VBT_B200_B_LDEXP + 1>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    if (dt == VBT_B200_I64) {
      if constexpr (binary_ext_int_ok(OP))
        st = launch_ew<BinaryExtF<OP, int64_t>, int64_t, int64_t, int64_t, int64_t, 2, -1, 0, true>(plan, {}, s);
    } else {
      VB_DISPATCH_FLOAT(dt, T, (st = launch_ew<BinaryExtF<OP, T>, T, T, T, T, 2, -1, 0, true>(plan, {}, s)));
    }
  });
  return st;
}

vbt_b200_status binary_scalar_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                  const void* scalar, int32_t scalar_on_left, void* stream) {
  const std::string name = binary_ext_name(op);
  VB_ARG(binary_ext_is_float_op(op), name + ": no scalar form");
  VB_TRY(check_float_ext(op, name, out, a, a->dtype));
  const int dt = a->dtype;
  VB_ARG(dt != VBT_B200_F16, name + ": Half CPU scalars not supported yet");
  VB_ARG(dt == VBT_B200_F32 || dt == VBT_B200_I64, name + ": unsupported dtype for scalar op");
  const vbt_b200_tensor* ops[2] = {out, a};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 2, name.c_str(), &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool left = scalar_on_left != 0;
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<VBT_B200_B_POW, VBT_B200_B_LDEXP + 1>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    if (dt == VBT_B200_I64) {
      if constexpr (binary_ext_int_ok(OP)) {
        int64_t v;
        std::memcpy(&v, scalar, 8);
        st = launch_ew<ScalarExtF<OP, int64_t>, int64_t, int64_t, int64_t, int64_t, 1, -1, 0, true>(plan, {v, left}, s);
      }
    } else {
      float v;
      std::memcpy(&v, scalar, 4);
      st = launch_ew<ScalarExtF<OP, float>, float, float, float, float, 1, -1, 0, true>(plan, {v, left}, s);
    }
  });
  return st;
}
}  // namespace vb
