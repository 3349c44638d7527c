// The long tail of vbt_b200_unary: the remaining float functors, the predicates that write
// BOOL, and bitwise_not.  Reached through vbt_b200_unary for op codes >= kUnaryCore.
#include "ew_functors_ext.cuh"
#include "ew_kernels.cuh"

namespace vb {
static const char* const kUnaryExtNames[VBT_B200_U_COUNT - kUnaryCore] = {
    "vt::exp2", "vt::log2", "vt::log10", "vt::sinh", "vt::cosh", "vt::asinh", "vt::acosh", "vt::atanh",
    "vt::tan", "vt::asin", "vt::acos", "vt::atan", "vt::erf", "vt::erfc", "vt::lgamma", "vt::sinc",
    "vt::frac", "vt::deg2rad", "vt::rad2deg", "vt::mish", "vt::selu", "vt::elu", "vt::hardsigmoid",
    "vt::hardshrink", "vt::softshrink", "vt::logit", "vt::angle", "vt::positive", "vt::sgn",
    "vt::nan_to_num", "vt::isfinite", "vt::isinf", "vt::isnan", "vt::isneginf", "vt::isposinf",
    "vt::signbit", "vt::logical_not", "vt::bitwise_not"};

template <class F, class TO, class T>
static vbt_b200_status lean1(const TiPlan& plan, cudaStream_t s) {
  return launch_ew<F, TO, T, T, T, 1, -1, 0, true>(plan, {}, s);
}

vbt_b200_status unary_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                          void* stream) {
  const std::string name = kUnaryExtNames[op - kUnaryCore];
  VB_ARG(out && a, name + ": null tensor descriptor");
  const int dt = a->dtype;
  const bool pred = unary_is_predicate(op);
  VB_ARG(out->dtype == (pred ? VBT_B200_BOOL : dt), name + (pred ? ": output must be a bool tensor" : ": dtype mismatch"));
  if (op == VBT_B200_U_BITWISE_NOT) {
    VB_ARG(dt == VBT_B200_I64 || dt == VBT_B200_I32 || dt == VBT_B200_BOOL,
           name + ": integral or bool tensor expected");
  } else if (pred) {
    VB_ARG(is_float_dtype(dt) || dt == VBT_B200_I64 || dt == VBT_B200_BOOL, name + ": unsupported dtype");
  } else if (op == VBT_B200_U_NAN_TO_NUM) {
    VB_ARG(dt == VBT_B200_F32, name + ": float32 tensor expected");
  } else if (op == VBT_B200_U_SGN && dt == VBT_B200_BOOL) {
    return fail(VBT_B200_INVALID_ARGUMENT, name + ": non-bool tensor expected");
  } else if (!is_float_dtype(dt)) {
    VB_ARG(dt == VBT_B200_I64 && unary_ext_int_ok(op),
           name + (dt == VBT_B200_I64 ? ": floating tensor expected" : ": unsupported dtype"));
  }
  const vbt_b200_tensor* ops[2] = {out, a};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 2, name.c_str(), &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<kUnaryCore, VBT_B200_U_COUNT>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    if constexpr (OP == VBT_B200_U_BITWISE_NOT) {
      // ~a == a ^ all-ones; BOOL flips 0/1 (the reference routes it to logical_not)
      if (dt == VBT_B200_I64) st = lean1<IntBinaryNotF<int64_t>, int64_t, int64_t>(plan, s);
      else if (dt == VBT_B200_I32) st = lean1<IntBinaryNotF<int32_t>, int32_t, int32_t>(plan, s);
      else st = lean1<PredicateF<VBT_B200_U_LOGICAL_NOT, uint8_t>, uint8_t, uint8_t>(plan, s);
    } else if constexpr (unary_is_predicate(OP)) {
      if (dt == VBT_B200_I64) st = lean1<PredicateF<OP, int64_t>, uint8_t, int64_t>(plan, s);
      else if (dt == VBT_B200_BOOL) st = lean1<PredicateF<OP, uint8_t>, uint8_t, uint8_t>(plan, s);
      else VB_DISPATCH_FLOAT(dt, T, (st = lean1<PredicateF<OP, T>, uint8_t, T>(plan, s)));
    } else if constexpr (OP == VBT_B200_U_NAN_TO_NUM) {
      st = lean1<UnaryExtF<OP, float>, float, float>(plan, s);
    } else {
      if (dt == VBT_B200_I64) {
        if constexpr (unary_ext_int_ok(OP)) st = lean1<UnaryExtF<OP, int64_t>, int64_t, int64_t>(plan, s);
      } else {
        VB_DISPATCH_FLOAT(dt, T, (st = lean1<UnaryExtF<OP, T>, T, T>(plan, s)));
      }
    }
  });
  return st;
}
}  // namespace vb
