// Integer and logical binary ops: bitwise and/or/xor (BOOL/I32/I64), shifts (I32/I64),
// gcd/lcm (I64), logical and/or/xor (-> BOOL).  The reference's binary_bitwise_dispatcher and
// the Bool output mode of binary_op_dispatcher (src/vbt/ops/cuda_elementwise.cu:3215-3350,
// :3489-3545).
#include "ew_functors_ext.cuh"
#include "ew_kernels.cuh"

namespace vb {
const char* binary_ext_name(int op);  // ew_binary_ext.cu

template <class F, class TO, class T>
static vbt_b200_status lean2(const TiPlan& plan, cudaStream_t s) {
  return launch_ew<F, TO, T, T, T, 2, -1, 0, true>(plan, {}, s);
}

vbt_b200_status binary_int_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                               const vbt_b200_tensor* b, void* stream) {
  const std::string name = binary_ext_name(op);
  VB_ARG(out && a && b, name + ": null tensor descriptor");
  const int dt = a->dtype;
  const bool logical = binary_is_logical(op);
  if (logical) {
    VB_ARG(dt == b->dtype, name + ": dtype mismatch");
    VB_ARG(is_float_dtype(dt) || dt == VBT_B200_I64 || dt == VBT_B200_BOOL, name + ": unsupported dtype");
    VB_ARG(out->dtype == VBT_B200_BOOL, name + ": output dtype mismatch");
  } else {
    const bool shift = op == VBT_B200_B_LSHIFT || op == VBT_B200_B_RSHIFT;
    const bool gl = op == VBT_B200_B_GCD || op == VBT_B200_B_LCM;
    auto int_like = [](int d) { return d == VBT_B200_I64 || d == VBT_B200_I32; };
    if (shift) VB_ARG(int_like(dt) && int_like(b->dtype), name + ": expected Int32/Int64 tensors");
    else if (gl) VB_ARG(dt == VBT_B200_I64 && b->dtype == VBT_B200_I64, name + ": expected Int64 tensors");
    else VB_ARG(int_like(dt) || dt == VBT_B200_BOOL, name + ": integral or bool tensors expected");
    VB_ARG(dt == b->dtype, name + ": dtype mismatch");
    VB_ARG(out->dtype == dt, name + ": output dtype mismatch");
  }
  const vbt_b200_tensor* ops[3] = {out, a, b};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 3, name.c_str(), &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<VBT_B200_B_BITWISE_AND, VBT_B200_B_COUNT>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    if constexpr (binary_is_logical(OP)) {
      if (dt == VBT_B200_I64) st = lean2<LogicalF<OP, int64_t>, uint8_t, int64_t>(plan, s);
      else if (dt == VBT_B200_BOOL) st = lean2<LogicalF<OP, uint8_t>, uint8_t, uint8_t>(plan, s);
      else VB_DISPATCH_FLOAT(dt, T, (st = lean2<LogicalF<OP, T>, uint8_t, T>(plan, s)));
    } else {
      if (dt == VBT_B200_I64) st = lean2<IntBinaryF<OP, int64_t>, int64_t, int64_t>(plan, s);
      else if constexpr (OP != VBT_B200_B_GCD && OP != VBT_B200_B_LCM) {
        if (dt == VBT_B200_I32) st = lean2<IntBinaryF<OP, int32_t>, int32_t, int32_t>(plan, s);
        else if constexpr (OP != VBT_B200_B_LSHIFT && OP != VBT_B200_B_RSHIFT)
          st = lean2<IntBinaryF<OP, uint8_t>, uint8_t, uint8_t>(plan, s);
      }
    }
  });
  return st;
}
}  // namespace vb
