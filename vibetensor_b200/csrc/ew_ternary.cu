// vbt_b200_ternary (clamp / lerp / threshold and the fused chains) and vbt_b200_where.
#include "ew_functors.cuh"
#include "ew_kernels.cuh"

namespace vb {
static const char* const kTernaryNames[VBT_B200_T_COUNT] = {
    "vt::clamp", "vt::lerp", "vt::threshold", "vt::addcmul", "vt::addcdiv", "vt::where_gt0_addcmul",
    "vt::huber_loss", "vt::smooth_l1_loss"};
}

extern "C" vbt_b200_status vbt_b200_ternary(int32_t op, const vbt_b200_tensor* out,
                                            const vbt_b200_tensor* a, const vbt_b200_tensor* b,
                                            const vbt_b200_tensor* c, void* stream) {
  using namespace vb;
  VB_ARG(op >= 0 && op < VBT_B200_T_COUNT, "ternary: unknown op code");
  const char* name = kTernaryNames[op];
  VB_ARG(out && a && b && c, std::string(name) + ": null tensor descriptor");
  VB_ARG(a->dtype == b->dtype && a->dtype == c->dtype && a->dtype == out->dtype,
         std::string(name) + ": dtype mismatch");
  VB_ARG(is_float_dtype(a->dtype), std::string(name) + ": floating tensor expected");
  const int dt = a->dtype;
  const vbt_b200_tensor* ops[4] = {out, a, b, c};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 4, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<0, VBT_B200_T_COUNT>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    // The fused chains also get a build where inputs 2 and 3 are known not to vary along
    // dim 1, so that their product is computed once per thread and reused for every row.
    // ... and where the first input is also a per-row scalar (broadcast along the output's
    // inner dim), which is the layout of a[n,1,h,1] + b[1,c,1,w] * c[n,c,1,w] written
    // channels-last: the per-element work shrinks to one add and one select.
    constexpr int INV = ternary_is_chain(OP) ? 6 : -1;
    constexpr int BC0 = ternary_is_chain(OP) ? 1 : 0;
    VB_DISPATCH_FLOAT(dt, T, (st = launch_ew<TernaryF<OP, T>, T, T, T, T, 3, INV, BC0>(plan, {}, s)));
  });
  return st;
}

extern "C" vbt_b200_status vbt_b200_where(const vbt_b200_tensor* out, const vbt_b200_tensor* cond,
                                          const vbt_b200_tensor* x, const vbt_b200_tensor* y,
                                          void* stream) {
  using namespace vb;
  const char* name = "vt::where";
  VB_ARG(out && cond && x && y, std::string(name) + ": null tensor descriptor");
  VB_ARG(cond->dtype == VBT_B200_BOOL, std::string(name) + ": condition must be a bool tensor");
  VB_ARG(x->dtype == y->dtype && x->dtype == out->dtype, std::string(name) + ": dtype mismatch");
  const vbt_b200_tensor* ops[4] = {out, cond, x, y};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 4, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (x->dtype) {
    case VBT_B200_BOOL:
      return launch_ew<WhereF<uint8_t>, uint8_t, uint8_t, uint8_t, uint8_t, 3>(plan, {}, s);
    case VBT_B200_F16:
    case VBT_B200_BF16:
      return launch_ew<WhereF<uint16_t>, uint16_t, uint8_t, uint16_t, uint16_t, 3>(plan, {}, s);
    case VBT_B200_F32:
      return launch_ew<WhereF<uint32_t>, uint32_t, uint8_t, uint32_t, uint32_t, 3>(plan, {}, s);
    case VBT_B200_I64:
      return launch_ew<WhereF<uint64_t>, uint64_t, uint8_t, uint64_t, uint64_t, 3>(plan, {}, s);
  }
  return fail(VBT_B200_INVALID_ARGUMENT, std::string(name) + ": unsupported dtype");
}
