// vbt_b200_unary, vbt_b200_copy and the named unary forms.
#include "ew_functors.cuh"
#include "ew_kernels.cuh"

namespace vb {
static const char* const kUnaryNames[kUnaryCore] = {
    "vt::relu", "vt::neg", "vt::abs", "vt::square", "vt::exp", "vt::log", "vt::sqrt", "vt::rsqrt",
    "vt::sin", "vt::cos", "vt::tanh", "vt::sigmoid", "vt::silu", "vt::gelu", "vt::reciprocal",
    "vt::sign", "vt::floor", "vt::ceil", "vt::trunc", "vt::round", "vt::expm1", "vt::log1p",
    "vt::softplus", "vt::relu6", "vt::hardtanh"};
vbt_b200_status unary_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                          void* stream);  // ew_unary_ext.cu
vbt_b200_status copy16(const TiPlan& plan, cudaStream_t s);  // ew_complex.cu
}  // namespace vb

extern "C" vbt_b200_status vbt_b200_unary(int32_t op, const vbt_b200_tensor* out,
                                          const vbt_b200_tensor* a, void* stream) {
  using namespace vb;
  VB_ARG(op >= 0 && op < VBT_B200_U_COUNT, "unary: unknown op code");
  if (op >= kUnaryCore) return unary_ext(op, out, a, stream);
  const char* name = kUnaryNames[op];
  VB_ARG(out && a, std::string(name) + ": null tensor descriptor");
  VB_ARG(out->dtype == a->dtype, std::string(name) + ": dtype mismatch");
  const int dt = a->dtype;
  if (dt == VBT_B200_I64 || dt == VBT_B200_I32 || dt == VBT_B200_BOOL)
    VB_ARG(dt == VBT_B200_I64 && unary_int_ok(op),
           std::string(name) + (dt == VBT_B200_I64 ? ": floating tensor expected" : ": unsupported dtype"));
  const vbt_b200_tensor* ops[2] = {out, a};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 2, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  const bool ok = dispatch_op<0, kUnaryCore>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    if (dt == VBT_B200_I64) {
      if constexpr (unary_int_ok(OP))
        st = launch_ew<UnaryF<OP, int64_t>, int64_t, int64_t, int64_t, int64_t, 1>(plan, {}, s);
    } else {
      const bool known = VB_DISPATCH_FLOAT(dt, T, (st = launch_ew<UnaryF<OP, T>, T, T, T, T, 1>(plan, {}, s)));
      if (!known) st = fail(VBT_B200_INVALID_ARGUMENT, std::string(name) + ": unsupported dtype");
    }
  });
  VB_ARG(ok, "unary: unknown op code");
  return st;
}

extern "C" vbt_b200_status vbt_b200_copy(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                         void* stream) {
  using namespace vb;
  VB_ARG(out && a, "copy: null tensor descriptor");
  VB_ARG(out->dtype == a->dtype, "copy: dtype mismatch");
  const vbt_b200_tensor* ops[2] = {out, a};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 2, "copy", &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (itemsize(a->dtype)) {
    case 1: return launch_ew<CopyF<uint8_t>, uint8_t, uint8_t, uint8_t, uint8_t, 1>(plan, {}, s);
    case 2: return launch_ew<CopyF<uint16_t>, uint16_t, uint16_t, uint16_t, uint16_t, 1>(plan, {}, s);
    case 4: return launch_ew<CopyF<uint32_t>, uint32_t, uint32_t, uint32_t, uint32_t, 1>(plan, {}, s);
    case 8: return launch_ew<CopyF<uint64_t>, uint64_t, uint64_t, uint64_t, uint64_t, 1>(plan, {}, s);
    case 16: return copy16(plan, s);
  }
  return fail(VBT_B200_INVALID_ARGUMENT, "copy: unsupported dtype");
}

extern "C" vbt_b200_status vbt_b200_relu(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                         void* stream) {
  return vbt_b200_unary(VBT_B200_U_RELU, out, a, stream);
}
