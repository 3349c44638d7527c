// vbt_b200_binary, vbt_b200_binary_scalar and the named binary forms.
#include "ew_functors.cuh"
#include "ew_kernels.cuh"

namespace vb {
static const char* const kBinaryNames[kBinaryCore] = {
    "vt::add", "vt::sub", "vt::mul", "vt::div", "vt::maximum", "vt::minimum", "vt::fmax", "vt::fmin",
    "vt::eq", "vt::ne", "vt::lt", "vt::gt", "vt::le", "vt::ge"};

static vbt_b200_status check_binary(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                    int b_dtype, const char** name_out) {
  VB_ARG(op >= 0 && op < kBinaryCore, "binary: unknown op code");
  const char* name = kBinaryNames[op];
  *name_out = name;
  VB_ARG(out && a, std::string(name) + ": null tensor descriptor");
  VB_ARG(a->dtype == b_dtype, std::string(name) + ": dtype mismatch");
  const bool cmp = binary_is_compare(op);
  VB_ARG(out->dtype == (cmp ? VBT_B200_BOOL : a->dtype), std::string(name) + ": output dtype mismatch");
  const int dt = a->dtype;
  VB_ARG(dt == VBT_B200_I64 || is_float_dtype(dt), std::string(name) + ": unsupported dtype");
  if (op == VBT_B200_B_DIV) VB_ARG(dt != VBT_B200_I64, std::string(name) + ": unsupported dtype");
  return VBT_B200_OK;
}
// ew_binary_ext.cu
vbt_b200_status binary_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                           const vbt_b200_tensor* b, void* stream);
vbt_b200_status binary_scalar_ext(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                  const void* scalar, int32_t scalar_on_left, void* stream);
// ew_complex.cu
vbt_b200_status complex_binary(int32_t op, const char* name, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                               const vbt_b200_tensor* b, void* stream);
}  // namespace vb

extern "C" vbt_b200_status vbt_b200_binary(int32_t op, const vbt_b200_tensor* out,
                                           const vbt_b200_tensor* a, const vbt_b200_tensor* b,
                                           void* stream) {
  using namespace vb;
  const char* name = "binary";
  VB_ARG(b != nullptr, "binary: null tensor descriptor");
  if (op >= kBinaryCore && op < VBT_B200_B_COUNT) return binary_ext(op, out, a, b, stream);
  if (out && a && op >= 0 && op < kBinaryCore && (a->dtype == VBT_B200_C64 || a->dtype == VBT_B200_C128))
    return complex_binary(op, kBinaryNames[op], out, a, b, stream);  // vt::add / vt::mul only (cuda_elementwise.cu:3169-3188)
  VB_TRY(check_binary(op, out, a, b->dtype, &name));
  const int dt = a->dtype;
  const vbt_b200_tensor* ops[3] = {out, a, b};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 3, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<0, kBinaryCore>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    if constexpr (binary_is_compare(OP)) {
      if (dt == VBT_B200_I64)
        st = launch_ew<CompareF<OP, int64_t>, uint8_t, int64_t, int64_t, int64_t, 2>(plan, {}, s);
      else
        VB_DISPATCH_FLOAT(dt, T, (st = launch_ew<CompareF<OP, T>, uint8_t, T, T, T, 2>(plan, {}, s)));
    } else {
      if (dt == VBT_B200_I64) {
        if constexpr (OP != VBT_B200_B_DIV)
          st = launch_ew<BinaryF<OP, int64_t>, int64_t, int64_t, int64_t, int64_t, 2>(plan, {}, s);
      } else {
        VB_DISPATCH_FLOAT(dt, T, (st = launch_ew<BinaryF<OP, T>, T, T, T, T, 2>(plan, {}, s)));
      }
    }
  });
  return st;
}

extern "C" vbt_b200_status vbt_b200_binary_scalar(int32_t op, const vbt_b200_tensor* out,
                                                  const vbt_b200_tensor* a, const void* scalar,
                                                  int32_t scalar_on_left, void* stream) {
  using namespace vb;
  const char* name = "binary";
  VB_ARG(a != nullptr && scalar != nullptr, "binary_scalar: null argument");
  if (op >= kBinaryCore && op < VBT_B200_B_COUNT)
    return binary_scalar_ext(op, out, a, scalar, scalar_on_left, stream);
  VB_TRY(check_binary(op, out, a, a->dtype, &name));
  const int dt = a->dtype;
  // the reference's scalar path takes Float32 / Int64 only (cuda_elementwise.cu:2953-2957)
  VB_ARG(dt != VBT_B200_F16, std::string(name) + ": Half CPU scalars not supported yet");
  VB_ARG(dt == VBT_B200_F32 || dt == VBT_B200_I64, std::string(name) + ": unsupported dtype for scalar op");
  const vbt_b200_tensor* ops[2] = {out, a};
  TiPlan plan;
  VB_TRY(build_ti_plan(ops, 2, name, &plan));
  DeviceScope scope(out->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool left = scalar_on_left != 0;
  vbt_b200_status st = VBT_B200_OK;
  dispatch_op<0, kBinaryCore>(op, [&](auto opc) {
    constexpr int OP = decltype(opc)::value;
    constexpr bool CMP = binary_is_compare(OP);
    if (dt == VBT_B200_I64) {
      if constexpr (OP != VBT_B200_B_DIV) {
        int64_t v;
        std::memcpy(&v, scalar, 8);
        using TO = std::conditional_t<CMP, uint8_t, int64_t>;
        st = launch_ew<ScalarF<OP, int64_t, CMP>, TO, int64_t, int64_t, int64_t, 1>(plan, {v, left}, s);
      }
    } else {
      float v;
      std::memcpy(&v, scalar, 4);
      using TO = std::conditional_t<CMP, uint8_t, float>;
      st = launch_ew<ScalarF<OP, float, CMP>, TO, float, float, float, 1>(plan, {v, left}, s);
    }
  });
  return st;
}

#define VB_NAMED_BINARY(fn, code)                                                              \
  extern "C" vbt_b200_status fn(const vbt_b200_tensor* out, const vbt_b200_tensor* a,         \
                                const vbt_b200_tensor* b, void* stream) {                      \
    return vbt_b200_binary(code, out, a, b, stream);                                           \
  }
VB_NAMED_BINARY(vbt_b200_add, VBT_B200_B_ADD)
VB_NAMED_BINARY(vbt_b200_sub, VBT_B200_B_SUB)
VB_NAMED_BINARY(vbt_b200_mul, VBT_B200_B_MUL)
VB_NAMED_BINARY(vbt_b200_div, VBT_B200_B_DIV)
VB_NAMED_BINARY(vbt_b200_gt, VBT_B200_B_GT)
