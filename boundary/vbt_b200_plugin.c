/*
 * VibeTensor plugin that serves the like-shaped vt:: elementwise ops from libvbt_b200.so.
 *
 * Built against the reference's stable plugin C ABI (include/vbt/plugin/vbt_plugin.h, v1.4):
 * exports vbt_plugin_get_abi_version and vbt_plugin_init (:315-318), registers kernels of type
 * vt_kernel2_fn (:44) and vt_kernel_boxed_fn (:81-84) for the CUDA dispatch key, takes every
 * output from host->tensor_new_dense_like (src/vbt/dispatch/plugin_loader.cc:1398-1441) and
 * reports errors as a vt_status plus host->set_last_error.  The sample it follows is
 * plugins/reference/vbt_reference_add_cuda.cu.
 *
 * What a plugin can and cannot carry: the host API can only allocate an output "dense like"
 * one of the inputs (same sizes, dtype, device).  So this file registers the ops whose result
 * has the dtype of their inputs and the shape of one of them -- unary math, same-dtype binary
 * ops (the other operand may broadcast INTO that shape), ternary ops and where(cond, x, y).
 * Comparisons and predicates (BOOL result), reductions and indexing (other shapes) need the
 * in-tree binding shown in vbt_b200_glue.cc.  The loader silently ignores a registration
 * for "vt::add" (plugin_loader.cc:1183-1185); it is registered anyway so that a host without
 * that quirk gets it.  Ops the host has no schema for are skipped, not treated as an error.
 */
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "vbt/plugin/vbt_plugin.h"
#include "vbt_b200.h"

#if defined(__GNUC__)
#define VBT_PLUGIN_EXPORT __attribute__((visibility("default")))
#else
#define VBT_PLUGIN_EXPORT
#endif

static const struct vbt_host_api* H;
static int g_registered; /* kernels the host accepted */
static int g_skipped;    /* names the host has no schema for */

static void set_err(const char* msg) {
  if (H && H->set_last_error) H->set_last_error(msg);
}

/* DLPack dtype -> vbt::core::ScalarType ordinal used by the library; -1 = not supported */
static int32_t dtype_code(DLDataType dt) {
  if (dt.lanes != 1) return -1;
  switch (dt.code) {
    case kDLFloat: return dt.bits == 32 ? VBT_B200_F32 : (dt.bits == 16 ? VBT_B200_F16 : -1);
    case kDLBfloat: return dt.bits == 16 ? VBT_B200_BF16 : -1;
    case kDLInt: return dt.bits == 64 ? VBT_B200_I64 : (dt.bits == 32 ? VBT_B200_I32 : -1);
    case kDLBool: return VBT_B200_BOOL;
    case kDLUInt: return dt.bits == 8 ? VBT_B200_BOOL : -1;
    default: return -1;
  }
}

/* borrowed view of a host tensor; data == NULL asks the host for the read-only pointer */
static int describe(vt_tensor t, void* data, vbt_b200_tensor* d) {
  const int32_t code = dtype_code(H->tensor_dtype(t));
  if (code < 0) return 0;
  d->data = data ? data : (void*)H->tensor_data(t);
  d->dtype = code;
  d->ndim = (int32_t)H->tensor_ndim(t);
  d->sizes = H->tensor_sizes(t);
  d->strides = H->tensor_strides(t);
  return 1;
}

static vt_status map_status(vbt_b200_status s) {
  set_err(vbt_b200_last_error());
  switch (s) {
    case VBT_B200_INVALID_ARGUMENT: return VT_STATUS_INVALID_ARG;
    case VBT_B200_OUT_OF_RANGE: return VT_STATUS_INVALID_ARG;
    case VBT_B200_CUDA_ERROR: return VT_STATUS_INTERNAL;
    default: return VT_STATUS_RUNTIME_ERROR;
  }
}

static int same_shape(const vbt_b200_tensor* t, const int64_t* sizes, int32_t nd) {
  if (t->ndim != nd) return 0;
  for (int32_t i = 0; i < nd; ++i)
    if (t->sizes[i] != sizes[i]) return 0;
  return 1;
}

/* The operand whose shape equals the broadcast shape of all `n` operands, preferring the
 * earliest one allowed by `like_mask`; NULL when no operand has that shape. */
static vt_tensor pick_like(const vt_tensor* args, const vbt_b200_tensor* d, int n, unsigned like_mask,
                           vt_status* st) {
  const vbt_b200_tensor* ptrs[4];
  int64_t shape[VBT_B200_MAX_NDIM];
  int32_t nd = 0;
  for (int i = 0; i < n; ++i) ptrs[i] = &d[i];
  const vbt_b200_status r = vbt_b200_broadcast_shape(ptrs, n, shape, &nd);
  if (r != VBT_B200_OK) {
    *st = map_status(r);
    return NULL;
  }
  for (int i = 0; i < n; ++i)
    if (((like_mask >> i) & 1u) && same_shape(&d[i], shape, nd)) return args[i];
  set_err("vbt_b200 plugin: the result shape equals none of the operands' shapes; the plugin host "
          "API can only allocate an output like an input (use the in-tree kernel)");
  *st = VT_STATUS_UNSUPPORTED;
  return NULL;
}

enum family { F_UNARY, F_BINARY, F_TERNARY, F_WHERE, F_POLYGAMMA };

/* one body for every registered op */
static vt_status run(enum family fam, int32_t op, vt_stream s, const vt_tensor* args, size_t nargs,
                     vt_tensor* out) {
  if (!out) {
    set_err("null out");
    return VT_STATUS_INVALID_ARG;
  }
  *out = NULL;
  if (!H) return VT_STATUS_INTERNAL;
  const size_t want = fam == F_UNARY ? 1 : ((fam == F_BINARY || fam == F_POLYGAMMA) ? 2 : 3);
  if (nargs != want || !args) {
    set_err("vbt_b200 plugin: wrong number of tensor arguments");
    return VT_STATUS_INVALID_ARG;
  }
  vbt_b200_tensor d[3];
  int32_t device = -1;
  for (size_t i = 0; i < nargs; ++i) {
    const DLDevice dev = H->tensor_device(args[i]);
    if (dev.device_type != kDLCUDA) {
      set_err("vbt_b200 plugin: expected CUDA tensors");
      return VT_STATUS_INVALID_ARG;
    }
    if (device < 0) device = dev.device_id;
    if (dev.device_id != device) {
      set_err("vbt_b200 plugin: tensors on different devices");
      return VT_STATUS_INVALID_ARG;
    }
    if (!describe(args[i], NULL, &d[i])) {
      set_err("vbt_b200 plugin: unsupported dtype");
      return VT_STATUS_UNSUPPORTED;
    }
  }
  /* where(cond, x, y): the result is like x or y, never like the BOOL condition */
  vt_status st = VT_STATUS_OK;
  /* polygamma(n, x): like x, never like the one-element order tensor */
  vt_tensor like = pick_like(args, d, (int)nargs, fam == F_WHERE ? 0x6u : (fam == F_POLYGAMMA ? 0x2u : 0x7u), &st);
  if (!like) return st;
  vt_tensor c = NULL;
  st = H->tensor_new_dense_like(like, &c);
  if (st != VT_STATUS_OK) return st;
  vbt_b200_tensor dc;
  void* cdata = H->tensor_mutable_data(c);
  if (!describe(c, cdata, &dc) || (!cdata && H->tensor_numel(c) != 0)) {
    set_err("vbt_b200 plugin: host returned an output without writable data");
    return VT_STATUS_INTERNAL; /* the host frees tensors a failing kernel created */
  }
  void* stream = (void*)(uintptr_t)s;
  vbt_b200_status r;
  switch (fam) {
    case F_UNARY: r = vbt_b200_unary(op, &dc, &d[0], stream); break;
    case F_BINARY: r = vbt_b200_binary(op, &dc, &d[0], &d[1], stream); break;
    case F_TERNARY: r = vbt_b200_ternary(op, &dc, &d[0], &d[1], &d[2], stream); break;
    case F_POLYGAMMA: r = vbt_b200_polygamma(&dc, &d[0], &d[1], stream); break;
    default: r = vbt_b200_where(&dc, &d[0], &d[1], &d[2], stream); break;
  }
  if (r != VBT_B200_OK) return map_status(r);
  *out = c; /* ownership passes to the host on OK (plugin_loader.cc:1097-1103) */
  return VT_STATUS_OK;
}

/* ---- the op table: one tiny entry function per op, generated from the lists below ---- */
#define UNARY_OPS(X)                                                                              \
  X(relu, RELU) X(neg, NEG) X(abs, ABS) X(square, SQUARE) X(exp, EXP) X(log, LOG) X(sqrt, SQRT)     \
  X(rsqrt, RSQRT) X(sin, SIN) X(cos, COS) X(tanh, TANH) X(sigmoid, SIGMOID) X(silu, SILU)           \
  X(gelu, GELU) X(reciprocal, RECIPROCAL) X(sign, SIGN) X(floor, FLOOR) X(ceil, CEIL)               \
  X(trunc, TRUNC) X(round, ROUND) X(expm1, EXPM1) X(log1p, LOG1P) X(softplus, SOFTPLUS)             \
  X(relu6, RELU6) X(hardtanh, HARDTANH) X(exp2, EXP2) X(log2, LOG2) X(log10, LOG10) X(sinh, SINH)   \
  X(cosh, COSH) X(asinh, ASINH) X(acosh, ACOSH) X(atanh, ATANH) X(tan, TAN) X(asin, ASIN)           \
  X(acos, ACOS) X(atan, ATAN) X(erf, ERF) X(erfc, ERFC) X(lgamma, LGAMMA) X(sinc, SINC)             \
  X(frac, FRAC) X(deg2rad, DEG2RAD) X(rad2deg, RAD2DEG) X(mish, MISH) X(selu, SELU) X(elu, ELU)     \
  X(celu, ELU) X(hardsigmoid, HARDSIGMOID) X(hardshrink, HARDSHRINK) X(softshrink, SOFTSHRINK)      \
  X(logit, LOGIT) X(angle, ANGLE) X(positive, POSITIVE) X(conj_physical, POSITIVE) X(sgn, SGN)      \
  X(nan_to_num, NAN_TO_NUM) X(bitwise_not, BITWISE_NOT)

#define BINARY_OPS(X)                                                                             \
  X(add, ADD) X(sub, SUB) X(mul, MUL) X(div, DIV) X(true_divide, DIV) X(maximum, MAXIMUM)           \
  X(minimum, MINIMUM) X(clamp_min, MAXIMUM) X(clamp_max, MINIMUM) X(fmax, FMAX) X(fmin, FMIN)       \
  X(pow, POW) X(float_power, POW) X(fmod, FMOD) X(remainder, REMAINDER) X(atan2, ATAN2)             \
  X(copysign, COPYSIGN) X(hypot, HYPOT) X(xlogy, XLOGY) X(xlog1py, XLOG1PY)                         \
  X(special_xlog1py, XLOG1PY) X(logaddexp, LOGADDEXP) X(logaddexp2, LOGADDEXP2)                     \
  X(nextafter, NEXTAFTER) X(heaviside, HEAVISIDE) X(rsub, RSUB) X(tanh_backward, TANH_BACKWARD)     \
  X(sigmoid_backward, SIGMOID_BACKWARD) X(silu_backward, SILU_BACKWARD)                             \
  X(logit_backward, LOGIT_BACKWARD) X(mse_loss, MSE_LOSS) X(ldexp, LDEXP)                           \
  X(bitwise_and, BITWISE_AND) X(bitwise_or, BITWISE_OR) X(bitwise_xor, BITWISE_XOR)                 \
  X(bitwise_left_shift, LSHIFT) X(bitwise_right_shift, RSHIFT) X(gcd, GCD) X(lcm, LCM)

#define TERNARY_OPS(X)                                                                            \
  X(clamp, CLAMP) X(clip, CLAMP) X(lerp, LERP) X(threshold, THRESHOLD) X(addcmul, ADDCMUL)          \
  X(addcdiv, ADDCDIV) X(huber_loss, HUBER_LOSS) X(smooth_l1_loss, SMOOTH_L1_LOSS)

#define DEF_UNARY(name, CODE)                                                                       \
  static vt_status k_##name(vt_stream s, const vt_tensor* a, size_t n, vt_tensor* out) {           \
    return run(F_UNARY, VBT_B200_U_##CODE, s, a, n, out);                                           \
  }
#define DEF_BINARY(name, CODE)                                                                      \
  static vt_status k_##name(vt_stream s, vt_tensor a, vt_tensor b, vt_tensor* out) {               \
    const vt_tensor args[2] = {a, b};                                                               \
    return run(F_BINARY, VBT_B200_B_##CODE, s, args, 2, out);                                       \
  }
#define DEF_TERNARY(name, CODE)                                                                     \
  static vt_status k_##name(vt_stream s, const vt_tensor* a, size_t n, vt_tensor* out) {           \
    return run(F_TERNARY, VBT_B200_T_##CODE, s, a, n, out);                                         \
  }
UNARY_OPS(DEF_UNARY)
BINARY_OPS(DEF_BINARY)
TERNARY_OPS(DEF_TERNARY)
static vt_status k_where(vt_stream s, const vt_tensor* a, size_t n, vt_tensor* out) {
  return run(F_WHERE, 0, s, a, n, out);
}
/* vt::polygamma(n, x): a binary schema, n a one-element tensor (cuda_elementwise.cu:3853-3876) */
static vt_status k_polygamma(vt_stream s, vt_tensor n, vt_tensor x, vt_tensor* out) {
  const vt_tensor args[2] = {n, x};
  return run(F_POLYGAMMA, 0, s, args, 2, out);
}
/* masked_fill(self, mask, value) = where(mask, value, self) (cuda_elementwise.cu:3924-3926) */
static vt_status k_masked_fill(vt_stream s, const vt_tensor* a, size_t n, vt_tensor* out) {
  if (n != 3 || !a) return run(F_WHERE, 0, s, a, n, out);
  const vt_tensor args[3] = {a[1], a[2], a[0]};
  return run(F_WHERE, 0, s, args, 3, out);
}

/* A name the host does not define is not an error for this plugin: it serves whatever subset
 * of the table the host has schemas for.  Anything else the host refuses ends init. */
static vt_status accept(vt_status st) {
  if (st == VT_STATUS_OK) {
    ++g_registered;
    return VT_STATUS_OK;
  }
  if (st == VT_STATUS_INVALID_ARG || st == VT_STATUS_NOT_FOUND) { /* "undefined op in VBT_IMPL_CUDA: ..." */
    ++g_skipped;
    set_err("");
    return VT_STATUS_OK;
  }
  return st;
}

VBT_PLUGIN_EXPORT uint32_t vbt_plugin_get_abi_version(void) { return VBT_PLUGIN_ABI_VERSION; }

VBT_PLUGIN_EXPORT vt_status vbt_plugin_init(const struct vbt_host_api* host, struct vbt_plugin_api* out_api) {
  if (!host || !out_api) return VT_STATUS_INVALID_ARG;
  if (host->host_abi_major != VBT_PLUGIN_ABI_VERSION_MAJOR) return VT_STATUS_ABI_MISMATCH;
  /* register_kernel_boxed / register_kernel2 arrived with v1.1 */
  if (host->host_abi_minor < 1 || !host->register_kernel2 || !host->register_kernel_boxed ||
      !host->tensor_new_dense_like || !host->tensor_mutable_data)
    return VT_STATUS_ABI_MISMATCH;
  if (vbt_b200_compiled_arch() != 100) return VT_STATUS_UNSUPPORTED;
  H = host;
  g_registered = g_skipped = 0;
  vt_status st;
#define REG_BOXED(name, CODE)                                                                       \
  st = accept(host->register_kernel_boxed("vt::" #name, kDLCUDA, &k_##name));                       \
  if (st != VT_STATUS_OK) return st;
#define REG_K2(name, CODE)                                                                          \
  st = accept(host->register_kernel2("vt::" #name, kDLCUDA, &k_##name));                            \
  if (st != VT_STATUS_OK) return st;
  UNARY_OPS(REG_BOXED)
  BINARY_OPS(REG_K2)
  TERNARY_OPS(REG_BOXED)
  REG_BOXED(where, 0)
  REG_BOXED(masked_fill, 0)
  REG_K2(polygamma, 0)
  out_api->abi_version = VBT_PLUGIN_ABI_VERSION;
  out_api->name = "vbt_b200: sm_100a elementwise kernels";
  return VT_STATUS_OK;
}

/* For tests and diagnostics: how many registrations the host accepted / had no schema for. */
VBT_PLUGIN_EXPORT int vbt_b200_plugin_registered(void) { return g_registered; }
VBT_PLUGIN_EXPORT int vbt_b200_plugin_skipped(void) { return g_skipped; }
