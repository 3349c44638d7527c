// Per-element functors.  Semantics follow the reference's functors
// (src/vbt/ops/cuda_elementwise.cu:155-160, :244-306, :590-1030, :1259-1277, :2399-2404):
// half / bfloat16 are widened to float, computed, and rounded to nearest-even once per op.
// The reference writes Silu, Gelu, Reciprocal, Sign, Softplus, Relu6 and Hardtanh in device
// fp64; here they are fp32 (an fp64 functor would make a memory-bound kernel compute-bound
// on B200), which stays within 1e-5 of the fp64 form.
#pragma once
#include "common.cuh"

namespace vb {

// Op codes below these bounds are served by ew_unary.cu / ew_binary.cu / ew_ternary.cu with
// every kernel variant; the codes above them by the *_ext translation units.
constexpr int kUnaryCore = VBT_B200_U_HARDTANH + 1;
constexpr int kBinaryCore = VBT_B200_B_GE + 1;
constexpr bool binary_is_compare(int op) { return op >= VBT_B200_B_EQ && op <= VBT_B200_B_GE; }
constexpr bool ternary_is_chain(int op) {
  return op >= VBT_B200_T_ADDCMUL && op <= VBT_B200_T_WHERE_GT0_ADDCMUL;
}

template <int OP>
__device__ __forceinline__ float unary_math(float a) {
  if constexpr (OP == VBT_B200_U_RELU) return a > 0.f ? a : 0.f;
  else if constexpr (OP == VBT_B200_U_NEG) return -a;
  else if constexpr (OP == VBT_B200_U_ABS) return fabsf(a);
  else if constexpr (OP == VBT_B200_U_SQUARE) return a * a;
  else if constexpr (OP == VBT_B200_U_EXP) return expf(a);
  else if constexpr (OP == VBT_B200_U_LOG) return logf(a);
  else if constexpr (OP == VBT_B200_U_SQRT) return sqrtf(a);
  else if constexpr (OP == VBT_B200_U_RSQRT) return rsqrtf(a);
  else if constexpr (OP == VBT_B200_U_SIN) return sinf(a);
  else if constexpr (OP == VBT_B200_U_COS) return cosf(a);
  else if constexpr (OP == VBT_B200_U_TANH) return tanhf(a);
  else if constexpr (OP == VBT_B200_U_SIGMOID) return 1.0f / (1.0f + expf(-a));
  else if constexpr (OP == VBT_B200_U_SILU) return a / (1.0f + expf(-a));
  else if constexpr (OP == VBT_B200_U_GELU) return 0.5f * a * (1.0f + erff(a * 0.70710678118654752440f));
  else if constexpr (OP == VBT_B200_U_RECIPROCAL) return 1.0f / a;
  else if constexpr (OP == VBT_B200_U_SIGN) return static_cast<float>((a > 0.f) - (a < 0.f));
  else if constexpr (OP == VBT_B200_U_FLOOR) return floorf(a);
  else if constexpr (OP == VBT_B200_U_CEIL) return ceilf(a);
  else if constexpr (OP == VBT_B200_U_TRUNC) return truncf(a);
  else if constexpr (OP == VBT_B200_U_ROUND) return nearbyintf(a);
  else if constexpr (OP == VBT_B200_U_EXPM1) return expm1f(a);
  else if constexpr (OP == VBT_B200_U_LOG1P) return log1pf(a);
  else if constexpr (OP == VBT_B200_U_SOFTPLUS) {
    if (a > 20.f) return a;
    if (a < -20.f) return expf(a);
    return log1pf(expf(a));
  } else if constexpr (OP == VBT_B200_U_RELU6) return a < 0.f ? 0.f : (a > 6.f ? 6.f : a);
  else if constexpr (OP == VBT_B200_U_HARDTANH) return a < -1.f ? -1.f : (a > 1.f ? 1.f : a);
  else return a;
}

// which unary ops accept INT64 (the rest reject integral inputs, :121-125)
constexpr bool unary_int_ok(int op) {
  return op == VBT_B200_U_RELU || op == VBT_B200_U_NEG || op == VBT_B200_U_ABS ||
         op == VBT_B200_U_SQUARE || op == VBT_B200_U_SIGN || op == VBT_B200_U_FLOOR ||
         op == VBT_B200_U_CEIL || op == VBT_B200_U_TRUNC || op == VBT_B200_U_ROUND;
}
template <int OP>
__device__ __forceinline__ int64_t unary_int(int64_t a) {
  const uint64_t ua = static_cast<uint64_t>(a);
  if constexpr (OP == VBT_B200_U_RELU) return a > 0 ? a : 0;
  else if constexpr (OP == VBT_B200_U_NEG) return static_cast<int64_t>(0ull - ua);
  else if constexpr (OP == VBT_B200_U_ABS) return a < 0 ? static_cast<int64_t>(0ull - ua) : a;
  else if constexpr (OP == VBT_B200_U_SQUARE) return static_cast<int64_t>(ua * ua);
  else if constexpr (OP == VBT_B200_U_SIGN) return (a > 0) - (a < 0);
  else return a;
}

template <int OP, class T>
struct UnaryF {
  static constexpr bool kFloatMath = is_float_storage<T>::value;
  __device__ __forceinline__ float fn(float a, float, float) const { return unary_math<OP>(a); }
  __device__ __forceinline__ T operator()(T a, T, T) const {
    if constexpr (is_float_storage<T>::value) return from_f<T>(unary_math<OP>(to_f(a)));
    else return static_cast<T>(unary_int<OP>(static_cast<int64_t>(a)));
  }
};

template <int OP>
__device__ __forceinline__ float binary_math(float a, float b) {
  if constexpr (OP == VBT_B200_B_ADD) return a + b;
  else if constexpr (OP == VBT_B200_B_SUB) return a - b;
  else if constexpr (OP == VBT_B200_B_MUL) return a * b;
  else if constexpr (OP == VBT_B200_B_DIV) return a / b;
  else if constexpr (OP == VBT_B200_B_MAXIMUM) return a != a ? a : (b != b ? b : fmaxf(a, b));
  else if constexpr (OP == VBT_B200_B_MINIMUM) return a != a ? a : (b != b ? b : fminf(a, b));
  else if constexpr (OP == VBT_B200_B_FMAX) return fmaxf(a, b);
  else return fminf(a, b);
}
template <int OP>
__device__ __forceinline__ int64_t binary_int(int64_t a, int64_t b) {
  const uint64_t ua = static_cast<uint64_t>(a), ub = static_cast<uint64_t>(b);
  if constexpr (OP == VBT_B200_B_ADD) return static_cast<int64_t>(ua + ub);
  else if constexpr (OP == VBT_B200_B_SUB) return static_cast<int64_t>(ua - ub);
  else if constexpr (OP == VBT_B200_B_MUL) return static_cast<int64_t>(ua * ub);
  else if constexpr (OP == VBT_B200_B_MAXIMUM || OP == VBT_B200_B_FMAX) return a > b ? a : b;
  else return a < b ? a : b;
}
template <int OP, class X>
__device__ __forceinline__ bool compare(X a, X b) {
  if constexpr (OP == VBT_B200_B_EQ) return a == b;
  else if constexpr (OP == VBT_B200_B_NE) return a != b;
  else if constexpr (OP == VBT_B200_B_LT) return a < b;
  else if constexpr (OP == VBT_B200_B_GT) return a > b;
  else if constexpr (OP == VBT_B200_B_LE) return a <= b;
  else return a >= b;
}

// Packed 16-bit arithmetic for add / sub / mul: one HADD2 / HMUL2 per two elements instead of
// widen-compute-round per element.  The result is the same bits as the float route: the
// float sum (product) of two 16-bit values is exact unless the exponents differ by more than
// the float significand allows, and in that case both routes return the larger operand, so a
// single rounding to 16 bits and "round to float, then to 16 bits" cannot disagree.
template <int OP>
__device__ __forceinline__ __nv_bfloat162 packed_math(__nv_bfloat162 a, __nv_bfloat162 b) {
  if constexpr (OP == VBT_B200_B_ADD) return __hadd2_rn(a, b);
  else if constexpr (OP == VBT_B200_B_SUB) return __hsub2_rn(a, b);
  else return __hmul2_rn(a, b);
}
template <int OP>
__device__ __forceinline__ __half2 packed_math(__half2 a, __half2 b) {
  if constexpr (OP == VBT_B200_B_ADD) return __hadd2_rn(a, b);
  else if constexpr (OP == VBT_B200_B_SUB) return __hsub2_rn(a, b);
  else return __hmul2_rn(a, b);
}
template <class T> struct Packed2 { using type = void; };
template <> struct Packed2<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Packed2<__half> { using type = __half2; };

template <int OP, class T>
struct BinaryF {
  static constexpr bool kFloatMath = is_float_storage<T>::value;
  static constexpr bool kPacked2 = sizeof(T) == 2 && is_float_storage<T>::value &&
                                   (OP == VBT_B200_B_ADD || OP == VBT_B200_B_SUB || OP == VBT_B200_B_MUL);
  __device__ __forceinline__ uint32_t pair(uint32_t a, uint32_t b) const {
    using P = typename Packed2<T>::type;
    if constexpr (kPacked2) {
      const P r = packed_math<OP>(*reinterpret_cast<const P*>(&a), *reinterpret_cast<const P*>(&b));
      return *reinterpret_cast<const uint32_t*>(&r);
    } else {
      return 0u;
    }
  }
  __device__ __forceinline__ float fn(float a, float b, float) const { return binary_math<OP>(a, b); }
  __device__ __forceinline__ T operator()(T a, T b, T) const {
    if constexpr (is_float_storage<T>::value) return from_f<T>(binary_math<OP>(to_f(a), to_f(b)));
    else return static_cast<T>(binary_int<OP>(a, b));
  }
};
template <int OP, class T>
struct CompareF {
  __device__ __forceinline__ uint8_t operator()(T a, T b, T) const {
    if constexpr (is_float_storage<T>::value) return compare<OP, float>(to_f(a), to_f(b));
    else return compare<OP, T>(a, b);
  }
};
// op(tensor, scalar) or op(scalar, tensor): the reference's CPU-scalar fast path
template <int OP, class T, bool CMP>
struct ScalarF {
  T s;
  bool left;
  __device__ __forceinline__ auto operator()(T a, T, T) const {
    const T x = left ? s : a, y = left ? a : s;
    if constexpr (CMP) return CompareF<OP, T>{}(x, y, T{});
    else return BinaryF<OP, T>{}(x, y, T{});
  }
};

// float in, float out; the caller rounds the result to T once.  Intermediates of the fused
// chains are rounded to T here, exactly where the reference's separate launches round.
template <int OP, class T>
struct TernaryF {
  static constexpr bool kFloatMath = true;
  __device__ __forceinline__ float fn(float a, float b, float c) const {
    if constexpr (OP == VBT_B200_T_CLAMP) {
      if (b != b || c != c) return __int_as_float(0x7fc00000);
      return a < b ? b : (a > c ? c : a);
    } else if constexpr (OP == VBT_B200_T_LERP) {
      return fmaf(c, b - a, a);
    } else if constexpr (OP == VBT_B200_T_THRESHOLD) {
      return a > b ? a : c;
    } else if constexpr (OP == VBT_B200_T_ADDCMUL) {
      return __fadd_rn(a, to_f(from_f<T>(__fmul_rn(b, c))));
    } else if constexpr (OP == VBT_B200_T_ADDCDIV) {
      return __fadd_rn(a, to_f(from_f<T>(__fdiv_rn(b, c))));
    } else if constexpr (OP == VBT_B200_T_HUBER_LOSS) {
      const float d = a - b, ad = fabsf(d);
      return ad < c ? 0.5f * d * d : c * (ad - 0.5f * c);
    } else if constexpr (OP == VBT_B200_T_SMOOTH_L1_LOSS) {
      const float d = a - b, ad = fabsf(d);
      return ad < c ? 0.5f * d * d / c : ad - 0.5f * c;
    } else {  // where(a > 0, a + b*c, 0): mul, add, gt, where of the reference, fused
      const float t2 = __fadd_rn(a, to_f(from_f<T>(__fmul_rn(b, c))));
      return a > 0.f ? t2 : 0.f;
    }
  }
  __device__ __forceinline__ T operator()(T ta, T tb, T tc) const {
    return from_f<T>(fn(to_f(ta), to_f(tb), to_f(tc)));
  }
  // Split form of the fused chains, fn(a, b, c) == fin(a, pre(b, c)): the kernel evaluates
  // pre once per thread when b and c do not change along the rows it walks.
  static constexpr bool kSplit = ternary_is_chain(OP);
  __device__ __forceinline__ float pre(float b, float c) const {
    if constexpr (OP == VBT_B200_T_ADDCDIV) return to_f(from_f<T>(__fdiv_rn(b, c)));
    else return to_f(from_f<T>(__fmul_rn(b, c)));
  }
  __device__ __forceinline__ float fin(float a, float t) const {
    const float r = __fadd_rn(a, t);
    if constexpr (OP == VBT_B200_T_WHERE_GT0_ADDCMUL) return a > 0.f ? r : 0.f;
    else return r;
  }
};

template <class T>
struct WhereF {
  __device__ __forceinline__ T operator()(uint8_t c, T x, T y) const { return c != 0 ? x : y; }
};
template <class T>
struct CopyF {
  __device__ __forceinline__ T operator()(T a, T, T) const { return a; }
};

// compile-time dispatch of a run-time op code
template <int OP, int COUNT, class Fn>
inline bool dispatch_op(int op, Fn&& fn) {
  if constexpr (OP < COUNT) {
    if (op == OP) {
      fn(std::integral_constant<int, OP>{});
      return true;
    }
    return dispatch_op<OP + 1, COUNT>(op, fn);
  } else {
    return false;
  }
}

}  // namespace vb
