// Functors of the long tail of the reference's elementwise table
// (src/vbt/ops/cuda_elementwise.cu:191-589 binary, :808-1252 unary, :1279-1287 logit,
// :1556-1572 nan_to_num).  Same conventions as ew_functors.cuh: 16-bit floats are widened to
// float, computed, rounded once; functors the reference writes in device fp64 (frac, sinc,
// deg2rad, mish, selu, hardsigmoid, the *_backward forms, ...) are fp32 here.
#pragma once
#include <cfloat>
#include <climits>

#include "ew_functors.cuh"

namespace vb {

constexpr bool unary_is_predicate(int op) {
  return op >= VBT_B200_U_ISFINITE && op <= VBT_B200_U_LOGICAL_NOT;
}
constexpr bool unary_ext_int_ok(int op) { return op == VBT_B200_U_POSITIVE || op == VBT_B200_U_SGN; }

template <int OP>
__device__ __forceinline__ float unary_ext_math(float a) {
  if constexpr (OP == VBT_B200_U_EXP2) return exp2f(a);
  else if constexpr (OP == VBT_B200_U_LOG2) return log2f(a);
  else if constexpr (OP == VBT_B200_U_LOG10) return log10f(a);
  else if constexpr (OP == VBT_B200_U_SINH) return sinhf(a);
  else if constexpr (OP == VBT_B200_U_COSH) return coshf(a);
  else if constexpr (OP == VBT_B200_U_ASINH) return asinhf(a);
  else if constexpr (OP == VBT_B200_U_ACOSH) return acoshf(a);
  else if constexpr (OP == VBT_B200_U_ATANH) return atanhf(a);
  else if constexpr (OP == VBT_B200_U_TAN) return tanf(a);
  else if constexpr (OP == VBT_B200_U_ASIN) return asinf(a);
  else if constexpr (OP == VBT_B200_U_ACOS) return acosf(a);
  else if constexpr (OP == VBT_B200_U_ATAN) return atanf(a);
  else if constexpr (OP == VBT_B200_U_ERF) return erff(a);
  else if constexpr (OP == VBT_B200_U_ERFC) return erfcf(a);
  else if constexpr (OP == VBT_B200_U_LGAMMA) return lgammaf(a);
  else if constexpr (OP == VBT_B200_U_SINC) {
    // sinpif reduces the argument exactly, so large |a| keeps the accuracy of the fp64 form
    return a == 0.f ? 1.f : sinpif(a) / (3.14159265358979323846f * a);
  } else if constexpr (OP == VBT_B200_U_FRAC) {
    float ip;
    return modff(a, &ip);
  } else if constexpr (OP == VBT_B200_U_DEG2RAD) return a * 0.017453292519943295f;
  else if constexpr (OP == VBT_B200_U_RAD2DEG) return a * 57.29577951308232f;
  else if constexpr (OP == VBT_B200_U_MISH) {
    const float sp = a > 20.f ? a : log1pf(expf(a));
    return a * tanhf(sp);
  } else if constexpr (OP == VBT_B200_U_SELU) {
    const float y = a > 0.f ? a : 1.6732632423543772f * expm1f(a);
    return 1.0507009873554805f * y;
  } else if constexpr (OP == VBT_B200_U_ELU) return a > 0.f ? a : expm1f(a);
  else if constexpr (OP == VBT_B200_U_HARDSIGMOID) {
    const float y = a / 6.0f + 0.5f;
    return y < 0.f ? 0.f : (y > 1.f ? 1.f : y);
  } else if constexpr (OP == VBT_B200_U_HARDSHRINK) return (a > 0.5f || a < -0.5f) ? a : 0.f;
  else if constexpr (OP == VBT_B200_U_SOFTSHRINK) return a > 0.5f ? a - 0.5f : (a < -0.5f ? a + 0.5f : 0.f);
  else if constexpr (OP == VBT_B200_U_LOGIT) return logf(a / (1.0f - a));
  else if constexpr (OP == VBT_B200_U_ANGLE) {
    if (a != a) return a;
    return a < 0.f ? 3.14159265358979323846f : 0.f;
  } else if constexpr (OP == VBT_B200_U_SGN) return a != a ? 0.f : static_cast<float>((a > 0.f) - (a < 0.f));
  else if constexpr (OP == VBT_B200_U_NAN_TO_NUM) {
    if (a != a) return 0.f;
    if (isinf(a)) return a > 0.f ? FLT_MAX : -FLT_MAX;
    return a;
  } else return a;  // POSITIVE
}

template <int OP, class T>
struct UnaryExtF {
  static constexpr bool kFloatMath = is_float_storage<T>::value;
  __device__ __forceinline__ float fn(float a, float, float) const { return unary_ext_math<OP>(a); }
  __device__ __forceinline__ T operator()(T a, T, T) const {
    if constexpr (is_float_storage<T>::value) return from_f<T>(unary_ext_math<OP>(to_f(a)));
    else if constexpr (OP == VBT_B200_U_SGN) return static_cast<T>((a > 0) - (a < 0));
    else return a;
  }
};

// value -> BOOL byte.  T: a float storage type, int64_t, or uint8_t (BOOL).
template <int OP, class T>
struct PredicateF {
  __device__ __forceinline__ uint8_t operator()(T a, T, T) const {
    if constexpr (is_float_storage<T>::value) {
      const float x = to_f(a);
      if constexpr (OP == VBT_B200_U_ISFINITE) return isfinite(x);
      else if constexpr (OP == VBT_B200_U_ISINF) return isinf(x);
      else if constexpr (OP == VBT_B200_U_ISNAN) return x != x;
      else if constexpr (OP == VBT_B200_U_ISNEGINF) return isinf(x) && x < 0.f;
      else if constexpr (OP == VBT_B200_U_ISPOSINF) return isinf(x) && x > 0.f;
      else if constexpr (OP == VBT_B200_U_SIGNBIT) return (__float_as_uint(x) >> 31) != 0u;
      else return !(x != 0.f);  // LOGICAL_NOT; NaN is truthy
    } else {
      if constexpr (OP == VBT_B200_U_ISFINITE) return 1;
      else if constexpr (OP == VBT_B200_U_SIGNBIT) return std::is_signed_v<T> ? a < 0 : 0;
      else if constexpr (OP == VBT_B200_U_LOGICAL_NOT) return a == 0;
      else return 0;
    }
  }
};

template <class T>
struct IntBinaryNotF {
  __device__ __forceinline__ T operator()(T a, T, T) const { return ~a; }
};

// ---------------------------------------------------------------------------- binary
constexpr bool binary_ext_is_float_op(int op) { return op >= VBT_B200_B_POW && op <= VBT_B200_B_LDEXP; }
constexpr bool binary_ext_int_ok(int op) {  // float ops that also take INT64
  return op == VBT_B200_B_FMOD || op == VBT_B200_B_REMAINDER || op == VBT_B200_B_HEAVISIDE ||
         op == VBT_B200_B_RSUB;
}
constexpr bool binary_is_intop(int op) { return op >= VBT_B200_B_BITWISE_AND && op <= VBT_B200_B_LCM; }
constexpr bool binary_is_logical(int op) { return op >= VBT_B200_B_LOGICAL_AND && op <= VBT_B200_B_LOGICAL_XOR; }

template <int OP>
__device__ __forceinline__ float binary_ext_math(float a, float b) {
  if constexpr (OP == VBT_B200_B_POW) return powf(a, b);
  else if constexpr (OP == VBT_B200_B_FMOD) return fmodf(a, b);
  else if constexpr (OP == VBT_B200_B_REMAINDER) {
    float r = fmodf(a, b);
    if (r != 0.f && ((r < 0.f) != (b < 0.f))) r += b;
    return r;
  } else if constexpr (OP == VBT_B200_B_ATAN2) return atan2f(a, b);
  else if constexpr (OP == VBT_B200_B_COPYSIGN) return copysignf(a, b);
  else if constexpr (OP == VBT_B200_B_HYPOT) return hypotf(a, b);
  else if constexpr (OP == VBT_B200_B_XLOGY) return a == 0.f ? 0.f : a * logf(b);
  else if constexpr (OP == VBT_B200_B_XLOG1PY) return a == 0.f ? 0.f : a * log1pf(b);
  else if constexpr (OP == VBT_B200_B_LOGADDEXP) {
    const float m = a > b ? a : b;
    if (isinf(m)) return m;
    return m + log1pf(expf(-fabsf(a - b)));
  } else if constexpr (OP == VBT_B200_B_LOGADDEXP2) {
    const float m = a > b ? a : b;
    if (isinf(m)) return m;
    return m + log2f(1.0f + exp2f(-fabsf(a - b)));
  } else if constexpr (OP == VBT_B200_B_NEXTAFTER) return nextafterf(a, b);
  else if constexpr (OP == VBT_B200_B_HEAVISIDE) return a < 0.f ? 0.f : (a > 0.f ? 1.f : b);
  else if constexpr (OP == VBT_B200_B_RSUB) return b - a;
  else if constexpr (OP == VBT_B200_B_TANH_BACKWARD) return a * (1.0f - b * b);
  else if constexpr (OP == VBT_B200_B_SIGMOID_BACKWARD) return a * b * (1.0f - b);
  else if constexpr (OP == VBT_B200_B_SILU_BACKWARD) {
    const float s = 1.0f / (1.0f + expf(-b));
    return a * (s * (1.0f + b * (1.0f - s)));
  } else if constexpr (OP == VBT_B200_B_LOGIT_BACKWARD) return a / (b * (1.0f - b));
  else if constexpr (OP == VBT_B200_B_MSE_LOSS) {
    const float d = a - b;
    return d * d;
  } else {  // LDEXP
    int e;
    if (b != b) e = 0;
    else if (b >= 2147483648.0f) e = INT_MAX;  // float(INT_MAX) is 2^31; the device cast saturates there
    else if (b < -2147483648.0f) e = INT_MIN;
    else e = static_cast<int>(b);
    return ldexpf(a, e);
  }
}

template <int OP>
__device__ __forceinline__ int64_t binary_ext_i64(int64_t a, int64_t b) {
  if constexpr (OP == VBT_B200_B_FMOD || OP == VBT_B200_B_REMAINDER) {
    if (b == 0) return 0;
    if (a == INT64_MIN && b == -1) return 0;
    int64_t r = a % b;
    if constexpr (OP == VBT_B200_B_REMAINDER)
      if (r != 0 && ((r < 0) != (b < 0))) r += b;
    return r;
  } else if constexpr (OP == VBT_B200_B_HEAVISIDE) {
    return a < 0 ? 0 : (a > 0 ? 1 : b);
  } else {  // RSUB
    return static_cast<int64_t>(static_cast<uint64_t>(b) - static_cast<uint64_t>(a));
  }
}

template <int OP, class T>
struct BinaryExtF {
  static constexpr bool kFloatMath = is_float_storage<T>::value;
  __device__ __forceinline__ float fn(float a, float b, float) const { return binary_ext_math<OP>(a, b); }
  __device__ __forceinline__ T operator()(T a, T b, T) const {
    if constexpr (is_float_storage<T>::value) return from_f<T>(binary_ext_math<OP>(to_f(a), to_f(b)));
    else return static_cast<T>(binary_ext_i64<OP>(a, b));
  }
};
template <int OP, class T>
struct ScalarExtF {
  T s;
  bool left;
  __device__ __forceinline__ T operator()(T a, T, T) const {
    return BinaryExtF<OP, T>{}(left ? s : a, left ? a : s, T{});
  }
};

// T: int64_t, int32_t, or uint8_t holding a BOOL (and/or/xor only; normalised to 0/1)
template <int OP, class T>
struct IntBinaryF {
  __device__ __forceinline__ T operator()(T a, T b, T) const {
    using U = std::make_unsigned_t<T>;
    constexpr int bits = static_cast<int>(sizeof(T) * 8);
    if constexpr (std::is_same_v<T, uint8_t>) {
      const bool x = a != 0, y = b != 0;
      if constexpr (OP == VBT_B200_B_BITWISE_AND) return x && y;
      else if constexpr (OP == VBT_B200_B_BITWISE_OR) return x || y;
      else return x != y;
    } else if constexpr (OP == VBT_B200_B_BITWISE_AND) return a & b;
    else if constexpr (OP == VBT_B200_B_BITWISE_OR) return a | b;
    else if constexpr (OP == VBT_B200_B_BITWISE_XOR) return a ^ b;
    else if constexpr (OP == VBT_B200_B_LSHIFT) {
      if (b < 0 || b >= bits) return 0;
      return static_cast<T>(static_cast<U>(a) << static_cast<int>(b));
    } else if constexpr (OP == VBT_B200_B_RSHIFT) {
      if (b < 0 || b >= bits) return a < 0 ? T(-1) : T(0);
      return a >> static_cast<int>(b);  // arithmetic shift: sign-fills, as the reference's fill mask
    } else {
      U ua = a < 0 ? U(0) - static_cast<U>(a) : static_cast<U>(a);
      U ub = b < 0 ? U(0) - static_cast<U>(b) : static_cast<U>(b);
      if constexpr (OP == VBT_B200_B_LCM)
        if (a == 0 || b == 0) return 0;
      U x = ua, y = ub;
      while (y != 0) {
        const U t = y;
        y = x % y;
        x = t;
      }
      if constexpr (OP == VBT_B200_B_GCD) return static_cast<T>(x);
      else return static_cast<T>((ua / x) * ub);
    }
  }
};
template <int OP, class T>
struct LogicalF {
  __device__ __forceinline__ uint8_t operator()(T a, T b, T) const {
    bool x, y;
    if constexpr (is_float_storage<T>::value) {
      x = to_f(a) != 0.f;
      y = to_f(b) != 0.f;
    } else {
      x = a != 0;
      y = b != 0;
    }
    if constexpr (OP == VBT_B200_B_LOGICAL_AND) return x && y;
    else if constexpr (OP == VBT_B200_B_LOGICAL_OR) return x || y;
    else return x != y;
  }
};

}  // namespace vb
