/*
 * TEST INFRASTRUCTURE ONLY -- the CPU oracle.  A plain-C, single-threaded restatement of
 * what VibeTensor's own implementation computes for the vt:: data-parallel op path, used
 * by tests/, the smoke check and the bench's CPU-baseline leg as the checker.  The product
 * (libvbt_b200.so and the vibetensor_b200 package) never links, loads or calls it.
 *
 * Parity of this restatement is pinned two ways (tests/test_oracle_*.py): against the
 * golden vectors of the reference's own unit tests, and against the reference's real CPU
 * code compiled from its sources (oracle/_ref/libvbt_ref_cpu.so, see build_ref.sh) on
 * seeded random inputs.  Paths with no CPU code in the reference (bf16/f16 elementwise,
 * where, softmax, RMSNorm) follow its CUDA functors / Triton kernels and are checked
 * against torch CPU with the reference tests' own tolerances.
 *
 * Citations are path:line in the NVlabs/vibetensor tree.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { DT_BOOL = 0, DT_I32 = 1, DT_I64 = 2, DT_F32 = 3, DT_F16 = 4, DT_BF16 = 5 };

static int itemsize(int dt) {
  switch (dt) {
    case DT_BOOL: return 1;
    case DT_I32: return 4;
    case DT_I64: return 8;
    case DT_F32: return 4;
    case DT_F16: return 2;
    case DT_BF16: return 2;
  }
  return 0;
}

/* ---- storage <-> float, as src/vbt/ops/cuda_elementwise.cu:135-140: widen to float,
 * compute, store with round-to-nearest-even (__float2bfloat16_rn / __float2half_rn). ---- */
static float bf16_to_f(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint16_t f_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN, canonical as the intrinsic */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float f16_to_f(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}
static uint16_t f_to_f16(float f) {
  _Float16 x = (_Float16)f;
  uint16_t h;
  memcpy(&h, &x, 2);
  if (f != f) h = 0x7fff;
  return h;
}
static float load_f(const void* p, int dt) {
  switch (dt) {
    case DT_F32: return *(const float*)p;
    case DT_F16: return f16_to_f(*(const uint16_t*)p);
    case DT_BF16: return bf16_to_f(*(const uint16_t*)p);
  }
  return 0.f;
}
static void store_f(void* p, int dt, float v) {
  switch (dt) {
    case DT_F32: *(float*)p = v; break;
    case DT_F16: *(uint16_t*)p = f_to_f16(v); break;
    case DT_BF16: *(uint16_t*)p = f_to_bf16(v); break;
  }
}
/* value after one store+load round trip: the per-op rounding of a chained expression */
static float round_to(int dt, float v) {
  if (dt == DT_F32) return v;
  if (dt == DT_F16) return f16_to_f(f_to_f16(v));
  return bf16_to_f(f_to_bf16(v));
}

/* ---- op codes: must match include/vbt_b200.h ---- */
enum {
  U_RELU, U_NEG, U_ABS, U_SQUARE, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_SIN, U_COS, U_TANH,
  U_SIGMOID, U_SILU, U_GELU, U_RECIPROCAL, U_SIGN, U_FLOOR, U_CEIL, U_TRUNC, U_ROUND,
  U_EXPM1, U_LOG1P, U_SOFTPLUS, U_RELU6, U_HARDTANH,
  U_EXP2, U_LOG2, U_LOG10, U_SINH, U_COSH, U_ASINH, U_ACOSH, U_ATANH, U_TAN, U_ASIN, U_ACOS,
  U_ATAN, U_ERF, U_ERFC, U_LGAMMA, U_SINC, U_FRAC, U_DEG2RAD, U_RAD2DEG, U_MISH, U_SELU, U_ELU,
  U_HARDSIGMOID, U_HARDSHRINK, U_SOFTSHRINK, U_LOGIT, U_ANGLE, U_POSITIVE, U_SGN, U_NAN_TO_NUM,
  U_ISFINITE, U_ISINF, U_ISNAN, U_ISNEGINF, U_ISPOSINF, U_SIGNBIT, U_LOGICAL_NOT, U_BITWISE_NOT,
  U_COUNT
};
enum {
  B_ADD, B_SUB, B_MUL, B_DIV, B_MAXIMUM, B_MINIMUM, B_FMAX, B_FMIN,
  B_EQ, B_NE, B_LT, B_GT, B_LE, B_GE,
  B_POW, B_FMOD, B_REMAINDER, B_ATAN2, B_COPYSIGN, B_HYPOT, B_XLOGY, B_XLOG1PY, B_LOGADDEXP,
  B_LOGADDEXP2, B_NEXTAFTER, B_HEAVISIDE, B_RSUB, B_TANH_BACKWARD, B_SIGMOID_BACKWARD,
  B_SILU_BACKWARD, B_LOGIT_BACKWARD, B_MSE_LOSS, B_LDEXP,
  B_BITWISE_AND, B_BITWISE_OR, B_BITWISE_XOR, B_LSHIFT, B_RSHIFT, B_GCD, B_LCM,
  B_LOGICAL_AND, B_LOGICAL_OR, B_LOGICAL_XOR, B_COUNT
};
enum { T_CLAMP, T_LERP, T_THRESHOLD, T_ADDCMUL, T_ADDCDIV, T_WHERE_GT0_ADDCMUL, T_HUBER_LOSS,
       T_SMOOTH_L1_LOSS, T_COUNT };

/* Functors on float: src/vbt/ops/cuda_elementwise.cu:590-900, :1622-1630.  Several are
 * written in double there (Silu, Gelu, Reciprocal, Sign, Softplus, Relu6, Hardtanh). */
static float unary_f(int op, float a) {
  switch (op) {
    case U_RELU: return a > 0.f ? a : 0.f;
    case U_NEG: return -a;
    case U_ABS: return fabsf(a);
    case U_SQUARE: return a * a;
    case U_EXP: return expf(a);
    case U_LOG: return logf(a);
    case U_SQRT: return sqrtf(a);
    case U_RSQRT: return (float)(1.0 / sqrt((double)a));
    case U_SIN: return sinf(a);
    case U_COS: return cosf(a);
    case U_TANH: return tanhf(a);
    case U_SIGMOID: return 1.0f / (1.0f + expf(-a));
    case U_SILU: { double x = a; return (float)(x * (1.0 / (1.0 + exp(-x)))); }
    case U_GELU: { double x = a; return (float)(0.5 * x * (1.0 + erf(x * 0.70710678118654752440))); }
    case U_RECIPROCAL: return (float)(1.0 / (double)a);
    case U_SIGN: { double x = a; return (float)((x > 0) - (x < 0)); }
    case U_FLOOR: return floorf(a);
    case U_CEIL: return ceilf(a);
    case U_TRUNC: return truncf(a);
    case U_ROUND: return nearbyintf(a);
    case U_EXPM1: return expm1f(a);
    case U_LOG1P: return log1pf(a);
    case U_SOFTPLUS: {
      double x = a;
      if (x > 20.0) return (float)x;
      if (x < -20.0) return (float)exp(x);
      return (float)log1p(exp(x));
    }
    case U_RELU6: { double x = a; if (x < 0.0) x = 0.0; if (x > 6.0) x = 6.0; return (float)x; }
    case U_HARDTANH: { double x = a; if (x < -1.0) x = -1.0; if (x > 1.0) x = 1.0; return (float)x; }
    /* :1151-1252: float math for T = float */
    case U_EXP2: return exp2f(a);
    case U_LOG2: return log2f(a);
    case U_LOG10: return log10f(a);
    case U_SINH: return sinhf(a);
    case U_COSH: return coshf(a);
    case U_ASINH: return asinhf(a);
    case U_ACOSH: return acoshf(a);
    case U_ATANH: return atanhf(a);
    case U_TAN: return tanf(a);
    case U_ASIN: return asinf(a);
    case U_ACOS: return acosf(a);
    case U_ATAN: return atanf(a);
    case U_ERF: return erff(a);
    case U_ERFC: return erfcf(a);
    case U_LGAMMA: return lgammaf(a);
    /* :808-850, :901-948: written in double */
    case U_SINC: { double x = a; if (x == 0.0) return 1.f; double pix = 3.14159265358979323846 * x; return (float)(sin(pix) / pix); }
    case U_FRAC: { double ip; return (float)modf((double)a, &ip); }
    case U_DEG2RAD: return (float)((double)a * (3.14159265358979323846 / 180.0));
    case U_RAD2DEG: return (float)((double)a * (180.0 / 3.14159265358979323846));
    case U_MISH: { double x = a; double sp = x > 20.0 ? x : log1p(exp(x)); return (float)(x * tanh(sp)); }
    case U_SELU: {
      double x = a;
      double y = x > 0.0 ? x : 1.6732632423543772848170429916717 * expm1(x);
      return (float)(1.0507009873554804934193349852946 * y);
    }
    case U_ELU: { double x = a; return (float)(x > 0.0 ? x : expm1(x)); }
    case U_HARDSIGMOID: { double y = (double)a / 6.0 + 0.5; if (y < 0.0) y = 0.0; if (y > 1.0) y = 1.0; return (float)y; }
    case U_HARDSHRINK: { double x = a; return (x > 0.5 || x < -0.5) ? (float)x : 0.f; }
    case U_SOFTSHRINK: { double x = a; if (x > 0.5) return (float)(x - 0.5); if (x < -0.5) return (float)(x + 0.5); return 0.f; }
    case U_LOGIT: return logf(a / (1.0f - a)); /* :1279-1287 */
    case U_ANGLE: { double x = a; if (x != x) return a; if (x == 0.0) return 0.f; return (float)(x < 0.0 ? 3.14159265358979323846 : 0.0); }
    case U_POSITIVE: return a;
    case U_SGN: { double x = a; if (x != x) return 0.f; return (float)((x > 0) - (x < 0)); }
    case U_NAN_TO_NUM: /* :1556-1572 */
      if (a != a) return 0.f;
      if (isinf(a)) return a > 0.f ? 3.402823466e+38F : -3.402823466e+38F;
      return a;
  }
  return 0.f;
}
/* Predicates -> bool: :1043-1149 */
static int pred_f(int op, float x) {
  switch (op) {
    case U_ISFINITE: return isfinite(x) != 0;
    case U_ISINF: return isinf(x) != 0;
    case U_ISNAN: return x != x;
    case U_ISNEGINF: return isinf(x) && x < 0.f;
    case U_ISPOSINF: return isinf(x) && x > 0.f;
    case U_SIGNBIT: return signbit(x) != 0;
    case U_LOGICAL_NOT: return !(x != 0.f);
  }
  return 0;
}
static int pred_i(int op, int64_t a, int is_signed) {
  switch (op) {
    case U_ISFINITE: return 1;
    case U_SIGNBIT: return is_signed ? a < 0 : 0;
    case U_LOGICAL_NOT: return a == 0;
  }
  return 0;
}
static int64_t unary_i64(int op, int64_t a, int* ok) {
  uint64_t ua = (uint64_t)a;
  switch (op) {
    case U_RELU: return a > 0 ? a : 0;
    case U_NEG: return (int64_t)(0u - ua);
    case U_ABS: return a < 0 ? (int64_t)(0u - ua) : a;
    case U_SQUARE: return (int64_t)(ua * ua);
    case U_SIGN: return (a > 0) - (a < 0);
    case U_FLOOR: case U_CEIL: case U_TRUNC: case U_ROUND: case U_POSITIVE: return a;
    case U_SGN: return (a > 0) - (a < 0);
  }
  *ok = 0; /* transcendental ops reject integral inputs (:121-125) */
  return 0;
}
static float binary_f(int op, float a, float b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_MAXIMUM: if (a != a) return a; if (b != b) return b; return fmaxf(a, b);
    case B_MINIMUM: if (a != a) return a; if (b != b) return b; return fminf(a, b);
    case B_FMAX: return fmaxf(a, b);
    case B_FMIN: return fminf(a, b);
    /* :307-589 (float branches), :851-876 and the backward forms in double, :1253-1258 */
    case B_POW: return powf(a, b);
    case B_FMOD: return fmodf(a, b);
    case B_REMAINDER: { float r = fmodf(a, b); if (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) r += b; return r; }
    case B_ATAN2: return atan2f(a, b);
    case B_COPYSIGN: return copysignf(a, b);
    case B_HYPOT: return hypotf(a, b);
    case B_XLOGY: return a == 0.f ? 0.f : a * logf(b);
    case B_XLOG1PY: return a == 0.f ? 0.f : a * log1pf(b);
    case B_LOGADDEXP: { float m = a > b ? a : b; if (isinf(m)) return m; return m + log1pf(expf(-fabsf(a - b))); }
    case B_LOGADDEXP2: { float m = a > b ? a : b; if (isinf(m)) return m; return m + log2f(1.0f + exp2f(-fabsf(a - b))); }
    case B_NEXTAFTER: return nextafterf(a, b);
    case B_HEAVISIDE: if (a < 0.f) return 0.f; if (a > 0.f) return 1.f; return b;
    case B_RSUB: return b - a;
    case B_TANH_BACKWARD: { double g = a, o = b; return (float)(g * (1.0 - o * o)); }
    case B_SIGMOID_BACKWARD: { double g = a, o = b; return (float)(g * o * (1.0 - o)); }
    case B_SILU_BACKWARD: { double g = a, x = b; double s = 1.0 / (1.0 + exp(-x)); return (float)(g * (s * (1.0 + x * (1.0 - s)))); }
    case B_LOGIT_BACKWARD: { double g = a, x = b; return (float)(g / (x * (1.0 - x))); }
    case B_MSE_LOSS: { float d = a - b; return d * d; }
    case B_LDEXP: { /* :463-478; the device cast of 2^31 saturates to INT_MAX */
      int e;
      if (b != b) e = 0;
      else if (b >= 2147483648.0f) e = 2147483647;
      else if (b < -2147483648.0f) e = -2147483647 - 1;
      else e = (int)b;
      return ldexpf(a, e);
    }
  }
  return 0.f;
}
static int compare_f(int op, float a, float b) {
  switch (op) {
    case B_EQ: return a == b;
    case B_NE: return a != b;
    case B_LT: return a < b;
    case B_GT: return a > b;
    case B_LE: return a <= b;
    case B_GE: return a >= b;
  }
  return 0;
}
static int64_t binary_i64(int op, int64_t a, int64_t b) {
  switch (op) {
    case B_ADD: return (int64_t)((uint64_t)a + (uint64_t)b);
    case B_SUB: return (int64_t)((uint64_t)a - (uint64_t)b);
    case B_MUL: return (int64_t)((uint64_t)a * (uint64_t)b);
    case B_MAXIMUM: case B_FMAX: return a > b ? a : b;
    case B_MINIMUM: case B_FMIN: return a < b ? a : b;
    case B_FMOD: case B_REMAINDER: { /* :322-330, :355-366 */
      if (b == 0) return 0;
      if (a == INT64_MIN && b == -1) return 0;
      int64_t r = a % b;
      if (op == B_REMAINDER && r != 0 && ((r < 0) != (b < 0))) r += b;
      return r;
    }
    case B_HEAVISIDE: if (a < 0) return 0; if (a > 0) return 1; return b;
    case B_RSUB: return (int64_t)((uint64_t)b - (uint64_t)a);
  }
  return 0;
}
/* bitwise / shift / gcd / lcm on a `bits`-wide signed integer held in int64 (:191-243,
 * :537-588); bits == 1 is BOOL (and/or/xor only). */
static int64_t intop(int op, int64_t a, int64_t b, int bits) {
  if (bits == 1) {
    int x = a != 0, y = b != 0;
    return op == B_BITWISE_AND ? (x && y) : op == B_BITWISE_OR ? (x || y) : (x != y);
  }
  switch (op) {
    case B_BITWISE_AND: return a & b;
    case B_BITWISE_OR: return a | b;
    case B_BITWISE_XOR: return a ^ b;
    case B_LSHIFT: {
      if (b < 0 || b >= bits) return 0;
      uint64_t r = (uint64_t)a << (int)b;
      return bits == 32 ? (int64_t)(int32_t)(uint32_t)r : (int64_t)r;
    }
    case B_RSHIFT: {
      if (b < 0 || b >= bits) return a < 0 ? -1 : 0;
      /* logical shift of the two's-complement pattern, then sign fill */
      uint64_t ua = bits == 32 ? (uint64_t)(uint32_t)(int32_t)a : (uint64_t)a;
      uint64_t r = ua >> (int)b;
      if (a < 0 && b > 0) {
        uint64_t all = bits == 32 ? 0xffffffffull : ~0ull;
        r |= (all << (bits - (int)b)) & all;
      }
      return bits == 32 ? (int64_t)(int32_t)(uint32_t)r : (int64_t)r;
    }
    case B_GCD: case B_LCM: {
      uint64_t ua = a < 0 ? 0ull - (uint64_t)a : (uint64_t)a;
      uint64_t ub = b < 0 ? 0ull - (uint64_t)b : (uint64_t)b;
      if (op == B_LCM && (a == 0 || b == 0)) return 0;
      uint64_t x = ua, y = ub;
      while (y != 0) { uint64_t t = y; y = x % y; x = t; }
      return op == B_GCD ? (int64_t)x : (int64_t)((ua / x) * ub);
    }
  }
  return 0;
}
static int logical(int op, int x, int y) {
  return op == B_LOGICAL_AND ? (x && y) : op == B_LOGICAL_OR ? (x || y) : (x != y);
}
static int compare_i64(int op, int64_t a, int64_t b) {
  switch (op) {
    case B_EQ: return a == b;
    case B_NE: return a != b;
    case B_LT: return a < b;
    case B_GT: return a > b;
    case B_LE: return a <= b;
    case B_GE: return a >= b;
  }
  return 0;
}
static float ternary_f(int op, int dt, float a, float b, float c) {
  switch (op) {
    case T_CLAMP: /* (v, mn, mx) :1259-1266 */
      if (b != b || c != c) return NAN;
      return a < b ? b : (a > c ? c : a);
    case T_LERP: return fmaf(c, b - a, a); /* start + weight*(end-start), contracted on device */
    case T_THRESHOLD: return a > b ? a : c;
    case T_ADDCMUL: return a + round_to(dt, b * c);        /* mul, then add (:3927-3931) */
    case T_ADDCDIV: return a + round_to(dt, b / c);
    case T_WHERE_GT0_ADDCMUL: {
      float t2 = round_to(dt, a + round_to(dt, b * c));
      return a > 0.f ? t2 : 0.f;
    }
    case T_HUBER_LOSS: { /* (input, target, delta) :1385-1395 */
      float d = a - b, ad = fabsf(d);
      return ad < c ? 0.5f * d * d : c * (ad - 0.5f * c);
    }
    case T_SMOOTH_L1_LOSS: { /* (input, target, beta) :1397-1407 */
      float d = a - b, ad = fabsf(d);
      return ad < c ? 0.5f * d * d / c : ad - 0.5f * c;
    }
  }
  return 0.f;
}

/* Generic N-d strided iteration in row-major order of `sizes`; strides in elements. */
#define MAXD 32
typedef struct {
  int ndim;
  int64_t sizes[MAXD];
  int64_t idx[MAXD];
} odo_t;
static int64_t numel_of(int ndim, const int64_t* sizes) {
  int64_t n = 1;
  for (int i = 0; i < ndim; ++i) n *= sizes[i];
  return n;
}
static void odo_init(odo_t* o, int ndim, const int64_t* sizes) {
  o->ndim = ndim;
  for (int i = 0; i < ndim; ++i) { o->sizes[i] = sizes[i]; o->idx[i] = 0; }
}
static void odo_next(odo_t* o) {
  for (int d = o->ndim - 1; d >= 0; --d) {
    if (++o->idx[d] < o->sizes[d]) return;
    o->idx[d] = 0;
  }
}
static int64_t odo_off(const odo_t* o, const int64_t* strides) {
  int64_t off = 0;
  for (int d = 0; d < o->ndim; ++d) off += o->idx[d] * strides[d];
  return off;
}

/* out = op(a [, b [, c]]).  nin = 1,2,3.  kind: 0 unary, 1 binary, 2 ternary, 3 where
 * (a = BOOL cond, b = x, c = y), 4 copy.  Comparison binaries write BOOL bytes. */
int vbo_elementwise(int kind, int op, int dtype, int ndim, const int64_t* sizes, void* out,
                    const int64_t* os, const void* a, const int64_t* as, const void* b,
                    const int64_t* bs, const void* c, const int64_t* cs) {
  if (ndim > MAXD) return 1;
  const int64_t n = numel_of(ndim, sizes);
  const int es = itemsize(dtype);
  const int is_cmp = (kind == 1 && op >= B_EQ && op <= B_GE);
  const int is_logical = (kind == 1 && op >= B_LOGICAL_AND && op <= B_LOGICAL_XOR);
  const int is_intop = (kind == 1 && op >= B_BITWISE_AND && op <= B_LCM);
  const int is_pred = (kind == 0 && op >= U_ISFINITE && op <= U_LOGICAL_NOT);
  const int oes = (is_cmp || is_logical || is_pred) ? 1 : es;
  odo_t o;
  odo_init(&o, ndim, sizes);
  for (int64_t i = 0; i < n; ++i, odo_next(&o)) {
    char* po = (char*)out + odo_off(&o, os) * oes;
    if (kind == 3) { /* where_ti_strided_kernel :2645-2662 */
      const uint8_t cond = *((const uint8_t*)a + odo_off(&o, as));
      const char* px = (const char*)b + odo_off(&o, bs) * es;
      const char* py = (const char*)c + odo_off(&o, cs) * es;
      memcpy(po, cond != 0 ? px : py, es);
      continue;
    }
    const char* pa = (const char*)a + odo_off(&o, as) * es;
    if (kind == 4) { memcpy(po, pa, es); continue; }
    const char* pb = b ? (const char*)b + odo_off(&o, bs) * es : 0;
    const char* pc = c ? (const char*)c + odo_off(&o, cs) * es : 0;
    if (is_intop || (kind == 0 && op == U_BITWISE_NOT)) {
      const int bits = dtype == DT_I64 ? 64 : dtype == DT_I32 ? 32 : dtype == DT_BOOL ? 1 : 0;
      if (bits == 0) return 1;
      if (bits == 1 && (op == B_LSHIFT || op == B_RSHIFT)) return 1;
      if (bits != 64 && (op == B_GCD || op == B_LCM) && kind == 1) return 1;
      int64_t av = bits == 64 ? *(const int64_t*)pa : bits == 32 ? *(const int32_t*)pa : *(const uint8_t*)pa;
      int64_t r;
      if (kind == 0) r = bits == 1 ? (av == 0) : ~av;
      else {
        int64_t bv = bits == 64 ? *(const int64_t*)pb : bits == 32 ? *(const int32_t*)pb : *(const uint8_t*)pb;
        r = intop(op, av, bv, bits);
      }
      if (bits == 64) *(int64_t*)po = r;
      else if (bits == 32) *(int32_t*)po = (int32_t)r;
      else *(uint8_t*)po = (uint8_t)r;
    } else if (dtype == DT_BOOL) { /* predicates and logical ops on BOOL bytes */
      const int av = *(const uint8_t*)pa;
      if (is_pred) *(uint8_t*)po = (uint8_t)pred_i(op, av, 0);
      else if (is_logical) *(uint8_t*)po = (uint8_t)logical(op, av != 0, *(const uint8_t*)pb != 0);
      else return 1;
    } else if (dtype == DT_I64) {
      int64_t av = *(const int64_t*)pa;
      if (is_pred) {
        *(uint8_t*)po = (uint8_t)pred_i(op, av, 1);
      } else if (is_logical) {
        *(uint8_t*)po = (uint8_t)logical(op, av != 0, *(const int64_t*)pb != 0);
      } else if (kind == 0) {
        int ok = 1;
        int64_t r = unary_i64(op, av, &ok);
        if (!ok) return 1;
        *(int64_t*)po = r;
      } else if (kind == 1) {
        int64_t bv = *(const int64_t*)pb;
        if (op == B_DIV || (op >= B_POW && op != B_FMOD && op != B_REMAINDER && op != B_HEAVISIDE &&
                            op != B_RSUB))
          return 1;
        if (is_cmp) *(uint8_t*)po = (uint8_t)compare_i64(op, av, bv);
        else *(int64_t*)po = binary_i64(op, av, bv);
      } else {
        return 1;
      }
    } else if (dtype == DT_F32 || dtype == DT_F16 || dtype == DT_BF16) {
      float av = load_f(pa, dtype);
      if (is_pred) *(uint8_t*)po = (uint8_t)pred_f(op, av);
      else if (kind == 0) {
        if (op == U_NAN_TO_NUM && dtype != DT_F32) return 1;
        store_f(po, dtype, unary_f(op, av));
      } else if (kind == 1) {
        float bv = load_f(pb, dtype);
        if (is_logical) *(uint8_t*)po = (uint8_t)logical(op, av != 0.f, bv != 0.f);
        else if (is_cmp) *(uint8_t*)po = (uint8_t)compare_f(op, av, bv);
        else store_f(po, dtype, binary_f(op, av, bv));
      } else {
        store_f(po, dtype, ternary_f(op, dtype, av, load_f(pb, dtype), load_f(pc, dtype)));
      }
    } else {
      return 1;
    }
  }
  return 0;
}

/* ---- reductions: x dense [outer, n, inner]; sequential left-to-right along n, as the
 * loop callbacks in src/vbt/python/tensor_bindings.cc:290-419, :630-682 and
 * vbt_default_sum_impl (src/vbt/ops/default_kernels.cc:748-805).  out dense [outer, inner].
 * op: 0 sum 1 mean 2 max 3 min 4 prod 5 argmax 6 argmin.  For F16/BF16 inputs the
 * accumulator is float and the result is rounded once to out_dtype (F32 or the input's). */
int vbo_reduce(int op, int dtype, int out_dtype, int64_t outer, int64_t n, int64_t inner,
               const void* x, void* out, int64_t* out_idx) {
  const int es = itemsize(dtype);
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t j = 0; j < inner; ++j) {
      const char* base = (const char*)x + (o * n * inner + j) * es;
      const int64_t step = inner * es;
      const int64_t oi = o * inner + j;
      if (dtype == DT_I64) {
        int64_t acc = 0, bi = 0;
        if (op == 0) { uint64_t s = 0; for (int64_t i = 0; i < n; ++i) s += *(const uint64_t*)(base + i * step); acc = (int64_t)s; }
        else if (op == 4) { uint64_t s = 1; for (int64_t i = 0; i < n; ++i) s *= *(const uint64_t*)(base + i * step); acc = (int64_t)s; }
        else if (op == 1) return 1;
        else {
          if (n == 0) return 2;
          acc = *(const int64_t*)base;
          for (int64_t i = 1; i < n; ++i) {
            int64_t v = *(const int64_t*)(base + i * step);
            if ((op == 2 || op == 5) ? (v > acc) : (v < acc)) { acc = v; bi = i; }
          }
        }
        if (out) ((int64_t*)out)[oi] = acc;
        if (out_idx) out_idx[oi] = bi;
      } else {
        float acc = 0.f;
        int64_t bi = 0;
        if (op == 0 || op == 1) {
          for (int64_t i = 0; i < n; ++i) acc += load_f(base + i * step, dtype);
          if (op == 1) acc = n == 0 ? NAN : acc / (float)(n > 0 ? n : 1);
        } else if (op == 4) {
          acc = 1.f;
          for (int64_t i = 0; i < n; ++i) acc *= load_f(base + i * step, dtype);
        } else {
          if (n == 0) return 2;
          acc = load_f(base, dtype);
          for (int64_t i = 1; i < n; ++i) {
            float v = load_f(base + i * step, dtype);
            if ((op == 2 || op == 5) ? (v > acc) : (v < acc)) { acc = v; bi = i; }
          }
        }
        if (out) store_f((char*)out + oi * itemsize(out_dtype), out_dtype, acc);
        if (out_idx) out_idx[oi] = bi;
      }
    }
  }
  return 0;
}

/* ---- indexing ---- */
/* policy 0 WRAP (indexing_advanced.cc:663-675), 1 STRICT (embedding_dispatch.cc:437-443),
 * 2 CLAMP (vibe_kernels/indexing/kernels.py:79-80).  Returns 0 or 3 (out of range). */
static int norm_index(int64_t* v, int64_t V, int policy) {
  int64_t i = *v;
  if (policy == 2) { if (i < 0) i = 0; if (i > V - 1) i = V - 1; *v = i; return V > 0 ? 0 : 3; }
  if (policy == 0 && i < 0) i += V;
  if (i < 0 || i >= V) return 3;
  *v = i;
  return 0;
}
/* out[i, :] = table[idx[i], :]; table strides (s0, s1) in elements; byte copy
 * (advanced_index_cpu, indexing_advanced.cc:1129-1263; CPU vt::embedding,
 * embedding_dispatch.cc:292-533).  All indices are validated before any copy. */
int vbo_gather_rows(int esize, int64_t V, int64_t D, const void* table, int64_t s0, int64_t s1,
                    const int64_t* idx, int64_t N, int policy, void* out) {
  for (int64_t i = 0; i < N; ++i) { int64_t v = idx[i]; if (norm_index(&v, V, policy)) return 3; }
  for (int64_t i = 0; i < N; ++i) {
    int64_t v = idx[i];
    norm_index(&v, V, policy);
    const char* src = (const char*)table + v * s0 * esize;
    char* dst = (char*)out + i * D * esize;
    if (s1 == 1) memcpy(dst, src, (size_t)(D * esize));
    else for (int64_t j = 0; j < D; ++j) memcpy(dst + j * esize, src + j * s1 * esize, esize);
  }
  return 0;
}
/* table[idx[i], :] (+)= values[i, :] in index order -- sequential accumulation
 * (advanced_index_put_cpu + accumulate_in_place, indexing_advanced.cc:1267-1473);
 * overwrite: last writer in linear order wins.  padding_idx rows are skipped when
 * use_padding != 0 (embedding backward, embedding_cuda.cu:66-87). */
int vbo_scatter_rows(int dtype, int64_t V, int64_t D, void* table, const int64_t* idx, int64_t N,
                     const void* values, int accumulate, int policy, int use_padding,
                     int64_t padding_idx) {
  const int es = itemsize(dtype);
  for (int64_t i = 0; i < N; ++i) { int64_t v = idx[i]; if (norm_index(&v, V, policy)) return 3; }
  for (int64_t i = 0; i < N; ++i) {
    int64_t v = idx[i];
    if (use_padding && v == padding_idx) continue;
    norm_index(&v, V, policy);
    char* dst = (char*)table + v * D * es;
    const char* src = (const char*)values + i * D * es;
    if (!accumulate) { memcpy(dst, src, (size_t)(D * es)); continue; }
    for (int64_t j = 0; j < D; ++j) {
      switch (dtype) {
        case DT_F32: ((float*)dst)[j] += ((const float*)src)[j]; break;
        case DT_I64: ((uint64_t*)dst)[j] += ((const uint64_t*)src)[j]; break;
        case DT_I32: ((uint32_t*)dst)[j] += ((const uint32_t*)src)[j]; break;
        default: return 1;
      }
    }
  }
  return 0;
}
/* Embedding backward with scale_grad_by_freq (embedding_count_by_freq_i64_kernel and
 * embedding_backward_accum_scaled_f32_kernel, src/vbt/ops/embedding_cuda.cu:89-131):
 * counts[row] = occurrences of row outside padding; gw[row, :] += grad[i, :] * (1 / counts[row]),
 * here in index order (the device order is undefined). */
int vbo_embedding_backward_by_freq(int64_t V, int64_t D, float* gw, const int64_t* idx, int64_t N,
                                   const float* grad, int use_padding, int64_t padding_idx) {
  int64_t* counts = (int64_t*)calloc((size_t)(V > 0 ? V : 1), sizeof(int64_t));
  for (int64_t i = 0; i < N; ++i) {
    const int64_t v = idx[i];
    if (use_padding && v == padding_idx) continue;
    if (v < 0 || v >= V) { free(counts); return 3; }
    counts[v]++;
  }
  for (int64_t i = 0; i < N; ++i) {
    const int64_t v = idx[i];
    if (use_padding && v == padding_idx) continue;
    const float scale = 1.0f / (float)counts[v];
    for (int64_t j = 0; j < D; ++j) gw[v * D + j] += grad[i * D + j] * scale;
  }
  free(counts);
  return 0;
}
/* out[b, k] = src[b*sb + idx[k]*sk]: the reference's CUDA last-dim pattern
 * (advanced_index_gather_1d_kernel, indexing_advanced_cuda.cu:953-978). */
int vbo_index_lastdim(int esize, int64_t B, int64_t K0, const void* src, int64_t sb, int64_t sk,
                      const int64_t* idx, int64_t K, int policy, void* out) {
  for (int64_t k = 0; k < K; ++k) { int64_t v = idx[k]; if (norm_index(&v, K0, policy)) return 3; }
  for (int64_t b = 0; b < B; ++b)
    for (int64_t k = 0; k < K; ++k) {
      int64_t v = idx[k];
      norm_index(&v, K0, policy);
      memcpy((char*)out + (b * K + k) * esize, (const char*)src + (b * sb + v * sk) * esize, esize);
    }
  return 0;
}
/* self[b, idx[k]] (+)= values[b, k]; self dense [B, K0]. */
int vbo_index_put_lastdim(int dtype, int64_t B, int64_t K0, void* self, const int64_t* idx,
                          int64_t K, const void* values, int accumulate, int policy) {
  const int es = itemsize(dtype);
  for (int64_t k = 0; k < K; ++k) { int64_t v = idx[k]; if (norm_index(&v, K0, policy)) return 3; }
  for (int64_t b = 0; b < B; ++b)
    for (int64_t k = 0; k < K; ++k) {
      int64_t v = idx[k];
      norm_index(&v, K0, policy);
      char* dst = (char*)self + (b * K0 + v) * es;
      const char* src = (const char*)values + (b * K + k) * es;
      if (!accumulate) { memcpy(dst, src, es); continue; }
      switch (dtype) {
        case DT_F32: *(float*)dst += *(const float*)src; break;
        case DT_I64: *(uint64_t*)dst += *(const uint64_t*)src; break;
        case DT_I32: *(uint32_t*)dst += *(const uint32_t*)src; break;
        default: return 1;
      }
    }
  return 0;
}

/* ---- row ops ---- */
/* Both Triton kernels reduce a row block by block: tl.sum over a block of BLOCK lanes (a
 * halving tree), block results accumulated in order.  The restatement keeps that shape so
 * that long rows see the same kind of rounding; the order inside tl.sum is Triton's own and
 * is not pinned by the reference, which is why these paths are tolerance-checked. */
static float block_tree_sum(const float* vals, int64_t n, int64_t block, float* tmp) {
  float acc = 0.f;
  for (int64_t start = 0; start < n; start += block) {
    for (int64_t i = 0; i < block; ++i) tmp[i] = (start + i < n) ? vals[start + i] : 0.f;
    for (int64_t s = block / 2; s > 0; s /= 2)
      for (int64_t i = 0; i < s; ++i) tmp[i] += tmp[i + s];
    acc += tmp[0];
  }
  return acc;
}
static int64_t next_pow2(int64_t v) { int64_t p = 1; while (p < v) p <<= 1; return p; }

/* Triton softmax_kernel (vibe_kernels/softmax/vbt_native.py:39-97): fp32 math,
 * m = max x; s = sum exp(x - m); s = max(s, 1e-20); y = exp(x - (log s + m));
 * log_softmax: y = x - (log s + m).  BLOCK_SIZE = clamp(round_up(cols, 128), 128, 1024)
 * (:240-252). */
int vbo_softmax(int dtype, int64_t rows, int64_t cols, const void* x, int64_t row_stride,
                void* out, int log_softmax) {
  const int es = itemsize(dtype);
  int64_t block = (cols + 127) / 128 * 128;
  if (block < 128) block = 128;
  if (block > 1024) block = 1024;
  block = next_pow2(block); /* tl.arange needs a power of two; 128..1024 */
  float* e = (float*)malloc(sizeof(float) * (size_t)(cols > 0 ? cols : 1));
  float* tmp = (float*)malloc(sizeof(float) * (size_t)block);
  for (int64_t r = 0; r < rows; ++r) {
    const char* px = (const char*)x + r * row_stride * es;
    char* po = (char*)out + r * cols * es;
    float m = -INFINITY;
    for (int64_t j = 0; j < cols; ++j) { float v = load_f(px + j * es, dtype); m = fmaxf(m, v); }
    for (int64_t j = 0; j < cols; ++j) e[j] = expf(load_f(px + j * es, dtype) - m);
    float s = block_tree_sum(e, cols, block, tmp);
    s = fmaxf(s, 1e-20f);
    const float lse = logf(s) + m;
    for (int64_t j = 0; j < cols; ++j) {
      float v = load_f(px + j * es, dtype) - lse;
      store_f(po + j * es, dtype, log_softmax ? v : expf(v));
    }
  }
  free(e);
  free(tmp);
  return 0;
}
/* Triton _rmsnorm_fwd_kernel (vibe_kernels/rmsnorm/vbt_native.py:55-103):
 * inv_rms = rsqrt(sum x^2 / cols + eps); y = x * inv_rms * gamma; output cast to the
 * input dtype (vibe_kernels/rmsnorm/impl/triton_impl.py:99-104).
 * BLOCK = min(256, next_pow2(hidden)) (:378-380). */
int vbo_rmsnorm(int dtype, int64_t rows, int64_t cols, const void* x, int64_t row_stride,
                const float* gamma, float eps, void* out, float* inv_rms) {
  const int es = itemsize(dtype);
  int64_t block = next_pow2(cols);
  if (block > 256) block = 256;
  float* sq = (float*)malloc(sizeof(float) * (size_t)(cols > 0 ? cols : 1));
  float* tmp = (float*)malloc(sizeof(float) * (size_t)block);
  for (int64_t r = 0; r < rows; ++r) {
    const char* px = (const char*)x + r * row_stride * es;
    char* po = (char*)out + r * cols * es;
    for (int64_t j = 0; j < cols; ++j) { float v = load_f(px + j * es, dtype); sq[j] = v * v; }
    const float ss = block_tree_sum(sq, cols, block, tmp);
    const float inv = (float)(1.0 / sqrt((double)(ss / (float)cols + eps)));
    if (inv_rms) inv_rms[r] = inv;
    for (int64_t j = 0; j < cols; ++j) {
      float v = load_f(px + j * es, dtype) * inv;
      if (gamma) v *= gamma[j];
      store_f(po + j * es, dtype, v);
    }
  }
  free(sq);
  free(tmp);
  return 0;
}

/* Softmax / log_softmax backward (SoftmaxBackward / LogSoftmaxBackward,
 * vibe_kernels/softmax/impl/cutedsl_softmax/softmax.py:405-423, :809-828):
 *   softmax:     dx = y * (dy - sum(dy*y));   log_softmax: dx = dy - exp(log_y) * sum(dy).
 * The row sum is a float reduction whose order is a schedule detail of the CuTe kernel; it is
 * accumulated in double here and rounded once, so any float order agrees to a few ulp. */
int vbo_softmax_backward(int dtype, int64_t rows, int64_t cols, const void* dy, int64_t dy_stride,
                         const void* y, int64_t y_stride, void* dx, int log_softmax) {
  const int es = itemsize(dtype);
  for (int64_t r = 0; r < rows; ++r) {
    const char* pd = (const char*)dy + r * dy_stride * es;
    const char* py = (const char*)y + r * y_stride * es;
    char* po = (char*)dx + r * cols * es;
    double acc = 0.0;
    for (int64_t j = 0; j < cols; ++j) {
      const float a = load_f(pd + j * es, dtype), b = load_f(py + j * es, dtype);
      acc += log_softmax ? (double)a : (double)a * (double)b;
    }
    const float s = (float)acc;
    for (int64_t j = 0; j < cols; ++j) {
      const float a = load_f(pd + j * es, dtype), b = load_f(py + j * es, dtype);
      store_f(po + j * es, dtype, log_softmax ? a - expf(b) * s : b * (a - s));
    }
  }
  return 0;
}

/* Triton _rmsnorm_bwd_kernel (vibe_kernels/rmsnorm/vbt_native.py:110-176): per row
 *   normed = x*inv_rms; dot = sum(dy*gamma*normed) (block sums per chunk of BLOCK, added chunk
 *   by chunk); dx = inv_rms*(dy*gamma - normed*dot/cols); grad_gamma[c] += dy*normed.
 * grad_gamma is a float atomic per element there (order undefined): accumulated in double
 * here and rounded once. */
int vbo_rmsnorm_backward(int dtype, int64_t rows, int64_t cols, const void* dy, int64_t dy_stride,
                         const void* x, int64_t x_stride, const float* inv_rms, const float* gamma,
                         void* dx, float* dgamma) {
  const int es = itemsize(dtype);
  int64_t block = next_pow2(cols);
  if (block > 256) block = 256;
  float* pr = (float*)malloc(sizeof(float) * (size_t)(cols > 0 ? cols : 1));
  float* tmp = (float*)malloc(sizeof(float) * (size_t)block);
  double* gg = (double*)calloc((size_t)(cols > 0 ? cols : 1), sizeof(double));
  for (int64_t r = 0; r < rows; ++r) {
    const char* pd = (const char*)dy + r * dy_stride * es;
    const char* px = (const char*)x + r * x_stride * es;
    char* po = (char*)dx + r * cols * es;
    const float inv = inv_rms[r];
    for (int64_t j = 0; j < cols; ++j) {
      const float a = load_f(pd + j * es, dtype), n = load_f(px + j * es, dtype) * inv;
      gg[j] += (double)a * (double)n;
      pr[j] = (gamma ? a * gamma[j] : a) * n;
    }
    const float dot_mean = block_tree_sum(pr, cols, block, tmp) / (float)cols;
    for (int64_t j = 0; j < cols; ++j) {
      const float a = load_f(pd + j * es, dtype), n = load_f(px + j * es, dtype) * inv;
      const float ds = gamma ? a * gamma[j] : a;
      store_f(po + j * es, dtype, inv * (ds - n * dot_mean));
    }
  }
  if (dgamma)
    for (int64_t j = 0; j < cols; ++j) dgamma[j] = (float)gg[j];
  free(pr);
  free(tmp);
  free(gg);
  return 0;
}

/* out[i] = cast(partial[i] * scale): finish of a sharded mean. */
int vbo_scale_cast(int out_dtype, const float* partial, int64_t n, float scale, void* out) {
  for (int64_t i = 0; i < n; ++i)
    store_f((char*)out + i * itemsize(out_dtype), out_dtype, partial[i] * scale);
  return 0;
}

/* Host mirror of the reference's device offset calculator compute_offset_elems
 * (include/vbt/core/tensor_iterator/cuda.h:25-42; the same mirror appears in
 * tests/cpp/tensor_iter_cuda_meta_test.cc:78-91): linear index -> element offset, sizes
 * and strides innermost-first. */
int64_t vbo_offset_elems(int64_t linear, int ndim, const int64_t* sizes, const int64_t* strides) {
  int64_t off = 0;
  for (int d = 0; d < ndim; ++d) {
    const int64_t sz = sizes[d];
    if (sz <= 0) continue;
    off += (linear % sz) * strides[d];
    linear /= sz;
  }
  return off;
}
