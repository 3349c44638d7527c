/*
 * vbt_b200.h -- C ABI of libvbt_b200.so: a from-scratch sm_100a implementation of the
 * CUDA backend behind VibeTensor's vt:: data-parallel ops.
 *
 * Every entry point takes plain pointers, sizes and strides.  A VibeTensor binding
 * fills a vbt_b200_tensor from a vbt::core::TensorImpl (data(), dtype(), sizes(),
 * strides()), allocates the output through VibeTensor's own stream-ordered caching
 * allocator, passes the current stream, and maps the returned status to the C++
 * exception class named beside each code.  Nothing here allocates device memory except
 * where a function says so; nothing synchronises the stream except where it says so.
 * All launches go to the `stream` argument (a cudaStream_t passed as void*; NULL is the
 * legacy default stream) on the device that owns the pointers; the library switches to
 * that device for the call and restores the previous one.
 *
 * "Reference" below means the NVlabs/vibetensor source tree; citations are
 * path:line inside it.
 */
#ifndef VBT_B200_H_
#define VBT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define VBT_B200_API __attribute__((visibility("default")))
#else
#define VBT_B200_API
#endif

/* ---- status codes: the exception the reference throws for the same condition ---- */
typedef int32_t vbt_b200_status;
#define VBT_B200_OK 0
#define VBT_B200_INVALID_ARGUMENT 1 /* std::invalid_argument -> Python ValueError  */
#define VBT_B200_RUNTIME_ERROR 2    /* std::runtime_error    -> Python RuntimeError */
#define VBT_B200_OUT_OF_RANGE 3     /* std::out_of_range     -> Python IndexError   */
#define VBT_B200_CUDA_ERROR 4       /* a CUDA runtime call failed                   */

/* Message of the last non-OK status on the calling thread (thread-local, never NULL). */
VBT_B200_API const char* vbt_b200_last_error(void);
/* Library version (major*1000 + minor) and the sm architecture it was compiled for. */
VBT_B200_API int32_t vbt_b200_version(void);
VBT_B200_API int32_t vbt_b200_compiled_arch(void);

/* ---- dtypes: ordinals of vbt::core::ScalarType (include/vbt/core/dtype.h:19-30) ---- */
#define VBT_B200_BOOL 0
#define VBT_B200_I32 1
#define VBT_B200_I64 2
#define VBT_B200_F32 3
#define VBT_B200_F16 4
#define VBT_B200_BF16 5
#define VBT_B200_F64 6   /* ordinal reserved (the reference has no Float64 CUDA kernels on this path) */
#define VBT_B200_C64 7   /* two float32: vt::add, vt::mul and copy only, as in the reference            */
#define VBT_B200_C128 8  /* two float64: likewise                                                       */

/* Maximum rank accepted, the reference's CUDA broadcast limit
 * (src/vbt/ops/cuda_elementwise.cu:2974-2979). */
#define VBT_B200_MAX_NDIM 25

/* A strided view of device memory.  `data` already includes the storage offset
 * (TensorImpl::data(), include/vbt/core/tensor.h:96-101); strides are in elements and
 * may be 0 (broadcast) or negative. */
typedef struct vbt_b200_tensor {
  void* data;
  int32_t dtype;
  int32_t ndim;
  const int64_t* sizes;
  const int64_t* strides;
} vbt_b200_tensor;

/* =====================================================================================
 * 1. TensorIterator elementwise ops over broadcast / strided views
 *    replaces: binary_op_dispatcher, unary_op_dispatcher, ternary_op_dispatcher,
 *    where_op_dispatcher and their *_ti_strided_kernel launches
 *    (src/vbt/ops/cuda_elementwise.cu:1786-1909, :2645-2782, :2845-2866, :2884-3211),
 *    the launcher ti_gpu_kernel (include/vbt/core/tensor_iterator/cuda_loops.h:16-48) and
 *    the offset calculator compute_offset_elems
 *    (include/vbt/core/tensor_iterator/cuda.h:25-42).
 *
 *    `out` is written in place and may be ANY strided view whose shape equals the
 *    broadcast of the inputs (the reference always allocates a dense output,
 *    cuda_elementwise.cu:96-110; a binding passes that allocation here).  Inputs must all
 *    have out's dtype, except: comparison, logical and predicate ops write BOOL, `where` takes
 *    a BOOL condition.
 *    No type promotion, as in the reference (:2887).
 * ===================================================================================== */

/* Broadcast shape of up to 4 operands (src/vbt/core/broadcast.cc); out_sizes has room for
 * VBT_B200_MAX_NDIM entries.  INVALID_ARGUMENT on incompatible shapes. */
VBT_B200_API vbt_b200_status vbt_b200_broadcast_shape(const vbt_b200_tensor* const* operands, int32_t n,
                                         int64_t* out_sizes, int32_t* out_ndim);

enum vbt_b200_unary_op {
  VBT_B200_U_RELU = 0,   /* vbt_cuda_relu_impl; relu(NaN)=0, relu(-0.0)=+0.0 (:1622-1630) */
  VBT_B200_U_NEG,        /* vbt_cuda_neg_impl; integers wrap (:619-628)                    */
  VBT_B200_U_ABS,        /* vbt_cuda_abs_impl; abs(INT64_MIN)=INT64_MIN (:590-618)         */
  VBT_B200_U_SQUARE,
  VBT_B200_U_EXP,
  VBT_B200_U_LOG,
  VBT_B200_U_SQRT,
  VBT_B200_U_RSQRT,
  VBT_B200_U_SIN,
  VBT_B200_U_COS,
  VBT_B200_U_TANH,
  VBT_B200_U_SIGMOID,    /* 1/(1+exp(-x))                                                 */
  VBT_B200_U_SILU,       /* reference computes in fp64 (:877-883); here fp32, |err|<=1e-6 */
  VBT_B200_U_GELU,       /* exact erf form (:884-891); here fp32 erff                     */
  VBT_B200_U_RECIPROCAL,
  VBT_B200_U_SIGN,
  VBT_B200_U_FLOOR,
  VBT_B200_U_CEIL,
  VBT_B200_U_TRUNC,
  VBT_B200_U_ROUND,      /* ties to even (:789-807)                                       */
  VBT_B200_U_EXPM1,
  VBT_B200_U_LOG1P,
  VBT_B200_U_SOFTPLUS,   /* thresholds +-20 (:892-900)                                    */
  VBT_B200_U_RELU6,
  VBT_B200_U_HARDTANH,
  /* the rest of the reference's unary table (:808-1252, :1279-1287); floating inputs only
   * unless noted, computed in fp32 where the reference writes fp64                        */
  VBT_B200_U_EXP2, VBT_B200_U_LOG2, VBT_B200_U_LOG10, VBT_B200_U_SINH, VBT_B200_U_COSH,
  VBT_B200_U_ASINH, VBT_B200_U_ACOSH, VBT_B200_U_ATANH, VBT_B200_U_TAN, VBT_B200_U_ASIN,
  VBT_B200_U_ACOS, VBT_B200_U_ATAN, VBT_B200_U_ERF, VBT_B200_U_ERFC, VBT_B200_U_LGAMMA,
  VBT_B200_U_SINC,       /* sin(pi x)/(pi x), sinc(0)=1 (:817-824)                         */
  VBT_B200_U_FRAC,       /* modf fraction, keeps the sign of x (:808-815)                  */
  VBT_B200_U_DEG2RAD, VBT_B200_U_RAD2DEG,
  VBT_B200_U_MISH,       /* x*tanh(softplus(x)), threshold 20 (:901-908)                   */
  VBT_B200_U_SELU, VBT_B200_U_ELU,   /* alpha = 1; vt::celu is the same functor (:909-930) */
  VBT_B200_U_HARDSIGMOID,            /* clamp(x/6 + 0.5, 0, 1)                             */
  VBT_B200_U_HARDSHRINK, VBT_B200_U_SOFTSHRINK,  /* lambda = 0.5 (:931-948)                */
  VBT_B200_U_LOGIT,      /* log(x/(1-x)) (:1279-1287)                                      */
  VBT_B200_U_ANGLE,      /* NaN -> NaN, x<0 -> pi, else 0 (:843-850)                       */
  VBT_B200_U_POSITIVE,   /* identity; also INT64 (vt::conj_physical is the same)           */
  VBT_B200_U_SGN,        /* sign with sgn(NaN)=0; also INT64 (:832-838)                    */
  VBT_B200_U_NAN_TO_NUM, /* F32 only: NaN->0, +-inf->+-FLT_MAX (:1556-1572)                */
  /* predicates: out dtype BOOL; input F32/F16/BF16/I64/BOOL (:1043-1149, :1995-2100)      */
  VBT_B200_U_ISFINITE, VBT_B200_U_ISINF, VBT_B200_U_ISNAN, VBT_B200_U_ISNEGINF,
  VBT_B200_U_ISPOSINF, VBT_B200_U_SIGNBIT, VBT_B200_U_LOGICAL_NOT,
  VBT_B200_U_BITWISE_NOT, /* I64/I32: ~a; BOOL: logical not (:3498-3506)                   */
  VBT_B200_U_COUNT
};

enum vbt_b200_binary_op {
  VBT_B200_B_ADD = 0,  /* vbt_cuda_add_impl (:3351-3356) */
  VBT_B200_B_SUB,
  VBT_B200_B_MUL,      /* vbt_cuda_mul_impl */
  VBT_B200_B_DIV,      /* INT64 rejected, as :2889-2891 */
  VBT_B200_B_MAXIMUM,  /* NaN from either side propagates (:244-306) */
  VBT_B200_B_MINIMUM,
  VBT_B200_B_FMAX,     /* NaN ignored (:1333-1350) */
  VBT_B200_B_FMIN,
  VBT_B200_B_EQ,       /* comparisons: out dtype BOOL (:2399-2404, :2406-2530) */
  VBT_B200_B_NE,
  VBT_B200_B_LT,
  VBT_B200_B_GT,
  VBT_B200_B_LE,
  VBT_B200_B_GE,
  /* floating dtypes only unless noted (:307-589, :851-876, :1253-1258, :3526-3640)        */
  VBT_B200_B_POW,        /* powf; vt::float_power is the same functor                      */
  VBT_B200_B_FMOD,       /* also INT64: b==0 -> 0, INT64_MIN % -1 -> 0 (:307-334)          */
  VBT_B200_B_REMAINDER,  /* sign of the divisor; also INT64 (:336-377)                     */
  VBT_B200_B_ATAN2, VBT_B200_B_COPYSIGN, VBT_B200_B_HYPOT,
  VBT_B200_B_XLOGY, VBT_B200_B_XLOG1PY,  /* x == 0 -> 0 even for NaN y                     */
  VBT_B200_B_LOGADDEXP, VBT_B200_B_LOGADDEXP2, VBT_B200_B_NEXTAFTER,
  VBT_B200_B_HEAVISIDE,  /* also INT64                                                     */
  VBT_B200_B_RSUB,       /* b - a; also INT64 (:3379-3384)                                 */
  VBT_B200_B_TANH_BACKWARD,    /* (grad, out): grad*(1-out^2)                              */
  VBT_B200_B_SIGMOID_BACKWARD, /* (grad, out): grad*out*(1-out)                            */
  VBT_B200_B_SILU_BACKWARD,    /* (grad, x)                                                */
  VBT_B200_B_LOGIT_BACKWARD,   /* (grad, x): grad/(x*(1-x))                                */
  VBT_B200_B_MSE_LOSS,   /* (a-b)^2, no reduction (:1365-1370)                             */
  VBT_B200_B_LDEXP,      /* a * 2^int(b), exponent clamped as :463-478                     */
  /* integer ops: dtype BOOL/I32/I64 for and/or/xor, I32/I64 for shifts, I64 for gcd/lcm;
   * a shift count outside [0, bits) gives 0 (right shift of a negative: -1) (:191-243)    */
  VBT_B200_B_BITWISE_AND, VBT_B200_B_BITWISE_OR, VBT_B200_B_BITWISE_XOR,
  VBT_B200_B_LSHIFT, VBT_B200_B_RSHIFT, VBT_B200_B_GCD, VBT_B200_B_LCM,
  /* out dtype BOOL; inputs F32/F16/BF16/I64/BOOL (:194-196, :3510-3512)                   */
  VBT_B200_B_LOGICAL_AND, VBT_B200_B_LOGICAL_OR, VBT_B200_B_LOGICAL_XOR,
  VBT_B200_B_COUNT
};

enum vbt_b200_ternary_op {
  VBT_B200_T_CLAMP = 0,  /* clamp(v, mn, mx); NaN bound -> NaN (:1259-1266)              */
  VBT_B200_T_LERP,       /* start + weight*(end-start) (:1267-1271)                      */
  VBT_B200_T_THRESHOLD,  /* x > thr ? x : value (:1273-1277)                             */
  VBT_B200_T_ADDCMUL,    /* a + b*c, ONE launch; the reference's vbt_cuda_addcmul_impl
                            is three launches with two temporaries (:3927-3931); each
                            intermediate is rounded to the storage dtype as there       */
  VBT_B200_T_ADDCDIV,    /* a + b/c, likewise (:3933-3937)                               */
  VBT_B200_T_WHERE_GT0_ADDCMUL, /* where(a > 0, a + b*c, 0) in one launch: the chain
                            mul -> add -> gt -> where of four reference ops with the same
                            per-op rounding, so results are bit-identical to the chain   */
  VBT_B200_T_HUBER_LOSS,     /* (input, target, delta), elementwise (:1385-1395)         */
  VBT_B200_T_SMOOTH_L1_LOSS, /* (input, target, beta) (:1397-1407)                       */
  VBT_B200_T_COUNT
};

VBT_B200_API vbt_b200_status vbt_b200_unary(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                               void* stream);
VBT_B200_API vbt_b200_status vbt_b200_binary(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                const vbt_b200_tensor* b, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_ternary(int32_t op, const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                                 const vbt_b200_tensor* b, const vbt_b200_tensor* c, void* stream);
/* vbt_cuda_where_impl / vbt_cuda_masked_fill_impl (:3921-3926): cond BOOL; x, y, out same
 * dtype in {F32, I64, BOOL, F16, BF16} (:2701-2712). */
VBT_B200_API vbt_b200_status vbt_b200_where(const vbt_b200_tensor* out, const vbt_b200_tensor* cond,
                               const vbt_b200_tensor* x, const vbt_b200_tensor* y, void* stream);
/* Binary op with a host scalar on one side: the reference's CPU 0-d scalar fast path
 * (:2893-2961).  `scalar` points at one host element of a's dtype (F32 or I64 only, as
 * there); scalar_on_left selects op(scalar, a) (the reference's ROp functors, :2934). */
VBT_B200_API vbt_b200_status vbt_b200_binary_scalar(int32_t op, const vbt_b200_tensor* out,
                                       const vbt_b200_tensor* a, const void* scalar,
                                       int32_t scalar_on_left, void* stream);
/* vt::polygamma(n, x) (vbt_cuda_polygamma_impl, src/vbt/ops/cuda_elementwise.cu:1288-1330, :3853-3876):
 * n is a ONE-element floating tensor on x's device and of x's dtype, out has x's shape and dtype.
 * As in the reference only order n == 2 is computed (any other order gives NaN): the recurrence
 * psi''(x) = psi''(x + 1) - 2 / x^3 up to x >= 10 (at most 100 steps), then the three-term
 * asymptotic series, all in double; poles (x a non-positive integer) and x < -1e6 give NaN.
 * Errors: "vt::polygamma: expected n to be a scalar tensor", "... expected n to have floating
 * dtype", "... dtype mismatch". */
VBT_B200_API vbt_b200_status vbt_b200_polygamma(const vbt_b200_tensor* out, const vbt_b200_tensor* n,
                                   const vbt_b200_tensor* x, void* stream);
/* Strided copy out <- a (same dtype, a broadcast to out's shape): clone_cuda /
 * clone_strided_to_contig_kernel (src/vbt/core/tensor_ops_cuda.cu:83-91). */
VBT_B200_API vbt_b200_status vbt_b200_copy(const vbt_b200_tensor* out, const vbt_b200_tensor* a, void* stream);

/* Named forms of the ops the benchmark configuration chains; each forwards to the
 * enum entry above.  vbt_cuda_{add,mul,sub,div,gt,relu}_impl (:3351-3393, :3486). */
VBT_B200_API vbt_b200_status vbt_b200_add(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                             const vbt_b200_tensor* b, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_sub(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                             const vbt_b200_tensor* b, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_mul(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                             const vbt_b200_tensor* b, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_div(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                             const vbt_b200_tensor* b, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_gt(const vbt_b200_tensor* out, const vbt_b200_tensor* a,
                            const vbt_b200_tensor* b, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_relu(const vbt_b200_tensor* out, const vbt_b200_tensor* a, void* stream);

/* Introspection of the iteration plan the host builds for an elementwise call: the
 * counterpart of TensorIterBase::export_device_meta / can_use_32bit_indexing
 * (src/vbt/core/tensor_iterator/core.cc:248-474).  Fills the coalesced iteration shape
 * (innermost first) and, per operand (out first), the element strides in that order.
 * `strides` has room for noperands*VBT_B200_MAX_NDIM entries, row per operand.
 * *kernel: 0 = flat vector kernel, 1 = tiled kernel (vector along dim 0), 2 = tiled
 * scalar kernel, 3 = shared-memory transposing kernel (an input is contiguous along another
 * dim than the output).  *pieces: number of 32-bit-safe launches the call is split into. */
VBT_B200_API vbt_b200_status vbt_b200_ti_plan(const vbt_b200_tensor* const* operands, int32_t noperands,
                                 int64_t* shape, int64_t* strides, int32_t* ndim,
                                 int32_t* kernel, int32_t* pieces);

/* =====================================================================================
 * 2. Dim reductions
 *    replaces: vbt_cuda_{sum,prod,min,max,mean}_impl -> cuda_reduce_dispatch and kernels
 *    K1/K2/K3 (src/vbt/ops/cuda_reduction.cu:254-416, :907-2070); adds argmax/argmin,
 *    which the reference only has on CPU (src/vbt/python/tensor_bindings.cc:630-889),
 *    and BF16/F16 inputs (FP32 accumulation).
 *
 *    `out` (and `out_index` for ARGMAX/ARGMIN; INT64) is a caller-allocated dense
 *    tensor whose shape is the reduced shape (keepdim decides whether reduced dims stay
 *    as size 1).  dims == NULL / ndims == 0 reduces everything.  Accumulation order is
 *    fixed by the shapes alone: results are run-to-run deterministic (no float atomics).
 *    SUM/PROD/MAX/MIN: F32 or I64 (out same dtype); BF16/F16 in -> out BF16/F16 or F32.
 *    MEAN: F32 ("mean: expected dtype=float32", cuda_reduction.cu:982) or BF16/F16.
 *    Reduced extent 0: SUM 0, PROD 1, MEAN NaN, MAX/MIN/ARG* -> RUNTIME_ERROR
 *    "amax: empty" / "amin: empty" (cuda_reduction.cu:1176-1216).
 *    MAX/MIN/ARGMAX/ARGMIN follow the CPU scan (tensor_bindings.cc:361-379, :630-655):
 *    strict compare from element 0, first extremum wins, a NaN wins only at position 0.
 * ===================================================================================== */
enum vbt_b200_reduce_op {
  VBT_B200_R_SUM = 0,
  VBT_B200_R_MEAN,
  VBT_B200_R_MAX,
  VBT_B200_R_MIN,
  VBT_B200_R_PROD,
  VBT_B200_R_ARGMAX,
  VBT_B200_R_ARGMIN,
  VBT_B200_R_COUNT
};

/* Bytes of scratch the call below needs for these arguments on the device that owns self
 * (0 for most shapes; the split reductions keep a VBT_B200_REDUCE_TICKET_BYTES area of ticket
 * counters at the start of it and per-block partials behind).  A binding takes it from the
 * caching allocator; for vbt_b200_reduce the contents need no initialisation. */
#define VBT_B200_REDUCE_TICKET_BYTES 4096
VBT_B200_API size_t vbt_b200_reduce_workspace_bytes(int32_t op, const vbt_b200_tensor* self,
                                       const int64_t* dims, int32_t ndims);
VBT_B200_API vbt_b200_status vbt_b200_reduce(int32_t op, const vbt_b200_tensor* out,
                                const vbt_b200_tensor* out_index, const vbt_b200_tensor* self,
                                const int64_t* dims, int32_t ndims, int32_t keepdim,
                                void* workspace, size_t workspace_bytes, void* stream);
/* The same call for a binding that KEEPS its workspace (one per stream, say): the first
 * VBT_B200_REDUCE_TICKET_BYTES of the workspace must be zero before the first call -- zero the
 * buffer once when it is created -- and every call leaves them zero again (the block that
 * draws the last ticket resets the counter), so the per-call clearing of the ticket counters
 * that vbt_b200_reduce enqueues in front of its kernel is not needed.  The rest of the
 * workspace needs no initialisation.  Results are bit-identical to vbt_b200_reduce.  Calls
 * that share a workspace must not overlap on the GPU. */
VBT_B200_API vbt_b200_status vbt_b200_reduce_zeroed_ws(int32_t op, const vbt_b200_tensor* out,
                                          const vbt_b200_tensor* out_index,
                                          const vbt_b200_tensor* self, const int64_t* dims,
                                          int32_t ndims, int32_t keepdim, void* workspace,
                                          size_t workspace_bytes, void* stream);
/* The same reduction for callers that cannot supply scratch memory (no counterpart in the
 * reference, whose kernels take their temporaries from its caching allocator).  Meant for
 * hosts that cannot allocate at call time -- a plugin whose host API only creates "dense
 * like" outputs, code running under an allocator lock, an embedder that bans cudaMalloc after
 * start-up.  The partials and ticket counters live in a fixed device array of
 * VBT_B200_NOALLOC_SCRATCH_BYTES inside the library (held by every GPU that loads it);
 * shapes that need more are rejected with INVALID_ARGUMENT.  No cudaMalloc / cudaFree or
 * other allocating call is made.  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress, cached): make that call before any stream capture.  Every
 * call on a device shares the array: calls that may overlap on the GPU race and must be
 * ordered by the caller.  Results are bit-identical to vbt_b200_reduce. */
#define VBT_B200_NOALLOC_SCRATCH_BYTES (2u << 20)
VBT_B200_API vbt_b200_status vbt_b200_reduce_noalloc(int32_t op, const vbt_b200_tensor* out,
                                        const vbt_b200_tensor* out_index,
                                        const vbt_b200_tensor* self, const int64_t* dims,
                                        int32_t ndims, int32_t keepdim, void* stream);
/* Reduced shape for (self, dims, keepdim): cuda_reduction.cu:749-810.  INVALID_ARGUMENT
 * "<op>: dim out of range" on a bad dim. */
VBT_B200_API vbt_b200_status vbt_b200_reduce_shape(const vbt_b200_tensor* self, const int64_t* dims,
                                      int32_t ndims, int32_t keepdim, int64_t* out_sizes,
                                      int32_t* out_ndim);

/* =====================================================================================
 * 3. Advanced indexing, row gather, scatter-add
 *    replaces: embedding_gather_f32_kernel / embedding_backward_accum_f32_kernel /
 *    embedding_bounds_check_i64_kernel (src/vbt/ops/embedding_cuda.cu:32-87, :225-302),
 *    advanced_index_gather_1d_kernel, advanced_index_cuda_kernel,
 *    advanced_index_put_cuda_kernel, advanced_index_bounds_normalize_kernel
 *    (src/vbt/core/indexing_advanced_cuda.cu:662-684, :953-978, :1325-1453) and the Triton
 *    gather/scatter_add kernels (vibe_kernels/indexing/kernels.py:13-186).
 *
 *    Index policy (how an index outside [0, V) is treated):
 *      WRAP   vt::index / index_put_: i in [-V, V) wraps once, else error
 *             (src/vbt/core/indexing_advanced.cc:663-675)
 *      STRICT vt::embedding: negative is an error (embedding_dispatch.cc:437-443)
 *      CLAMP  Triton scatter/gather-2d: clamp into range, never an error
 *             (vibe_kernels/indexing/kernels.py:79-80)
 *    Errors are detected ON DEVICE: a bad index is skipped (gather writes zeros for that
 *    row, scatter drops it) and recorded in the caller's 16-byte `index_status` block
 *    {int64 count, int64 first_bad_value}, which the caller zeroes once and may share
 *    between calls.  vbt_b200_index_status_check copies it back (this one synchronises
 *    the stream) and returns OUT_OF_RANGE with the reference's message.  index_status may
 *    be NULL to skip recording.
 * ===================================================================================== */
#define VBT_B200_INDEX_WRAP 0
#define VBT_B200_INDEX_STRICT 1
#define VBT_B200_INDEX_CLAMP 2

/* out[i, :] = table[idx[i], :].  table [V, D] with arbitrary row stride and unit or
 * non-unit column stride, any dtype (byte copy, bit exact); idx I64 or I32, any rank,
 * contiguous; out dense [idx.shape..., D]. */
VBT_B200_API vbt_b200_status vbt_b200_index_rows(const vbt_b200_tensor* out, const vbt_b200_tensor* table,
                                    const vbt_b200_tensor* idx, int32_t policy,
                                    void* index_status, void* stream);
/* table[idx[i], :] = values[i, :]            (accumulate == 0; duplicate rows: one of the
 *                                             writers wins, as on the reference's CUDA path)
 * table[idx[i], :] += values[i, :]           (accumulate != 0; F32, I64, I32, BF16/F16)
 * table dense rows ([V, D], column stride 1), values [N, D] dense.  Duplicates are
 * pre-summed inside each thread block (1024 consecutive updates, sorted by row in shared
 * memory) before one atomic per distinct row and column vector reaches memory.  I64/I32 results are exact (wrap-around); F32 is order-free
 * only up to rounding.  Uses no scratch memory. */
VBT_B200_API vbt_b200_status vbt_b200_index_put_rows(const vbt_b200_tensor* table, const vbt_b200_tensor* idx,
                                        const vbt_b200_tensor* values, int32_t accumulate,
                                        int32_t policy, void* index_status, void* stream);
/* table[idx[i], :] += values[i, :] by bringing the updates of one destination row TOGETHER first:
 * the counterpart of the accumulate path above that adds run sums instead of single updates --
 * the fast one for 64-bit integers and for large update counts.  It does what the reference's
 * opt-in sort + reduce-by-key path does (advanced_index_put_make_kv_cuda_kernel + CUB SortPairs +
 * ReduceByKey + scatter, src/vbt/core/indexing_advanced_cuda.cu:1460-1557, :2888-3055) with
 * an LSD radix sort written here.  Tables of 4-byte elements with more than 65536 rows are not
 * sorted by row but grouped by a 16-bit hash of the row (two passes whatever the height): equal
 * rows still end up next to each other, in update order, unless another row of the same hash
 * bucket falls between them, which costs that row one more add.  A warp walks 256 consecutive
 * entries, sums every run of equal rows in update order and adds the run's sum to the row once
 * (row += u1 + u2 + ...); a run that crosses a slice boundary is finished by the next warp with
 * an add of its own.  INT64 / INT32 exact; F32 bit-identical to a sequential loop for every row
 * that starts at zero (or is updated once) and whose updates form one run.  `workspace` (16-byte
 * aligned, vbt_b200_index_put_rows_sorted_workspace_bytes(N) bytes, about 18 bytes per
 * index) needs no initialisation.  Shapes the sorted kernels do not take (rows that are not
 * whole 16-byte chunks) are served by the atomic path with the same result. */
VBT_B200_API size_t vbt_b200_index_put_rows_sorted_workspace_bytes(int64_t num_indices);
VBT_B200_API vbt_b200_status vbt_b200_index_put_rows_sorted(const vbt_b200_tensor* table,
                                               const vbt_b200_tensor* idx,
                                               const vbt_b200_tensor* values, int32_t policy,
                                               void* index_status, void* workspace,
                                               size_t workspace_bytes, void* stream);
/* The reference's CUDA advanced-index pattern: one index tensor applied to the LAST dim
 * (indexing_advanced_cuda.cu:2139-2177): out[b, k] = src[b, idx[k]]; src [B, K0] strided. */
VBT_B200_API vbt_b200_status vbt_b200_index_lastdim(const vbt_b200_tensor* out, const vbt_b200_tensor* src,
                                       const vbt_b200_tensor* idx, int32_t policy,
                                       void* index_status, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_index_put_lastdim(const vbt_b200_tensor* self, const vbt_b200_tensor* idx,
                                           const vbt_b200_tensor* values, int32_t accumulate,
                                           int32_t policy, void* index_status, void* stream);
/* vt::embedding forward (F32 weight [V, D] with non-negative strides, I64 contiguous
 * indices, STRICT policy) and the dense-gradient backward gw[idx[i], :] += grad[i, :],
 * skipping rows whose index equals padding_idx (embedding_cuda.cu:66-87). */
VBT_B200_API vbt_b200_status vbt_b200_embedding(const vbt_b200_tensor* out, const vbt_b200_tensor* weight,
                                   const vbt_b200_tensor* idx, void* index_status, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_embedding_backward(const vbt_b200_tensor* grad_weight,
                                            const vbt_b200_tensor* idx,
                                            const vbt_b200_tensor* grad_out, int64_t padding_idx,
                                            void* index_status, void* stream);
/* The same with scale_grad_by_freq: every row's gradient is divided by the number of times the
 * row occurs in idx (padding excluded) -- embedding_count_by_freq_i64_kernel +
 * embedding_backward_accum_scaled_f32_kernel (embedding_cuda.cu:89-131).  `counts` is scratch,
 * 4 bytes per weight row, cleared by the call. */
VBT_B200_API vbt_b200_status vbt_b200_embedding_backward_by_freq(const vbt_b200_tensor* grad_weight,
                                                    const vbt_b200_tensor* idx,
                                                    const vbt_b200_tensor* grad_out, int64_t padding_idx,
                                                    void* counts, size_t counts_bytes,
                                                    void* index_status, void* stream);
/* Boolean mask -> ascending INT64 indices of its true elements, on the stream, without a host
 * pass over the mask.  Replaces the reference's bool-mask front end of advanced indexing
 * (indexing_advanced_cuda.cu:2191-2429: CUB count + select, or D2H mask / host scan / H2D
 * indices).  mask: BOOL, rank 1, any non-negative stride.  *count_out (device, 8 bytes)
 * receives the number of true elements; positions are written to out_indices[0 .. min(count,
 * capacity)).  Either call once with capacity = mask length, or call with capacity = 0, read
 * the count, allocate, and call again.  workspace: 8-byte aligned, size from
 * vbt_b200_mask_select_workspace_bytes(mask length).  The indices feed vbt_b200_index_lastdim /
 * vbt_b200_index_rows like any other index tensor. */
VBT_B200_API vbt_b200_status vbt_b200_mask_select_workspace_bytes(int64_t n, size_t* bytes);
VBT_B200_API vbt_b200_status vbt_b200_mask_select(const vbt_b200_tensor* mask, int64_t* out_indices,
                                     int64_t capacity, uint64_t* count_out, void* workspace,
                                     size_t workspace_bytes, void* stream);
/* Synchronises `stream`, reads the status block; OK if count == 0, else OUT_OF_RANGE with
 * message "<what>: index out of range ..." and clears the block. */
VBT_B200_API vbt_b200_status vbt_b200_index_status_check(void* index_status, const char* what, int64_t dim_size,
                                            void* stream);

/* =====================================================================================
 * 4. Row ops
 *    replaces: Triton softmax_kernel + host wrapper (vibe_kernels/softmax/vbt_native.py:39-97,
 *    :193-259), log_softmax (:262-328) and Triton _rmsnorm_fwd_kernel + host wrapper
 *    (vibe_kernels/rmsnorm/vbt_native.py:55-103, :340-406).  One global read and one
 *    global write per element.  x is [rows, cols] with column stride 1 and any row stride;
 *    out dense, same dtype (F32, BF16, F16); math in FP32.
 *    softmax:  m = max x;  s = max(sum exp(x-m), 1e-20);  y = exp(x-m)/s
 *    rmsnorm:  r = rsqrt(sum x^2 / cols + eps);  y = x*r*gamma;  inv_rms[row] = r
 *              gamma: F32 [cols] or NULL;  inv_rms: F32 [rows] or NULL.
 * ===================================================================================== */
VBT_B200_API vbt_b200_status vbt_b200_softmax(void* out, const void* x, int32_t dtype, int64_t rows,
                                 int64_t cols, int64_t x_row_stride, int32_t log_softmax,
                                 void* stream);
VBT_B200_API vbt_b200_status vbt_b200_rmsnorm(void* out, float* inv_rms, const void* x, const float* gamma,
                                 int32_t dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                 float eps, void* stream);

/* Backward of the row ops.  dy and y / x are [rows, cols] with column stride 1 and any row
 * stride, dx is dense, all of one dtype (F32, BF16, F16); math in FP32.
 *   softmax_backward      dx = y * (dy - sum(dy*y));  log_softmax: dx = dy - exp(y)*sum(dy)
 *                         (SoftmaxBackward / LogSoftmaxBackward of
 *                         vibe_kernels/softmax/impl/cutedsl_softmax/softmax.py:236-423, :640-828)
 *   rmsnorm_backward      n = x*inv_rms; dx = inv_rms*(dy*gamma - n*mean(dy*gamma*n));
 *                         dgamma[c] = sum over rows of dy*n  (F32 [cols], or NULL to skip)
 *                         replaces Triton _rmsnorm_bwd_kernel + host wrapper
 *                         (vibe_kernels/rmsnorm/vbt_native.py:110-176, :409-492), whose dgamma
 *                         is a float atomic per element; here per-block partial rows in
 *                         `workspace` (F32, 16-byte aligned; size from
 *                         vbt_b200_rmsnorm_backward_workspace_bytes for the device the call
 *                         runs on; only needed when dgamma != NULL) are folded in a fixed order
 *                         by a second launch, so dgamma is reproducible run to run.          */
VBT_B200_API vbt_b200_status vbt_b200_softmax_backward(void* dx, const void* dy, const void* y, int32_t dtype,
                                          int64_t rows, int64_t cols, int64_t dy_row_stride,
                                          int64_t y_row_stride, int32_t log_softmax, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_rmsnorm_backward_workspace_bytes(int64_t rows, int64_t cols, int32_t dtype,
                                                          int32_t device, size_t* bytes);
VBT_B200_API vbt_b200_status vbt_b200_rmsnorm_backward(void* dx, float* dgamma, const void* dy, const void* x,
                                          const float* inv_rms, const float* gamma, int32_t dtype,
                                          int64_t rows, int64_t cols, int64_t dy_row_stride,
                                          int64_t x_row_stride, void* workspace, size_t workspace_bytes,
                                          void* stream);

/* =====================================================================================
 * 5. Fabric: sharded reductions and elementwise on a row-sharded tensor
 *    sits behind FabricTensor.sharded_1d_row (python/vibetensor/fabric.py:483-533) and
 *    replaces fabric_binary_kernel (src/vbt/cuda/fabric_elementwise.cu:122-162).
 *    Each rank reduces its own shard to an FP32 (or I64) partial with the call below;
 *    the ranks' partials are then combined by an NCCL all-reduce on the same stream, and
 *    MEAN is finished with vbt_b200_scale_cast once the global row count is known.
 *    vbt_b200_binary / vbt_b200_unary accept pointers into a peer GPU's memory for the
 *    INPUTS (plain loads over NVLink, as the reference's Fabric kernel does); outputs
 *    must be local.
 * ===================================================================================== */
/* Lets kernels launched on `compute_device` load from `peer_device` memory: the step the
 * reference performs before a cross-device fabric op (enable_peer_access_or_throw,
 * src/vbt/cuda/fabric_elementwise.cu:255-279).  Idempotent.  RUNTIME_ERROR when the two
 * devices have no P2P path.  Passing a peer pointer to an elementwise entry WITHOUT this
 * (or the host framework's equivalent) is an invalid-address fault, so bindings must call it
 * first. */
VBT_B200_API vbt_b200_status vbt_b200_enable_peer_access(int32_t compute_device, int32_t peer_device);
/* vt::fabric_add / vt::fabric_mul (any binary op code is accepted): a and b have equal shapes
 * and dtypes and may live on two GPUs of this process
 * (vbt_cuda_fabric_{add,mul}_impl(a, b, compute_device, require_fabric, use_copy_fallback),
 * src/vbt/cuda/fabric_elementwise.cu:820-1042, :1052-1115).
 *   same device            the ordinary op there                          *mode = FK_LOCAL
 *   two devices, P2P       compute_device (one of the two; owns `out`) reads the remote operand
 *                          in place with loads over NVLink                *mode = FK_PEER_LOAD
 *   two devices, no P2P    use_copy_fallback != 0 and require_fabric == 0: the remote operand
 *                          (contiguous) is copied into `scratch` (numel * itemsize bytes on
 *                          compute_device) and the op runs locally       *mode = FK_COPY_FALLBACK
 *                          otherwise RUNTIME_ERROR "[Fabric] ...: peer access not available ..."
 * use_copy_fallback == 2 takes the copy path even when P2P exists (the reference's dry-run
 * mode), for comparing the two.  Errors carry the reference's "[Fabric] " prefix. */
VBT_B200_API vbt_b200_status vbt_b200_fabric_binary(int32_t op, const vbt_b200_tensor* out,
                                       const vbt_b200_tensor* a, const vbt_b200_tensor* b,
                                       int32_t compute_device, int32_t require_fabric,
                                       int32_t use_copy_fallback, void* scratch, size_t scratch_bytes,
                                       int32_t* mode_out, void* stream);
/* partial (F32/I64, dense, reduced shape) = local SUM/MAX/MIN of the shard; BF16/F16
 * shards accumulate and emit FP32.  Workspace as for vbt_b200_reduce.  flags:
 *   VBT_B200_PARTIAL_WS_ZEROED  the vbt_b200_reduce_zeroed_ws contract holds for `workspace`
 *   VBT_B200_PARTIAL_NOT_FIRST  the shard does not hold the first element of the global
 *                               tensor: MAX / MIN then skip the "a NaN at position 0 wins" rule,
 *                               which belongs to the global position 0 only */
#define VBT_B200_PARTIAL_WS_ZEROED 1
#define VBT_B200_PARTIAL_NOT_FIRST 2
VBT_B200_API vbt_b200_status vbt_b200_reduce_partial(int32_t op, const vbt_b200_tensor* partial,
                                        const vbt_b200_tensor* shard, const int64_t* dims,
                                        int32_t ndims, int32_t keepdim, void* workspace,
                                        size_t workspace_bytes, int32_t flags, void* stream);
/* ---- the fused form: local reduction + cross-GPU combine + scale + cast in ONE launch ----
 * Each rank owns an exchange buffer; ranks swap a handle to it once and map each other's
 * buffer (IPC between processes, plain peer access between GPUs of one process).  After that
 * vbt_b200_reduce_exchange is the whole sharded reduction: the block that finishes a tile of
 * the local result writes every value, as one 8-byte word that also holds the call's epoch,
 * into every rank's buffer with peer stores over NVLink, reads its own buffer until all ranks'
 * words carry that epoch -- at most a few seconds, then it records an error instead -- folds
 * the `world` values in rank order (so every rank ends with the same bits), scales, casts and
 * stores.  No collective library call and no kernel behind it.
 * All ranks must make the same sequence of calls on a comm (as with any collective).
 *
 * vbt_b200_fabric_comm_create is the one place in this library that allocates device memory
 * (cudaMalloc of 2*world*slot_floats*8 + 256 bytes, at set-up; freed by _destroy).
 * slot_floats bounds the number of output elements of a fused call. */
#define VBT_B200_FABRIC_MAX_RANKS 8
#define VBT_B200_FABRIC_HANDLE_BYTES 128
typedef struct vbt_b200_fabric_comm vbt_b200_fabric_comm;
VBT_B200_API vbt_b200_status vbt_b200_fabric_comm_create(int32_t device, int32_t rank, int32_t world,
                                            size_t slot_floats, vbt_b200_fabric_comm** out);
/* handle_out: VBT_B200_FABRIC_HANDLE_BYTES bytes to hand to every other rank. */
VBT_B200_API vbt_b200_status vbt_b200_fabric_comm_handle(const vbt_b200_fabric_comm* comm, void* handle_out);
/* handles: world * VBT_B200_FABRIC_HANDLE_BYTES bytes, rank r's handle at offset r * BYTES.
 * RUNTIME_ERROR when a peer's buffer cannot be mapped (no P2P path, IPC refused). */
VBT_B200_API vbt_b200_status vbt_b200_fabric_comm_connect(vbt_b200_fabric_comm* comm, const void* handles);
/* Synchronises `stream` and reports (RUNTIME_ERROR) if an exchange on this rank gave up waiting. */
VBT_B200_API vbt_b200_status vbt_b200_fabric_comm_status(vbt_b200_fabric_comm* comm, void* stream);
VBT_B200_API vbt_b200_status vbt_b200_fabric_comm_destroy(vbt_b200_fabric_comm* comm);
/* out (F32/BF16/F16, dense, reduced shape) = cast(scale * combine over ranks of the local
 * SUM/MAX/MIN of `shard`).  Supported layouts: everything reduced to one value, and reductions
 * over the leading dim(s) of a tensor whose last kept dim is contiguous (mean(dim=0) of a
 * row-sharded matrix); others return INVALID_ARGUMENT and the caller uses
 * vbt_b200_reduce_partial + an all-reduce.  flags: VBT_B200_PARTIAL_WS_ZEROED.
 * first_owner_rank: the rank whose shard holds global row 0 (its NaN-at-position-0 rule is the
 * one that counts for MAX / MIN). */
VBT_B200_API vbt_b200_status vbt_b200_reduce_exchange(int32_t op, const vbt_b200_tensor* out,
                                         const vbt_b200_tensor* shard, const int64_t* dims,
                                         int32_t ndims, int32_t keepdim, void* workspace,
                                         size_t workspace_bytes, int32_t flags,
                                         vbt_b200_fabric_comm* comm, int32_t first_owner_rank,
                                         float scale, void* stream);
/* out[i] = cast(partial[i] * scale): the "divide by the global N and cast" step of a
 * sharded mean.  partial F32 [n]; out F32/BF16/F16 [n]. */
VBT_B200_API vbt_b200_status vbt_b200_scale_cast(void* out, int32_t out_dtype, const float* partial, int64_t n,
                                    float scale, void* stream);

/* =====================================================================================
 * 6. Observability
 *    stands in for the reference's test hooks and counters: TensorIterStats
 *    (cuda_ti_kernel_launches, num_32bit_splits; include/vbt/core/tensor_iterator/core.h:559-600)
 *    and CudaReductionLastStats (selected kernel, grid, block, slice length, workspace bytes;
 *    include/vbt/cuda/reduction_env.h:97-138).  Host-side bookkeeping only: nothing here
 *    touches the device.
 * ===================================================================================== */
#define VBT_B200_FAMILY_NONE 0
#define VBT_B200_FAMILY_ELEMENTWISE 1
#define VBT_B200_FAMILY_REDUCE 2
#define VBT_B200_FAMILY_INDEX 3
#define VBT_B200_FAMILY_ROWOP 4
#define VBT_B200_FAMILY_FABRIC 5
#define VBT_B200_FAMILY_COUNT 6
/* `kernel` values.  ELEMENTWISE: the codes of vbt_b200_ti_plan (0 flat, 1 tiled vector,
 * 2 tiled scalar, 3 transposing).  REDUCE: */
#define VBT_B200_RK_ROW_WARP 1     /* one warp per output                                   */
#define VBT_B200_RK_ROW_BLOCK 2    /* `splits` blocks per output, ticket fold                */
#define VBT_B200_RK_COL 3          /* column tiles, `splits` blocks along the reduced dim   */
#define VBT_B200_RK_COL_CLUSTER 4  /* the same folded inside a thread-block cluster         */
#define VBT_B200_RK_GENERIC 5
#define VBT_B200_RK_FILL 6         /* empty reduction domain: constant fill                 */
#define VBT_B200_RK_ROW_ONCE 7     /* a 128-thread block per slice, one unrolled pass       */
/* INDEX: */
#define VBT_B200_IK_ROWS_COPY 1
#define VBT_B200_IK_ROWS_COPY_ELEM 2
#define VBT_B200_IK_SCATTER_ADD 3
#define VBT_B200_IK_SCATTER_ADD_ELEM 4
#define VBT_B200_IK_SCATTER_ADD_SORTED 5
#define VBT_B200_IK_LASTDIM 6
#define VBT_B200_IK_LASTDIM_STAGED 7  /* rows staged in shared memory by bulk copies, index
                                         list in registers; `splits` = pieces per row       */
#define VBT_B200_IK_MASK_SELECT 8
#define VBT_B200_IK_LASTDIM_WIDE 9    /* 4-byte rows of up to 65 536 elements: outputs in registers,
                                         all shared memory for the row; `splits` = pieces   */
/* ROWOP: */
#define VBT_B200_WK_GROUP 1
#define VBT_B200_WK_BLOCK 2
#define VBT_B200_WK_STREAM 3
#define VBT_B200_WK_BACKWARD 4
#define VBT_B200_WK_SCALE_CAST 5
/* FABRIC: */
#define VBT_B200_FK_PEER_LOAD 1      /* the elementwise kernel reads the peer operand over NVLink */
#define VBT_B200_FK_COPY_FALLBACK 2  /* peer operand copied to local scratch first           */
#define VBT_B200_FK_LOCAL 3          /* both operands on the compute device                  */

typedef struct vbt_b200_launch_info {
  int32_t family;           /* VBT_B200_FAMILY_*; NONE when the call launched nothing         */
  int32_t kernel;           /* per-family code above (the call's main kernel)                 */
  uint32_t grid[3];
  uint32_t block[3];
  int32_t vec;              /* elements per vector access                                     */
  int32_t splits;           /* reductions: blocks that share one output                       */
  int32_t cluster;          /* thread-block cluster size, 0 = none                            */
  int32_t launches;         /* stream operations the call enqueued (kernels + memsets/copies) */
  int64_t out_numel;
  int64_t slice_len;        /* reductions: reduced extent; indexing: indices                  */
  uint64_t workspace_bytes; /* scratch bytes the launch used                                  */
  void* stream;
} vbt_b200_launch_info;

/* What the last successful launching call on the CALLING THREAD enqueued. */
VBT_B200_API vbt_b200_status vbt_b200_last_launch_info(vbt_b200_launch_info* out);
VBT_B200_API void vbt_b200_reset_last_launch_info(void);
/* Process-wide launch counts per family (counts[f], f < VBT_B200_FAMILY_COUNT) since load or
 * the last reset. */
VBT_B200_API vbt_b200_status vbt_b200_launch_counts(uint64_t* counts, int32_t n);
VBT_B200_API void vbt_b200_reset_launch_counts(void);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* VBT_B200_H_ */
