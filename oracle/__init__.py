"""TEST INFRASTRUCTURE ONLY -- Python face of the CPU oracle.

Two checkers live here, both driven through ctypes on numpy arrays:

* ``port``  -- ``_build/libvbt_oracle.so``, the plain-C restatement in ``vbt_oracle.c``.
* ``ref``   -- ``_ref/libvbt_ref_cpu.so``, VibeTensor's own CPU sources compiled by
  ``build_ref.sh`` (present only where that build ran; the built file travels).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference legs
may import this package.  The product package never does.

bf16 / f16 arrays are carried as ``numpy.uint16`` bit patterns together with an explicit
dtype code (the ordinals of ``vbt::core::ScalarType``, include/vbt/core/dtype.h:19-30).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "_build", "libvbt_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libvbt_ref_cpu.so")

BOOL, I32, I64, F32, F16, BF16 = 0, 1, 2, 3, 4, 5
ITEMSIZE = {BOOL: 1, I32: 4, I64: 8, F32: 4, F16: 2, BF16: 2}
NP_STORAGE = {BOOL: np.uint8, I32: np.int32, I64: np.int64, F32: np.float32, F16: np.uint16,
              BF16: np.uint16}

UNARY = ["relu", "neg", "abs", "square", "exp", "log", "sqrt", "rsqrt", "sin", "cos", "tanh",
         "sigmoid", "silu", "gelu", "reciprocal", "sign", "floor", "ceil", "trunc", "round",
         "expm1", "log1p", "softplus", "relu6", "hardtanh",
         "exp2", "log2", "log10", "sinh", "cosh", "asinh", "acosh", "atanh", "tan", "asin", "acos",
         "atan", "erf", "erfc", "lgamma", "sinc", "frac", "deg2rad", "rad2deg", "mish", "selu", "elu",
         "hardsigmoid", "hardshrink", "softshrink", "logit", "angle", "positive", "sgn", "nan_to_num",
         "isfinite", "isinf", "isnan", "isneginf", "isposinf", "signbit", "logical_not", "bitwise_not"]
UNARY_TO_BOOL = {"isfinite", "isinf", "isnan", "isneginf", "isposinf", "signbit", "logical_not"}
BINARY = ["add", "sub", "mul", "div", "maximum", "minimum", "fmax", "fmin", "eq", "ne", "lt",
          "gt", "le", "ge",
          "pow", "fmod", "remainder", "atan2", "copysign", "hypot", "xlogy", "xlog1py", "logaddexp",
          "logaddexp2", "nextafter", "heaviside", "rsub", "tanh_backward", "sigmoid_backward",
          "silu_backward", "logit_backward", "mse_loss", "ldexp", "bitwise_and", "bitwise_or",
          "bitwise_xor", "lshift", "rshift", "gcd", "lcm", "logical_and", "logical_or", "logical_xor"]
BINARY_TO_BOOL = {"eq", "ne", "lt", "gt", "le", "ge", "logical_and", "logical_or", "logical_xor"}
TERNARY = ["clamp", "lerp", "threshold", "addcmul", "addcdiv", "where_gt0_addcmul", "huber_loss",
           "smooth_l1_loss"]
REDUCE = ["sum", "mean", "max", "min", "prod", "argmax", "argmin"]
WRAP, STRICT, CLAMP = 0, 1, 2

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i64p = ctypes.POINTER(ctypes.c_int64)
_int = ctypes.c_int


def build(ref_dir=None) -> None:
    """Compile the restatement (always) and, given a reference checkout (ref_dir, or
    VBT_REFERENCE_DIR in the environment), the reference's own CPU sources into _ref."""
    subprocess.run(["make", "-s", "-C", HERE, "_build/libvbt_oracle.so"], check=True)
    ref_dir = ref_dir or os.environ.get("VBT_REFERENCE_DIR")
    if ref_dir and os.path.isdir(os.path.join(ref_dir, "src", "vbt")):
        subprocess.run(["bash", os.path.join(HERE, "build_ref.sh"), ref_dir], check=True,
                       stdout=subprocess.DEVNULL)


def _arr(vals):
    vals = [int(v) for v in vals]
    return (ctypes.c_int64 * max(len(vals), 1))(*vals)


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def _estrides(a: np.ndarray):
    return [s // a.itemsize for s in a.strides]


# ----------------------------------------------------------------------------------------
# bf16 / f16 helpers (bit patterns in uint16)
# ----------------------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit pattern (NaN -> 0x7fff)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = 0x7FFF
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_storage(x: np.ndarray, dtype: int) -> np.ndarray:
    """float32 values -> storage array of the given dtype code."""
    if dtype == BF16:
        return f32_to_bf16_bits(x).reshape(x.shape)
    if dtype == F16:
        return np.asarray(x, dtype=np.float16).view(np.uint16)
    return np.asarray(x, dtype=NP_STORAGE[dtype])


def to_f32(a: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == BF16:
        return bf16_bits_to_f32(np.ascontiguousarray(a)).reshape(a.shape)
    if dtype == F16:
        return np.ascontiguousarray(a).view(np.float16).astype(np.float32)
    return np.asarray(a, dtype=np.float32)


# ----------------------------------------------------------------------------------------
# the plain-C restatement
# ----------------------------------------------------------------------------------------
class Port:
    def __init__(self):
        if not os.path.exists(PORT_SO):
            build(ref=False)
        L = ctypes.CDLL(PORT_SO)
        L.vbo_elementwise.argtypes = [_int, _int, _int, _int, _i64p, _vp, _i64p, _vp, _i64p, _vp,
                                      _i64p, _vp, _i64p]
        L.vbo_reduce.argtypes = [_int, _int, _int, _i64, _i64, _i64, _vp, _vp, _vp]
        L.vbo_gather_rows.argtypes = [_int, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _int, _vp]
        L.vbo_scatter_rows.argtypes = [_int, _i64, _i64, _vp, _vp, _i64, _vp, _int, _int, _int, _i64]
        L.vbo_embedding_backward_by_freq.argtypes = [_i64, _i64, _vp, _vp, _i64, _vp, _int, _i64]
        L.vbo_index_lastdim.argtypes = [_int, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _int, _vp]
        L.vbo_index_put_lastdim.argtypes = [_int, _i64, _i64, _vp, _vp, _i64, _vp, _int, _int]
        L.vbo_softmax.argtypes = [_int, _i64, _i64, _vp, _i64, _vp, _int]
        L.vbo_rmsnorm.argtypes = [_int, _i64, _i64, _vp, _i64, _vp, ctypes.c_float, _vp, _vp]
        L.vbo_softmax_backward.argtypes = [_int, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _int]
        L.vbo_rmsnorm_backward.argtypes = [_int, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp]
        L.vbo_scale_cast.argtypes = [_int, _vp, _i64, ctypes.c_float, _vp]
        L.vbo_offset_elems.argtypes = [_i64, _int, _i64p, _i64p]
        L.vbo_offset_elems.restype = _i64
        self.L = L

    # -- elementwise -------------------------------------------------------------------
    def _ew(self, kind, op, dtype, out, ins):
        shape = out.shape
        bc = [np.broadcast_to(a, shape) if a is not None else None for a in ins]
        args = []
        for a in bc + [None] * (3 - len(bc)):
            if a is None:
                args += [None, _arr([0])]
            else:
                args += [_ptr(a), _arr(_estrides(a))]
        rc = self.L.vbo_elementwise(kind, op, dtype, out.ndim, _arr(shape), _ptr(out),
                                    _arr(_estrides(out)), *args)
        if rc:
            raise ValueError(f"oracle elementwise rejected kind={kind} op={op} dtype={dtype}")
        return out

    def _out_like(self, dtype, arrays, out, out_dtype=None):
        shape = np.broadcast_shapes(*[a.shape for a in arrays])
        if out is None:
            out = np.zeros(shape, NP_STORAGE[dtype if out_dtype is None else out_dtype])
        assert tuple(out.shape) == tuple(shape)
        return out

    def unary(self, name, a, dtype, out=None):
        out = self._out_like(dtype, [a], out, BOOL if name in UNARY_TO_BOOL else None)
        return self._ew(0, UNARY.index(name), dtype, out, [a])

    def binary(self, name, a, b, dtype, out=None):
        op = BINARY.index(name)
        out = self._out_like(dtype, [a, b], out, BOOL if name in BINARY_TO_BOOL else None)
        return self._ew(1, op, dtype, out, [a, b])

    def ternary(self, name, a, b, c, dtype, out=None):
        out = self._out_like(dtype, [a, b, c], out)
        return self._ew(2, TERNARY.index(name), dtype, out, [a, b, c])

    def where(self, cond, x, y, dtype, out=None):
        out = self._out_like(dtype, [cond, x, y], out)
        return self._ew(3, 0, dtype, out, [cond.view(np.uint8), x, y])

    def copy(self, a, dtype, out):
        return self._ew(4, 0, dtype, out, [a])

    # -- reductions ----------------------------------------------------------------------
    def reduce(self, name, x, dtype, dim=None, keepdim=False, out_dtype=None):
        """Single-dim (or all, dim=None) reduction.  Non-contiguous input is cloned first,
        as reduce_value_cpu does (src/vbt/python/tensor_bindings.cc:469-472)."""
        op = REDUCE.index(name)
        x = np.ascontiguousarray(x)
        if dim is None:
            outer, n, inner = 1, x.size, 1
            oshape = ()
        else:
            d = dim % x.ndim
            outer = int(np.prod(x.shape[:d], dtype=np.int64))
            n = x.shape[d]
            inner = int(np.prod(x.shape[d + 1:], dtype=np.int64))
            oshape = x.shape[:d] + ((1,) if keepdim else ()) + x.shape[d + 1:]
        if out_dtype is None:
            out_dtype = dtype
        vals = np.zeros(oshape, NP_STORAGE[out_dtype])
        idx = np.zeros(oshape, np.int64) if op >= 5 else None
        rc = self.L.vbo_reduce(op, dtype, out_dtype, outer, n, inner, _ptr(x), _ptr(vals),
                               _ptr(idx) if idx is not None else None)
        if rc == 2:
            raise RuntimeError(("amin" if name in ("min", "argmin") else "amax") + ": empty")
        if rc:
            raise ValueError(f"oracle reduce rejected {name} dtype={dtype}")
        return (vals, idx) if idx is not None else vals

    # -- indexing ------------------------------------------------------------------------
    def gather_rows(self, table, idx, policy=WRAP):
        V, D = table.shape
        s0, s1 = _estrides(table)
        idx = np.ascontiguousarray(idx, np.int64)
        out = np.zeros(idx.shape + (D,), table.dtype)
        rc = self.L.vbo_gather_rows(table.itemsize, V, D, _ptr(table), s0, s1, _ptr(idx), idx.size,
                                    policy, _ptr(out))
        if rc:
            raise IndexError("index out of range")
        return out

    def scatter_rows(self, table, idx, values, dtype, accumulate=True, policy=WRAP,
                     padding_idx=None):
        assert table.flags.c_contiguous and values.flags.c_contiguous
        V, D = table.shape
        idx = np.ascontiguousarray(idx, np.int64)
        rc = self.L.vbo_scatter_rows(dtype, V, D, _ptr(table), _ptr(idx), idx.size, _ptr(values),
                                     int(accumulate), policy, int(padding_idx is not None),
                                     int(padding_idx or 0))
        if rc == 3:
            raise IndexError("index out of range")
        if rc:
            raise ValueError("oracle scatter rejected dtype")
        return table

    def embedding_backward_by_freq(self, grad, idx, num_weights, padding_idx=None):
        grad = np.ascontiguousarray(grad, np.float32)
        idx = np.ascontiguousarray(idx, np.int64)
        gw = np.zeros((num_weights, grad.shape[1]), np.float32)
        rc = self.L.vbo_embedding_backward_by_freq(num_weights, grad.shape[1], _ptr(gw), _ptr(idx), idx.size,
                                                   _ptr(grad), int(padding_idx is not None), int(padding_idx or 0))
        if rc:
            raise IndexError("index out of range")
        return gw

    def index_lastdim(self, src, idx, policy=WRAP):
        B, K0 = src.shape
        sb, sk = _estrides(src)
        idx = np.ascontiguousarray(idx, np.int64)
        out = np.zeros((B, idx.size), src.dtype)
        rc = self.L.vbo_index_lastdim(src.itemsize, B, K0, _ptr(src), sb, sk, _ptr(idx), idx.size,
                                      policy, _ptr(out))
        if rc:
            raise IndexError("index out of range")
        return out

    def index_put_lastdim(self, self_, idx, values, dtype, accumulate, policy=WRAP):
        assert self_.flags.c_contiguous and values.flags.c_contiguous
        B, K0 = self_.shape
        idx = np.ascontiguousarray(idx, np.int64)
        rc = self.L.vbo_index_put_lastdim(dtype, B, K0, _ptr(self_), _ptr(idx), idx.size,
                                          _ptr(values), int(accumulate), policy)
        if rc == 3:
            raise IndexError("index out of range")
        if rc:
            raise ValueError("oracle index_put rejected dtype")
        return self_

    # -- row ops -------------------------------------------------------------------------
    def softmax(self, x, dtype, log=False):
        assert x.ndim == 2 and x.strides[1] == x.itemsize
        out = np.zeros(x.shape, x.dtype)
        self.L.vbo_softmax(dtype, x.shape[0], x.shape[1], _ptr(x), _estrides(x)[0], _ptr(out),
                           int(log))
        return out

    def rmsnorm(self, x, gamma, eps, dtype):
        assert x.ndim == 2 and x.strides[1] == x.itemsize
        out = np.zeros(x.shape, x.dtype)
        inv = np.zeros(x.shape[0], np.float32)
        g = None if gamma is None else np.ascontiguousarray(gamma, np.float32)
        self.L.vbo_rmsnorm(dtype, x.shape[0], x.shape[1], _ptr(x), _estrides(x)[0],
                           _ptr(g) if g is not None else None, float(eps), _ptr(out), _ptr(inv))
        return out, inv

    def softmax_backward(self, dy, y, dtype, log=False):
        assert dy.shape == y.shape and y.ndim == 2
        assert dy.strides[1] == dy.itemsize and y.strides[1] == y.itemsize
        dx = np.zeros(y.shape, y.dtype)
        self.L.vbo_softmax_backward(dtype, y.shape[0], y.shape[1], _ptr(dy), _estrides(dy)[0], _ptr(y),
                                    _estrides(y)[0], _ptr(dx), int(log))
        return dx

    def rmsnorm_backward(self, dy, x, inv_rms, gamma, dtype):
        assert dy.shape == x.shape and x.ndim == 2
        assert dy.strides[1] == dy.itemsize and x.strides[1] == x.itemsize
        dx = np.zeros(x.shape, x.dtype)
        inv = np.ascontiguousarray(inv_rms, np.float32)
        g = None if gamma is None else np.ascontiguousarray(gamma, np.float32)
        dg = None if gamma is None else np.zeros(x.shape[1], np.float32)
        self.L.vbo_rmsnorm_backward(dtype, x.shape[0], x.shape[1], _ptr(dy), _estrides(dy)[0], _ptr(x),
                                    _estrides(x)[0], _ptr(inv), _ptr(g) if g is not None else None,
                                    _ptr(dx), _ptr(dg) if dg is not None else None)
        return dx, dg

    def scale_cast(self, partial, scale, out_dtype):
        partial = np.ascontiguousarray(partial, np.float32)
        out = np.zeros(partial.shape, NP_STORAGE[out_dtype])
        self.L.vbo_scale_cast(out_dtype, _ptr(partial), partial.size, float(scale), _ptr(out))
        return out

    def offset_elems(self, linear, sizes, strides):
        return self.L.vbo_offset_elems(int(linear), len(sizes), _arr(sizes), _arr(strides))

    # The tail of the elementwise table, restated in numpy (elementwise, a handful of operations per
    # element; numpy rounds every float32 / float64 operation separately, which is what the reference's
    # expressions do without contraction).
    @staticmethod
    def complex_binary(name, a, b):
        """vt::add / vt::mul on Complex64 / Complex128 (src/vbt/ops/cuda_elementwise.cu:162-190):
        add = (a.re + b.re, a.im + b.im); mul = (a.re*b.re - a.im*b.im, a.re*b.im + a.im*b.re)."""
        a, b = np.broadcast_arrays(np.asarray(a), np.asarray(b))
        assert a.dtype == b.dtype and a.dtype in (np.complex64, np.complex128)
        f = np.float32 if a.dtype == np.complex64 else np.float64
        ar, ai, br, bi = (np.ascontiguousarray(v, f) for v in (a.real, a.imag, b.real, b.imag))
        if name == "add":
            re, im = ar + br, ai + bi
        elif name == "mul":
            re, im = ar * br - ai * bi, ar * bi + ai * br
        else:
            raise ValueError(f"vt::{name}: unsupported dtype")
        out = np.empty(a.shape, a.dtype)
        out.real, out.imag = re, im
        return out

    @staticmethod
    def polygamma(n, x, dtype):
        """vt::polygamma (src/vbt/ops/cuda_elementwise.cu:1288-1330): only order 2 is computed, in
        double: NaN at the poles and below -1e6; psi''(x) -= 2/x^3, x += 1 while x < 10 (at most 100
        steps); then -1/x^2 - 1/x^3 - 1/(2 x^4); rounded to the tensor's dtype.  x in storage form."""
        xs = np.asarray(x)
        xf = to_f32(xs, dtype).astype(np.float64)
        nan = np.full(xf.shape, np.nan)
        if float(n) != 2.0:
            return to_storage(nan.astype(np.float32), dtype)
        xx = xf.copy()
        bad = ((xx <= 0.0) & (xx == np.floor(xx))) | (xx < -1e6) | np.isnan(xx)
        xx[bad] = 1.0
        acc = np.zeros_like(xx)
        for _ in range(100):
            m = xx < 10.0
            if not m.any():
                break
            acc[m] -= 2.0 / (xx[m] * xx[m] * xx[m])
            xx[m] += 1.0
        i1 = 1.0 / xx
        i2 = i1 * i1
        i3 = i2 * i1
        i4 = i3 * i1
        res = acc + (-i2 - i3 - 0.5 * i4)
        res[bad] = np.nan
        return to_storage(res.astype(np.float32), dtype)


# ----------------------------------------------------------------------------------------
# the reference's own CPU code
# ----------------------------------------------------------------------------------------
class Ref:
    """VibeTensor's CPU kernels, compiled from its sources (oracle/build_ref.sh)."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        L = ctypes.CDLL(REF_SO)
        L.vref_last_error.restype = ctypes.c_char_p
        L.vref_sum_mean.argtypes = [_int, _vp, _int, _int, _i64p, _i64p, _i64p, _int, _int, _vp]
        L.vref_minmax.argtypes = [_int, _vp, _int, _int, _i64p, _i64p, _i64, _vp, _vp]
        L.vref_elementwise.argtypes = [ctypes.c_char_p, _vp, _int, _int, _i64p, _i64p, _vp, _int,
                                       _int, _i64p, _i64p, _vp, _i64p, ctypes.POINTER(_int)]
        L.vref_index_rows.argtypes = [_vp, _int, _i64, _i64, _i64, _i64, _vp, _i64, _vp]
        L.vref_index_put_rows.argtypes = [_vp, _int, _i64, _i64, _vp, _i64, _vp, _int]
        L.vref_index_1d.argtypes = [_vp, _int, _i64, _vp, _i64, _vp]
        L.vref_index_put_1d.argtypes = [_vp, _int, _i64, _vp, _i64, _vp, _int]
        L.vref_embedding.argtypes = [_vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]
        self.L = L

    def _check(self, rc):
        if rc == 0:
            return
        msg = self.L.vref_last_error().decode()
        raise {1: ValueError, 2: RuntimeError, 3: IndexError}.get(rc, RuntimeError)(msg)

    def sum(self, x, dtype, dims=(), keepdim=False, mean=False):
        dims = list(dims)
        nd = [d % x.ndim for d in dims] if dims else list(range(x.ndim))
        oshape = tuple((1 if i in nd else s) for i, s in enumerate(x.shape) if keepdim or i not in nd)
        out = np.zeros(oshape, NP_STORAGE[dtype])
        self._check(self.L.vref_sum_mean(int(mean), _ptr(x), dtype, x.ndim, _arr(x.shape),
                                         _arr(_estrides(x)), _arr(dims), len(dims), int(keepdim),
                                         _ptr(out)))
        return out

    def minmax(self, kind, x, dtype, dim=None):
        """kind: 'amax' | 'amin' | 'argmax' -> values (and int64 indices for argmax)."""
        k = {"amax": 0, "amin": 1, "argmax": 2}[kind]
        if dim is None:
            oshape, d = (), -(2 ** 63)
        else:
            dd = dim % x.ndim
            oshape, d = x.shape[:dd] + x.shape[dd + 1:], dim
        vals = np.zeros(oshape, NP_STORAGE[dtype])
        idx = np.zeros(oshape, np.int64)
        self._check(self.L.vref_minmax(k, _ptr(x), dtype, x.ndim, _arr(x.shape), _arr(_estrides(x)),
                                       d, _ptr(vals), _ptr(idx)))
        return (vals, idx) if k == 2 else vals

    def elementwise(self, op, a, b, dtype, out_dtype=None):
        shape = np.broadcast_shapes(a.shape, b.shape) if b is not None else a.shape
        out = np.zeros(shape, NP_STORAGE[dtype if out_dtype is None else out_dtype])
        osz = (ctypes.c_int64 * 32)()
        ond = _int()
        self._check(self.L.vref_elementwise(
            ("vt::" + op).encode(), _ptr(a), dtype, a.ndim, _arr(a.shape), _arr(_estrides(a)),
            _ptr(b) if b is not None else None, dtype, b.ndim if b is not None else 0,
            _arr(b.shape) if b is not None else _arr([0]),
            _arr(_estrides(b)) if b is not None else _arr([0]), _ptr(out), osz, ctypes.byref(ond)))
        assert tuple(osz[:ond.value]) == tuple(shape)
        return out

    # The reference wraps negative indices IN PLACE in the caller's contiguous int64 index
    # tensor (indexing_advanced.cc:653-676), so every call here works on a private copy.
    def index_rows(self, table, idx, dtype):
        V, D = table.shape
        s0, s1 = _estrides(table)
        idx = np.array(idx, np.int64, copy=True)
        out = np.zeros((idx.size, D), table.dtype)
        self._check(self.L.vref_index_rows(_ptr(table), dtype, V, D, s0, s1, _ptr(idx), idx.size,
                                           _ptr(out)))
        return out

    def index_put_rows(self, table, idx, values, dtype, accumulate):
        assert table.flags.c_contiguous and values.flags.c_contiguous
        V, D = table.shape
        idx = np.array(idx, np.int64, copy=True)
        self._check(self.L.vref_index_put_rows(_ptr(table), dtype, V, D, _ptr(idx), idx.size,
                                               _ptr(values), int(accumulate)))
        return table

    def index_1d(self, x, idx, dtype):
        idx = np.array(idx, np.int64, copy=True)
        out = np.zeros(idx.size, x.dtype)
        self._check(self.L.vref_index_1d(_ptr(x), dtype, x.size, _ptr(idx), idx.size, _ptr(out)))
        return out

    def index_put_1d(self, x, idx, values, dtype, accumulate):
        idx = np.array(idx, np.int64, copy=True)
        self._check(self.L.vref_index_put_1d(_ptr(x), dtype, x.size, _ptr(idx), idx.size,
                                             _ptr(values), int(accumulate)))
        return x

    def embedding(self, weight, idx):
        V, D = weight.shape
        s0, s1 = _estrides(weight)
        idx = np.array(idx, np.int64, copy=True)
        out = np.zeros((idx.size, D), np.float32)
        self._check(self.L.vref_embedding(_ptr(weight), V, D, s0, s1, _ptr(idx), idx.size,
                                          _ptr(out)))
        return out


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref() -> Ref:
    global _ref
    if _ref is None:
        _ref = Ref()
    return _ref


def have_ref() -> bool:
    return os.path.exists(REF_SO)
