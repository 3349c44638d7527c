"""vt:: ops on CUDA tensors, served by libvbt_b200.so.

Mirrors the operator surface of the reference for this path -- ``vibetensor.torch.ops.vt.*``
(python/vibetensor/torch/ops.py:36-80) and the ``Tensor`` reduction / indexing methods
(src/vbt/python/tensor_bindings.cc:2219-2573) -- with the same argument meaning, dtype
rules and error classes.  Tensors are ``torch.Tensor`` objects on a CUDA device: torch
provides memory and the current stream, nothing else.  Every function launches on the
current stream and returns without synchronising, except where stated.

Each elementwise op also takes ``out=``: any strided view of the broadcast shape (the
reference allocates a dense result for every op, src/vbt/ops/cuda_elementwise.cu:96-110).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import check, desc, i64_array, lib, stream_ptr

UNARY = ["relu", "neg", "abs", "square", "exp", "log", "sqrt", "rsqrt", "sin", "cos", "tanh",
         "sigmoid", "silu", "gelu", "reciprocal", "sign", "floor", "ceil", "trunc", "round",
         "expm1", "log1p", "softplus", "relu6", "hardtanh",
         "exp2", "log2", "log10", "sinh", "cosh", "asinh", "acosh", "atanh", "tan", "asin", "acos",
         "atan", "erf", "erfc", "lgamma", "sinc", "frac", "deg2rad", "rad2deg", "mish", "selu", "elu",
         "hardsigmoid", "hardshrink", "softshrink", "logit", "angle", "positive", "sgn", "nan_to_num",
         "isfinite", "isinf", "isnan", "isneginf", "isposinf", "signbit", "logical_not", "bitwise_not"]
UNARY_TO_BOOL = {"isfinite", "isinf", "isnan", "isneginf", "isposinf", "signbit", "logical_not"}
BINARY = ["add", "sub", "mul", "div", "maximum", "minimum", "fmax", "fmin", "eq", "ne", "lt", "gt",
          "le", "ge",
          "pow", "fmod", "remainder", "atan2", "copysign", "hypot", "xlogy", "xlog1py", "logaddexp",
          "logaddexp2", "nextafter", "heaviside", "rsub", "tanh_backward", "sigmoid_backward",
          "silu_backward", "logit_backward", "mse_loss", "ldexp", "bitwise_and", "bitwise_or",
          "bitwise_xor", "lshift", "rshift", "gcd", "lcm", "logical_and", "logical_or", "logical_xor"]
BINARY_TO_BOOL = {"eq", "ne", "lt", "gt", "le", "ge", "logical_and", "logical_or", "logical_xor"}
TERNARY = ["clamp", "lerp", "threshold", "addcmul", "addcdiv", "where_gt0_addcmul", "huber_loss",
           "smooth_l1_loss"]
REDUCE = ["sum", "mean", "max", "min", "prod", "argmax", "argmin"]
INDEX_WRAP, INDEX_STRICT, INDEX_CLAMP = 0, 1, 2


_peer_enabled: set = set()  # (compute device index, peer device index) pairs opened so far


def enable_peer_access(compute_device: int, peer_device: int) -> None:
    """Allow kernels on ``compute_device`` to read ``peer_device`` memory (needed before an
    elementwise op takes an INPUT that lives on another GPU)."""
    check(lib().vbt_b200_enable_peer_access(int(compute_device), int(peer_device)))
    _peer_enabled.add((int(compute_device), int(peer_device)))


def _require_cuda(*ts: torch.Tensor) -> None:
    """All tensors on CUDA; the first one (the output, or the tensor the output is allocated
    like) fixes the compute device, and every other tensor must live there or on a device
    whose memory has been opened with enable_peer_access."""
    dev0 = None
    for t in ts:
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise ValueError("vibetensor_b200 ops take CUDA tensors (there is no CPU path)")
        if dev0 is None:
            dev0 = t.device.index
        elif t.device.index != dev0 and (dev0, t.device.index) not in _peer_enabled:
            raise ValueError(f"operand on cuda:{t.device.index} but the op computes on cuda:{dev0}: "
                             "call ops.enable_peer_access(compute_device, peer_device) first")


def _alloc_out(out, shape, dtype, like):
    """The library computes on the device that owns the output, and the launch goes to that
    device's current stream (every caller below passes stream_ptr(output))."""
    if out is None:
        return torch.empty(tuple(shape), dtype=dtype, device=like.device)
    if tuple(out.shape) != tuple(shape):
        raise ValueError("out= has the wrong shape for the broadcast result")
    return out


def _bshape(*ts):
    try:
        return torch.broadcast_shapes(*[tuple(t.shape) for t in ts])
    except RuntimeError:
        raise ValueError("shape mismatch: operands cannot be broadcast together") from None


# --------------------------------------------------------------------------------------
# elementwise
# --------------------------------------------------------------------------------------
def unary(name: str, a: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _require_cuda(*([out] if out is not None else []), a)
    o = _alloc_out(out, a.shape, torch.bool if name in UNARY_TO_BOOL else a.dtype, a)
    do, da = desc(o), desc(a)
    check(lib().vbt_b200_unary(UNARY.index(name), do.ref, da.ref, stream_ptr(o)))
    return o


def binary(name: str, a, b, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a, b: CUDA tensors of one dtype, or one of them a Python number (the reference's CPU
    0-d scalar operand, float32 / int64 tensors only)."""
    op = BINARY.index(name)
    cmp_ = name in BINARY_TO_BOOL
    a_t, b_t = isinstance(a, torch.Tensor), isinstance(b, torch.Tensor)
    if a_t and b_t:
        _require_cuda(*([out] if out is not None else []), a, b)
        o = _alloc_out(out, _bshape(a, b), torch.bool if cmp_ else a.dtype, a)
        do, da, db = desc(o), desc(a), desc(b)
        check(lib().vbt_b200_binary(op, do.ref, da.ref, db.ref, stream_ptr(o)))
        return o
    t, s, left = (a, b, False) if a_t else (b, a, True)
    _require_cuda(t)
    o = _alloc_out(out, t.shape, torch.bool if cmp_ else t.dtype, t)
    if t.dtype == torch.float32:
        sv = ctypes.c_float(float(s))
    elif t.dtype == torch.int64:
        sv = ctypes.c_int64(int(s))
    elif t.dtype == torch.float16:
        raise ValueError(f"vt::{name}: Half CPU scalars not supported yet")
    else:
        raise ValueError(f"vt::{name}: unsupported dtype for scalar op")
    do, dt_ = desc(o), desc(t)
    check(lib().vbt_b200_binary_scalar(op, do.ref, dt_.ref, ctypes.byref(sv), int(left), stream_ptr(o)))
    return o


def ternary(name: str, a, b, c, out=None) -> torch.Tensor:
    _require_cuda(*([out] if out is not None else []), a, b, c)
    o = _alloc_out(out, _bshape(a, b, c), a.dtype, a)
    do, da, db, dc = desc(o), desc(a), desc(b), desc(c)
    check(lib().vbt_b200_ternary(TERNARY.index(name), do.ref, da.ref, db.ref, dc.ref, stream_ptr(o)))
    return o


def where(cond, x, y, out=None) -> torch.Tensor:
    _require_cuda(*([out] if out is not None else []), x, cond, y)
    o = _alloc_out(out, _bshape(cond, x, y), x.dtype, x)
    do, dc, dx, dy = desc(o), desc(cond), desc(x), desc(y)
    check(lib().vbt_b200_where(do.ref, dc.ref, dx.ref, dy.ref, stream_ptr(o)))
    return o


def polygamma(n: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """vt::polygamma(n, x): n a one-element floating tensor of x's dtype on x's device.  As in the
    reference only order 2 is computed; other orders give NaN (cuda_elementwise.cu:1288-1330)."""
    _require_cuda(n, x)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    do, dn, dx = desc(out), desc(n), desc(x)
    check(lib().vbt_b200_polygamma(do.ref, dn.ref, dx.ref, stream_ptr(out)))
    return out


def masked_fill(self_, mask, value, out=None):
    """vt::masked_fill = where(mask, value, self) (cuda_elementwise.cu:3924-3926)."""
    return where(mask, value, self_, out=out)


def copy_(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """Strided copy (src broadcast to dst)."""
    _require_cuda(dst, src)
    dd, ds = desc(dst), desc(src)
    check(lib().vbt_b200_copy(dd.ref, ds.ref, stream_ptr(dst)))
    return dst


def contiguous(a: torch.Tensor) -> torch.Tensor:
    """clone_cuda: dense row-major copy of a strided view."""
    return copy_(torch.empty(a.shape, dtype=a.dtype, device=a.device), a)


def _mk_unary(n):
    def f(a, out=None):
        return unary(n, a, out=out)
    f.__name__ = n
    f.__doc__ = f"vt::{n}"
    return f


def _mk_binary(n):
    def f(a, b, out=None):
        return binary(n, a, b, out=out)
    f.__name__ = n
    f.__doc__ = f"vt::{n}"
    return f


def _mk_ternary(n):
    def f(a, b, c, out=None):
        return ternary(n, a, b, c, out=out)
    f.__name__ = n
    f.__doc__ = f"vt::{n}"
    return f


for _n in UNARY:
    globals()[_n if _n != "round" else "round_"] = _mk_unary(_n)
for _n in BINARY:
    globals()[_n] = _mk_binary(_n)
for _n in TERNARY:
    globals()[_n] = _mk_ternary(_n)
clamp_min = globals()["maximum"]   # cuda_elementwise.cu:3912-3917
clamp_max = globals()["minimum"]
clip = globals()["clamp"]
# names the reference registers on the same functors (cuda_elementwise.cu:3957-4276)
true_divide = globals()["div"]
celu = globals()["elu"]
conj_physical = globals()["positive"]
float_power = globals()["pow"]
special_xlog1py = globals()["xlog1py"]
bitwise_left_shift = globals()["lshift"]
bitwise_right_shift = globals()["rshift"]


def ti_plan(out: torch.Tensor, *inputs: torch.Tensor):
    """The iteration plan the library builds for (out, inputs): (shape, strides-per-operand,
    kernel kind, pieces), dims innermost first.  Host-only; works on any device's tensors."""
    ds = [desc(out)] + [desc(t) for t in inputs]
    arr = (ctypes.POINTER(_lib.VbtTensor) * len(ds))(*[ctypes.pointer(d.struct) for d in ds])
    shape = (ctypes.c_int64 * _lib.MAX_NDIM)()
    strides = (ctypes.c_int64 * (_lib.MAX_NDIM * len(ds)))()
    nd, kern, pieces = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    check(lib().vbt_b200_ti_plan(arr, len(ds), shape, strides, ctypes.byref(nd), ctypes.byref(kern),
                                 ctypes.byref(pieces)))
    n = nd.value
    return (list(shape[:n]),
            [list(strides[k * _lib.MAX_NDIM:k * _lib.MAX_NDIM + n]) for k in range(len(ds))],
            kern.value, pieces.value)


# --------------------------------------------------------------------------------------
# reductions
# --------------------------------------------------------------------------------------
def _norm_dims(dim) -> list:
    if dim is None:
        return []
    if isinstance(dim, int):
        return [dim]
    return list(dim)


def reduce_shape(x: torch.Tensor, dims: Sequence[int], keepdim: bool):
    dx = desc(x)
    out = (ctypes.c_int64 * _lib.MAX_NDIM)()
    nd = ctypes.c_int32()
    check(lib().vbt_b200_reduce_shape(dx.ref, i64_array(dims), len(dims), int(keepdim), out,
                                      ctypes.byref(nd)))
    return tuple(out[:nd.value])


_ws_cache: dict = {}
_reduce_ws_cache: dict = {}


def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    """General scratch (contents undefined).  One buffer per (device, stream), grown on demand
    and reused: work on one stream is ordered, so successive calls cannot overlap."""
    if nbytes == 0:
        return None
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


def _reduce_workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    """Scratch of the split reductions, one per (device, stream) like the buffer above but used
    by reductions only and ZEROED when it is created: the kernels return its ticket counters to
    zero, so no call has to clear them (vbt_b200_reduce_zeroed_ws)."""
    if nbytes == 0:
        return None
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _reduce_ws_cache.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 4 << 20), dtype=torch.uint8, device=device)
        _reduce_ws_cache[key] = ws
    return ws


def reduce(name: str, x: torch.Tensor, dim=None, keepdim: bool = False,
           out_dtype: Optional[torch.dtype] = None, partial: bool = False,
           out: Optional[torch.Tensor] = None, first_shard: bool = True):
    """sum / mean / max / min / prod -> values; argmax / argmin -> (values, int64 indices).
    partial=True is the per-shard step of a sharded reduction (FP32 / INT64 partials).
    out= reuses a result buffer of the reduced shape (values only).  first_shard=False (partial
    only): the shard does not start at the global position 0, so max / min ignore a NaN at its
    own position 0."""
    _require_cuda(x)
    op = REDUCE.index(name)
    dims = _norm_dims(dim)
    if out is None:
        oshape = reduce_shape(x, dims, keepdim)
        if out_dtype is None:
            out_dtype = x.dtype
            if partial and x.dtype in (torch.float16, torch.bfloat16):
                out_dtype = torch.float32
        o = torch.empty(oshape, dtype=out_dtype, device=x.device)
    else:
        o = out
    oi = torch.empty(o.shape, dtype=torch.int64, device=x.device) if op >= 5 else None
    dx, do = desc(x), desc(o)
    di = desc(oi) if oi is not None else None
    da = i64_array(dims)
    nbytes = lib().vbt_b200_reduce_workspace_bytes(op, dx.ref, da, len(dims))
    ws = _reduce_workspace(nbytes, x.device)
    wp = ctypes.c_void_p(ws.data_ptr()) if ws is not None else None
    if partial:
        check(lib().vbt_b200_reduce_partial(op, do.ref, dx.ref, da, len(dims), int(keepdim), wp,
                                            nbytes, 1 | (0 if first_shard else 2), stream_ptr(o)))
    else:
        check(lib().vbt_b200_reduce_zeroed_ws(op, do.ref, di.ref if di else None, dx.ref, da, len(dims),
                                              int(keepdim), wp, nbytes, stream_ptr(o)))
    return (o, oi) if oi is not None else o


class PreparedReduce:
    """reduce() with everything but the launch done ahead: output, workspace and the ctypes
    argument list are built once, run() is a single C-ABI call on the current stream of the
    output's device.  The input's storage must stay where it is; the result tensor (``out``)
    is overwritten by every run.  Values only (no argmax / argmin)."""

    def __init__(self, name: str, x: torch.Tensor, dim=None, keepdim: bool = False, partial: bool = False,
                 first_shard: bool = True):
        _require_cuda(x)
        op = REDUCE.index(name)
        if op >= 5:
            raise ValueError("PreparedReduce: argmax / argmin are not supported")
        dims = _norm_dims(dim)
        out_dtype = x.dtype
        if partial and x.dtype in (torch.float16, torch.bfloat16):
            out_dtype = torch.float32
        self.x = x
        self.out = torch.empty(reduce_shape(x, dims, keepdim), dtype=out_dtype, device=x.device)
        self._dx, self._do, self._da = desc(x), desc(self.out), i64_array(dims)
        nbytes = lib().vbt_b200_reduce_workspace_bytes(op, self._dx.ref, self._da, len(dims))
        self._ws = _reduce_workspace(nbytes, x.device)
        wp = ctypes.c_void_p(self._ws.data_ptr()) if self._ws is not None else None
        if partial:
            self._fn = lib().vbt_b200_reduce_partial
            self._args = (op, self._do.ref, self._dx.ref, self._da, len(dims), int(keepdim), wp, nbytes,
                          1 | (0 if first_shard else 2))
        else:
            self._fn = lib().vbt_b200_reduce_zeroed_ws
            self._args = (op, self._do.ref, None, self._dx.ref, self._da, len(dims), int(keepdim), wp, nbytes)

    def run(self) -> torch.Tensor:
        check(self._fn(*self._args, stream_ptr(self.out)))
        return self.out


class PreparedScaleCast:
    """scale_cast() with its output and argument list built once."""

    def __init__(self, partial: torch.Tensor, scale: float, out_dtype: torch.dtype):
        _require_cuda(partial)
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise ValueError("scale_cast: partial must be contiguous float32")
        self.src = partial
        self.out = torch.empty(partial.shape, dtype=out_dtype, device=partial.device)
        self._args = (ctypes.c_void_p(self.out.data_ptr()), _lib.dtype_code(out_dtype),
                      ctypes.c_void_p(partial.data_ptr()), partial.numel(), float(scale))

    def run(self) -> torch.Tensor:
        check(lib().vbt_b200_scale_cast(*self._args, stream_ptr(self.out)))
        return self.out


def sum(x, dim=None, keepdim=False):  # noqa: A001 - mirrors Tensor.sum
    return reduce("sum", x, dim, keepdim)


def mean(x, dim=None, keepdim=False):
    return reduce("mean", x, dim, keepdim)


def amax(x, dim=None, keepdim=False):
    return reduce("max", x, dim, keepdim)


def amin(x, dim=None, keepdim=False):
    return reduce("min", x, dim, keepdim)


def prod(x, dim=None, keepdim=False):
    return reduce("prod", x, dim, keepdim)


def argmax(x, dim=None, keepdim=False):
    return reduce("argmax", x, dim, keepdim)[1]


def argmin(x, dim=None, keepdim=False):
    return reduce("argmin", x, dim, keepdim)[1]


def max_dim(x, dim, keepdim=False):
    """Tensor.max(dim) -> (values, indices) (tensor_bindings.cc:2538-2573)."""
    return reduce("argmax", x, dim, keepdim)


def min_dim(x, dim, keepdim=False):
    return reduce("argmin", x, dim, keepdim)


# --------------------------------------------------------------------------------------
# indexing
# --------------------------------------------------------------------------------------
class IndexStatus:
    """Device-side record of out-of-range indices: {count, first bad value}.  Kernels skip a
    bad index and note it here; ``check`` synchronises and raises IndexError."""

    def __init__(self, device):
        self.buf = torch.zeros(2, dtype=torch.int64, device=device)

    @property
    def ptr(self):
        return ctypes.c_void_p(self.buf.data_ptr())

    def check(self, what: str, dim_size: int) -> None:
        check(lib().vbt_b200_index_status_check(self.ptr, what.encode(), int(dim_size),
                                                stream_ptr(self.buf)))


def _status(status, eager, device):
    if status is not None:
        return status, False
    return (IndexStatus(device), True) if eager else (None, False)


def index_rows(table: torch.Tensor, idx: torch.Tensor, policy: int = INDEX_WRAP,
               status: Optional[IndexStatus] = None, eager_check: bool = True,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``table[idx]`` for a 2-D table: out[..., :] = table[idx[...], :].  eager_check=True
    reproduces the reference's immediate IndexError (which costs a stream sync, as its own
    bounds check does, src/vbt/ops/embedding_cuda.cu:282-299); pass a shared ``status``
    and check it later to stay asynchronous."""
    _require_cuda(table, idx)
    st, own = _status(status, eager_check, table.device)
    o = _alloc_out(out, tuple(idx.shape) + (table.shape[1],), table.dtype, table)
    do, dt_, di = desc(o), desc(table), desc(idx.contiguous())
    check(lib().vbt_b200_index_rows(do.ref, dt_.ref, di.ref, policy, st.ptr if st else None,
                                    stream_ptr(table)))
    if own:
        st.check("index", table.shape[0])
    return o


def grouping_engine_pays(dtype: torch.dtype, num_updates: int) -> bool:
    """Whether ``index_put_(accumulate=True)`` on a table of `dtype` with `num_updates` updates runs
    faster through the grouping engine (radix passes + per-run sums) than through block-local
    aggregation + atomics -- the measured crossovers on B200 with 1 - 2 KiB rows."""
    if dtype in (torch.int64, torch.int32):
        return num_updates >= (1 << 19)
    return dtype == torch.float32 and num_updates >= (1 << 21)


def index_put_rows_(table: torch.Tensor, idx: torch.Tensor, values: torch.Tensor,
                    accumulate: bool = False, policy: int = INDEX_WRAP,
                    status: Optional[IndexStatus] = None, eager_check: bool = True,
                    deterministic: Optional[bool] = None) -> torch.Tensor:
    """``table.index_put_((idx,), values, accumulate)`` for a 2-D table and [N, D] values.

    accumulate=True has two engines: block-local aggregation + atomics (no scratch), and
    group-by-row + per-run sums (scratch of ~18 bytes per index; a radix sort by row, or by a
    16-bit hash of the row for 4-byte tables of more than 65536 rows; integer results are exact
    and order-independent, a float row receives a few large partial sums instead of many updates).
    ``deterministic=None`` picks the grouping engine where it measured faster -- integer tables from
    2^19 updates on (int64 rows of 2 KiB into 2^20 rows: 0.18 against 0.20 ms at 2^18 updates, 0.65
    against 0.53 ms at 2^20), float32 tables from 2^21 on (4 M updates of 1 KiB into 2^20 rows: 0.88 against
    0.94 ms with Zipf(1.1) rows, 1.30 against 1.86 ms with uniform ones; at 2^20 updates the two are
    level, below that the sort costs more than it saves); True / False force the choice."""
    _require_cuda(table, idx, values)
    st, own = _status(status, eager_check, table.device)
    dt_, di, dv = desc(table), desc(idx.contiguous()), desc(values)
    if deterministic is None:
        deterministic = accumulate and grouping_engine_pays(table.dtype, idx.numel())
    if accumulate and deterministic:
        nbytes = lib().vbt_b200_index_put_rows_sorted_workspace_bytes(idx.numel())
        ws = _workspace(nbytes, table.device)
        check(lib().vbt_b200_index_put_rows_sorted(dt_.ref, di.ref, dv.ref, policy, st.ptr if st else None,
                                                   ctypes.c_void_p(ws.data_ptr()) if ws is not None else None,
                                                   nbytes, stream_ptr(table)))
    else:
        check(lib().vbt_b200_index_put_rows(dt_.ref, di.ref, dv.ref, int(accumulate), policy,
                                            st.ptr if st else None, stream_ptr(table)))
    if own:
        st.check("index_put_", table.shape[0])
    return table


def index_lastdim(src: torch.Tensor, idx: torch.Tensor, status=None, eager_check=True):
    """The reference's CUDA advanced-index form ``src[..., idx]``: src of any rank >= 1 and
    any strides, one index tensor (any shape) applied to the last dim; the result is dense
    ``src.shape[:-1] + idx.shape`` (src/vbt/core/indexing_advanced_cuda.cu:2156-2177)."""
    _require_cuda(src, idx)
    if src.dim() < 1:
        raise ValueError("index: advanced indexing is not supported for 0-d tensors on CUDA")
    if idx.dim() < 1:
        raise ValueError("index: advanced tensor indices must have dim() > 0")
    st, own = _status(status, eager_check, src.device)
    o = torch.empty(tuple(src.shape[:-1]) + tuple(idx.shape), dtype=src.dtype, device=src.device)
    do, ds, di = desc(o), desc(src), desc(idx.contiguous())
    check(lib().vbt_b200_index_lastdim(do.ref, ds.ref, di.ref, INDEX_WRAP, st.ptr if st else None,
                                       stream_ptr(o)))
    if own:
        st.check("index", src.shape[-1])
    return o


def mask_select(mask: torch.Tensor):
    """Device part of bool-mask indexing, no host round trip: returns (indices, count) where
    ``indices`` is an int64 buffer as long as the mask whose first ``count`` entries are the
    ascending positions of the true elements and ``count`` is a 1-element int64 device tensor."""
    _require_cuda(mask)
    if mask.dtype != torch.bool:
        raise ValueError("index: mask must be a bool tensor")
    if mask.dim() != 1:
        raise ValueError("index: CUDA advanced indexing does not support boolean mask indices of rank other than 1")
    n = mask.numel()
    need = ctypes.c_size_t()
    check(lib().vbt_b200_mask_select_workspace_bytes(n, ctypes.byref(need)))
    ws = _workspace(max(need.value, 8), mask.device)
    idx = torch.empty((n,), dtype=torch.int64, device=mask.device)
    count = torch.empty((1,), dtype=torch.int64, device=mask.device)
    dm = desc(mask)
    check(lib().vbt_b200_mask_select(dm.ref, ctypes.c_void_p(idx.data_ptr()), n, ctypes.c_void_p(count.data_ptr()),
                                     ctypes.c_void_p(ws.data_ptr()), ws.numel(), stream_ptr(idx)))
    return idx, count


def mask_to_indices(mask: torch.Tensor) -> torch.Tensor:
    """Ascending int64 positions of the true elements of a 1-D bool mask, computed on the
    device.  Reads the count back (one 8-byte D2H copy and a stream synchronise, as the
    reference's bool-mask path does) to size the result."""
    idx, count = mask_select(mask)
    return idx[: int(count.item())]


def index_mask_lastdim(src: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """``src[..., mask]`` for 2-D src and a 1-D bool mask over its last dim: the form the
    reference's CUDA bool-mask indexing takes (float32 / int64 data only, as there)."""
    if src.dtype not in (torch.float32, torch.int64):
        raise ValueError("index: CUDA advanced indexing does not support boolean mask indices")
    if mask.dim() != 1 or mask.numel() != src.shape[-1]:
        raise ValueError("index: CUDA advanced indexing does not support boolean mask indices")
    return index_lastdim(src, mask_to_indices(mask), eager_check=False)


def index_mask_rows(src: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """``src[mask]`` for a 1-D bool mask over dim 0 (row compaction)."""
    if mask.dim() != 1 or mask.numel() != src.shape[0]:
        raise ValueError("index: mask length must equal the size of dim 0")
    return index_rows(src, mask_to_indices(mask), eager_check=False)


def index_put_lastdim_(self_: torch.Tensor, idx, values, accumulate=False, status=None,
                       eager_check=True):
    _require_cuda(self_, idx, values)
    st, own = _status(status, eager_check, self_.device)
    ds, di, dv = desc(self_), desc(idx.contiguous()), desc(values)
    check(lib().vbt_b200_index_put_lastdim(ds.ref, di.ref, dv.ref, int(accumulate), INDEX_WRAP,
                                           st.ptr if st else None, stream_ptr(self_)))
    if own:
        st.check("index_put_", self_.shape[-1])
    return self_


def embedding(weight: torch.Tensor, indices: torch.Tensor, status=None, eager_check=True):
    """vt::embedding forward (src/vbt/ops/embedding_dispatch.cc:536-709)."""
    _require_cuda(weight, indices)
    st, own = _status(status, eager_check, weight.device)
    o = torch.empty(tuple(indices.shape) + (weight.shape[1],), dtype=weight.dtype, device=weight.device)
    do, dw, di = desc(o), desc(weight), desc(indices)
    check(lib().vbt_b200_embedding(do.ref, dw.ref, di.ref, st.ptr if st else None, stream_ptr(weight)))
    if own:
        st.check("vt::embedding", weight.shape[0])
    return o


def embedding_backward(grad_out: torch.Tensor, indices: torch.Tensor, num_weights: int,
                       padding_idx: int = -1, status=None, eager_check=True,
                       scale_grad_by_freq: bool = False) -> torch.Tensor:
    """Dense weight gradient: gw[idx[i], :] += grad_out[i, :], padding_idx rows skipped; with
    scale_grad_by_freq every row's gradient is divided by the row's number of occurrences."""
    _require_cuda(grad_out, indices)
    st, own = _status(status, eager_check, grad_out.device)
    D = grad_out.shape[-1]
    gw = torch.zeros((num_weights, D), dtype=grad_out.dtype, device=grad_out.device)
    dg, di, do = desc(gw), desc(indices), desc(grad_out.reshape(-1, D))
    if scale_grad_by_freq:
        counts = torch.empty((max(num_weights, 1),), dtype=torch.int32, device=grad_out.device)
        check(lib().vbt_b200_embedding_backward_by_freq(dg.ref, di.ref, do.ref, int(padding_idx),
                                                        ctypes.c_void_p(counts.data_ptr()), counts.numel() * 4,
                                                        st.ptr if st else None, stream_ptr(gw)))
    else:
        check(lib().vbt_b200_embedding_backward(dg.ref, di.ref, do.ref, int(padding_idx),
                                                st.ptr if st else None, stream_ptr(gw)))
    if own:
        st.check("vt::embedding", num_weights)
    return gw


FABRIC_MODES = {1: "peer_load", 2: "copy_fallback", 3: "local"}


def fabric_binary(name: str, a: torch.Tensor, b: torch.Tensor, compute_device: Optional[int] = None,
                  require_fabric: bool = False, use_copy_fallback=True, out: Optional[torch.Tensor] = None):
    """vt::fabric_add / vt::fabric_mul (src/vbt/cuda/fabric_elementwise.cu:820-1042): a and b
    of equal shape and dtype on one or two GPUs of this process; the result lives on
    ``compute_device`` (default: a's device).  Returns (out, mode) with mode one of
    "local", "peer_load" (the remote operand is read in place over NVLink) or "copy_fallback"
    (it is copied to the compute device first).  ``use_copy_fallback="always"`` takes the copy
    path even when peer access exists."""
    for t in (a, b):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"[Fabric] vt::fabric_{name}: expects CUDA tensors")
    dev = a.device.index if compute_device is None else int(compute_device)
    if out is None:
        out = torch.empty(a.shape, dtype=a.dtype, device=torch.device("cuda", dev))
    policy = 2 if use_copy_fallback == "always" else int(bool(use_copy_fallback))
    scratch = None
    if a.device != b.device and policy:
        scratch = torch.empty(max(a.numel() * a.element_size(), 16), dtype=torch.uint8, device=out.device)
    mode = ctypes.c_int32()
    do, da, db = desc(out), desc(a), desc(b)
    with torch.cuda.device(out.device):
        check(lib().vbt_b200_fabric_binary(BINARY.index(name), do.ref, da.ref, db.ref, dev, int(require_fabric), policy,
                                           ctypes.c_void_p(scratch.data_ptr()) if scratch is not None else None,
                                           scratch.numel() if scratch is not None else 0, ctypes.byref(mode),
                                           stream_ptr(out)))
    if mode.value == 1 and a.device != b.device:
        _peer_enabled.add((dev, (b if a.device.index == dev else a).device.index))
    return out, FABRIC_MODES.get(mode.value, "none")


def scale_cast(partial: torch.Tensor, scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """out = cast(partial * scale): the last step of a sharded mean (float32 partials)."""
    _require_cuda(partial)
    if partial.dtype != torch.float32:
        if scale == 1.0 and partial.dtype == out_dtype:
            return partial
        raise ValueError("scale_cast: partial must be float32")
    p = partial.contiguous()
    o = torch.empty(p.shape, dtype=out_dtype, device=p.device)
    check(lib().vbt_b200_scale_cast(ctypes.c_void_p(o.data_ptr()), _lib.dtype_code(out_dtype),
                                    ctypes.c_void_p(p.data_ptr()), p.numel(), float(scale),
                                    stream_ptr(p)))
    return o
