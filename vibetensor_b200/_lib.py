"""ctypes binding of libvbt_b200.so (the C ABI declared in include/vbt_b200.h).

PyTorch is used here only as plumbing: it owns device memory and streams.  Every compute
call goes through the C ABI with raw pointers; there is no fallback of any kind -- if the
shared library is missing or an entry point fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libvbt_b200.so")

BOOL, I32, I64, F32, F16, BF16 = 0, 1, 2, 3, 4, 5
C64, C128 = 7, 8  # vt::add, vt::mul and copy only
_TORCH_TO_CODE = {
    torch.bool: BOOL, torch.int32: I32, torch.int64: I64, torch.float32: F32,
    torch.float16: F16, torch.bfloat16: BF16, torch.uint8: BOOL,
    torch.complex64: C64, torch.complex128: C128,
}
MAX_NDIM = 25
FABRIC_HANDLE_BYTES = 128


class LaunchInfo(ctypes.Structure):
    """vbt_b200_launch_info: what the last launching call on this thread enqueued."""
    _fields_ = [("family", ctypes.c_int32), ("kernel", ctypes.c_int32), ("grid", ctypes.c_uint32 * 3),
                ("block", ctypes.c_uint32 * 3), ("vec", ctypes.c_int32), ("splits", ctypes.c_int32),
                ("cluster", ctypes.c_int32), ("launches", ctypes.c_int32), ("out_numel", ctypes.c_int64),
                ("slice_len", ctypes.c_int64), ("workspace_bytes", ctypes.c_uint64), ("stream", ctypes.c_void_p)]


class VbtTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("sizes", ctypes.POINTER(ctypes.c_int64)), ("strides", ctypes.POINTER(ctypes.c_int64))]


_P = ctypes.POINTER(VbtTensor)
_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64
_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)

# name -> (restype, argtypes); mirrors include/vbt_b200.h one to one
SIGNATURES = {
    "vbt_b200_last_error": (ctypes.c_char_p, []),
    "vbt_b200_version": (_i32, []),
    "vbt_b200_compiled_arch": (_i32, []),
    "vbt_b200_broadcast_shape": (_i32, [ctypes.POINTER(_P), _i32, _i64p, _i32p]),
    "vbt_b200_unary": (_i32, [_i32, _P, _P, _vp]),
    "vbt_b200_binary": (_i32, [_i32, _P, _P, _P, _vp]),
    "vbt_b200_ternary": (_i32, [_i32, _P, _P, _P, _P, _vp]),
    "vbt_b200_where": (_i32, [_P, _P, _P, _P, _vp]),
    "vbt_b200_binary_scalar": (_i32, [_i32, _P, _P, _vp, _i32, _vp]),
    "vbt_b200_polygamma": (_i32, [_P, _P, _P, _vp]),
    "vbt_b200_copy": (_i32, [_P, _P, _vp]),
    "vbt_b200_add": (_i32, [_P, _P, _P, _vp]),
    "vbt_b200_sub": (_i32, [_P, _P, _P, _vp]),
    "vbt_b200_mul": (_i32, [_P, _P, _P, _vp]),
    "vbt_b200_div": (_i32, [_P, _P, _P, _vp]),
    "vbt_b200_gt": (_i32, [_P, _P, _P, _vp]),
    "vbt_b200_relu": (_i32, [_P, _P, _vp]),
    "vbt_b200_ti_plan": (_i32, [ctypes.POINTER(_P), _i32, _i64p, _i64p, _i32p, _i32p, _i32p]),
    "vbt_b200_reduce_workspace_bytes": (ctypes.c_size_t, [_i32, _P, _i64p, _i32]),
    "vbt_b200_reduce": (_i32, [_i32, _P, _P, _P, _i64p, _i32, _i32, _vp, ctypes.c_size_t, _vp]),
    "vbt_b200_reduce_zeroed_ws": (_i32, [_i32, _P, _P, _P, _i64p, _i32, _i32, _vp, ctypes.c_size_t, _vp]),
    "vbt_b200_reduce_noalloc": (_i32, [_i32, _P, _P, _P, _i64p, _i32, _i32, _vp]),
    "vbt_b200_reduce_shape": (_i32, [_P, _i64p, _i32, _i32, _i64p, _i32p]),
    "vbt_b200_index_rows": (_i32, [_P, _P, _P, _i32, _vp, _vp]),
    "vbt_b200_index_put_rows": (_i32, [_P, _P, _P, _i32, _i32, _vp, _vp]),
    "vbt_b200_index_put_rows_sorted_workspace_bytes": (ctypes.c_size_t, [_i64]),
    "vbt_b200_index_put_rows_sorted": (_i32, [_P, _P, _P, _i32, _vp, _vp, ctypes.c_size_t, _vp]),
    "vbt_b200_index_lastdim": (_i32, [_P, _P, _P, _i32, _vp, _vp]),
    "vbt_b200_index_put_lastdim": (_i32, [_P, _P, _P, _i32, _i32, _vp, _vp]),
    "vbt_b200_embedding": (_i32, [_P, _P, _P, _vp, _vp]),
    "vbt_b200_embedding_backward": (_i32, [_P, _P, _P, _i64, _vp, _vp]),
    "vbt_b200_mask_select_workspace_bytes": (_i32, [_i64, ctypes.POINTER(ctypes.c_size_t)]),
    "vbt_b200_mask_select": (_i32, [_P, _vp, _i64, _vp, _vp, ctypes.c_size_t, _vp]),
    "vbt_b200_embedding_backward_by_freq": (_i32, [_P, _P, _P, _i64, _vp, ctypes.c_size_t, _vp, _vp]),
    "vbt_b200_index_status_check": (_i32, [_vp, ctypes.c_char_p, _i64, _vp]),
    "vbt_b200_softmax": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _i32, _vp]),
    "vbt_b200_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, ctypes.c_float, _vp]),
    "vbt_b200_softmax_backward": (_i32, [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _vp]),
    "vbt_b200_rmsnorm_backward_workspace_bytes": (_i32, [_i64, _i64, _i32, _i32, ctypes.POINTER(ctypes.c_size_t)]),
    "vbt_b200_rmsnorm_backward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _vp,
                                         ctypes.c_size_t, _vp]),
    "vbt_b200_enable_peer_access": (_i32, [_i32, _i32]),
    "vbt_b200_reduce_partial": (_i32, [_i32, _P, _P, _i64p, _i32, _i32, _vp, ctypes.c_size_t, _i32, _vp]),
    "vbt_b200_scale_cast": (_i32, [_vp, _i32, _vp, _i64, ctypes.c_float, _vp]),
    "vbt_b200_fabric_binary": (_i32, [_i32, _P, _P, _P, _i32, _i32, _i32, _vp, ctypes.c_size_t, _i32p, _vp]),
    "vbt_b200_fabric_comm_create": (_i32, [_i32, _i32, _i32, ctypes.c_size_t, ctypes.POINTER(_vp)]),
    "vbt_b200_fabric_comm_handle": (_i32, [_vp, _vp]),
    "vbt_b200_fabric_comm_connect": (_i32, [_vp, _vp]),
    "vbt_b200_fabric_comm_status": (_i32, [_vp, _vp]),
    "vbt_b200_fabric_comm_destroy": (_i32, [_vp]),
    "vbt_b200_reduce_exchange": (_i32, [_i32, _P, _P, _i64p, _i32, _i32, _vp, ctypes.c_size_t, _i32, _vp, _i32,
                                        ctypes.c_float, _vp]),
    "vbt_b200_last_launch_info": (_i32, [ctypes.POINTER(LaunchInfo)]),
    "vbt_b200_reset_last_launch_info": (None, []),
    "vbt_b200_launch_counts": (_i32, [ctypes.POINTER(ctypes.c_uint64), _i32]),
    "vbt_b200_reset_launch_counts": (None, []),
}

_EXC = {1: ValueError, 2: RuntimeError, 3: IndexError, 4: RuntimeError}
_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m vibetensor_b200.build` "
                "(vibetensor_b200 has no fallback compute path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = lib().vbt_b200_last_error().decode()
        raise _EXC.get(status, RuntimeError)(msg)


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_CODE[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}") from None


class Desc:
    """Keeps the ctypes arrays of one tensor descriptor alive for the duration of a call."""

    __slots__ = ("t", "sizes", "strides", "struct")

    def __init__(self, t: torch.Tensor):
        nd = t.dim()
        if nd > 64:
            raise ValueError("rank too large")
        self.t = t
        self.sizes = (ctypes.c_int64 * max(nd, 1))(*t.shape)
        self.strides = (ctypes.c_int64 * max(nd, 1))(*t.stride())
        self.struct = VbtTensor(t.data_ptr() if t.numel() else (t.data_ptr() or 0), dtype_code(t.dtype),
                                nd, self.sizes, self.strides)

    @property
    def ref(self):
        return ctypes.byref(self.struct)


def desc(t: torch.Tensor) -> Desc:
    return Desc(t)


def stream_ptr(t: torch.Tensor | None = None) -> ctypes.c_void_p:
    """Current torch stream of the tensor's device as a cudaStream_t."""
    dev = t.device if t is not None else None
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


FAMILIES = ("none", "elementwise", "reduce", "index", "rowop", "fabric")


def last_launch_info() -> LaunchInfo:
    info = LaunchInfo()
    check(lib().vbt_b200_last_launch_info(ctypes.byref(info)))
    return info


def launch_counts() -> dict:
    """Process-wide launch counts per kernel family since load (or the last reset)."""
    arr = (ctypes.c_uint64 * len(FAMILIES))()
    check(lib().vbt_b200_launch_counts(arr, len(FAMILIES)))
    return {name: int(arr[i]) for i, name in enumerate(FAMILIES)}


def i64_array(vals):
    vals = [int(v) for v in vals]
    return (ctypes.c_int64 * max(len(vals), 1))(*vals)
