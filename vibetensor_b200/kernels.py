"""Row ops and gather / scatter_add with the call signatures of the reference's
``vibe_kernels.*.vbt_native`` modules, served by plain CUDA in libvbt_b200.so instead of
Triton kernels compiled at run time:

* ``softmax`` / ``log_softmax``  -- vibe_kernels/softmax/vbt_native.py:193-328
* ``rmsnorm``                    -- vibe_kernels/rmsnorm/vbt_native.py:340-406
* ``rmsnorm_backward``           -- vibe_kernels/rmsnorm/vbt_native.py:409-492
* ``softmax_backward`` / ``log_softmax_backward``
                                 -- vibe_kernels/softmax/impl/cutedsl_softmax/softmax.py:992-1017
* ``gather`` / ``scatter_add``   -- vibe_kernels/indexing/vbt_native.py:197-280, :490-580

Same argument meaning and the same exception classes for the same misuse (RuntimeError for a
non-CUDA tensor, TypeError for a dtype, NotImplementedError for an unsupported dim); float16
and bfloat16 inputs are accepted in addition to the reference's float32.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import ops as _ops
from ._lib import check, dtype_code, lib, stream_ptr

_FLOATS = (torch.float32, torch.float16, torch.bfloat16)


def _rows_view(x: torch.Tensor, what: str):
    """(rows, cols, row_stride) of x seen as a stack of last-dim rows, the reference's 2-D
    view (rows = product of leading dims, row stride = strides[-2])."""
    if not x.is_cuda:
        raise RuntimeError(f"{what} requires CUDA tensors")
    if x.dtype not in _FLOATS:
        raise TypeError(f"{what} requires float32, float16 or bfloat16")
    if x.dim() == 0:
        return x.reshape(1, 1), 1, 1, 1
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if x.dim() >= 2:
        lead_ok = x.stride(-1) == 1 or cols <= 1
        # leading dims must collapse onto one row stride
        expect = x.stride(-2)
        for d in range(x.dim() - 3, -1, -1):
            expect *= x.shape[d + 1]
            if x.shape[d] != 1 and x.stride(d) != expect:
                lead_ok = False
        if not lead_ok:
            x = _ops.contiguous(x)
        row_stride = x.stride(-2) if x.shape[-2] != 1 else max(cols, 1)
    else:
        if x.stride(-1) != 1 and cols > 1:
            x = _ops.contiguous(x)
        row_stride = cols
    return x, rows, cols, row_stride


def _softmax(x: torch.Tensor, dim: int, log: bool) -> torch.Tensor:
    what = "log_softmax" if log else "softmax"
    nd = x.dim()
    d = dim + nd if dim < 0 else dim
    if nd and d != nd - 1:
        raise NotImplementedError(f"{what} currently only supports dim=-1 (last dimension)")
    xv, rows, cols, rs = _rows_view(x, what)
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if rows == 0 or cols == 0:
        return out
    check(lib().vbt_b200_softmax(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(xv.data_ptr()),
                                 dtype_code(x.dtype), rows, cols, rs, int(log), stream_ptr(x)))
    return out


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return _softmax(x, dim, False)


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return _softmax(x, dim, True)


def rmsnorm(x: torch.Tensor, gamma: Optional[torch.Tensor] = None, eps: float = 1e-6):
    """Returns (out, inv_rms): out has x's shape and dtype, inv_rms is float32 [rows]."""
    xv, rows, cols, rs = _rows_view(x, "rmsnorm")
    if gamma is not None:
        if not gamma.is_cuda:
            raise RuntimeError("rmsnorm requires CUDA tensors")
        if gamma.dtype != torch.float32 or gamma.numel() != cols:
            raise TypeError("gamma must be float32 of shape [hidden_size]")
        gamma = gamma.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    inv = torch.empty((rows,), dtype=torch.float32, device=x.device)
    if rows == 0 or cols == 0:
        return out, inv
    check(lib().vbt_b200_rmsnorm(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(inv.data_ptr()),
                                 ctypes.c_void_p(xv.data_ptr()),
                                 ctypes.c_void_p(gamma.data_ptr()) if gamma is not None else None,
                                 dtype_code(x.dtype), rows, cols, rs, float(eps), stream_ptr(x)))
    return out, inv


def _softmax_backward(dy: torch.Tensor, y: torch.Tensor, log: bool) -> torch.Tensor:
    what = "log_softmax_backward" if log else "softmax_backward"
    if dy.shape != y.shape:
        raise ValueError(f"{what}: dy and y must have the same shape")
    if dy.dtype != y.dtype:
        raise TypeError(f"{what}: dy and y must have the same dtype")
    dyv, rows, cols, rs_dy = _rows_view(dy, what)
    yv, _, _, rs_y = _rows_view(y, what)
    dx = torch.empty(y.shape, dtype=y.dtype, device=y.device)
    if rows == 0 or cols == 0:
        return dx
    check(lib().vbt_b200_softmax_backward(ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dyv.data_ptr()),
                                          ctypes.c_void_p(yv.data_ptr()), dtype_code(y.dtype), rows, cols,
                                          rs_dy, rs_y, int(log), stream_ptr(y)))
    return dx


def softmax_backward(dy: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """dx of y = softmax(x, -1): y * (dy - sum(dy * y))."""
    return _softmax_backward(dy, y, False)


def log_softmax_backward(dy: torch.Tensor, log_y: torch.Tensor) -> torch.Tensor:
    """dx of log_y = log_softmax(x, -1): dy - exp(log_y) * sum(dy)."""
    return _softmax_backward(dy, log_y, True)


def rmsnorm_backward(grad_output: torch.Tensor, x: torch.Tensor, inv_rms: torch.Tensor,
                     gamma: Optional[torch.Tensor] = None):
    """Returns (grad_input, grad_gamma); grad_gamma is None when gamma is None, float32
    [hidden_size] otherwise.  inv_rms is the second result of ``rmsnorm``."""
    what = "rmsnorm_backward"
    if grad_output.shape != x.shape:
        raise ValueError(f"{what}: grad_output and x must have the same shape")
    if grad_output.dtype != x.dtype:
        raise TypeError(f"{what}: grad_output and x must have the same dtype")
    xv, rows, cols, rs_x = _rows_view(x, what)
    gv, _, _, rs_g = _rows_view(grad_output, what)
    if not inv_rms.is_cuda:
        raise RuntimeError(f"{what} requires CUDA tensors")
    if inv_rms.dtype != torch.float32 or inv_rms.numel() != rows:
        raise TypeError("inv_rms must be float32 of shape [rows]")
    inv_rms = inv_rms.contiguous()
    if gamma is not None:
        if not gamma.is_cuda:
            raise RuntimeError(f"{what} requires CUDA tensors")
        if gamma.dtype != torch.float32 or gamma.numel() != cols:
            raise TypeError("gamma must be float32 of shape [hidden_size]")
        gamma = gamma.contiguous()
    dx = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    dgamma = torch.empty((cols,), dtype=torch.float32, device=x.device) if gamma is not None else None
    ws, ws_bytes = None, 0
    if dgamma is not None and cols:
        need = ctypes.c_size_t()
        check(lib().vbt_b200_rmsnorm_backward_workspace_bytes(rows, cols, dtype_code(x.dtype), x.device.index,
                                                              ctypes.byref(need)))
        # the dgamma partial rows live in the general scratch buffer of this (device, stream)
        ws = _ops._workspace(max(need.value, 16), x.device)
        ws_bytes = ws.numel()
    if cols == 0:
        return dx, dgamma
    check(lib().vbt_b200_rmsnorm_backward(
        ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dgamma.data_ptr()) if dgamma is not None else None,
        ctypes.c_void_p(gv.data_ptr()), ctypes.c_void_p(xv.data_ptr()), ctypes.c_void_p(inv_rms.data_ptr()),
        ctypes.c_void_p(gamma.data_ptr()) if gamma is not None else None, dtype_code(x.dtype), rows, cols,
        rs_g, rs_x, ctypes.c_void_p(ws.data_ptr()) if ws is not None else None, ws_bytes, stream_ptr(x)))
    return dx, dgamma


def _check_gather_args(src, dim, index, what):
    if not src.is_cuda:
        raise RuntimeError(f"{what} requires CUDA tensors")
    if not index.is_cuda:
        raise RuntimeError("index must be on CUDA")
    if index.dtype != torch.int64:
        raise TypeError("index must be int64")
    nd = src.dim()
    d = dim + nd if dim < 0 else dim
    if d != 0:
        raise NotImplementedError(f"{what} currently only supports dim=0")
    if index.dim() != 1:
        raise NotImplementedError(f"{what} currently only supports 1D index")


def gather(src: torch.Tensor, dim: int, index: torch.Tensor, status=None) -> torch.Tensor:
    """out[i, ...] = src[index[i], ...] (dim 0, 1-D int64 index).  The Triton kernel reads
    whatever an out-of-range index points at; here such a row comes back as zeros and is
    counted in ``status`` (an ops.IndexStatus) when one is given."""
    _check_gather_args(src, dim, index, "gather")
    src2 = src.reshape(src.shape[0], -1) if src.dim() != 2 else src
    out = _ops.index_rows(src2, index, policy=_ops.INDEX_STRICT, status=status, eager_check=False)
    return out.reshape((index.numel(),) + tuple(src.shape[1:]))


def scatter_add(out: torch.Tensor, dim: int, index: torch.Tensor, src: torch.Tensor, status=None):
    """out[index[i], ...] += src[i, ...] in place (dim 0, 1-D int64 index); indices are
    clamped into range as the Triton kernel does (vibe_kernels/indexing/kernels.py:79-80)."""
    _check_gather_args(out, dim, index, "scatter_add")
    if out.dtype != src.dtype:
        raise TypeError("out and src must have the same dtype")
    out2 = out.view(out.shape[0], -1) if out.dim() != 2 else out
    src2 = src.reshape(index.numel(), -1)
    _ops.index_put_rows_(out2, index, src2, accumulate=True, policy=_ops.INDEX_CLAMP, status=status,
                         eager_check=False)
    return out
