"""Helpers shared by the parity tests: numpy <-> torch <-> oracle storage conversions."""
import numpy as np
import torch

import oracle

CODE = {torch.float32: oracle.F32, torch.float16: oracle.F16, torch.bfloat16: oracle.BF16,
        torch.int64: oracle.I64, torch.int32: oracle.I32, torch.bool: oracle.BOOL}


def to_np(t: torch.Tensor) -> np.ndarray:
    """Device tensor -> oracle storage array (bf16 / f16 as uint16 bit patterns).  Keeps
    the logical shape; the result is contiguous."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.bool:
        return t.numpy().view(np.uint8)
    return t.numpy()


def from_np(a: np.ndarray, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    """Oracle storage array -> device tensor of the given torch dtype."""
    a = np.ascontiguousarray(a)
    if dtype in (torch.bfloat16, torch.float16):
        return torch.from_numpy(a.view(np.int16)).view(dtype).to(device)
    if dtype == torch.bool:
        return torch.from_numpy(a.view(np.uint8)).to(device).view(torch.bool)
    return torch.from_numpy(a).to(device)


def rand_storage(rng, shape, dtype: torch.dtype, scale=1.0):
    """Seeded N(0, scale) values (or small ints) in oracle storage form."""
    if dtype == torch.int64:
        return rng.integers(-1000, 1001, shape).astype(np.int64)
    x = (scale * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
    return oracle.to_storage(x, CODE[dtype])


def as_f32(a: np.ndarray, dtype: torch.dtype) -> np.ndarray:
    if dtype == torch.int64:
        return a.astype(np.float64)
    return oracle.to_f32(a, CODE[dtype])


def strided_like(t_np: np.ndarray, dtype, strides_elems, storage_elems, offset=0, device="cuda"):
    """A device tensor with the given shape/strides holding t_np's values, plus the numpy
    view with the same strides (for the oracle)."""
    base_np = np.zeros(storage_elems, t_np.dtype)
    view_np = np.lib.stride_tricks.as_strided(base_np[offset:], t_np.shape,
                                              [s * t_np.itemsize for s in strides_elems])
    view_np[...] = t_np
    base_t = from_np(base_np, dtype, device)
    view_t = torch.as_strided(base_t, t_np.shape, strides_elems, offset)
    return view_t, view_np


WORST: dict = {}  # label -> (largest error / scale seen in this run, bound); printed at the end of the run


def note_worst(label: str, err_over_scale: float, bound: float) -> None:
    prev = WORST.get(label, (0.0, bound))[0]
    WORST[label] = (max(prev, float(err_over_scale)), bound)
