"""vbt_b200_reduce_noalloc: the reduction entry for callers that cannot allocate scratch
(plugin hosts that can only create "dense like" outputs, code under an allocator lock,
embedders that forbid cudaMalloc after start-up).  Called through the C ABI and compared
with vbt_b200_reduce given an ordinary workspace: same kernels, same order of additions, so
the outputs must be bit-identical -- on two calls in a row, because the fixed scratch array
is shared and keeps the previous call's contents.  Collected last on purpose."""
import ctypes

import pytest
import torch

from vibetensor_b200 import _lib

pytestmark = pytest.mark.gpu
SUM, MEAN, MAX, ARGMAX = 0, 1, 2, 5


def _reduce(L, op, x, dims, noalloc):
    dx = _lib.desc(x)
    da = _lib.i64_array(dims)
    shape = (ctypes.c_int64 * 25)()
    nd = ctypes.c_int32()
    _lib.check(L.vbt_b200_reduce_shape(dx.ref, da, len(dims), 0, shape, ctypes.byref(nd)))
    oshape = tuple(shape[:nd.value])
    out = torch.empty(oshape, dtype=x.dtype, device=x.device)
    idx = torch.empty(oshape, dtype=torch.int64, device=x.device) if op == ARGMAX else None
    do = _lib.desc(out)
    di = _lib.desc(idx) if idx is not None else None
    stream = _lib.stream_ptr(x)
    if noalloc:
        _lib.check(L.vbt_b200_reduce_noalloc(op, do.ref, di.ref if di else None, dx.ref, da, len(dims), 0,
                                             stream))
    else:
        need = L.vbt_b200_reduce_workspace_bytes(op, dx.ref, da, len(dims))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
        _lib.check(L.vbt_b200_reduce(op, do.ref, di.ref if di else None, dx.ref, da, len(dims), 0,
                                     ctypes.c_void_p(ws.data_ptr()), need, stream))
    torch.cuda.synchronize()
    return out, idx


CASES = [
    (SUM, (1 << 22,), []),            # one long row: chunk partials + one ticket
    (MEAN, (4096, 1024), [0]),        # column reduction split over rows
    (MAX, (3, 1 << 20), [1]),
    (ARGMAX, (1 << 21,), []),
    (SUM, (512, 512), [1]),           # needs no scratch at all
]


@pytest.mark.parametrize("op,shape,dims", CASES)
def test_noalloc_matches_workspace_entry_twice_in_a_row(op, shape, dims):
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(1234)
    for call in range(2):  # the second call sees the first one's leftovers in the scratch
        x = torch.randn(shape, device="cuda", generator=g)
        want, want_i = _reduce(L, op, x, dims, noalloc=False)
        got, got_i = _reduce(L, op, x, dims, noalloc=True)
        assert torch.equal(got, want), f"call {call}: values differ"
        if want_i is not None:
            assert torch.equal(got_i, want_i), f"call {call}: indices differ"


def test_noalloc_rejects_shapes_beyond_its_fixed_scratch():
    L = _lib.lib()
    # argmax over dim 0 of a bf16 [65536, 256] tensor splits the rows over many blocks and
    # keeps a 16-byte (value, index) partial per column and block: more than the fixed 2 MiB
    x = torch.zeros((65536, 256), dtype=torch.bfloat16, device="cuda")
    dx = _lib.desc(x)
    dims = _lib.i64_array([0])
    need = L.vbt_b200_reduce_workspace_bytes(ARGMAX, dx.ref, dims, 1)
    assert need > (2 << 20)
    out = torch.empty((256,), dtype=torch.bfloat16, device="cuda")
    idx = torch.empty((256,), dtype=torch.int64, device="cuda")
    do, di = _lib.desc(out), _lib.desc(idx)
    rc = L.vbt_b200_reduce_noalloc(ARGMAX, do.ref, di.ref, dx.ref, dims, 1, 0, _lib.stream_ptr(out))
    assert rc == 1
    msg = L.vbt_b200_last_error().decode()
    assert "bytes of scratch" in msg and "vbt_b200_reduce with a workspace" in msg
    # the ordinary entry point takes the same call with a caller workspace
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    _lib.check(L.vbt_b200_reduce(ARGMAX, do.ref, di.ref, dx.ref, dims, 1, 0, ctypes.c_void_p(ws.data_ptr()),
                                 need, _lib.stream_ptr(out)))
    torch.cuda.synchronize()
    assert idx.tolist() == [0] * 256
