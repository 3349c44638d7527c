"""Out-of-bounds-write detection without a memory checker: every kernel family writes its
output into the MIDDLE of a sentinel-filled buffer, for ragged shapes (sizes that are not
multiples of a vector, a tile or a block), and the sentinels on both sides are checked
afterwards.  A store one vector past a ragged row, or before the start of an output whose base
is not 16-byte aligned, shows up here even when every in-range value is right."""
import ctypes

import numpy as np
import pytest
import torch

from vibetensor_b200 import _lib

pytestmark = pytest.mark.gpu
GUARD = 2048  # elements on each side
SENT = {torch.float32: 12345.0, torch.bfloat16: 12345.0, torch.float16: 12345.0, torch.int64: -7777777,
        torch.int32: -7777777, torch.bool: True, torch.uint8: 0xA5}


class Guarded:
    """A dense tensor of `shape` carved out of a sentinel-filled buffer; `offset` extra elements
    in front make the output's base address unaligned for vector stores."""

    def __init__(self, shape, dtype, offset=0):
        n = int(np.prod(shape)) if len(shape) else 1
        fill_dtype = torch.uint8 if dtype == torch.bool else dtype
        self.buf = torch.full((n + 2 * GUARD + offset,), SENT[fill_dtype if dtype != torch.bool else torch.uint8],
                              dtype=fill_dtype, device="cuda")
        self.lo, self.hi = GUARD + offset, GUARD + offset + n
        inner = self.buf[self.lo:self.hi]
        self.t = (inner.view(torch.bool) if dtype == torch.bool else inner).view(shape)
        self.sent = SENT[fill_dtype if dtype != torch.bool else torch.uint8]

    def check(self, what):
        torch.cuda.synchronize()
        assert bool((self.buf[:self.lo] == self.sent).all()), f"{what}: wrote before the output"
        assert bool((self.buf[self.hi:] == self.sent).all()), f"{what}: wrote past the output"


@pytest.fixture(scope="module")
def ops():
    from vibetensor_b200 import ops as o
    return o


RAGGED = [(1,), (7,), (33, 5), (129, 67), (5, 4099), (3, 2, 1031), (1025, 3), (64, 64), (4097,)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.bool])
@pytest.mark.parametrize("offset", [0, 1, 3])
def test_elementwise_families(ops, dtype, offset):
    g = torch.Generator(device="cuda").manual_seed(7)
    for shape in RAGGED:
        if dtype == torch.bool:
            a = torch.rand(shape, device="cuda", generator=g) < 0.5
            out = Guarded(shape, dtype, offset)
            ops.logical_not(a, out=out.t)
            out.check(f"logical_not {shape}")
            assert torch.equal(out.t, ~a)
            continue
        a = (torch.randn(shape, device="cuda", generator=g) * 5).to(dtype)
        b = (torch.randn(shape[-1:], device="cuda", generator=g) * 5).to(dtype)     # broadcast along rows
        out = Guarded(shape, dtype, offset)
        ops.add(a, b, out=out.t)                                                     # flat / tiled
        out.check(f"add {shape}")
        assert torch.equal(out.t, a + b)
        if len(shape) >= 2:
            # output written through a transposed view: tiled kernels with a strided output, and
            # the transposing kernels when the input is contiguous along the other dim
            tshape = shape[:-2] + (shape[-1], shape[-2])
            outt = Guarded(tshape, dtype, offset)
            ops.copy_(outt.t.transpose(-1, -2), a)
            outt.check(f"copy into transposed {shape}")
            assert torch.equal(outt.t.transpose(-1, -2), a)
            out2 = Guarded(tshape, dtype, offset)
            ops.copy_(out2.t, a.transpose(-1, -2))                                  # transposed INPUT
            out2.check(f"contiguous of transposed {shape}")
            assert torch.equal(out2.t, a.transpose(-1, -2))
        if dtype != torch.int64:
            o3 = Guarded(shape, dtype, offset)
            ops.where_gt0_addcmul(a, b, a, out=o3.t)
            o3.check(f"fused chain {shape}")
            cmp_out = Guarded(shape, torch.bool, offset)
            ops.gt(a, b, out=cmp_out.t)
            cmp_out.check(f"gt {shape}")
            assert torch.equal(cmp_out.t, a > b)


RED_SHAPES = [((7, 1031), -1), ((1031, 7), 0), ((4099,), None), ((3, 5, 129), 1), ((70000, 3), 0), ((3, 70000), 1),
              ((2, 300001), None), ((513, 515), 0), ((1 << 22,), None)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_reductions_write_only_their_output(ops, dtype):
    g = torch.Generator(device="cuda").manual_seed(8)
    for shape, dim in RED_SHAPES:
        x = (torch.randn(shape, device="cuda", generator=g) * 3).to(dtype)
        for name in ("sum", "max", "argmax"):
            oshape = ops.reduce_shape(x, [] if dim is None else [dim], False)
            if name == "argmax":
                # values and indices both guarded, through the C ABI
                vals, idx = Guarded(oshape, dtype, 1), Guarded(oshape, torch.int64, 1)
                L = _lib.lib()
                dx, dv, di = _lib.desc(x), _lib.desc(vals.t), _lib.desc(idx.t)
                da = _lib.i64_array([] if dim is None else [dim])
                nd = 0 if dim is None else 1
                need = L.vbt_b200_reduce_workspace_bytes(5, dx.ref, da, nd)
                ws = Guarded((max(need, 16),), torch.uint8)
                _lib.check(L.vbt_b200_reduce(5, dv.ref, di.ref, dx.ref, da, nd, 0, ctypes.c_void_p(ws.t.data_ptr()),
                                             need, _lib.stream_ptr(x)))
                vals.check(f"argmax values {shape}")
                idx.check(f"argmax indices {shape}")
                ws.check(f"argmax workspace {shape}")      # the scratch the call was told about, not more
                want = x.float().reshape(-1).argmax() if dim is None else x.float().argmax(dim)
                xf = x.float()
                got_v = xf.reshape(-1)[idx.t] if dim is None else xf.gather(dim, idx.t.unsqueeze(dim)).squeeze(dim)
                assert torch.equal(got_v, xf.reshape(-1)[want] if dim is None else xf.gather(dim, want.unsqueeze(dim)).squeeze(dim))
            else:
                out = Guarded(oshape, dtype, 1)
                ops.reduce(name, x, dim, False, out=out.t)
                out.check(f"{name} {shape} dim={dim}")


def test_gather_scatter_and_lastdim(ops):
    g = torch.Generator(device="cuda").manual_seed(9)
    for V, D, N in ((50, 7, 133), (1000, 260, 999), (64, 4, 5000), (3, 1031, 77)):
        table = torch.randn((V, D), device="cuda", generator=g)
        idx = torch.randint(0, V, (N,), device="cuda", generator=g)
        out = Guarded((N, D), torch.float32, 0 if D % 4 == 0 else 1)
        ops.index_rows(table, idx, out=out.t)
        out.check(f"gather {V}x{D}")
        assert torch.equal(out.t, table[idx])
        for dt in (torch.float32, torch.int64):
            for det in (False, True):
                acc = Guarded((V, D), dt)
                acc.t.zero_()
                upd = (torch.randn((N, D), device="cuda", generator=g) * 4).to(dt)
                ops.index_put_rows_(acc.t, idx, upd, accumulate=True, deterministic=det)
                acc.check(f"scatter_add {V}x{D} {dt} sorted={det}")
        tgt = Guarded((V, D), torch.float32)
        ops.index_put_rows_(tgt.t, idx[:V].unique(), torch.ones((idx[:V].unique().numel(), D), device="cuda"))
        tgt.check(f"scatter overwrite {V}x{D}")
    L = _lib.lib()
    for B, K0, K in ((5, 77, 33), (40, 70001, 30000), (33, 16384, 16384), (64, 50000, 40000), (32, 40000, 8191),
                     (33, 65536, 65536), (12, 100003, 50001)):
        src = torch.randn((B, K0), device="cuda", generator=g)
        idx = torch.randint(-K0, K0, (K,), device="cuda", generator=g)
        out = Guarded((B, K), torch.float32, 1)
        do, ds, di = _lib.desc(out.t), _lib.desc(src), _lib.desc(idx)
        _lib.check(L.vbt_b200_index_lastdim(do.ref, ds.ref, di.ref, 0, None, _lib.stream_ptr(src)))
        out.check(f"index lastdim {B}x{K0} K={K}")
        assert torch.equal(out.t, src[:, idx])
        selfg = Guarded((B, K0), torch.float32)
        selfg.t.zero_()
        vals = torch.randn((B, K), device="cuda", generator=g)
        ds2, dv = _lib.desc(selfg.t), _lib.desc(vals)
        _lib.check(L.vbt_b200_index_put_lastdim(ds2.ref, di.ref, dv.ref, 1, 0, None, _lib.stream_ptr(src)))
        selfg.check(f"index_put lastdim {B}x{K0}")


def test_mask_select_and_scale_cast(ops):
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(10)
    for n in (1, 15, 4097, 16384, 16385, 100003, 1 << 20):
        mask = torch.rand(n, device="cuda", generator=g) < 0.37
        need = ctypes.c_size_t()
        _lib.check(L.vbt_b200_mask_select_workspace_bytes(n, ctypes.byref(need)))
        ws = Guarded(((need.value + 7) // 8,), torch.int64)
        idx = Guarded((n,), torch.int64, 1)
        cnt = Guarded((1,), torch.int64)
        dm = _lib.desc(mask)
        _lib.check(L.vbt_b200_mask_select(dm.ref, ctypes.c_void_p(idx.t.data_ptr()), n, ctypes.c_void_p(cnt.t.data_ptr()),
                                          ctypes.c_void_p(ws.t.data_ptr()), need.value, _lib.stream_ptr(mask)))
        for b, w in ((ws, "workspace"), (idx, "indices"), (cnt, "count")):
            b.check(f"mask_select {w} n={n}")
        k = int(cnt.t.item())
        assert torch.equal(idx.t[:k], torch.nonzero(mask).reshape(-1))
        # a capacity smaller than the count: nothing is written past it
        cap = max(k // 2, 1)
        small = Guarded((cap,), torch.int64, 1)
        _lib.check(L.vbt_b200_mask_select(dm.ref, ctypes.c_void_p(small.t.data_ptr()), cap, ctypes.c_void_p(cnt.t.data_ptr()),
                                          ctypes.c_void_p(ws.t.data_ptr()), need.value, _lib.stream_ptr(mask)))
        small.check(f"mask_select capacity n={n}")
        assert torch.equal(small.t[:min(cap, k)], torch.nonzero(mask).reshape(-1)[:cap])
    for n in (1, 7, 1031, 4096):
        part = torch.randn(n, device="cuda", generator=g)
        for dt in (torch.float32, torch.bfloat16):
            out = Guarded((n,), dt, 1)
            _lib.check(L.vbt_b200_scale_cast(ctypes.c_void_p(out.t.data_ptr()), _lib.dtype_code(dt),
                                             ctypes.c_void_p(part.data_ptr()), n, 0.5, _lib.stream_ptr(part)))
            out.check(f"scale_cast {n} {dt}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_ops_forward_and_backward(dtype):
    L = _lib.lib()
    code = _lib.dtype_code(dtype)
    g = torch.Generator(device="cuda").manual_seed(11)

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    cases = [(5, 1), (7, 33), (9, 129), (130, 200), (3, 1031), (2, 5000), (3, 20001), (70, 128), (17, 4096), (33, 8192)]
    for (rows, cols), off in [(c, o) for c in cases for o in (0, 1)]:
        x = (3 * torch.randn((rows, cols), device="cuda", generator=g)).to(dtype)
        dy = torch.randn((rows, cols), device="cuda", generator=g).to(dtype)
        gamma = torch.rand(cols, device="cuda", generator=g) + 0.5
        st = _lib.stream_ptr(x)
        for log in (0, 1):
            y = Guarded((rows, cols), dtype, off)
            _lib.check(L.vbt_b200_softmax(p(y.t), p(x), code, rows, cols, cols, log, st))
            y.check(f"softmax {rows}x{cols}")
            dx = Guarded((rows, cols), dtype, off)
            yc = y.t.contiguous()
            _lib.check(L.vbt_b200_softmax_backward(p(dx.t), p(dy), p(yc), code, rows, cols, cols, cols, log, st))
            dx.check(f"softmax_backward {rows}x{cols}")
        o, inv = Guarded((rows, cols), dtype, off), Guarded((rows,), torch.float32, off)
        _lib.check(L.vbt_b200_rmsnorm(p(o.t), p(inv.t), p(x), p(gamma), code, rows, cols, cols, 1e-6, st))
        o.check(f"rmsnorm out {rows}x{cols}")
        inv.check(f"rmsnorm inv {rows}x{cols}")
        need = ctypes.c_size_t()
        _lib.check(L.vbt_b200_rmsnorm_backward_workspace_bytes(rows, cols, code, 0, ctypes.byref(need)))
        ws = Guarded((max(need.value // 4, 4),), torch.float32)
        dxg, dg = Guarded((rows, cols), dtype, off), Guarded((cols,), torch.float32, off)
        invc = inv.t.contiguous()
        _lib.check(L.vbt_b200_rmsnorm_backward(p(dxg.t), p(dg.t), p(dy), p(x), p(invc), p(gamma), code, rows, cols,
                                               cols, cols, p(ws.t), ws.t.numel() * 4, st))
        for b, w in ((dxg, "dx"), (dg, "dgamma"), (ws, "workspace")):
            b.check(f"rmsnorm_backward {w} {rows}x{cols}")
