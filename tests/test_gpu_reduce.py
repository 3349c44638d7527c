"""CUDA dim reductions vs the CPU oracle through the C ABI.

Bit-exact: int64 everything, amax / amin / argmax / argmin (values and indices).
fp32 sum / mean: |delta| <= 1e-5 * scale against the fp64 truth, scale = max(|truth|,
sigma * sqrt(N)) of the reduced slice (sigma * sqrt(N) computed as sqrt(sum x^2)); the oracle's
own left-to-right fp32 sum is held to the same bound, and the worst observed error of each is
reported on failure.  bf16 / f16: 1e-2 on the same scale."""
import os

import numpy as np
import pytest
import torch

import oracle
from tests.util import CODE, as_f32, from_np, note_worst, rand_storage, to_np

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


@pytest.fixture(scope="module")
def ops():
    from vibetensor_b200 import ops as o
    return o


def _check(ops, port, name, x_np, dtype, dim, view=None, keepdim=False):
    t = from_np(x_np, dtype) if view is None else view
    got = ops.reduce(name, t, dim, keepdim)
    want = port.reduce(name, x_np, CODE[dtype], dim=dim, keepdim=keepdim)
    if name in ("argmax", "argmin"):
        np.testing.assert_array_equal(to_np(got[0]), want[0], err_msg=f"{name} values")
        np.testing.assert_array_equal(to_np(got[1]), want[1], err_msg=f"{name} indices")
        return
    g = to_np(got)
    assert g.shape == want.shape
    if dtype == torch.int64 or name in ("max", "min"):
        np.testing.assert_array_equal(g, want, err_msg=name)
        return
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    xf = as_f32(x_np, dtype).astype(np.float64)
    if name == "prod":
        np.testing.assert_allclose(as_f32(g, dtype), as_f32(want, dtype), rtol=1e-4 if tol < 1e-3 else 3e-2)
        return
    ax = None if dim is None else dim
    truth = xf.sum(axis=ax, keepdims=keepdim)
    scale = np.maximum(np.abs(truth), np.sqrt((xf * xf).sum(axis=ax, keepdims=keepdim)))
    if name == "mean":
        n = xf.size if dim is None else xf.shape[dim]
        scale, truth = scale / n, truth / n
    err = np.abs(as_f32(g, dtype).astype(np.float64) - truth)
    ref_err = np.abs(as_f32(want, dtype).astype(np.float64) - truth)
    worst, ref_worst = float((err / (scale + 1e-300)).max()), float((ref_err / (scale + 1e-300)).max())
    note_worst(f"reduce {name} {str(dtype)[6:]}", worst, tol)
    assert (err <= tol * scale + 1e-30).all(), \
        f"{name}: worst error {worst:.3e} of scale (oracle's own: {ref_worst:.3e}), bound {tol:.0e}"


SHAPES = [((64, 96), -1), ((64, 96), 0), ((4096, 17), 0), ((17, 4096), -1), ((3, 5000), 1),
          ((5000, 3), 0), ((7, 33, 9), 1), ((1, 300000), 1), ((300000,), 0), ((2, 3, 4, 5), 2),
          ((257, 129), None), ((1, 1), 0), ((8, 16384), -1), ((16384, 8), 0)]


@pytest.mark.parametrize("shape,dim", SHAPES)
@pytest.mark.parametrize("name", ["sum", "mean", "max", "min", "argmax", "argmin"])
def test_fp32(ops, port, name, shape, dim):
    rng = np.random.default_rng(abs(hash((shape, dim))) % 2 ** 31)
    x = rng.standard_normal(shape, dtype=np.float32)
    _check(ops, port, name, x, torch.float32, dim)


@pytest.mark.parametrize("shape,dim", SHAPES[:8])
@pytest.mark.parametrize("name", ["sum", "max", "min", "prod", "argmax"])
def test_int64_exact(ops, port, name, shape, dim):
    rng = np.random.default_rng(21)
    x = rng.integers(-3, 4, shape).astype(np.int64) if name == "prod" else \
        rng.integers(-2 ** 40, 2 ** 40, shape).astype(np.int64)
    _check(ops, port, name, x, torch.int64, dim)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,dim", [((512, 200), 0), ((200, 512), -1), ((3000,), 0), ((64, 8, 33), 1)])
@pytest.mark.parametrize("name", ["sum", "mean", "max", "argmax"])
def test_half_types(ops, port, name, dtype, shape, dim):
    rng = np.random.default_rng(22)
    x = rand_storage(rng, shape, dtype)
    _check(ops, port, name, x, dtype, dim)


ONCE = [  # (dtype, base shape, columns kept, kernel the sum takes: 7 = one-pass block per slice)
    (torch.float32, (200, 2004), 2003, 7),    # 500 vectors + 3 tail elements, 128 threads
    (torch.float32, (200, 1004), 1003, 1),    # 4 KiB and less: one warp per slice
    (torch.float32, (64, 4096), 4096, 7),     # exactly 256 threads x 4 vectors
    (torch.float32, (100, 4), 3, 1),          # no whole vector: the tail path holds element 0
    (torch.float32, (70, 2052), 2049, 7),     # 512 vectors + 1: 256 threads, last pass nearly empty
    (torch.bfloat16, (300, 8192), 8190, 7),   # 8-element vectors, 6 tail elements
    (torch.int64, (128, 2048), 2047, 7),      # 2-element vectors
    (torch.float32, (63, 4096), 4096, 2),     # fewer than 64 slices: the general block kernel
    (torch.float32, (64, 4100), 4100, 2)]     # one vector too long for one pass


@pytest.mark.parametrize("dtype,base,cols,kernel", ONCE)
def test_one_pass_row_kernel(ops, port, dtype, base, cols, kernel):
    """Slices of at most 1024 vectors with 64 or more outputs take the one-pass kernel (a block per
    slice, straight-line code): whole and partial last vectors, both block sizes, every vector
    width, ties and a NaN at position 0 for the extrema, and the shapes just outside its range."""
    from vibetensor_b200 import _lib
    rng = np.random.default_rng(51)
    x = rand_storage(rng, base, dtype)
    t = from_np(x, dtype)[:, :cols]
    xv = np.ascontiguousarray(x[:, :cols])
    for name in ("sum", "mean", "max", "min", "argmax", "argmin") if dtype != torch.int64 else ("sum", "max", "argmin"):
        _check(ops, port, name, xv, dtype, -1, view=t)
        if name == "sum":
            info = _lib.last_launch_info()
            assert (info.family, info.kernel) == (2, kernel), (info.family, info.kernel)
    if dtype == torch.float32:
        y = xv.copy()
        y[::3, 0] = np.nan                       # NaN at position 0 wins for max / min ...
        y[1::3, min(5, cols - 1)] = np.nan       # ... and is ignored anywhere else (rows that have both keep rule 1)
        y[2::3, :] = 1.5                         # all ties: the first index
        ty = torch.from_numpy(np.ascontiguousarray(y)).cuda()
        for name in ("max", "min", "argmax", "argmin"):
            _check(ops, port, name, np.ascontiguousarray(y), dtype, -1, view=ty)


def test_argmax_long_slices_take_one_warp_per_slice(ops, port):
    """argmax / argmin over many slices of 4 - 32 KiB: one warp per slice, four accumulators per lane;
    ties across accumulators, lanes and the tail must still resolve to the first index."""
    from vibetensor_b200 import _lib
    rng = np.random.default_rng(52)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows = sms * 16 + 5
    for cols in (4096, 1500, 8190):
        x = rng.integers(-3, 4, (rows, cols)).astype(np.float32)   # few distinct values: ties everywhere
        x[7, :] = 2.0
        x[8, 0] = np.nan
        t = torch.from_numpy(x).cuda()
        for name in ("argmax", "argmin"):
            _check(ops, port, name, x, torch.float32, -1, view=t)
            info = _lib.last_launch_info()
            assert (info.family, info.kernel) == (2, 1), (info.family, info.kernel)


def test_keepdim_and_multi_dim(ops, port, ref):
    x = GOLD["red3_x"]
    t = torch.from_numpy(x).cuda()
    np.testing.assert_allclose(ops.reduce("sum", t, (0, 2)).cpu().numpy(), GOLD["red3_sum_02"], rtol=1e-5, atol=1e-5)
    got = ops.reduce("mean", t, (1, 2), keepdim=True).cpu().numpy()
    assert got.shape == (5, 1, 1)
    np.testing.assert_allclose(got, GOLD["red3_mean_12_keep"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ops.reduce("sum", t, 1).cpu().numpy(), GOLD["red3_sum_1"], rtol=1e-5, atol=1e-5)
    assert ops.reduce("sum", t, -1, keepdim=True).shape == (5, 7, 1)


def test_golden_reference_vectors(ops):
    x = torch.from_numpy(GOLD["red_x"]).cuda()
    np.testing.assert_allclose(ops.sum(x, -1).cpu().numpy(), GOLD["red_sum_m1"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(ops.mean(x, 0).cpu().numpy(), GOLD["red_mean_0"], rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(ops.amax(x, -1).cpu().numpy(), GOLD["red_amax_m1"])
    np.testing.assert_array_equal(ops.amin(x, 0).cpu().numpy(), GOLD["red_amin_0"])
    np.testing.assert_array_equal(ops.argmax(x, -1).cpu().numpy(), GOLD["red_argmax_m1_idx"])
    np.testing.assert_array_equal(ops.argmax(x.t(), -1).cpu().numpy(), GOLD["red_t_argmax_m1_idx"])
    np.testing.assert_allclose(ops.sum(x.t(), -1).cpu().numpy(), GOLD["red_t_sum_m1"], rtol=1e-5, atol=1e-5)
    xt = torch.from_numpy(GOLD["red_tie_x"]).cuda()
    np.testing.assert_array_equal(ops.argmax(xt, -1).cpu().numpy(), GOLD["red_tie_argmax_idx"])
    np.testing.assert_array_equal(ops.argmax(xt, 0).cpu().numpy(), GOLD["red_tie_argmax0_idx"])
    xi = torch.from_numpy(GOLD["red_i64_x"]).cuda()
    np.testing.assert_array_equal(ops.sum(xi, -1).cpu().numpy(), GOLD["red_i64_sum_m1"])
    np.testing.assert_array_equal(ops.amax(xi, 0).cpu().numpy(), GOLD["red_i64_amax_0"])
    np.testing.assert_array_equal(ops.argmax(xi, -1).cpu().numpy(), GOLD["red_i64_argmax_m1_idx"])


def test_config1_shapes_contiguous_and_transposed(ops, port):
    """[4096,4096] fp32 N(0,1) seed 0: sum(-1), mean(0), amax(-1), argmax(-1) on the tensor
    and on its transposed view."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4096, 4096), dtype=np.float32)
    t = torch.from_numpy(x).cuda()
    for view_np, view_t in ((x, t), (x.T, t.t())):
        _check(ops, port, "sum", view_np, torch.float32, -1, view=view_t)
        _check(ops, port, "mean", view_np, torch.float32, 0, view=view_t)
        _check(ops, port, "max", view_np, torch.float32, -1, view=view_t)
        _check(ops, port, "argmax", view_np, torch.float32, -1, view=view_t)


def test_nan_and_inf_rules(ops):
    nan, inf = float("nan"), float("inf")
    t = lambda v: torch.tensor(v, dtype=torch.float32, device="cuda")  # noqa: E731
    assert np.isnan(ops.amax(t([nan, 1.0, 2.0])).item())
    assert ops.amax(t([1.0, nan, 2.0])).item() == 2.0
    v, i = ops.reduce("argmax", t([[1.0, nan, 5.0, 5.0]]), 1)
    assert v.item() == 5.0 and i.item() == 2
    v, i = ops.reduce("argmax", t([[nan, 9.0]]), 1)
    assert np.isnan(v.item()) and i.item() == 0
    # tests/py/test_cuda_reduction.py:122-150 of the reference
    assert ops.amin(t([inf, inf])).item() == inf
    assert ops.amax(t([-inf, -inf])).item() == -inf
    assert ops.amin(t([1.0, inf])).item() == 1.0
    assert ops.amax(t([-inf, 2.0])).item() == 2.0
    assert ops.argmax(t([-inf, -inf, -inf])).item() == 0


@pytest.mark.parametrize("shape,dim", [((3, 70000), 1), ((700, 300), 0), ((5, 64, 33), 1), ((40, 9), 1)])
def test_arg_ops_when_nothing_beats_the_identity(ops, port, shape, dim):
    """Slices that hold only -inf / NaN (argmax), +inf (argmin) or INT64_MIN: index 0, as the
    CPU scan that starts from element 0; plus ties, where the first position wins."""
    x = np.full(shape, -np.inf, np.float32)
    x[0] = np.nan if dim != 0 else -np.inf
    x.flat[5::7] = np.nan
    x[-1] = 3.0                                   # a slice (or part of each) with ties everywhere
    for name, arr in (("argmax", x), ("argmin", -x)):
        v, i = ops.reduce(name, torch.from_numpy(arr).cuda(), dim)
        wv, wi = port.reduce(name, arr, oracle.F32, dim=dim)
        np.testing.assert_array_equal(i.cpu().numpy(), wi)
        np.testing.assert_array_equal(v.cpu().numpy(), wv)
    xi = np.full(shape, np.iinfo(np.int64).min, np.int64)
    xi[-1] = 4
    v, i = ops.reduce("argmax", torch.from_numpy(xi).cuda(), dim)
    wv, wi = port.reduce("argmax", xi, oracle.I64, dim=dim)
    np.testing.assert_array_equal(i.cpu().numpy(), wi)
    np.testing.assert_array_equal(v.cpu().numpy(), wv)


def test_empty_semantics_and_errors(ops):
    x = torch.zeros((3, 0), device="cuda")
    assert ops.sum(x, 1).tolist() == [0.0, 0.0, 0.0]
    assert ops.prod(x, 1).tolist() == [1.0, 1.0, 1.0]
    assert torch.isnan(ops.mean(x, 1)).all()
    with pytest.raises(RuntimeError, match="amax: empty"):
        ops.amax(x, 1)
    with pytest.raises(RuntimeError, match="amin: empty"):
        ops.argmin(x, 1)
    assert ops.sum(x, 0).shape == (0,)          # empty output, not an error
    assert ops.amax(x, 0).shape == (0,)
    with pytest.raises(ValueError, match="dim out of range"):
        ops.sum(torch.zeros(3, device="cuda"), 2)
    with pytest.raises(ValueError, match="mean: expected dtype=float32"):
        ops.mean(torch.zeros(3, dtype=torch.int64, device="cuda"))
    with pytest.raises(ValueError, match="unsupported dtype"):
        ops.sum(torch.zeros(3, dtype=torch.int32, device="cuda"))


def test_run_to_run_determinism(ops):
    x = torch.randn(1 << 24, device="cuda")
    a = ops.sum(x)
    for _ in range(3):
        assert torch.equal(ops.sum(x), a)
    y = torch.randn((8192, 512), device="cuda")
    b = ops.mean(y, 0)
    for _ in range(3):
        assert torch.equal(ops.mean(y, 0), b)


def test_generic_layout(ops, port):
    rng = np.random.default_rng(23)
    x = rng.standard_normal((6, 7, 8), dtype=np.float32)
    t = torch.from_numpy(x).cuda().permute(2, 0, 1)  # sizes [8,6,7], no unit-stride kept dim last
    xp = x.transpose(2, 0, 1)
    for dim in (0, 1, 2):
        _check(ops, port, "sum", xp, torch.float32, dim, view=t)
        _check(ops, port, "argmax", xp, torch.float32, dim, view=t)


def test_large_sum_properties(ops):
    """2^28 fp32 elements: linearity and agreement with an fp64 fold of chunk sums."""
    n = 1 << 28
    x = torch.randn(n, device="cuda")
    s = ops.sum(x).item()
    truth = x.double().sum().item()
    scale = max(abs(truth), float(x.double().pow(2).sum().sqrt().item()))
    note_worst("reduce sum float32 [2^28]", abs(s - truth) / scale, 1e-5)
    assert abs(s - truth) <= 1e-5 * scale
    s2 = ops.sum(ops.mul(x, 2.0)).item()
    assert s2 == 2.0 * s  # scaling by 2 is exact, so the fixed-order sum doubles exactly
    assert ops.amax(x).item() == x.max().item()
    assert ops.argmax(x).item() == int(torch.argmax(x).item()) or x[ops.argmax(x)] == x.max()
