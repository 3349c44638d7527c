"""Row-wise softmax / log_softmax / RMSNorm vs the CPU oracle through the C ABI.
Tolerances are the ones the task states for this path: 1e-5 relative for fp32, 1e-2 for
bf16 (f16: 2e-3); softmax rows must also sum to one."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CODE, as_f32, from_np, to_np

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 2e-3}
# one shape per kernel variant: group G=8/16/32, VPL 1/2/4, block 128/256, stream, ragged
COLS = [8, 24, 64, 128, 200, 512, 1000, 1024, 2048, 4096, 5000, 8192, 16384, 20000, 33, 1]


@pytest.fixture(scope="module")
def kernels():
    from vibetensor_b200 import kernels as k
    return k


def _x(rng, rows, cols, dtype, sigma=3.0):
    return oracle.to_storage(sigma * rng.standard_normal((rows, cols), dtype=np.float32), CODE[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", COLS)
def test_softmax(kernels, port, dtype, cols):
    rng = np.random.default_rng(3)
    rows = 70 if cols <= 4096 else 9
    x = _x(rng, rows, cols, dtype)
    tol = TOL[dtype]
    got = as_f32(to_np(kernels.softmax(from_np(x, dtype))), dtype)
    want = as_f32(port.softmax(x, CODE[dtype]), dtype)
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol * 1e-2 if dtype == torch.float32 else tol * 0.05)
    np.testing.assert_allclose(got.sum(-1), 1.0, atol=1e-5 if dtype == torch.float32 else 2e-2)
    gl = as_f32(to_np(kernels.log_softmax(from_np(x, dtype))), dtype)
    wl = as_f32(port.softmax(x, CODE[dtype], log=True), dtype)
    np.testing.assert_allclose(gl, wl, rtol=tol, atol=tol * 10)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", COLS)
def test_rmsnorm(kernels, port, dtype, cols):
    rng = np.random.default_rng(3)
    rows = 70 if cols <= 4096 else 9
    x = _x(rng, rows, cols, dtype)
    gamma = (1 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
    tol = TOL[dtype]
    y, inv = kernels.rmsnorm(from_np(x, dtype), torch.from_numpy(gamma).cuda(), 1e-6)
    wy, winv = port.rmsnorm(x, gamma, 1e-6, CODE[dtype])
    np.testing.assert_allclose(as_f32(to_np(y), dtype), as_f32(wy, dtype), rtol=tol, atol=tol * 0.1)
    np.testing.assert_allclose(inv.cpu().numpy(), winv, rtol=1e-5)
    y2, _ = kernels.rmsnorm(from_np(x, dtype))  # no gamma
    wy2, _ = port.rmsnorm(x, None, 1e-6, CODE[dtype])
    np.testing.assert_allclose(as_f32(to_np(y2), dtype), as_f32(wy2, dtype), rtol=tol, atol=tol * 0.1)


def test_matches_torch_like_the_reference_tests(kernels):
    # vibe_kernels/rmsnorm/tests/test_rmsnorm.py:19-46 (atol 1e-4 fp32, 1e-2 bf16)
    torch.manual_seed(0)
    x = torch.randn(64, 4096, device="cuda")
    g = torch.randn(4096, device="cuda")
    y, _ = kernels.rmsnorm(x, g, 1e-6)
    torch.testing.assert_close(y, torch.nn.functional.rms_norm(x, (4096,), g, 1e-6), atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(kernels.softmax(x), torch.softmax(x, -1), atol=1e-6, rtol=1e-5)
    xb = x.bfloat16()
    yb, _ = kernels.rmsnorm(xb, g, 1e-6)
    torch.testing.assert_close(yb.float(), torch.nn.functional.rms_norm(xb.float(), (4096,), g, 1e-6), atol=3e-2, rtol=1e-2)


def test_row_strided_and_nd_views(kernels, port):
    rng = np.random.default_rng(4)
    big = (3 * rng.standard_normal((40, 300), dtype=np.float32))
    t = torch.from_numpy(big).cuda()
    got = kernels.softmax(t[:, :128]).cpu().numpy()          # row stride 300, 128 columns
    np.testing.assert_allclose(got, port.softmax(np.ascontiguousarray(big[:, :128]), oracle.F32), rtol=1e-5, atol=1e-7)
    got = kernels.softmax(t[:, 1:130]).cpu().numpy()         # misaligned start -> scalar kernel
    np.testing.assert_allclose(got, port.softmax(np.ascontiguousarray(big[:, 1:130]), oracle.F32), rtol=1e-5, atol=1e-7)
    x3 = t.reshape(5, 8, 300)
    got = kernels.softmax(x3).cpu().numpy().reshape(40, 300)
    np.testing.assert_allclose(got, port.softmax(big, oracle.F32), rtol=1e-5, atol=1e-7)
    got = kernels.softmax(t.t()).cpu().numpy()               # column stride != 1 -> copied first
    np.testing.assert_allclose(got, port.softmax(np.ascontiguousarray(big.T), oracle.F32), rtol=1e-5, atol=1e-7)


def test_edge_values(kernels):
    ninf = float("-inf")
    x = torch.tensor([[0.0, ninf, 1.0, ninf], [ninf] * 4, [1e4, -1e4, 0.0, 5.0]], device="cuda")
    y = kernels.softmax(x)
    assert y[0, 1].item() == 0.0 and abs(y[0].sum().item() - 1) < 1e-6
    assert torch.isnan(y[1]).all()          # all -inf row: NaN, as the reference's formula gives
    assert y[2].tolist() == [1.0, 0.0, 0.0, 0.0]
    assert kernels.softmax(torch.empty((0, 5), device="cuda")).shape == (0, 5)
    assert kernels.softmax(torch.empty((5, 0), device="cuda")).shape == (5, 0)
    with pytest.raises(NotImplementedError):
        kernels.softmax(torch.zeros((3, 4), device="cuda"), dim=0)
    with pytest.raises(TypeError):
        kernels.softmax(torch.zeros((3, 4), dtype=torch.int64, device="cuda"))
    with pytest.raises(RuntimeError):
        kernels.softmax(torch.zeros((3, 4)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(32768, 4096), (262144, 128)])
def test_config4_full_size_properties(kernels, dtype, shape):
    """Full benchmark shapes, N(0,3): softmax rows sum to 1 and are invariant to a per-row
    shift; RMSNorm output has unit RMS (gamma = 1) and inv_rms matches a float64 recompute on
    a sample of rows."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = (3 * torch.randn(shape, device="cuda", generator=g)).to(dtype)
    y = kernels.softmax(x)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (y.float().sum(-1) - 1).abs().max().item() < tol
    shift = torch.arange(shape[0], device="cuda").remainder(5).float().reshape(-1, 1)
    if dtype == torch.float32:
        y2 = kernels.softmax(x + shift)
        assert (y2 - y).abs().max().item() < 1e-5
    o, inv = kernels.rmsnorm(x)
    rms = o.float().pow(2).mean(-1).sqrt()
    assert (rms - 1).abs().max().item() < (1e-4 if dtype == torch.float32 else 1e-2)
    rows = torch.arange(0, shape[0], max(1, shape[0] // 257), device="cuda")
    want = (x[rows].double().pow(2).mean(-1) + 1e-6).rsqrt()
    torch.testing.assert_close(inv[rows].double(), want, rtol=1e-5, atol=0)


# ---- backward ------------------------------------------------------------------------------
BWD_COLS = [8, 32, 64, 200, 256, 512, 1000, 1024, 2048, 4096, 8192, 16384, 20000, 33, 1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", BWD_COLS)
def test_softmax_backward(kernels, port, dtype, cols):
    rng = np.random.default_rng(31)
    rows = 70 if cols <= 4096 else 9
    tol = TOL[dtype]
    dy = _x(rng, rows, cols, dtype, 1.0)
    for log in (False, True):
        y = port.softmax(_x(rng, rows, cols, dtype), CODE[dtype], log=log)
        fn = kernels.log_softmax_backward if log else kernels.softmax_backward
        got = as_f32(to_np(fn(from_np(dy, dtype), from_np(y, dtype))), dtype)
        want = as_f32(port.softmax_backward(dy, y, CODE[dtype], log=log), dtype)
        # dx is a difference of O(|dy|) terms: absolute bound of a few float ulps of |dy| ~ 1
        np.testing.assert_allclose(got, want, rtol=tol, atol=tol if dtype == torch.float32 else tol * 0.1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", BWD_COLS)
def test_rmsnorm_backward(kernels, port, dtype, cols):
    rng = np.random.default_rng(32)
    rows = 700 if cols <= 256 else 70 if cols <= 4096 else 9
    tol = TOL[dtype]
    x = _x(rng, rows, cols, dtype)
    dy = _x(rng, rows, cols, dtype, 1.0)
    gamma = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    _, inv = port.rmsnorm(x, gamma, 1e-6, CODE[dtype])
    tg = torch.from_numpy(gamma).cuda()
    dx, dg = kernels.rmsnorm_backward(from_np(dy, dtype), from_np(x, dtype), torch.from_numpy(inv).cuda(), tg)
    wdx, wdg = port.rmsnorm_backward(dy, x, inv, gamma, CODE[dtype])
    np.testing.assert_allclose(as_f32(to_np(dx), dtype), as_f32(wdx, dtype), rtol=tol, atol=tol * 0.1)
    # the reference's own test bound for fp32 RMSNorm (vibe_kernels/rmsnorm/tests/test_rmsnorm.py:19-46)
    np.testing.assert_allclose(dg.cpu().numpy(), wdg, rtol=1e-4, atol=1e-4)
    dx2, dg2 = kernels.rmsnorm_backward(from_np(dy, dtype), from_np(x, dtype), torch.from_numpy(inv).cuda())
    assert dg2 is None
    wdx2, _ = port.rmsnorm_backward(dy, x, inv, None, CODE[dtype])
    np.testing.assert_allclose(as_f32(to_np(dx2), dtype), as_f32(wdx2, dtype), rtol=tol, atol=tol * 0.1)


def test_backward_matches_torch_autograd_and_is_reproducible(kernels):
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((513, 1536), device="cuda", generator=g, requires_grad=True)
    dy = torch.randn((513, 1536), device="cuda", generator=g)
    gamma = torch.rand((1536,), device="cuda", generator=g, requires_grad=True) + 0.5
    gamma = gamma.detach().requires_grad_(True)
    y, inv = kernels.rmsnorm(x.detach(), gamma.detach(), 1e-6)
    dx, dg = kernels.rmsnorm_backward(dy, x.detach(), inv, gamma.detach())
    wdx, wdg = torch.autograd.grad(torch.nn.functional.rms_norm(x, (1536,), gamma, 1e-6), (x, gamma), dy)
    torch.testing.assert_close(dx, wdx, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dg, wdg, rtol=1e-4, atol=1e-4)
    for _ in range(3):  # fixed-order fold of the partial rows: bit-identical run to run
        dx_b, dg_b = kernels.rmsnorm_backward(dy, x.detach(), inv, gamma.detach())
        assert torch.equal(dg_b, dg) and torch.equal(dx_b, dx)
    p = kernels.softmax(x.detach())
    (w,) = torch.autograd.grad(torch.softmax(x, -1), x, dy)
    torch.testing.assert_close(kernels.softmax_backward(dy, p), w, rtol=1e-4, atol=1e-6)
    lp = kernels.log_softmax(x.detach())
    (w,) = torch.autograd.grad(torch.log_softmax(x, -1), x, dy)
    torch.testing.assert_close(kernels.log_softmax_backward(dy, lp), w, rtol=1e-4, atol=1e-5)


def test_backward_row_strided_views_and_errors(kernels, port):
    rng = np.random.default_rng(33)
    base = oracle.to_storage(rng.standard_normal((40, 768), dtype=np.float32), oracle.F32)
    dyb = oracle.to_storage(rng.standard_normal((40, 768), dtype=np.float32), oracle.F32)
    x, dy = base[:, :512], dyb[:, 256:]                       # row stride 768, 512 columns
    tx, tdy = torch.from_numpy(base).cuda()[:, :512], torch.from_numpy(dyb).cuda()[:, 256:]
    gamma = np.ones(512, np.float32)
    _, inv = port.rmsnorm(np.ascontiguousarray(x), gamma, 1e-6, oracle.F32)
    dx, dg = kernels.rmsnorm_backward(tdy, tx, torch.from_numpy(inv).cuda(), torch.from_numpy(gamma).cuda())
    wdx, wdg = port.rmsnorm_backward(dy, x, inv, gamma, oracle.F32)
    np.testing.assert_allclose(dx.cpu().numpy(), wdx, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(dg.cpu().numpy(), wdg, rtol=1e-4, atol=1e-4)
    y = port.softmax(np.ascontiguousarray(x), oracle.F32)
    got = kernels.softmax_backward(tdy, torch.from_numpy(y).cuda())
    np.testing.assert_allclose(got.cpu().numpy(), port.softmax_backward(np.ascontiguousarray(dy), y, oracle.F32),
                               rtol=1e-5, atol=1e-7)
    with pytest.raises(TypeError):
        kernels.softmax_backward(tdy, tx.bfloat16())
    with pytest.raises(ValueError):
        kernels.softmax_backward(tdy[:, :100], tx)
    with pytest.raises(RuntimeError):
        kernels.rmsnorm_backward(tdy.cpu(), tx.cpu(), torch.from_numpy(inv))
    e = torch.empty((0, 16), device="cuda")
    dx, dg = kernels.rmsnorm_backward(e, e, torch.empty((0,), device="cuda"), torch.ones(16, device="cuda"))
    assert dx.shape == (0, 16) and dg.tolist() == [0.0] * 16
