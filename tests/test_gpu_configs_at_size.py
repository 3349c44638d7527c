"""The benchmark configurations at their STATED sizes, CUDA path vs the CPU oracle.

The small-shape files prove the kernels on every code path; here the same comparisons run at
the sizes the configurations name, where 64-bit offsets, grid limits and the split / ticket
paths are really exercised.  Where the oracle over the whole output would take minutes, a
seeded sample of rows or planes is compared and the rest is covered by a structural check; the
sampling is stated in each test.

  C2  table [1 048 576 x 256], 4 194 304 indices (seed 2): gather bit-exact over the WHOLE
      output; scatter_add int64 bit-exact and fp32 within 1e-5 of the per-element mass, through
      both engines (atomics, sorted), with the oracle fed chunks of <= 390 625 indices in index
      order as the reference's 1e8-element cap forces (src/vbt/core/indexing_advanced.cc:100-103).
      The reference's CUDA advanced-index form x[..., idx] on [4096, 65536] fp32 with 65 536
      uniform int64 indices, and a bool mask of 2^28 elements turned into indices: 64 sampled
      rows against the oracle plus the whole output against a second, independent gather;
      the mask's indices against numpy on sampled windows plus count and monotonicity.
  C3  bf16 where(a > 0, a + b*c, 0) into the transpose(1,3) view of a [64,1024,512,128] output
      (seed 1): 64 sampled [128 x 1024] planes bit-exact, guard bands around the storage intact.
  C4  softmax / RMSNorm forward and backward on [32768,4096] and [262144,128], fp32 and bf16
      (seed 3): 257 sampled rows at 1e-5 / 1e-2; dgamma against the oracle over ALL rows.
  C5  sum and amax of [2^32] fp32 and bf16 mean(dim=0) of [1 048 576, 4096] on one GPU (seed 4):
      against the fp64 truth and against the reference's own sequential fp32 sum on a 2^28 slice.
"""
import numpy as np
import pytest
import torch

import oracle
from tests.util import CODE, as_f32, from_np, note_worst, to_np

pytestmark = pytest.mark.gpu
CHUNK = 390_625  # indices per oracle call


@pytest.fixture(scope="module")
def ops():
    from vibetensor_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def kernels():
    from vibetensor_b200 import kernels as k
    return k


# ------------------------------------------------------------------------------------------
# C2
# ------------------------------------------------------------------------------------------
V, D, N = 1 << 20, 256, 1 << 22


@pytest.fixture(scope="module")
def c2():
    rng = np.random.default_rng(2)
    table = rng.standard_normal((V, D), dtype=np.float32)
    idx_u = rng.integers(0, V, N).astype(np.int64)
    p = np.arange(1, V + 1, dtype=np.float64) ** -1.1
    ranks = np.searchsorted(np.cumsum(p / p.sum()), rng.random(N))
    idx_z = rng.permutation(V)[np.minimum(ranks, V - 1)].astype(np.int64)
    return {"rng": rng, "table": table, "idx_u": idx_u, "idx_z": idx_z}


def test_c2_gather_whole_output_bit_exact(ops, port, c2):
    table, idx = c2["table"], c2["idx_u"]
    out = ops.index_rows(torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda())
    assert out.shape == (N, D)
    for c0 in range(0, N, CHUNK):
        want = port.gather_rows(table, idx[c0:c0 + CHUNK])
        np.testing.assert_array_equal(out[c0:c0 + CHUNK].cpu().numpy(), want, err_msg=f"rows {c0}..")


def _oracle_scatter(port, idx, upd, code, dtype):
    acc = np.zeros((V, D), dtype)
    for c0 in range(0, N, CHUNK):
        port.scatter_rows(acc, idx[c0:c0 + CHUNK], upd[c0:c0 + CHUNK], code)
    return acc


def test_c2_scatter_add_fp32_both_engines(ops, port, c2):
    idx = c2["idx_z"]
    upd = c2["rng"].standard_normal((N, D), dtype=np.float32)
    want = _oracle_scatter(port, idx, upd, oracle.F32, np.float32)
    mass = np.zeros((V, D), np.float32)
    for c0 in range(0, N, CHUNK):
        port.scatter_rows(mass, idx[c0:c0 + CHUNK], np.abs(upd[c0:c0 + CHUNK]), oracle.F32)
    ti, tu = torch.from_numpy(idx).cuda(), torch.from_numpy(upd).cuda()
    del upd
    for deterministic in (False, True):
        acc = torch.zeros((V, D), device="cuda")
        ops.index_put_rows_(acc, ti, tu, accumulate=True, deterministic=deterministic)
        got = acc.cpu().numpy()
        err = np.abs(got.astype(np.float64) - want)
        bound = 1e-5 * mass.astype(np.float64)
        note_worst(f"C2 scatter_add fp32 {'sorted' if deterministic else 'atomics'} (of per-element mass)",
                   float((err / np.maximum(mass, 1e-30)).max()), 1e-5)
        assert (err <= bound + 1e-30).all(), f"deterministic={deterministic}: {float(err.max())}"
        # rows no index names stay exactly zero
        untouched = np.ones(V, bool)
        untouched[idx] = False
        assert not got[untouched].any()
        del acc, got


def test_c2_scatter_add_int64_both_engines_bit_exact(ops, port, c2):
    idx = c2["idx_z"]
    upd = c2["rng"].integers(-1000, 1001, (N, D)).astype(np.int64)
    want = _oracle_scatter(port, idx, upd, oracle.I64, np.int64)
    ti, tu = torch.from_numpy(idx).cuda(), torch.from_numpy(upd).cuda()
    del upd
    for deterministic in (True, False):
        acc = torch.zeros((V, D), device="cuda", dtype=torch.int64)
        ops.index_put_rows_(acc, ti, tu, accumulate=True, deterministic=deterministic)
        np.testing.assert_array_equal(acc.cpu().numpy(), want, err_msg=f"deterministic={deterministic}")
        del acc


def test_c2_index_lastdim_at_size_sampled_rows_and_whole_output(ops, port):
    """x[..., idx] at the bench shape: the register-output kernel with two index chunks.  64
    sampled rows bit-exact against the oracle; every row against torch's own gather (an
    independent implementation, here only as a second checker); wrapped negative indices."""
    from vibetensor_b200 import _lib
    rng = np.random.default_rng(5)
    B, K0 = 4096, 65536
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    x = torch.randn((B, K0), device="cuda", generator=g)
    idx = rng.integers(-K0, K0, K0).astype(np.int64)
    ti = torch.from_numpy(idx).cuda()
    got = ops.index_lastdim(x, ti)
    info = _lib.last_launch_info()
    assert (info.family, info.kernel) == (3, 9), "expected the register-output last-dim kernel"
    rows = np.sort(rng.choice(B, 64, replace=False))
    xs = x[torch.from_numpy(rows).cuda()].cpu().numpy()
    np.testing.assert_array_equal(got[torch.from_numpy(rows).cuda()].cpu().numpy(), port.index_lastdim(xs, idx))
    pos = torch.from_numpy(np.where(idx < 0, idx + K0, idx)).cuda()
    for r0 in range(0, B, 512):   # in slabs: the second checker's output is as large as ours
        assert torch.equal(got[r0:r0 + 512], x[r0:r0 + 512][:, pos]), f"rows {r0}.."


def test_c2_mask_to_indices_at_size(ops):
    """bool mask of 2^28 elements, about half true: ascending int64 indices of the true
    elements.  Count, strict monotonicity and membership over the whole output; exact
    positions against numpy on sampled windows."""
    n = 1 << 28
    g = torch.Generator(device="cuda")
    g.manual_seed(6)
    mask = torch.rand(n, device="cuda", generator=g) < 0.5
    idx = ops.mask_to_indices(mask)
    assert idx.dtype == torch.int64 and idx.numel() == int(mask.sum().item())
    assert bool((idx[1:] > idx[:-1]).all())
    assert bool(mask[idx].all())
    m = mask.cpu().numpy()
    got = idx.cpu().numpy()
    for lo in (0, 12_345_678, n - (1 << 20)):
        hi = lo + (1 << 20)
        want = lo + np.flatnonzero(m[lo:hi])
        a, b = np.searchsorted(got, lo), np.searchsorted(got, hi)
        np.testing.assert_array_equal(got[a:b], want)


# ------------------------------------------------------------------------------------------
# C3
# ------------------------------------------------------------------------------------------
def test_c3_fused_chain_at_size_sampled_planes_and_guard_bands(ops, port):
    rng = np.random.default_rng(1)
    a = oracle.f32_to_bf16_bits(rng.standard_normal((64, 1, 512, 1), dtype=np.float32)).reshape(64, 1, 512, 1)
    b = oracle.f32_to_bf16_bits(rng.standard_normal((1, 128, 1, 1024), dtype=np.float32)).reshape(1, 128, 1, 1024)
    c = oracle.f32_to_bf16_bits(rng.standard_normal((64, 128, 1, 1024), dtype=np.float32)).reshape(64, 128, 1, 1024)
    numel = 64 * 1024 * 512 * 128
    guard = 1 << 16
    sentinel = 0x7FC1  # a NaN pattern no computation here produces
    buf = torch.full((numel + 2 * guard,), sentinel, dtype=torch.int16, device="cuda").view(torch.bfloat16)
    base = buf[guard:guard + numel].view(64, 1024, 512, 128)
    outv = base.transpose(1, 3)  # sizes [64,128,512,1024], strides (67108864, 1, 128, 65536)
    assert outv.stride() == (67108864, 1, 128, 65536)
    ta, tb, tc = (from_np(v, torch.bfloat16) for v in (a, b, c))
    ops.where_gt0_addcmul(ta, tb, tc, out=outv)
    torch.cuda.synchronize()
    gb = buf.view(torch.int16)
    assert bool((gb[:guard] == sentinel).all()) and bool((gb[-guard:] == sentinel).all()), "write outside the output"
    pick = np.random.default_rng(11)
    planes = {(0, 0), (63, 511), (0, 511), (63, 0)}
    while len(planes) < 64:
        planes.add((int(pick.integers(0, 64)), int(pick.integers(0, 512))))
    for n, h in sorted(planes):
        want = port.ternary("where_gt0_addcmul", a[n, :, h, :], b[0, :, 0, :], c[n, :, 0, :], oracle.BF16)
        got = to_np(outv[n, :, h, :])
        np.testing.assert_array_equal(got, want.reshape(128, 1024), err_msg=f"plane n={n} h={h}")
    # every element was written: no sentinel is left inside the output
    assert not bool((base.view(torch.int16) == sentinel).any())


# ------------------------------------------------------------------------------------------
# C4
# ------------------------------------------------------------------------------------------
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(32768, 4096), (262144, 128)])
def test_c4_row_ops_at_size_sampled_rows(kernels, port, dtype, shape):
    rows, cols = shape
    rng = np.random.default_rng(3)
    code, tol = CODE[dtype], TOL[dtype]
    x = oracle.to_storage(3.0 * rng.standard_normal(shape, dtype=np.float32), code)
    gamma = (1 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
    dy = oracle.to_storage(rng.standard_normal(shape, dtype=np.float32), code)
    tx, tdy, tg = from_np(x, dtype), from_np(dy, dtype), torch.from_numpy(gamma).cuda()
    pick = np.unique(np.concatenate([[0, rows - 1], np.random.default_rng(13).integers(0, rows, 257)]))
    tp = torch.from_numpy(pick).cuda()
    xs, dys = np.ascontiguousarray(x[pick]), np.ascontiguousarray(dy[pick])

    def sample(t):
        return as_f32(to_np(t[tp]), dtype)

    for log in (False, True):
        y = kernels.log_softmax(tx) if log else kernels.softmax(tx)
        want_y = port.softmax(xs, code, log=log)
        np.testing.assert_allclose(sample(y), as_f32(want_y, dtype), rtol=tol,
                                   atol=(tol * 10) if log else (tol * 1e-2 if dtype == torch.float32 else tol * 0.05))
        fn = kernels.log_softmax_backward if log else kernels.softmax_backward
        dx = fn(tdy, y)
        # the oracle's backward takes the kernel's own forward rows as the saved tensor
        want_dx = port.softmax_backward(dys, to_np(y[tp]), code, log=log)
        np.testing.assert_allclose(sample(dx), as_f32(want_dx, dtype), rtol=tol,
                                   atol=tol if dtype == torch.float32 else tol * 0.1)
        del y, dx
    y, inv = kernels.rmsnorm(tx, tg, 1e-6)
    want_y, want_inv = port.rmsnorm(xs, gamma, 1e-6, code)
    np.testing.assert_allclose(sample(y), as_f32(want_y, dtype), rtol=tol, atol=tol * 0.1)
    np.testing.assert_allclose(inv[tp].cpu().numpy(), want_inv, rtol=1e-5)
    del y
    dx, dg = kernels.rmsnorm_backward(tdy, tx, inv, tg)
    inv_all = inv.cpu().numpy()
    want_dx, want_dg = port.rmsnorm_backward(dy, x, inv_all, gamma, code)  # all rows: dgamma sums over them
    np.testing.assert_allclose(sample(dx), as_f32(np.ascontiguousarray(want_dx[pick]), dtype), rtol=tol, atol=tol * 0.1)
    # dgamma[c] sums `rows` terms of size O(1): the bound scales with sqrt(rows), like any sum
    scale = np.sqrt(rows)
    err = np.abs(dg.cpu().numpy().astype(np.float64) - want_dg) / scale
    note_worst(f"C4 rmsnorm dgamma {str(dtype)[6:]} {list(shape)} (of sqrt(rows))", float(err.max()), 1e-4)
    assert err.max() <= 1e-4


# ------------------------------------------------------------------------------------------
# C5 (one GPU)
# ------------------------------------------------------------------------------------------
def test_c5_sum_and_amax_of_2p32_fp32_against_truth_and_the_reference_sum(ops, port):
    n = 1 << 32
    g = torch.Generator(device="cuda").manual_seed(4000)
    x = torch.empty(n, device="cuda", dtype=torch.float32)
    step = 1 << 28
    for o in range(0, n, step):
        x[o:o + step].normal_(generator=g)
    s = ops.sum(x).item()
    truth, sq = 0.0, 0.0
    for o in range(0, n, step):
        d = x[o:o + step].double()
        truth += d.sum().item()
        sq += d.pow(2).sum().item()
    scale = max(abs(truth), sq ** 0.5)  # max(|truth|, sigma * sqrt(N))
    note_worst("C5 sum fp32 [2^32] vs fp64 truth", abs(s - truth) / scale, 1e-5)
    assert abs(s - truth) <= 1e-5 * scale
    m = ops.amax(x).item()
    assert m == max(x[o:o + step].max().item() for o in range(0, n, step))
    # the reference's own sum on a 2^28 slice: a sequential fp32 accumulation, which drifts from
    # the truth far more than the kernel's fixed-order tree; both deltas are recorded
    sl = x[:step]
    host = sl.cpu().numpy()
    ours = ops.sum(sl).item()
    t28 = sl.double().sum().item()
    sc28 = max(abs(t28), float(sl.double().pow(2).sum().sqrt().item()))
    seq = float(oracle.ref().sum(host, oracle.F32, [])) if oracle.have_ref() else float(port.reduce("sum", host, oracle.F32))
    note_worst("C5 sum fp32 2^28 slice: kernel vs fp64 truth", abs(ours - t28) / sc28, 1e-5)
    note_worst("C5 sum fp32 2^28 slice: reference's sequential fp32 sum vs fp64 truth (reported, not asserted)",
               abs(seq - t28) / sc28, float("inf"))
    assert abs(ours - t28) <= 1e-5 * sc28
    # the kernel is at least as close to the truth as the reference's own loop
    assert abs(ours - t28) <= abs(seq - t28) + 1e-5 * sc28
    assert ops.amax(sl).item() == float(port.reduce("max", host, oracle.F32))


def test_c5_bf16_mean_dim0_of_1m_by_4096_against_truth(ops):
    rows, cols = 1 << 20, 4096
    g = torch.Generator(device="cuda").manual_seed(4001)
    x = torch.empty((rows, cols), device="cuda", dtype=torch.bfloat16)
    for o in range(0, rows, 1 << 14):
        x[o:o + (1 << 14)].normal_(generator=g)
    got = ops.mean(x, 0)
    assert got.dtype == torch.bfloat16 and got.shape == (cols,)
    truth = torch.zeros(cols, device="cuda", dtype=torch.float64)
    sq = torch.zeros(cols, device="cuda", dtype=torch.float64)
    for o in range(0, rows, 1 << 16):
        d = x[o:o + (1 << 16)].double()
        truth += d.sum(0)
        sq += d.pow(2).sum(0)
    scale = torch.maximum(truth.abs(), sq.sqrt()) / rows
    err = (got.double() - truth / rows).abs() / scale
    note_worst("C5 mean(dim=0) bf16 [1048576,4096] vs fp64 truth", float(err.max().item()), 1e-2)
    assert err.max().item() <= 1e-2
    # the fp32 partial (what a rank hands to the all-reduce) at the fp32 bound
    part = ops.reduce("sum", x, 0, False, partial=True)
    assert part.dtype == torch.float32
    perr = (part.double() - truth).abs() / torch.maximum(truth.abs(), sq.sqrt())
    note_worst("C5 column sums fp32 partial of bf16 [1048576,4096] vs fp64 truth", float(perr.max().item()), 1e-5)
    assert perr.max().item() <= 1e-5
