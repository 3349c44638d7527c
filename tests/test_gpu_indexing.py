"""Row gather / scatter(-add) / last-dim index vs the CPU oracle through the C ABI.
Gather, overwrite-scatter with distinct rows and int64 / int32 scatter-add are bit-exact;
fp32 scatter-add is compared with 1e-5 * (sum of |updates| per destination element) because
atomics do not fix the order of additions (neither does the reference's CUDA path)."""
import os

import numpy as np
import pytest
import torch

import oracle
from tests.util import CODE, from_np, to_np

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


@pytest.fixture(scope="module")
def ops():
    from vibetensor_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def kernels():
    from vibetensor_b200 import kernels as k
    return k


def zipf_indices(rng, V, N, s=1.1):
    """Bounded Zipf(s) over ranks 1..V, ranks scattered over rows by a permutation."""
    p = np.arange(1, V + 1, dtype=np.float64) ** -s
    ranks = np.searchsorted(np.cumsum(p / p.sum()), rng.random(N))
    return rng.permutation(V)[np.minimum(ranks, V - 1)].astype(np.int64)


def test_known_answers_from_reference_tests(ops):
    # tests/cpp/indexing_advanced_cpu_kernel_test.cc:57-96, :149-226
    base = torch.tensor([[10.], [11.], [12.], [13.], [14.]], device="cuda")
    out = ops.index_rows(base, torch.tensor([0, 4, 2], device="cuda"))
    assert out.flatten().tolist() == [10.0, 14.0, 12.0]
    b = torch.zeros((4, 1), device="cuda")
    ops.index_put_rows_(b, torch.tensor([1, 3], device="cuda"), torch.tensor([[5.], [7.]], device="cuda"))
    assert b.flatten().tolist() == [0.0, 5.0, 0.0, 7.0]
    ops.index_put_rows_(b, torch.tensor([1, 1], device="cuda"), torch.tensor([[1.], [2.]], device="cuda"),
                        accumulate=True)
    assert b[1, 0].item() == 8.0
    # tests/py/test_tensor_index_put_accumulate_cub_env.py:47-80
    idx = torch.tensor([0, 1, 0, 4], device="cuda")
    x = torch.zeros((5, 1), device="cuda")
    ops.index_put_rows_(x, idx, torch.tensor([[1.], [2.], [3.], [4.]], device="cuda"), accumulate=True)
    assert x.flatten().tolist() == [4.0, 2.0, 0.0, 0.0, 4.0]
    xi = torch.zeros((5, 1), dtype=torch.int64, device="cuda")
    ops.index_put_rows_(xi, idx, torch.tensor([[1], [2], [3], [4]], device="cuda"), accumulate=True)
    assert xi.flatten().tolist() == [4, 2, 0, 0, 4]


def test_golden_reference_vectors(ops):
    table, idx = torch.from_numpy(GOLD["ix_table"]).cuda(), torch.from_numpy(GOLD["ix_idx"]).cuda()
    np.testing.assert_array_equal(ops.index_rows(table, idx).cpu().numpy(), GOLD["ix_gather"])
    np.testing.assert_array_equal(ops.embedding(table, idx % 50).cpu().numpy(), GOLD["ix_embedding"])
    acc = torch.zeros((50, 12), device="cuda")
    ops.index_put_rows_(acc, idx, torch.from_numpy(GOLD["ix_vals"]).cuda(), accumulate=True)
    np.testing.assert_allclose(acc.cpu().numpy(), GOLD["ix_put_acc"], rtol=1e-5, atol=1e-5)
    acci = torch.zeros((50, 12), dtype=torch.int64, device="cuda")
    ops.index_put_rows_(acci, idx, torch.from_numpy(GOLD["ix_vals_i64"]).cuda(), accumulate=True)
    np.testing.assert_array_equal(acci.cpu().numpy(), GOLD["ix_put_acc_i64"])
    t2 = table.clone()
    ops.index_put_rows_(t2, torch.from_numpy(GOLD["ix_perm"]).cuda(),
                        torch.from_numpy(GOLD["ix_vals"][:30].copy()).cuda())
    np.testing.assert_array_equal(t2.cpu().numpy(), GOLD["ix_put_overwrite"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.int32, torch.bool])
@pytest.mark.parametrize("V,D,N", [(1000, 256, 5000), (333, 7, 1000), (64, 4, 300), (50, 1024, 200),
                                   (10, 2048 + 4, 100), (5, 1, 0)])
def test_gather_rows_bit_exact(ops, port, dtype, V, D, N):
    rng = np.random.default_rng(31)
    if dtype in (torch.float32,):
        table = rng.standard_normal((V, D), dtype=np.float32)
    elif dtype == torch.bfloat16:
        table = rng.integers(0, 2 ** 16, (V, D)).astype(np.uint16)
    elif dtype == torch.bool:
        table = rng.integers(0, 2, (V, D)).astype(np.uint8)
    else:
        table = rng.integers(-10 ** 6, 10 ** 6, (V, D)).astype(np.int64 if dtype == torch.int64 else np.int32)
    idx = rng.integers(-V, V, N).astype(np.int64)
    got = to_np(ops.index_rows(from_np(table, dtype), torch.from_numpy(idx).cuda()))
    np.testing.assert_array_equal(got.view(table.dtype), port.gather_rows(table, idx))


def test_gather_strided_table_and_int32_index(ops, port):
    rng = np.random.default_rng(32)
    big = rng.standard_normal((200, 96), dtype=np.float32)
    tb = torch.from_numpy(big).cuda()
    idx = rng.integers(0, 200, 777)
    for view_np, view_t in ((big[:, 8:72], tb[:, 8:72]), (big[::2], tb[::2]), (big.T[:50], tb.t()[:50])):
        i = idx % view_np.shape[0]
        got = ops.index_rows(view_t, torch.from_numpy(i.astype(np.int32)).cuda()).cpu().numpy()
        np.testing.assert_array_equal(got, port.gather_rows(view_np, i))
    # 2-D index
    i2 = (idx[:60] % 200).reshape(6, 10)
    got = ops.index_rows(tb, torch.from_numpy(i2).cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, port.gather_rows(big, i2))


@pytest.mark.parametrize("V,D,N", [(1000, 256, 20000), (97, 64, 5000), (40, 8, 3000), (16, 516, 999),
                                   (300, 3, 2000)])
def test_scatter_add_zipf(ops, port, V, D, N):
    rng = np.random.default_rng(33)
    idx = zipf_indices(rng, V, N)
    ti = torch.from_numpy(idx).cuda()
    # int64: exact whatever the order
    vi = rng.integers(-1000, 1001, (N, D)).astype(np.int64)
    acc = torch.zeros((V, D), dtype=torch.int64, device="cuda")
    ops.index_put_rows_(acc, ti, torch.from_numpy(vi).cuda(), accumulate=True)
    np.testing.assert_array_equal(acc.cpu().numpy(), port.scatter_rows(np.zeros((V, D), np.int64), idx, vi, oracle.I64))
    v32 = vi.astype(np.int32)
    acc32 = torch.zeros((V, D), dtype=torch.int32, device="cuda")
    ops.index_put_rows_(acc32, ti, torch.from_numpy(v32).cuda(), accumulate=True)
    np.testing.assert_array_equal(acc32.cpu().numpy(), port.scatter_rows(np.zeros((V, D), np.int32), idx, v32, oracle.I32))
    # fp32: tolerance relative to the mass added into each element
    vf = rng.standard_normal((N, D), dtype=np.float32)
    init = rng.standard_normal((V, D), dtype=np.float32)
    accf = torch.from_numpy(init.copy()).cuda()
    ops.index_put_rows_(accf, ti, torch.from_numpy(vf).cuda(), accumulate=True)
    want = port.scatter_rows(init.copy(), idx, vf, oracle.F32)
    mass = port.scatter_rows(np.abs(init), idx, np.abs(vf), oracle.F32)
    err = np.abs(accf.cpu().numpy().astype(np.float64) - want)
    assert (err <= 1e-5 * mass + 1e-30).all(), err.max()


def test_scatter_overwrite_unique_rows_and_negative(ops, port):
    rng = np.random.default_rng(34)
    V, D = 500, 64
    table = rng.standard_normal((V, D), dtype=np.float32)
    idx = rng.permutation(V)[:300].astype(np.int64)
    idx[::3] -= V
    vals = rng.standard_normal((300, D), dtype=np.float32)
    t = torch.from_numpy(table.copy()).cuda()
    ops.index_put_rows_(t, torch.from_numpy(idx).cuda(), torch.from_numpy(vals).cuda())
    np.testing.assert_array_equal(t.cpu().numpy(), port.scatter_rows(table.copy(), idx, vals, oracle.F32, accumulate=False))


def test_out_of_range_is_reported_not_faulted(ops):
    table = torch.arange(12, dtype=torch.float32, device="cuda").reshape(4, 3)
    for bad in ([1, 4], [-5, 0]):
        with pytest.raises(IndexError, match="out of range"):
            ops.index_rows(table, torch.tensor(bad, device="cuda"))
    with pytest.raises(IndexError, match="vt::embedding"):
        ops.embedding(table, torch.tensor([-1], device="cuda"))
    # lazy mode: the good rows are produced, the bad one is zero, the status says so
    st = ops.IndexStatus("cuda")
    out = ops.index_rows(table, torch.tensor([3, 9, 0], device="cuda"), status=st)
    assert out.tolist() == [[9., 10., 11.], [0., 0., 0.], [0., 1., 2.]]
    with pytest.raises(IndexError):
        st.check("index", 4)
    st.check("index", 4)  # cleared after reporting
    t2 = torch.zeros((4, 3), device="cuda")
    with pytest.raises(IndexError):
        ops.index_put_rows_(t2, torch.tensor([0, 7], device="cuda"), torch.ones((2, 3), device="cuda"), accumulate=True)
    assert t2.tolist()[0] == [1., 1., 1.] and t2.sum().item() == 3.0
    with pytest.raises(ValueError, match="Int32 and Int64"):
        ops.index_rows(table, torch.tensor([0.0], device="cuda"))


def test_embedding_backward_duplicates_and_padding(ops):
    # tests/py/test_embedding_backward_cuda.py:31-60 of the reference
    idx = torch.tensor([0, 2, 2, 2, 1], device="cuda")
    g = torch.arange(15, dtype=torch.float32, device="cuda").reshape(5, 3)
    gw = ops.embedding_backward(g, idx, 5, padding_idx=1).cpu().numpy()
    gn = g.cpu().numpy()
    exp = np.zeros((5, 3), np.float32)
    exp[0] += gn[0]
    exp[2] += gn[1] + gn[2] + gn[3]
    np.testing.assert_allclose(gw, exp, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("D", [3, 64, 256, 1000])
def test_embedding_backward_scale_grad_by_freq(ops, port, D):
    rng = np.random.default_rng(36)
    V, N = 300, 5000
    ranks = np.minimum((rng.pareto(1.1, N) * 3).astype(np.int64), V - 1)     # heavy duplicates
    idx = rng.permutation(V)[ranks].astype(np.int64)
    g = rng.standard_normal((N, D)).astype(np.float32)
    pad = int(idx[0])
    got = ops.embedding_backward(torch.from_numpy(g).cuda(), torch.from_numpy(idx).cuda(), V, padding_idx=pad,
                                 scale_grad_by_freq=True).cpu().numpy()
    want = port.embedding_backward_by_freq(g, idx, V, padding_idx=pad)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
    assert not got[pad].any()
    with pytest.raises(IndexError):
        ops.embedding_backward(torch.from_numpy(g).cuda(), torch.from_numpy(idx + V).cuda(), V,
                               scale_grad_by_freq=True)


def test_lastdim_index_and_put(ops, port):
    rng = np.random.default_rng(35)
    src = rng.standard_normal((37, 50), dtype=np.float32)
    idx = rng.integers(-50, 50, 123).astype(np.int64)
    ts = torch.from_numpy(src).cuda()
    np.testing.assert_array_equal(ops.index_lastdim(ts, torch.from_numpy(idx).cuda()).cpu().numpy(),
                                  port.index_lastdim(src, idx))
    np.testing.assert_array_equal(ops.index_lastdim(ts.t(), torch.from_numpy(idx[:20] % 37).cuda()).cpu().numpy(),
                                  port.index_lastdim(src.T, idx[:20] % 37))
    vals = rng.integers(-9, 10, (37, 123)).astype(np.int64)
    self_ = np.zeros((37, 50), np.int64)
    t = torch.from_numpy(self_.copy()).cuda()
    ops.index_put_lastdim_(t, torch.from_numpy(idx).cuda(), torch.from_numpy(vals).cuda(), accumulate=True)
    np.testing.assert_array_equal(t.cpu().numpy(), port.index_put_lastdim(self_.copy(), idx, vals, oracle.I64, True))


def test_vibe_kernels_gather_scatter_add_surface(kernels, port):
    # vibe_kernels/indexing/tests/test_vbt_native.py:45-66 of the reference
    src = np.arange(32, dtype=np.float32).reshape(4, 8)
    idx = np.array([1, 3, 0], np.int64)
    out = kernels.gather(torch.from_numpy(src).cuda(), 0, torch.from_numpy(idx).cuda())
    np.testing.assert_array_equal(out.cpu().numpy(), src[idx])
    dst = torch.zeros((4, 8), device="cuda")
    kernels.scatter_add(dst, 0, torch.tensor([1, 1, 9], device="cuda"), torch.ones((3, 8), device="cuda"))
    assert dst[1].tolist() == [2.0] * 8 and dst[3].tolist() == [1.0] * 8  # 9 is clamped to row 3
    with pytest.raises(NotImplementedError):
        kernels.gather(torch.from_numpy(src).cuda(), 1, torch.from_numpy(idx).cuda())
    with pytest.raises(TypeError):
        kernels.gather(torch.from_numpy(src).cuda(), 0, torch.from_numpy(idx.astype(np.int32)).cuda())


def test_config2_scale_roundtrip_properties(ops):
    """Full table shape of the benchmark configuration ([1,048,576 x 256] fp32), reduced
    index count: gather(idx) of a table whose row r is filled with r returns idx; scatter-add
    of ones counts occurrences exactly (small integers are exact in fp32)."""
    V, D, N = 1 << 20, 256, 1 << 18
    rng = np.random.default_rng(2)
    idx = zipf_indices(rng, V, N)
    ti = torch.from_numpy(idx).cuda()
    table = torch.arange(V, dtype=torch.float32, device="cuda").reshape(V, 1).expand(V, D).contiguous()
    out = ops.index_rows(table, ti)
    assert torch.equal(out[:, 0].long(), ti) and torch.equal(out[:, -1].long(), ti)
    acc = torch.zeros((V, D), device="cuda")
    ops.index_put_rows_(acc, ti, torch.ones((N, D), device="cuda"), accumulate=True)
    counts = torch.bincount(ti, minlength=V).float()
    assert torch.equal(acc[:, 0], counts) and torch.equal(acc[:, 255], counts)
    acci = torch.zeros((V, D), dtype=torch.int64, device="cuda")
    ops.index_put_rows_(acci, ti, torch.full((N, D), 3, dtype=torch.int64, device="cuda"), accumulate=True)
    assert torch.equal(acci[:, 17], 3 * counts.long())


@pytest.mark.parametrize("V,D,N", [(1000, 256, 20000), (97, 64, 5000), (5000, 8, 4097), (16, 516, 999),
                                   (300, 4, 31), (70000, 4, 300000), (3, 4, 1)])
def test_sorted_scatter_add(ops, port, V, D, N):
    """The sort-based accumulate engine: exact for integers, within tolerance for fp32, and
    exact for fp32 too when no row is updated twice."""
    rng = np.random.default_rng(36)
    idx = zipf_indices(rng, V, N)
    idx[::7] -= V                                   # negative indices wrap
    ti = torch.from_numpy(idx).cuda()
    vi = rng.integers(-1000, 1001, (N, D)).astype(np.int64)
    init = rng.integers(-5, 6, (V, D)).astype(np.int64)
    acc = torch.from_numpy(init.copy()).cuda()
    ops.index_put_rows_(acc, ti, torch.from_numpy(vi).cuda(), accumulate=True, deterministic=True)
    np.testing.assert_array_equal(acc.cpu().numpy(), port.scatter_rows(init.copy(), idx, vi, oracle.I64))
    v32 = vi.astype(np.int32)
    acc32 = torch.zeros((V, D), dtype=torch.int32, device="cuda")
    ops.index_put_rows_(acc32, ti, torch.from_numpy(v32).cuda(), accumulate=True, deterministic=True)
    np.testing.assert_array_equal(acc32.cpu().numpy(),
                                  port.scatter_rows(np.zeros((V, D), np.int32), idx, v32, oracle.I32))
    vf = rng.standard_normal((N, D), dtype=np.float32)
    initf = rng.standard_normal((V, D), dtype=np.float32)
    accf = torch.from_numpy(initf.copy()).cuda()
    ops.index_put_rows_(accf, ti, torch.from_numpy(vf).cuda(), accumulate=True, deterministic=True)
    want = port.scatter_rows(initf.copy(), idx, vf, oracle.F32)
    mass = port.scatter_rows(np.abs(initf), idx, np.abs(vf), oracle.F32)
    err = np.abs(accf.cpu().numpy().astype(np.float64) - want)
    assert (err <= 1e-5 * mass + 1e-30).all(), err.max()


@pytest.mark.parametrize("V", [4000, 200000])   # a full sort by row / rows grouped by a 16-bit hash (4-byte tables, > 65536 rows)
def test_sorted_scatter_add_unique_rows_is_bit_exact_and_flags_bad_indices(ops, port, V):
    rng = np.random.default_rng(37)
    D, N = 64, 3000
    idx = rng.permutation(V)[:N].astype(np.int64)
    vf = rng.standard_normal((N, D), dtype=np.float32)
    init = rng.standard_normal((V, D), dtype=np.float32)
    acc = torch.from_numpy(init.copy()).cuda()
    ops.index_put_rows_(acc, torch.from_numpy(idx).cuda(), torch.from_numpy(vf).cuda(), accumulate=True,
                        deterministic=True)
    np.testing.assert_array_equal(acc.cpu().numpy(), port.scatter_rows(init.copy(), idx, vf, oracle.F32))
    # zero-initialised destination, duplicates: every row summed from one slice is the
    # sequential sum; compare all rows with few updates bit for bit
    idx2 = rng.integers(0, V, 6000).astype(np.int64)
    v2 = rng.standard_normal((6000, D), dtype=np.float32)
    a2 = torch.zeros((V, D), device="cuda")
    ops.index_put_rows_(a2, torch.from_numpy(idx2).cuda(), torch.from_numpy(v2).cuda(), accumulate=True,
                        deterministic=True)
    want = port.scatter_rows(np.zeros((V, D), np.float32), idx2, v2, oracle.F32)
    got = a2.cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    assert (got == want).all(axis=1).mean() > 0.9
    # out-of-range updates are dropped and reported
    bad = idx.copy()
    bad[5] = V + 3
    acc3 = torch.zeros((V, D), device="cuda")
    with pytest.raises(IndexError):
        ops.index_put_rows_(acc3, torch.from_numpy(bad).cuda(), torch.from_numpy(vf).cuda(), accumulate=True,
                            deterministic=True)
    keep = np.ones(N, bool)
    keep[5] = False
    np.testing.assert_array_equal(
        acc3.cpu().numpy(), port.scatter_rows(np.zeros((V, D), np.float32), idx[keep], vf[keep], oracle.F32))


@pytest.mark.parametrize("n", [1, 15, 16, 4095, 4096, 4097, 100003, 5_000_000])
@pytest.mark.parametrize("density", [0.0, 0.01, 0.5, 1.0])
def test_mask_to_indices(ops, n, density):
    rng = np.random.default_rng(37)
    m = rng.random(n) < density
    got = ops.mask_to_indices(torch.from_numpy(m).cuda())
    np.testing.assert_array_equal(got.cpu().numpy(), np.flatnonzero(m))


def test_mask_strided_unaligned_and_truthy_bytes(ops):
    rng = np.random.default_rng(38)
    raw = rng.integers(0, 3, 30001).astype(np.uint8)          # bytes 0 / 1 / 2: any non-zero is true
    t = torch.from_numpy(raw).cuda()
    for view, ref in ((t[1:], raw[1:]), (t[::3], raw[::3]), (t[5::7], raw[5::7])):
        got = ops.mask_to_indices(view.view(torch.bool))
        np.testing.assert_array_equal(got.cpu().numpy(), np.flatnonzero(ref))
    # dense and aligned (the 16-byte path, whole tiles fetched ahead, and a ragged last tile): every byte value
    full = rng.integers(0, 256, 16384 * 5 + 77).astype(np.uint8)
    full[rng.random(full.size) < 0.5] = 0
    got = ops.mask_to_indices(torch.from_numpy(full).cuda().view(torch.bool))
    np.testing.assert_array_equal(got.cpu().numpy(), np.flatnonzero(full))
    assert ops.mask_to_indices(torch.zeros((0,), dtype=torch.bool, device="cuda")).numel() == 0
    with pytest.raises(ValueError, match="boolean mask"):
        ops.mask_to_indices(torch.ones((2, 2), dtype=torch.bool, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.int64])
def test_bool_mask_indexing(ops, port, dtype):
    rng = np.random.default_rng(39)
    src = rng.integers(-99, 100, (37, 501)).astype(np.float32 if dtype == torch.float32 else np.int64)
    m = rng.random(501) < 0.3
    ts = torch.from_numpy(src).cuda()
    got = ops.index_mask_lastdim(ts, torch.from_numpy(m).cuda())
    np.testing.assert_array_equal(got.cpu().numpy(), port.index_lastdim(src, np.flatnonzero(m)))
    mr = rng.random(37) < 0.5
    got = ops.index_mask_rows(ts, torch.from_numpy(mr).cuda())
    np.testing.assert_array_equal(got.cpu().numpy(), port.gather_rows(src, np.flatnonzero(mr)))
    with pytest.raises(ValueError, match="boolean mask"):
        ops.index_mask_lastdim(ts.bfloat16() if dtype == torch.float32 else ts.int(), torch.from_numpy(m).cuda())
    with pytest.raises(ValueError, match="boolean mask"):
        ops.index_mask_lastdim(ts, torch.from_numpy(m[:100]).cuda())


@pytest.mark.parametrize("dtype,shape,K", [(torch.float32, (5, 70001), 10000), (torch.int64, (3, 30000), 9000),
                                           (torch.bfloat16, (4, 50001), 20000), (torch.float32, (2, 8192), 8192),
                                           (torch.float32, (7, 25001), 9001), (torch.int64, (3, 12800), 8200)])
def test_index_lastdim_long_rows_few_of_them(ops, port, dtype, shape, K):
    """Long rows, many indices, only a handful of rows (the direct kernel): rows whose base is not
    16-byte aligned, negative (wrapped) indices, a strided source view."""
    rng = np.random.default_rng(40)
    if dtype == torch.int64:
        src = rng.integers(-10 ** 12, 10 ** 12, shape).astype(np.int64)
    else:
        src = oracle.to_storage(rng.standard_normal(shape, dtype=np.float32), CODE[dtype])
    idx = rng.integers(-shape[1], shape[1], K).astype(np.int64)
    ts, ti = from_np(src, dtype), torch.from_numpy(idx).cuda()
    got = to_np(ops.index_lastdim(ts, ti))
    np.testing.assert_array_equal(got, port.index_lastdim(src, idx))
    # the same through a view with a column stride of 2
    wide = np.zeros((shape[0], 2 * shape[1]), src.dtype)
    wide[:, ::2] = src
    tv = from_np(wide, dtype)[:, ::2]
    np.testing.assert_array_equal(to_np(ops.index_lastdim(tv, ti)), got)
    # out-of-range positions come back as zeros and are counted once each
    bad = idx.copy()
    bad[::1000] = shape[1] + 5
    st = ops.IndexStatus(ts.device)
    got_bad = to_np(ops.index_lastdim(ts, torch.from_numpy(bad).cuda(), status=st, eager_check=False))
    assert not got_bad[:, ::1000].any()
    keep = np.ones(K, bool)
    keep[::1000] = False
    np.testing.assert_array_equal(got_bad[:, keep], got[:, keep])
    with pytest.raises(IndexError, match=f"{len(bad[::1000])} bad indices"):
        st.check("index", shape[1])


def _lastdim_oracle(port, src_view_np, idx):
    """x[..., idx] for an N-d view through the 2-D oracle entry (rows = the flattened leading dims)."""
    k0 = src_view_np.shape[-1]
    flat = np.ascontiguousarray(src_view_np).reshape(-1, k0)
    return port.index_lastdim(flat, idx.reshape(-1)).reshape(src_view_np.shape[:-1] + idx.shape)


# (dtype, shape, index count, kernel id: 7 = output tile in shared memory, 9 = outputs in registers)
STAGED = [(torch.float32, (40, 60001), 32768, 7),    # 4 pieces, rows not 16-byte aligned: plain staging loads, 2 index chunks
          (torch.float32, (33, 65536), 65536, 9),    # 4 pieces of 64 KiB, two index chunks side by side
          (torch.bfloat16, (64, 50000), 40000, 7),   # one piece, two index chunks
          (torch.int64, (32, 12800), 8000, 7),       # one piece of exactly 100 KiB
          (torch.float32, (35, 16384), 16384, 7),
          (torch.float32, (34, 16384), 16380, 7),    # output rows not 16-byte aligned: scalar tile write-out
          (torch.bool, (32, 40000), 8192, 7),
          (torch.bfloat16, (32, 200000), 100000, 7),  # 400 KB rows: six pieces, four index chunks
          (torch.float32, (32, 100001), 65536, 7),    # nine pieces, rows not 16-byte aligned (plain staging loads)
          (torch.float32, (33, 40000), 50000, 9),     # three pieces; the second chunk's tile is partly empty
          (torch.float32, (32, 65536), 32770, 9),     # output rows not 16-byte aligned: scalar stores; a 2-entry tile
          (torch.int32, (64, 30000), 30000, 9),       # two pieces, one chunk
          (torch.float32, (64, 16000), 32768, 9),     # one piece
          (torch.float32, (150, 65532), 65536, 9)]    # more rows than row lanes; last piece shorter


@pytest.mark.parametrize("dtype,shape,K,kernel", STAGED)
def test_index_lastdim_staged_rows(ops, port, dtype, shape, K, kernel):
    """Shapes that take the staged kernels (rows brought into shared memory by bulk copies, the
    index list held in registers, outputs collected in a shared-memory tile or -- long 4-byte
    rows -- in registers): every element size, one and several pieces per row, one and several
    index chunks, aligned and unaligned rows and outputs, wrapped negative indices, bad indices."""
    from vibetensor_b200 import _lib
    rng = np.random.default_rng(44)
    if dtype == torch.int64:
        src = rng.integers(-10 ** 12, 10 ** 12, shape).astype(np.int64)
    elif dtype == torch.int32:
        src = rng.integers(-2 ** 31, 2 ** 31, shape).astype(np.int32)
    elif dtype == torch.bool:
        src = (rng.random(shape) < 0.5).astype(np.uint8)
    else:
        src = oracle.to_storage(rng.standard_normal(shape, dtype=np.float32), CODE[dtype])
    idx = rng.integers(-shape[1], shape[1], K).astype(np.int64)
    ts, ti = from_np(src, dtype), torch.from_numpy(idx).cuda()
    got = to_np(ops.index_lastdim(ts, ti))
    info = _lib.last_launch_info()
    assert (info.family, info.kernel) == (3, kernel), "expected the staged last-dim kernel"
    np.testing.assert_array_equal(got, port.index_lastdim(src, idx))
    bad = idx.copy()
    bad[::997] = shape[1] + 3
    st = ops.IndexStatus(ts.device)
    got_bad = to_np(ops.index_lastdim(ts, torch.from_numpy(bad).cuda(), status=st, eager_check=False))
    assert not got_bad[:, ::997].any()
    keep = np.ones(K, bool)
    keep[::997] = False
    np.testing.assert_array_equal(got_bad[:, keep], got[:, keep])
    with pytest.raises(IndexError, match=f"{len(bad[::997])} bad indices"):
        st.check("index", shape[1])
    st.check("index", shape[1])  # the block is clear again and no staged copy timed out


def test_index_lastdim_nd_strided_self(ops, port):
    """The index applies to the last dim of an N-d strided base
    (src/vbt/core/indexing_advanced_cuda.cu:2156-2177): leading dims that do not collapse onto
    one stride, a multi-dim index tensor, both kernels, and index_put_ on the same views."""
    from vibetensor_b200 import _lib
    rng = np.random.default_rng(45)
    base = rng.standard_normal((8, 10, 40000), dtype=np.float32)
    tb = torch.from_numpy(base).cuda()
    idx = rng.integers(-32768, 32768, (4, 5000)).astype(np.int64)
    ti = torch.from_numpy(idx).cuda()
    for sl, kernel in (((slice(None), slice(None, None, 2), slice(0, 32768)), 9),      # aligned rows: bulk copies
                       ((slice(None), slice(None, None, 2), slice(1, 32769)), 7)):     # rows start 4 bytes off
        got = ops.index_lastdim(tb[sl], ti)
        assert (_lib.last_launch_info().family, _lib.last_launch_info().kernel) == (3, kernel)
        assert got.shape == (8, 5, 4, 5000)
        np.testing.assert_array_equal(got.cpu().numpy(), _lastdim_oracle(port, base[sl], idx))
    # small N-d shapes on the direct kernel: permuted leading dims, rank 1, rank 4
    small = rng.standard_normal((3, 4, 5, 50), dtype=np.float32)
    tsm = torch.from_numpy(small).cuda()
    i2 = rng.integers(-50, 50, (7, 3)).astype(np.int64)
    ti2 = torch.from_numpy(i2).cuda()
    for view_np, view_t in ((small, tsm), (small.transpose(1, 0, 2, 3), tsm.permute(1, 0, 2, 3)),
                            (small[:, ::2, 1:4], tsm[:, ::2, 1:4]), (small[0, 0, 0], tsm[0, 0, 0]),
                            (small.transpose(0, 1, 3, 2)[..., :4], tsm.permute(0, 1, 3, 2)[..., :4])):
        k0 = view_np.shape[-1]
        ii = np.mod(i2, k0) - (k0 if k0 > 4 else 0) * (i2 < 0)
        got = ops.index_lastdim(view_t, torch.from_numpy(ii).cuda())
        assert _lib.last_launch_info().kernel == 6
        np.testing.assert_array_equal(got.cpu().numpy(), _lastdim_oracle(port, view_np, ii))
    # index_put_ through a permuted 3-D view, accumulate with duplicates (int64: exact)
    self_np = rng.integers(-5, 5, (4, 6, 30)).astype(np.int64)
    t = torch.from_numpy(self_np.copy()).cuda()
    view_t, view_np = t.permute(1, 0, 2), self_np.transpose(1, 0, 2)
    ip = rng.integers(-30, 30, 77).astype(np.int64)
    vals = rng.integers(-9, 10, (6, 4, 77)).astype(np.int64)
    ops.index_put_lastdim_(view_t, torch.from_numpy(ip).cuda(), torch.from_numpy(vals).cuda(), accumulate=True)
    want = np.ascontiguousarray(view_np).reshape(24, 30)
    port.index_put_lastdim(want, ip, vals.reshape(24, 77), oracle.I64, True)
    np.testing.assert_array_equal(view_t.cpu().numpy(), want.reshape(6, 4, 30))
    with pytest.raises(ValueError, match="0-d"):
        ops.index_lastdim(torch.zeros((), device="cuda"), ti2)
