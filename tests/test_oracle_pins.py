"""Pins the CPU oracle (oracle/vbt_oracle.c) before anything is checked against it:

1. known-answer vectors carried by the reference's own unit tests (values only);
2. tests/golden/ref_vectors.npz -- outputs of the reference's compiled CPU code on seeded
   inputs (made by tests/golden/make_golden.py);
3. where oracle/_ref is present, live comparison with the reference's CPU code on fresh
   random inputs;
4. torch CPU for the paths that have no CPU code in the reference (softmax, RMSNorm, bf16),
   with the tolerances of the reference's own tests (vibe_kernels/rmsnorm/tests/
   test_rmsnorm.py:19-46: 1e-4 fp32, 1e-2 bf16).
"""
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import BF16, BOOL, F16, F32, I64

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


# ---- 1. known answers from the reference's unit tests -------------------------------------
def test_gather_1d_known_answer(port):
    # tests/cpp/indexing_advanced_cpu_kernel_test.cc:57-96
    base = (10 + np.arange(5)).astype(np.float32).reshape(5, 1)
    out = port.gather_rows(base, np.array([0, 4, 2]))
    assert out.ravel().tolist() == [10.0, 14.0, 12.0]


def test_scatter_overwrite_then_duplicate_accumulate_known_answer(port):
    # tests/cpp/indexing_advanced_cpu_kernel_test.cc:149-226
    base = np.zeros((4, 1), np.float32)
    port.scatter_rows(base, np.array([1, 3]), np.array([[5.0], [7.0]], np.float32), F32,
                      accumulate=False)
    assert base.ravel().tolist() == [0.0, 5.0, 0.0, 7.0]
    port.scatter_rows(base, np.array([1, 1]), np.array([[1.0], [2.0]], np.float32), F32,
                      accumulate=True)
    assert base[1, 0] == 8.0


def test_index_put_accumulate_fp32_and_int64_known_answer(port):
    # tests/py/test_tensor_index_put_accumulate_cub_env.py:47-80
    idx = np.array([0, 1, 0, 4])
    x = np.zeros((5, 1), np.float32)
    port.scatter_rows(x, idx, np.array([[1.0], [2.0], [3.0], [4.0]], np.float32), F32)
    assert x.ravel().tolist() == [4.0, 2.0, 0.0, 0.0, 4.0]
    xi = np.zeros((5, 1), np.int64)
    port.scatter_rows(xi, idx, np.array([[1], [2], [3], [4]], np.int64), I64)
    assert xi.ravel().tolist() == [4, 2, 0, 0, 4]


def test_row_sums_known_answer(port):
    # tests/cpp/tensor_iter_reduction_test.cc:207-253
    x = (np.arange(6) + 1).astype(np.float32).reshape(2, 3)
    assert port.reduce("sum", x, F32, dim=1).tolist() == [6.0, 15.0]
    xi = (np.arange(6) + 1).astype(np.int64).reshape(2, 3)
    assert port.reduce("sum", xi, I64, dim=1).tolist() == [6, 15]


@pytest.mark.parametrize("vals,kind,expected", [
    ([np.inf, np.inf], "min", np.inf), ([-np.inf, -np.inf], "max", -np.inf),
    ([1.0, np.inf], "min", 1.0), ([-np.inf, 2.0], "max", 2.0)])
def test_min_max_inf_identities(port, vals, kind, expected):
    # tests/py/test_cuda_reduction.py:122-150
    assert port.reduce(kind, np.array(vals, np.float32), F32) == expected


def test_broadcast_add_known_answer(port):
    # tests/cpp/cuda_elementwise_test.cc:343-394
    rows, cols = 2, 256
    a = (np.arange(rows)[:, None] * 1000 + np.arange(cols)[None, :]).astype(np.float32)
    b = (1.5 * np.arange(cols)).astype(np.float32)
    np.testing.assert_array_equal(port.binary("add", a, b, F32), a + b)


def test_offset_calculator_known_answer(port):
    # tests/cpp/tensor_iter_cuda_meta_test.cc:353-400: [2,256] with a [256] broadcast operand;
    # meta dims are innermost-first.
    rows, cols = 2, 256
    for li in range(rows * cols):
        r, c = divmod(li, cols)
        assert port.offset_elems(li, [cols, rows], [1, cols]) == r * cols + c
        assert port.offset_elems(li, [cols, rows], [1, 0]) == c


def test_embedding_backward_duplicates_and_padding_known_answer(port):
    # tests/py/test_embedding_backward_cuda.py:31-60
    idx = np.array([0, 2, 2, 2, 1])
    g = np.arange(15, dtype=np.float32).reshape(5, 3)
    gw = np.zeros((5, 3), np.float32)
    port.scatter_rows(gw, idx, g, F32, accumulate=True, policy=oracle.STRICT, padding_idx=1)
    exp = np.zeros((5, 3), np.float32)
    exp[0] += g[0]
    exp[2] += g[1] + g[2] + g[3]
    np.testing.assert_allclose(gw, exp, rtol=1e-6, atol=1e-6)


def test_empty_reduction_semantics(port):
    # src/vbt/ops/cuda_reduction.cu:1176-1216 / tensor_bindings.cc:476-494
    x = np.zeros((3, 0), np.float32)
    assert port.reduce("sum", x, F32, dim=1).tolist() == [0.0, 0.0, 0.0]
    assert np.isnan(port.reduce("mean", x, F32, dim=1)).all()
    assert port.reduce("prod", x, F32, dim=1).tolist() == [1.0, 1.0, 1.0]
    with pytest.raises(RuntimeError, match="amax: empty"):
        port.reduce("max", x, F32, dim=1)


def test_nan_rules_of_max_scan(port):
    # tensor_bindings.cc:361-379: NaN survives only at position 0
    assert np.isnan(port.reduce("max", np.array([np.nan, 1, 2], np.float32), F32))
    assert port.reduce("max", np.array([1, np.nan, 2], np.float32), F32) == 2.0
    v, i = port.reduce("argmax", np.array([[1, np.nan, 5, 5]], np.float32), F32, dim=1)
    assert v[0] == 5.0 and i[0] == 2


# ---- 2. committed outputs of the reference's compiled CPU code ----------------------------
def test_golden_reductions(port):
    x = GOLD["red_x"]
    np.testing.assert_array_equal(port.reduce("sum", x, F32, dim=-1), GOLD["red_sum_m1"])
    np.testing.assert_array_equal(port.reduce("sum", x, F32, dim=0), GOLD["red_sum_0"])
    np.testing.assert_array_equal(port.reduce("mean", x, F32, dim=0), GOLD["red_mean_0"])
    np.testing.assert_array_equal(port.reduce("sum", x, F32), GOLD["red_sum_all"])
    np.testing.assert_array_equal(port.reduce("max", x, F32, dim=-1), GOLD["red_amax_m1"])
    np.testing.assert_array_equal(port.reduce("min", x, F32, dim=0), GOLD["red_amin_0"])
    v, i = port.reduce("argmax", x, F32, dim=-1)
    np.testing.assert_array_equal(v, GOLD["red_argmax_m1_val"])
    np.testing.assert_array_equal(i, GOLD["red_argmax_m1_idx"])
    np.testing.assert_array_equal(port.reduce("sum", x.T, F32, dim=-1), GOLD["red_t_sum_m1"])
    np.testing.assert_array_equal(port.reduce("argmax", x.T, F32, dim=-1)[1],
                                  GOLD["red_t_argmax_m1_idx"])
    xt = GOLD["red_tie_x"]
    np.testing.assert_array_equal(port.reduce("argmax", xt, F32, dim=-1)[1],
                                  GOLD["red_tie_argmax_idx"])
    np.testing.assert_array_equal(port.reduce("argmax", xt, F32, dim=0)[1],
                                  GOLD["red_tie_argmax0_idx"])
    xi = GOLD["red_i64_x"]
    np.testing.assert_array_equal(port.reduce("sum", xi, I64, dim=-1), GOLD["red_i64_sum_m1"])
    np.testing.assert_array_equal(port.reduce("max", xi, I64, dim=0), GOLD["red_i64_amax_0"])
    np.testing.assert_array_equal(port.reduce("argmax", xi, I64, dim=-1)[1],
                                  GOLD["red_i64_argmax_m1_idx"])
    np.testing.assert_array_equal(port.reduce("sum", GOLD["red3_x"], F32, dim=1), GOLD["red3_sum_1"])


def test_golden_elementwise(port):
    a, b = GOLD["ew_a"], GOLD["ew_b"]
    for op in ["add", "sub", "mul", "div"]:
        np.testing.assert_array_equal(port.binary(op, a, b, F32), GOLD["ew_" + op])
    for op in ["eq", "ne", "lt", "gt", "le", "ge"]:
        np.testing.assert_array_equal(port.binary(op, a, b, F32), GOLD["ew_" + op])
    for op in ["relu", "abs", "neg", "reciprocal"]:
        np.testing.assert_array_equal(port.unary(op, a, F32), GOLD["ew_" + op])
    ai, bi = GOLD["ew_ai"], GOLD["ew_bi"]
    for op in ["add", "sub", "mul"]:
        np.testing.assert_array_equal(port.binary(op, ai, bi, I64), GOLD["ew_i64_" + op])


def test_golden_indexing(port):
    table, idx = GOLD["ix_table"], GOLD["ix_idx"]
    np.testing.assert_array_equal(port.gather_rows(table, idx), GOLD["ix_gather"])
    np.testing.assert_array_equal(port.gather_rows(table, idx % 50, oracle.STRICT),
                                  GOLD["ix_embedding"])
    got = port.scatter_rows(np.zeros((50, 12), np.float32), idx, GOLD["ix_vals"], F32)
    np.testing.assert_array_equal(got, GOLD["ix_put_acc"])
    got = port.scatter_rows(np.zeros((50, 12), np.int64), idx, GOLD["ix_vals_i64"], I64)
    np.testing.assert_array_equal(got, GOLD["ix_put_acc_i64"])
    got = port.scatter_rows(table.copy(), GOLD["ix_perm"], GOLD["ix_vals"][:30].copy(), F32,
                            accumulate=False)
    np.testing.assert_array_equal(got, GOLD["ix_put_overwrite"])


# ---- 3. live against the reference's CPU code ----------------------------------------------
@pytest.mark.parametrize("shape,dim", [((33, 257), -1), ((33, 257), 0), ((7, 5, 11), 1),
                                       ((1, 1000), 1), ((1000, 1), 0)])
def test_live_reductions_bit_exact(port, ref, shape, dim):
    rng = np.random.default_rng(abs(hash((shape, dim))) % 2 ** 31)
    x = rng.standard_normal(shape, dtype=np.float32)
    np.testing.assert_array_equal(port.reduce("sum", x, F32, dim=dim), ref.sum(x, F32, [dim]))
    np.testing.assert_array_equal(port.reduce("mean", x, F32, dim=dim),
                                  ref.sum(x, F32, [dim], mean=True))
    np.testing.assert_array_equal(port.reduce("max", x, F32, dim=dim), ref.minmax("amax", x, F32, dim))
    v, i = ref.minmax("argmax", x, F32, dim)
    pv, pi = port.reduce("argmax", x, F32, dim=dim)
    np.testing.assert_array_equal(pv, v)
    np.testing.assert_array_equal(pi, i)


def test_live_transposed_view(port, ref):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((128, 64), dtype=np.float32).T  # sizes [64,128], strides (1,64)
    np.testing.assert_array_equal(port.reduce("sum", x, F32, dim=-1), ref.sum(x, F32, [-1]))
    np.testing.assert_array_equal(port.reduce("argmax", x, F32, dim=-1)[1],
                                  ref.minmax("argmax", x, F32, -1)[1])


def test_live_rows_gather_scatter(port, ref):
    rng = np.random.default_rng(2)
    V, D, N = 300, 20, 5000
    table = rng.standard_normal((V, D), dtype=np.float32)
    p = np.arange(1, V + 1, dtype=np.float64) ** -1.1
    idx = rng.permutation(V)[np.searchsorted(np.cumsum(p / p.sum()), rng.random(N))].astype(np.int64)
    np.testing.assert_array_equal(port.gather_rows(table, idx), ref.index_rows(table, idx, F32))
    vals = rng.standard_normal((N, D), dtype=np.float32)
    np.testing.assert_array_equal(
        port.scatter_rows(np.zeros((V, D), np.float32), idx, vals, F32),
        ref.index_put_rows(np.zeros((V, D), np.float32), idx, vals, F32, True))
    vi = rng.integers(-1000, 1001, (N, D)).astype(np.int64)
    np.testing.assert_array_equal(
        port.scatter_rows(np.zeros((V, D), np.int64), idx, vi, I64),
        ref.index_put_rows(np.zeros((V, D), np.int64), idx, vi, I64, True))


def test_live_index_errors(port, ref):
    table = np.zeros((4, 3), np.float32)
    for bad in ([4], [-5]):
        with pytest.raises(IndexError):
            ref.index_rows(table, bad, F32)
        with pytest.raises(IndexError):
            port.gather_rows(table, np.array(bad))
    with pytest.raises(IndexError):
        ref.embedding(table, [-1])
    with pytest.raises(IndexError):
        port.gather_rows(table, np.array([-1]), oracle.STRICT)


# ---- 4. paths with no CPU code in the reference: torch CPU as the cross-check ---------------
def _bf(x):
    return oracle.to_storage(x, BF16)


@pytest.mark.parametrize("dtype,tol", [(F32, 1e-5), (BF16, 1e-2), (F16, 2e-3)])
def test_softmax_rmsnorm_vs_torch(port, dtype, tol):
    rng = np.random.default_rng(3)
    xf = (3.0 * rng.standard_normal((37, 300), dtype=np.float32))
    xs = oracle.to_storage(xf, dtype)
    xr = torch.from_numpy(oracle.to_f32(xs, dtype))
    got = oracle.to_f32(port.softmax(xs, dtype), dtype)
    np.testing.assert_allclose(got, torch.softmax(xr, -1).numpy(), rtol=tol, atol=tol)
    got = oracle.to_f32(port.softmax(xs, dtype, log=True), dtype)
    np.testing.assert_allclose(got, torch.log_softmax(xr, -1).numpy(), rtol=tol, atol=tol * 10)
    gamma = (1 + 0.02 * rng.standard_normal(300)).astype(np.float32)
    y, inv = port.rmsnorm(xs, gamma, 1e-6, dtype)
    want = torch.nn.functional.rms_norm(xr, (300,), torch.from_numpy(gamma), 1e-6).numpy()
    np.testing.assert_allclose(oracle.to_f32(y, dtype), want, rtol=max(tol, 1e-4), atol=max(tol, 1e-4))
    np.testing.assert_allclose(inv, 1 / np.sqrt((xr.numpy() ** 2).mean(-1) + 1e-6), rtol=1e-5)


def test_bf16_chain_matches_torch_per_op_rounding(port):
    # config-3 expression: where(a > 0, a + b*c, 0), each op rounded to bf16
    rng = np.random.default_rng(1)
    a = _bf(rng.standard_normal((4, 1, 6, 1), dtype=np.float32))
    b = _bf(rng.standard_normal((1, 5, 1, 8), dtype=np.float32))
    c = _bf(rng.standard_normal((4, 5, 1, 8), dtype=np.float32))
    ta, tb, tc = [torch.from_numpy(oracle.to_f32(v, BF16)).bfloat16() for v in (a, b, c)]
    want = torch.where(ta > 0, ta + tb * tc, torch.zeros((), dtype=torch.bfloat16))
    fused = port.ternary("where_gt0_addcmul", a, b, c, BF16)
    np.testing.assert_array_equal(oracle.to_f32(fused, BF16), want.float().numpy())
    # the same through the four separate ops
    t1 = port.binary("mul", b, c, BF16)
    t2 = port.binary("add", a, t1, BF16)
    m = port.binary("gt", a, np.zeros((1,), np.uint16), BF16)
    out = port.where(m, t2, np.zeros((1,), np.uint16), BF16)
    np.testing.assert_array_equal(out, fused)


def test_bf16_storage_roundtrip():
    x = np.array([1.0, 1.00390625, -2.5, 3.3895314e38, np.inf, np.nan], np.float32)
    want = torch.from_numpy(x).bfloat16().float().numpy()
    got = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(x))
    np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
    np.testing.assert_array_equal(got[~np.isnan(got)], want[~np.isnan(want)])


def test_unary_float_ops_vs_torch(port):
    rng = np.random.default_rng(5)
    x = (4 * rng.standard_normal(2000)).astype(np.float32)
    t = torch.from_numpy(x)
    pos = np.abs(x) + 0.1
    tp = torch.from_numpy(pos)
    cases = {
        "relu": (x, torch.relu(t)), "neg": (x, -t), "abs": (x, t.abs()), "square": (x, t * t),
        "exp": (x, t.exp()), "log": (pos, tp.log()), "sqrt": (pos, tp.sqrt()),
        "rsqrt": (pos, tp.rsqrt()), "sin": (x, t.sin()), "cos": (x, t.cos()),
        "tanh": (x, t.tanh()), "sigmoid": (x, t.sigmoid()),
        "silu": (x, torch.nn.functional.silu(t)), "gelu": (x, torch.nn.functional.gelu(t)),
        "reciprocal": (pos, tp.reciprocal()), "sign": (x, t.sign()), "floor": (x, t.floor()),
        "ceil": (x, t.ceil()), "trunc": (x, t.trunc()), "round": (x, t.round()),
        "expm1": (x, t.expm1()), "log1p": (pos, tp.log1p()),
        "softplus": (x, torch.nn.functional.softplus(t)),
        "relu6": (x, torch.nn.functional.relu6(t)), "hardtanh": (x, torch.nn.functional.hardtanh(t)),
    }
    unit = np.clip(x / 16, -0.99, 0.99).astype(np.float32)
    tu = torch.from_numpy(unit)
    p01 = (np.abs(unit) * 0.98 + 0.01).astype(np.float32)
    tp01 = torch.from_numpy(p01)
    F = torch.nn.functional
    cases.update({
        "exp2": (x, t.exp2()), "log2": (pos, tp.log2()), "log10": (pos, tp.log10()), "sinh": (x, t.sinh()),
        "cosh": (x, t.cosh()), "asinh": (x, t.asinh()), "acosh": (pos + 1, (tp + 1).acosh()),
        "atanh": (unit, tu.atanh()), "tan": (unit, tu.tan()), "asin": (unit, tu.asin()),
        "acos": (unit, tu.acos()), "atan": (x, t.atan()), "erf": (x, t.erf()), "erfc": (x, t.erfc()),
        "lgamma": (pos, tp.lgamma()), "sinc": (x, t.sinc()), "frac": (x, t.frac()),
        "deg2rad": (x, t.deg2rad()), "rad2deg": (x, t.rad2deg()), "mish": (x, F.mish(t)),
        "selu": (x, F.selu(t)), "elu": (x, F.elu(t)), "hardsigmoid": (x, F.hardsigmoid(t)),
        "hardshrink": (x, F.hardshrink(t)), "softshrink": (x, F.softshrink(t)),
        "logit": (p01, tp01.logit()), "angle": (x, t.angle()), "positive": (x, t.positive()),
        "sgn": (x, t.sgn()), "nan_to_num": (x, t.nan_to_num()),
    })
    assert set(cases) == set(oracle.UNARY) - oracle.UNARY_TO_BOOL - {"bitwise_not"}
    for name, (inp, want) in cases.items():
        got = port.unary(name, inp, F32)
        np.testing.assert_allclose(got, want.numpy(), rtol=1e-5, atol=1e-6, err_msg=name)


def test_predicates_and_bitwise_not_vs_torch(port):
    x = np.array([0.0, -0.0, 1.5, -2.0, np.inf, -np.inf, np.nan, 1e-40], np.float32)
    t = torch.from_numpy(x)
    want = {"isfinite": t.isfinite(), "isinf": t.isinf(), "isnan": t.isnan(), "isneginf": t.isneginf(),
            "isposinf": t.isposinf(), "signbit": t.signbit(), "logical_not": t.logical_not()}
    assert set(want) == oracle.UNARY_TO_BOOL
    for dt, code in ((torch.float32, F32), (torch.bfloat16, BF16), (torch.float16, oracle.F16)):
        xs = oracle.to_storage(x, code)
        for name, w in want.items():
            w = getattr(t.to(dt), name)() if name != "logical_not" else t.to(dt).logical_not()
            keep = ~np.isnan(x) if name == "signbit" else np.ones(8, bool)  # a NaN's sign is payload
            np.testing.assert_array_equal(port.unary(name, xs, code)[keep], w.numpy().view(np.uint8)[keep],
                                          err_msg=name)
    xi = np.array([0, -1, 5, np.iinfo(np.int64).min], np.int64)
    ti = torch.from_numpy(xi)
    for name in ("isfinite", "isinf", "isnan", "signbit", "logical_not"):
        np.testing.assert_array_equal(port.unary(name, xi, I64), getattr(ti, name)().numpy().view(np.uint8))
    np.testing.assert_array_equal(port.unary("bitwise_not", xi, I64), (~ti).numpy())
    x32 = xi[:3].astype(np.int32)
    np.testing.assert_array_equal(port.unary("bitwise_not", x32, oracle.I32), ~x32)
    xb = np.array([0, 1, 1, 0], np.uint8)
    np.testing.assert_array_equal(port.unary("bitwise_not", xb, oracle.BOOL), 1 - xb)
    np.testing.assert_array_equal(port.unary("logical_not", xb, oracle.BOOL), 1 - xb)


def test_binary_tail_float_ops_vs_torch(port):
    rng = np.random.default_rng(6)
    a = (3 * rng.standard_normal(3000)).astype(np.float32)
    b = (3 * rng.standard_normal(3000)).astype(np.float32)
    a[:8] = [0.0, -0.0, 5.5, -5.5, 5.5, -5.5, np.inf, np.nan]
    b[:8] = [1.0, 2.0, 2.0, 2.0, -2.0, -2.0, 3.0, 1.0]
    ta, tb = torch.from_numpy(a), torch.from_numpy(b)
    pa, pb = np.abs(a) + 0.1, np.abs(b) + 0.1
    tpa, tpb = torch.from_numpy(pa), torch.from_numpy(pb)
    u = (np.abs(np.tanh(b)) * 0.98 + 0.01).astype(np.float32)
    tu = torch.from_numpy(u)
    e = np.round(b).astype(np.float32)
    cases = {
        "pow": (pa, b, tpa.pow(tb)), "fmod": (a, b, ta.fmod(tb)), "remainder": (a, b, ta.remainder(tb)),
        "atan2": (a, b, ta.atan2(tb)), "copysign": (a, b, ta.copysign(tb)), "hypot": (a, b, ta.hypot(tb)),
        "xlogy": (a, pb, ta.xlogy(tpb)), "xlog1py": (a, pb, torch.special.xlog1py(ta, tpb)),
        "logaddexp": (a, b, ta.logaddexp(tb)), "logaddexp2": (a, b, ta.logaddexp2(tb)),
        "nextafter": (a, b, ta.nextafter(tb)), "heaviside": (a, b, ta.heaviside(tb)),
        "rsub": (a, b, tb - ta), "tanh_backward": (a, u, ta * (1 - tu * tu)),
        "sigmoid_backward": (a, u, ta * tu * (1 - tu)),
        "silu_backward": (a, b, ta * (tb.sigmoid() * (1 + tb * (1 - tb.sigmoid())))),
        "logit_backward": (a, u, ta / (tu * (1 - tu))), "mse_loss": (a, b, (ta - tb) ** 2),
        "ldexp": (a, e, ta.ldexp(torch.from_numpy(e))),
    }
    exact = {"fmod", "remainder", "copysign", "nextafter", "heaviside", "rsub", "mse_loss", "ldexp"}
    for name, (x, y, want) in cases.items():
        got = port.binary(name, x, y, F32)
        w = want.numpy()
        if name == "heaviside":  # heaviside(NaN, y): the reference's functor falls through to y, torch gives 0
            assert got[7] == y[7]
            got, w = np.delete(got, 7), np.delete(w, 7)
        np.testing.assert_array_equal(np.isnan(got), np.isnan(w), err_msg=name)
        if name in exact:
            np.testing.assert_array_equal(got[~np.isnan(w)], w[~np.isnan(w)], err_msg=name)
        else:
            fin = np.isfinite(w)
            np.testing.assert_allclose(got[fin], w[fin], rtol=2e-5, atol=1e-6, err_msg=name)
    tail = oracle.BINARY[oracle.BINARY.index("pow"):oracle.BINARY.index("bitwise_and")]
    assert set(cases) == set(tail)


def test_integer_and_logical_ops_vs_torch(port):
    rng = np.random.default_rng(7)
    a = rng.integers(-2 ** 40, 2 ** 40, 2000).astype(np.int64)
    b = rng.integers(-50, 50, 2000).astype(np.int64)
    a[:4] = [np.iinfo(np.int64).min, 0, -7, 7]
    b[:4] = [-1, 0, 2, -2]
    ta, tb = torch.from_numpy(a), torch.from_numpy(b)
    sh = np.abs(b) % 70
    tsh = torch.from_numpy(sh)
    want = {"bitwise_and": ta & tb, "bitwise_or": ta | tb, "bitwise_xor": ta ^ tb,
            "gcd": torch.gcd(ta, tb), "remainder": None, "fmod": None}
    for name in ("bitwise_and", "bitwise_or", "bitwise_xor", "gcd"):
        np.testing.assert_array_equal(port.binary(name, a, b, I64), want[name].numpy(), err_msg=name)
    small = rng.integers(-1000, 1000, 2000).astype(np.int64)
    np.testing.assert_array_equal(port.binary("lcm", small, b, I64),
                                  torch.lcm(torch.from_numpy(small), tb).abs().numpy())
    nz = b != 0
    ok = nz & ~((a == np.iinfo(np.int64).min) & (b == -1))
    np.testing.assert_array_equal(port.binary("remainder", a, b, I64)[ok], ta.remainder(torch.where(tb == 0, 1, tb)).numpy()[ok])
    np.testing.assert_array_equal(port.binary("fmod", a, b, I64)[ok], ta.fmod(torch.where(tb == 0, 1, tb)).numpy()[ok])
    assert (port.binary("remainder", a, b, I64)[~ok] == 0).all()  # b == 0 and INT64_MIN % -1 give 0
    # shifts: counts in [0, 64) agree with torch; counts outside give 0 / the sign fill
    inr = sh < 64
    np.testing.assert_array_equal(port.binary("lshift", a, sh, I64)[inr], (ta << tsh).numpy()[inr])
    np.testing.assert_array_equal(port.binary("rshift", a, sh, I64)[inr], (ta >> tsh).numpy()[inr])
    assert (port.binary("lshift", a, sh, I64)[~inr] == 0).all()
    np.testing.assert_array_equal(port.binary("rshift", a, sh, I64)[~inr], np.where(a[~inr] < 0, -1, 0))
    assert (port.binary("rshift", a, -1 - sh, I64) == np.where(a < 0, -1, 0)).all()
    a32, s32 = (a % 2 ** 31).astype(np.int32) * np.where(a < 0, -1, 1).astype(np.int32), (sh % 32).astype(np.int32)
    t32, ts32 = torch.from_numpy(a32), torch.from_numpy(s32)
    np.testing.assert_array_equal(port.binary("lshift", a32, s32, oracle.I32), (t32 << ts32).numpy())
    np.testing.assert_array_equal(port.binary("rshift", a32, s32, oracle.I32), (t32 >> ts32).numpy())
    np.testing.assert_array_equal(port.binary("bitwise_xor", a32, s32, oracle.I32), a32 ^ s32)
    xb, yb = (a & 1).astype(np.uint8), (b & 1).astype(np.uint8)
    for name, w in (("bitwise_and", xb & yb), ("bitwise_or", xb | yb), ("bitwise_xor", xb ^ yb),
                    ("logical_and", xb & yb), ("logical_or", xb | yb), ("logical_xor", xb ^ yb)):
        np.testing.assert_array_equal(port.binary(name, xb, yb, oracle.BOOL), w, err_msg=name)
    fa = np.where(a % 3 == 0, 0.0, a).astype(np.float32)
    fb = np.where(b % 2 == 0, 0.0, np.nan).astype(np.float32)
    for name in ("logical_and", "logical_or", "logical_xor"):
        w = getattr(torch, name)(torch.from_numpy(fa), torch.from_numpy(fb)).numpy().view(np.uint8)
        np.testing.assert_array_equal(port.binary(name, fa, fb, F32), w, err_msg=name)
        wi = getattr(torch, name)(ta, tb).numpy().view(np.uint8)
        np.testing.assert_array_equal(port.binary(name, a, b, I64), wi, err_msg=name)


def test_loss_ternaries_vs_torch(port):
    rng = np.random.default_rng(8)
    a = rng.standard_normal(500).astype(np.float32) * 2
    b = rng.standard_normal(500).astype(np.float32) * 2
    d = np.full(500, 1.25, np.float32)
    F = torch.nn.functional
    ta, tb = torch.from_numpy(a), torch.from_numpy(b)
    np.testing.assert_allclose(port.ternary("huber_loss", a, b, d, F32),
                               F.huber_loss(ta, tb, reduction="none", delta=1.25).numpy(), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(port.ternary("smooth_l1_loss", a, b, d, F32),
                               F.smooth_l1_loss(ta, tb, reduction="none", beta=1.25).numpy(), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("dtype,tol", [(F32, 2e-5), (BF16, 2e-2)])
def test_row_op_backwards_vs_torch_autograd(port, dtype, tol):
    """No CPU code for these in the reference: the restatement of its CuTe / Triton backward
    kernels is pinned on torch autograd of the same forward, in float32 on the stored values."""
    rng = np.random.default_rng(9)
    rows, cols = 7, 300
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 2
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    xs, dys = oracle.to_storage(x, dtype), oracle.to_storage(dy, dtype)
    tx = torch.from_numpy(oracle.to_f32(xs, dtype)).requires_grad_(True)
    tdy = torch.from_numpy(oracle.to_f32(dys, dtype))
    for log in (False, True):
        ty = torch.log_softmax(tx, -1) if log else torch.softmax(tx, -1)
        (want,) = torch.autograd.grad(ty, tx, tdy)
        ys = oracle.to_storage(ty.detach().numpy(), dtype)
        got = oracle.to_f32(port.softmax_backward(dys, ys, dtype, log=log), dtype)
        np.testing.assert_allclose(got, want.numpy(), rtol=tol, atol=tol)
    tg = torch.from_numpy(gamma).requires_grad_(True)
    ty = torch.nn.functional.rms_norm(tx, (cols,), tg, 1e-6)
    wdx, wdg = torch.autograd.grad(ty, (tx, tg), tdy)
    _, inv = port.rmsnorm(xs, gamma, 1e-6, dtype)
    dx, dg = port.rmsnorm_backward(dys, xs, inv, gamma, dtype)
    np.testing.assert_allclose(oracle.to_f32(dx, dtype), wdx.numpy(), rtol=tol, atol=tol)
    np.testing.assert_allclose(dg, wdg.numpy(), rtol=1e-4, atol=1e-4)
    dx2, dg2 = port.rmsnorm_backward(dys, xs, inv, None, dtype)
    assert dg2 is None
    (wdx2,) = torch.autograd.grad(torch.nn.functional.rms_norm(tx, (cols,), None, 1e-6), tx, tdy)
    np.testing.assert_allclose(oracle.to_f32(dx2, dtype), wdx2.numpy(), rtol=tol, atol=tol)


def test_embedding_backward_scale_grad_by_freq_vs_torch(port):
    rng = np.random.default_rng(10)
    idx = rng.integers(0, 50, 400).astype(np.int64)
    g = rng.standard_normal((400, 24)).astype(np.float32)
    w = torch.zeros((50, 24), requires_grad=True)
    out = torch.nn.functional.embedding(torch.from_numpy(idx), w, padding_idx=3, scale_grad_by_freq=True)
    out.backward(torch.from_numpy(g))
    np.testing.assert_allclose(port.embedding_backward_by_freq(g, idx, 50, padding_idx=3), w.grad.numpy(),
                               rtol=1e-5, atol=1e-6)
