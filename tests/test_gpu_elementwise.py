"""CUDA elementwise path vs the CPU oracle, through the C ABI (vibetensor_b200.ops is a thin
ctypes layer).  Bit-exact for add/sub/mul/div, comparisons, where, copies, integer ops and
the fused chains; 1e-5 (fp32) / 1e-2 (bf16, f16: one storage ulp) for transcendental ops."""
import os

import numpy as np
import pytest
import torch

import oracle
from tests.util import CODE, as_f32, from_np, rand_storage, strided_like, to_np

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))
FLOATS = [torch.float32, torch.bfloat16, torch.float16]


@pytest.fixture(scope="module")
def ops():
    from vibetensor_b200 import ops as o
    return o


EXACT_UNARY = ["relu", "neg", "abs", "square", "sign", "floor", "ceil", "trunc", "round", "relu6",
               "hardtanh", "sqrt", "frac", "hardshrink", "softshrink", "angle", "positive", "sgn",
               "nan_to_num"]
FLOAT_UNARY = [n for n in oracle.UNARY if n not in oracle.UNARY_TO_BOOL and n != "bitwise_not"]
CORE_BINARY = oracle.BINARY[:oracle.BINARY.index("pow")]
TAIL_FLOAT_BINARY = oracle.BINARY[oracle.BINARY.index("pow"):oracle.BINARY.index("bitwise_and")]
EXACT_TAIL_BINARY = {"fmod", "remainder", "copysign", "nextafter", "heaviside", "rsub", "mse_loss", "ldexp"}


def _check_unary(ops, port, name, x_np, dtype):
    got = to_np(ops.unary(name, from_np(x_np, dtype)))
    want = port.unary(name, x_np, CODE[dtype])
    if dtype == torch.int64 or name in EXACT_UNARY:
        np.testing.assert_array_equal(got, want, err_msg=name)
    else:
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        g, w = as_f32(got, dtype), as_f32(want, dtype)
        fin = np.isfinite(w)
        np.testing.assert_array_equal(np.isnan(g), np.isnan(w), err_msg=name)
        np.testing.assert_allclose(g[fin], w[fin], rtol=tol, atol=tol if dtype != torch.float32 else 1e-6,
                                   err_msg=name)


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("name", FLOAT_UNARY)
def test_unary_float(ops, port, name, dtype):
    rng = np.random.default_rng(11)
    x = 4 * rng.standard_normal((37, 129), dtype=np.float32)
    if name in ("log", "sqrt", "rsqrt", "log1p", "reciprocal", "log2", "log10", "lgamma"):
        x = np.abs(x) + 0.05
    elif name == "acosh":
        x = np.abs(x) + 1.0
    elif name in ("atanh", "asin", "acos"):
        x = 0.99 * np.tanh(x)
    elif name == "logit":
        x = 0.01 + 0.98 / (1.0 + np.exp(-x))
    x.flat[:6] = [0.0, -0.0, 25.0, -25.0, 0.5, 2.5]
    x.flat[6:9] = [np.inf, -np.inf, np.nan]
    if name == "nan_to_num" and dtype != torch.float32:
        with pytest.raises(ValueError, match="float32 tensor expected"):
            ops.nan_to_num(from_np(oracle.to_storage(x, CODE[dtype]), dtype))
        return
    _check_unary(ops, port, name, oracle.to_storage(x, CODE[dtype]), dtype)


@pytest.mark.parametrize("dtype", FLOATS + [torch.int64, torch.bool])
@pytest.mark.parametrize("name", sorted(oracle.UNARY_TO_BOOL))
def test_predicates_write_bool(ops, port, name, dtype):
    rng = np.random.default_rng(21)
    if dtype == torch.bool:
        x = rng.integers(0, 2, (9, 70)).astype(np.uint8)
    elif dtype == torch.int64:
        x = rng.integers(-3, 4, (9, 70)).astype(np.int64)
        x.flat[:2] = [np.iinfo(np.int64).min, np.iinfo(np.int64).max]
    else:
        v = rng.standard_normal((9, 70), dtype=np.float32)
        v.flat[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 65536.0 * 65536.0]
        v.flat[8::7] = 0.0
        x = oracle.to_storage(v, CODE[dtype])
    got = ops.unary(name, from_np(x, dtype))
    assert got.dtype == torch.bool
    want = port.unary(name, x, CODE[dtype])
    if name == "signbit" and dtype != torch.bool and dtype != torch.int64:
        keep = ~np.isnan(as_f32(x, dtype))          # the sign of a NaN is payload, not semantics
        np.testing.assert_array_equal(to_np(got)[keep], want[keep])
    else:
        np.testing.assert_array_equal(to_np(got), want)
    # into a strided bool view
    base = torch.zeros((70, 9), dtype=torch.bool, device="cuda")
    ops.unary(name, from_np(x, dtype), out=base.t())
    assert torch.equal(base.t(), got)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32, torch.bool])
def test_bitwise_not(ops, port, dtype):
    rng = np.random.default_rng(22)
    if dtype == torch.bool:
        x = rng.integers(0, 2, (5, 333)).astype(np.uint8)
    else:
        npdt = np.int64 if dtype == torch.int64 else np.int32
        x = rng.integers(np.iinfo(npdt).min, np.iinfo(npdt).max, (5, 333), dtype=npdt)
    np.testing.assert_array_equal(to_np(ops.bitwise_not(from_np(x, dtype))), port.unary("bitwise_not", x, CODE[dtype]))
    with pytest.raises(ValueError, match="integral or bool tensor expected"):
        ops.bitwise_not(torch.ones(4, device="cuda"))


@pytest.mark.parametrize("name", ["relu", "neg", "abs", "square", "sign", "floor", "round", "positive", "sgn"])
def test_unary_int64(ops, port, name):
    rng = np.random.default_rng(12)
    x = rng.integers(-2 ** 62, 2 ** 62, (33, 65)).astype(np.int64)
    x.flat[:3] = [np.iinfo(np.int64).min, 0, np.iinfo(np.int64).max]
    _check_unary(ops, port, name, x, torch.int64)


def test_unary_rejects_integral_for_transcendental(ops):
    with pytest.raises(ValueError, match="floating tensor expected"):
        ops.exp(torch.ones(4, dtype=torch.int64, device="cuda"))


@pytest.mark.parametrize("dtype", FLOATS + [torch.int64])
@pytest.mark.parametrize("name", CORE_BINARY)
def test_binary_broadcast_bit_exact(ops, port, name, dtype):
    if dtype == torch.int64 and name == "div":
        with pytest.raises(ValueError):
            ops.div(torch.ones(2, dtype=dtype, device="cuda"), torch.ones(2, dtype=dtype, device="cuda"))
        return
    rng = np.random.default_rng(13)
    a = rand_storage(rng, (6, 1, 40), dtype)
    b = rand_storage(rng, (5, 40), dtype)
    if dtype != torch.int64:
        a.flat[0] = oracle.to_storage(np.array([np.nan], np.float32), CODE[dtype])[0]
        b.flat[1] = a.flat[0]
        b.flat[2] = a.flat[2]  # an equal pair for eq/le/ge
    got = to_np(ops.binary(name, from_np(a, dtype), from_np(b, dtype)))
    want = port.binary(name, a, b, CODE[dtype])
    if dtype == torch.int64 or name in ("eq", "ne", "lt", "gt", "le", "ge"):
        np.testing.assert_array_equal(got, want)
    else:
        g, w = as_f32(got, dtype), as_f32(want, dtype)
        np.testing.assert_array_equal(np.isnan(g), np.isnan(w))
        np.testing.assert_array_equal(g[~np.isnan(g)], w[~np.isnan(w)])


def _tail_inputs(rng, name, dtype):
    a = 3 * rng.standard_normal((6, 1, 40), dtype=np.float32)
    b = 3 * rng.standard_normal((5, 40), dtype=np.float32)
    if name == "pow":
        a = np.abs(a) + 0.1
    elif name in ("xlogy", "xlog1py"):
        b = np.abs(b) + 0.1
        a.flat[3:6] = 0.0
    elif name in ("tanh_backward", "sigmoid_backward", "logit_backward"):
        b = 0.01 + 0.98 / (1.0 + np.exp(-b))
    elif name == "ldexp":
        b = np.round(4 * b)
    elif name == "heaviside":
        a.flat[3:9] = [0.0, -0.0, 0.0, 1.0, -1.0, np.nan]
    elif name in ("fmod", "remainder"):
        a.flat[3:9] = [5.5, -5.5, 5.5, -5.5, 0.0, np.inf]
        b.flat[3:9] = [2.0, 2.0, -2.0, -2.0, 3.0, 2.0]
    a.flat[0] = np.nan
    b.flat[1] = np.nan
    return oracle.to_storage(a, CODE[dtype]), oracle.to_storage(b, CODE[dtype])


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("name", TAIL_FLOAT_BINARY)
def test_binary_tail_float(ops, port, name, dtype):
    rng = np.random.default_rng(23)
    a, b = _tail_inputs(rng, name, dtype)
    got = to_np(ops.binary(name, from_np(a, dtype), from_np(b, dtype)))
    want = port.binary(name, a, b, CODE[dtype])
    g, w = as_f32(got, dtype), as_f32(want, dtype)
    np.testing.assert_array_equal(np.isnan(g), np.isnan(w), err_msg=name)
    if name in EXACT_TAIL_BINARY:
        np.testing.assert_array_equal(got[~np.isnan(w)], want[~np.isnan(w)], err_msg=name)
    else:
        fin = np.isfinite(w)
        np.testing.assert_array_equal(g[~fin & ~np.isnan(w)], w[~fin & ~np.isnan(w)], err_msg=name)
        tol = 2e-5 if dtype == torch.float32 else 1e-2
        np.testing.assert_allclose(g[fin], w[fin], rtol=tol, atol=1e-6 if dtype == torch.float32 else tol,
                                   err_msg=name)


@pytest.mark.parametrize("name", ["fmod", "remainder", "heaviside", "rsub"])
def test_binary_tail_int64(ops, port, name):
    rng = np.random.default_rng(24)
    a = rng.integers(-2 ** 62, 2 ** 62, (7, 1, 33)).astype(np.int64)
    b = rng.integers(-9, 10, (5, 33)).astype(np.int64)          # includes zeros
    a.flat[:3] = [np.iinfo(np.int64).min, 0, np.iinfo(np.int64).max]
    b.flat[:3] = [-1, 0, -1]
    got = to_np(ops.binary(name, from_np(a, torch.int64), from_np(b, torch.int64)))
    np.testing.assert_array_equal(got, port.binary(name, a, b, oracle.I64))
    for bad in ("pow", "atan2", "hypot", "ldexp"):
        with pytest.raises(ValueError, match="floating tensor expected"):
            ops.binary(bad, from_np(a, torch.int64), from_np(b, torch.int64))
    with pytest.raises(ValueError, match="boolean not supported"):
        ops.fmod(torch.ones(3, dtype=torch.bool, device="cuda"), torch.ones(3, dtype=torch.bool, device="cuda"))


@pytest.mark.parametrize("left", [False, True])
def test_binary_tail_scalar_operand(ops, port, left):
    rng = np.random.default_rng(25)
    a = np.abs(rng.standard_normal((19, 31), dtype=np.float32)) + 0.25
    ta = torch.from_numpy(a).cuda()
    s = np.array(2.5, np.float32)
    for name in ("pow", "fmod", "remainder", "atan2", "rsub", "mse_loss"):
        got = to_np(ops.binary(name, 2.5, ta) if left else ops.binary(name, ta, 2.5))
        want = port.binary(name, s, a, oracle.F32) if left else port.binary(name, a, s, oracle.F32)
        if name in EXACT_TAIL_BINARY:
            np.testing.assert_array_equal(got, want, err_msg=name)
        else:
            np.testing.assert_allclose(got, want, rtol=2e-5, err_msg=name)
    ai = rng.integers(-1000, 1000, (19, 31)).astype(np.int64)
    ti = torch.from_numpy(ai).cuda()
    si = np.array(7, np.int64)
    for name in ("remainder", "fmod", "rsub"):
        got = to_np(ops.binary(name, 7, ti) if left else ops.binary(name, ti, 7))
        want = port.binary(name, si, ai, oracle.I64) if left else port.binary(name, ai, si, oracle.I64)
        np.testing.assert_array_equal(got, want, err_msg=name)
    with pytest.raises(ValueError, match="no scalar form"):
        ops.binary("bitwise_and", ti, 1)


def _int_storage(rng, shape, dtype, lo=None, hi=None):
    if dtype == torch.bool:
        return rng.integers(0, 2, shape).astype(np.uint8)
    npdt = np.int64 if dtype == torch.int64 else np.int32
    info = np.iinfo(npdt)
    return rng.integers(info.min if lo is None else lo, info.max if hi is None else hi, shape, dtype=npdt)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32, torch.bool])
@pytest.mark.parametrize("name", ["bitwise_and", "bitwise_or", "bitwise_xor", "lshift", "rshift", "gcd", "lcm"])
def test_integer_binary_ops(ops, port, name, dtype):
    rng = np.random.default_rng(26)
    shift = name in ("lshift", "rshift")
    gl = name in ("gcd", "lcm")
    ta1 = torch.ones(3, dtype=dtype, device="cuda")
    if (shift and dtype == torch.bool) or (gl and dtype != torch.int64):
        with pytest.raises(ValueError, match="expected Int"):
            ops.binary(name, ta1, ta1)
        return
    a = _int_storage(rng, (6, 1, 70), dtype)
    if shift:
        b = _int_storage(rng, (4, 70), dtype, -4, 70)      # counts below 0 and beyond the width too
    elif gl:
        a = _int_storage(rng, (6, 1, 70), dtype, -5000, 5000)
        b = _int_storage(rng, (4, 70), dtype, -60, 60)
        a.flat[:2] = [0, np.iinfo(np.int64).min]
        b.flat[:2] = [0, 6]
    else:
        b = _int_storage(rng, (4, 70), dtype)
    got = to_np(ops.binary(name, from_np(a, dtype), from_np(b, dtype)))
    np.testing.assert_array_equal(got, port.binary(name, a, b, CODE[dtype]))
    with pytest.raises(ValueError):
        ops.binary(name, torch.ones(3, device="cuda"), torch.ones(3, device="cuda"))


@pytest.mark.parametrize("dtype", FLOATS + [torch.int64, torch.bool])
@pytest.mark.parametrize("name", ["logical_and", "logical_or", "logical_xor"])
def test_logical_ops_write_bool(ops, port, name, dtype):
    rng = np.random.default_rng(27)
    if dtype in (torch.int64, torch.bool):
        a = _int_storage(rng, (8, 1, 50), dtype, -1, 2)
        b = _int_storage(rng, (3, 50), dtype, -1, 2)
    else:
        va = rng.integers(-1, 2, (8, 1, 50)).astype(np.float32)
        vb = rng.integers(-1, 2, (3, 50)).astype(np.float32)
        va.flat[:3] = [np.nan, -0.0, 1e-40]
        a, b = oracle.to_storage(va, CODE[dtype]), oracle.to_storage(vb, CODE[dtype])
    got = ops.binary(name, from_np(a, dtype), from_np(b, dtype))
    assert got.dtype == torch.bool
    np.testing.assert_array_equal(to_np(got), port.binary(name, a, b, CODE[dtype]))


def test_binary_golden_reference_vectors(ops):
    a, b = GOLD["ew_a"], GOLD["ew_b"]
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    for op in ["add", "sub", "mul", "div"]:
        np.testing.assert_array_equal(ops.binary(op, ta, tb).cpu().numpy(), GOLD["ew_" + op])
    for op in ["eq", "ne", "lt", "gt", "le", "ge"]:
        np.testing.assert_array_equal(to_np(ops.binary(op, ta, tb)), GOLD["ew_" + op])
    for op in ["relu", "abs", "neg", "reciprocal"]:
        np.testing.assert_array_equal(ops.unary(op, ta).cpu().numpy(), GOLD["ew_" + op])
    ai, bi = torch.from_numpy(GOLD["ew_ai"]).cuda(), torch.from_numpy(GOLD["ew_bi"]).cuda()
    for op in ["add", "sub", "mul"]:
        np.testing.assert_array_equal(ops.binary(op, ai, bi).cpu().numpy(), GOLD["ew_i64_" + op])


def test_broadcast_add_known_answer(ops):
    # tests/cpp/cuda_elementwise_test.cc:343-394 of the reference
    rows, cols = 2, 256
    a = (np.arange(rows)[:, None] * 1000 + np.arange(cols)[None, :]).astype(np.float32)
    b = (1.5 * np.arange(cols)).astype(np.float32)
    got = ops.add(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, a + b)


@pytest.mark.parametrize("left", [False, True])
@pytest.mark.parametrize("name", ["add", "sub", "mul", "div", "gt", "maximum"])
def test_binary_scalar_operand(ops, port, name, left):
    rng = np.random.default_rng(14)
    a = rng.standard_normal((17, 33), dtype=np.float32)
    s = np.array(1.25, np.float32)
    ta = torch.from_numpy(a).cuda()
    got = to_np(ops.binary(name, 1.25, ta) if left else ops.binary(name, ta, 1.25))
    want = port.binary(name, s, a, oracle.F32) if left else port.binary(name, a, s, oracle.F32)
    np.testing.assert_array_equal(got, want)
    with pytest.raises(ValueError, match="unsupported dtype for scalar op"):
        ops.add(ta.bfloat16(), 1.0)
    with pytest.raises(ValueError, match="Half CPU scalars"):
        ops.add(ta.half(), 1.0)


def test_dtype_mismatch_and_shape_errors(ops):
    a = torch.ones(4, device="cuda")
    with pytest.raises(ValueError, match="vt::add: dtype mismatch"):
        ops.add(a, a.bfloat16())
    with pytest.raises(ValueError, match="shape mismatch"):
        ops.add(torch.ones(3, device="cuda"), torch.ones(4, device="cuda"), out=torch.ones(4, device="cuda"))
    with pytest.raises(ValueError, match="25D"):
        ops.add(torch.ones([1] * 26, device="cuda"), torch.ones([1] * 26, device="cuda"))
    big = torch.ones([2] + [1] * 24, device="cuda")
    assert ops.add(big, big).shape == big.shape  # rank 25 is accepted


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("name", oracle.TERNARY)
def test_ternary_bit_exact(ops, port, name, dtype):
    rng = np.random.default_rng(15)
    a = rand_storage(rng, (4, 1, 24, 1), dtype)
    b = rand_storage(rng, (1, 16, 1, 8), dtype)
    c = rand_storage(rng, (4, 16, 1, 8), dtype)
    if name == "clamp":
        b, c = port.binary("minimum", b, c, CODE[dtype]), port.binary("maximum", b, c, CODE[dtype])
    if name in ("huber_loss", "smooth_l1_loss"):
        c = port.unary("abs", c, CODE[dtype])
    got = to_np(ops.ternary(name, from_np(a, dtype), from_np(b, dtype), from_np(c, dtype)))
    want = port.ternary(name, a, b, c, CODE[dtype])
    if name in ("addcdiv", "huber_loss", "smooth_l1_loss"):
        np.testing.assert_allclose(as_f32(got, dtype), as_f32(want, dtype), rtol=1e-6 if dtype == torch.float32 else 1e-2)
    else:
        np.testing.assert_array_equal(got, want)


def _config3(rng, n0, d1, d2, d3):
    a = rand_storage(rng, (n0, 1, d2, 1), torch.bfloat16)
    b = rand_storage(rng, (1, d1, 1, d3), torch.bfloat16)
    c = rand_storage(rng, (n0, d1, 1, d3), torch.bfloat16)
    return a, b, c


@pytest.mark.parametrize("shape", [(4, 16, 24, 8), (3, 128, 40, 16), (2, 24, 7, 5), (2, 8, 1, 8)])
def test_config3_chain_into_transposed_output(ops, port, shape):
    """where(a > 0, a + b*c, 0) in bf16 written into out_base.transpose(1, 3): the fused
    entry, the four separate ops with out=, and the oracle all agree bit for bit."""
    n0, d1, d2, d3 = shape
    rng = np.random.default_rng(1)
    a, b, c = _config3(rng, *shape)
    ta, tb, tc = [from_np(v, torch.bfloat16) for v in (a, b, c)]
    want = port.ternary("where_gt0_addcmul", a, b, c, oracle.BF16)  # [n0,d1,d2,d3]
    base = torch.full((n0, d3, d2, d1), 7.0, dtype=torch.bfloat16, device="cuda")
    out = base.transpose(1, 3)
    ops.where_gt0_addcmul(ta, tb, tc, out=out)
    np.testing.assert_array_equal(to_np(out), want)
    # storage really is [n0, d3, d2, d1]
    np.testing.assert_array_equal(to_np(base), np.ascontiguousarray(want.transpose(0, 3, 2, 1)))
    # the same as the reference would chain it: mul -> add -> gt -> where
    t1 = ops.mul(tb, tc)
    t2 = ops.add(ta, t1)
    m = ops.gt(ta, torch.zeros(1, dtype=torch.bfloat16, device="cuda"))
    base2 = torch.zeros_like(base)
    ops.where(m, t2, torch.zeros(1, dtype=torch.bfloat16, device="cuda"), out=base2.transpose(1, 3))
    assert torch.equal(base2, base)
    plan = ops.ti_plan(out, ta, tb, tc)
    assert plan[0][0] == d1 and plan[1][0][0] == 1  # dim 0 is the dim the output is contiguous in


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.bool])
def test_where_and_masked_fill(ops, port, dtype):
    rng = np.random.default_rng(16)
    cond = rng.integers(0, 2, (5, 1, 33)).astype(np.uint8)
    if dtype == torch.bool:
        x = rng.integers(0, 2, (5, 4, 33)).astype(np.uint8)
        y = rng.integers(0, 2, (1, 33)).astype(np.uint8)
    else:
        x = rand_storage(rng, (5, 4, 33), dtype)
        y = rand_storage(rng, (1, 33), dtype)
    got = to_np(ops.where(from_np(cond, torch.bool), from_np(x, dtype), from_np(y, dtype)))
    want = port.where(cond, x, y, CODE[dtype])
    np.testing.assert_array_equal(got, want)
    with pytest.raises(ValueError, match="bool"):
        ops.where(torch.ones(4, device="cuda"), torch.ones(4, device="cuda"), torch.ones(4, device="cuda"))


def test_strided_inputs_and_outputs(ops, port):
    rng = np.random.default_rng(17)
    a_np = rng.standard_normal((9, 14), dtype=np.float32)
    b_np = rng.standard_normal((9, 14), dtype=np.float32)
    ta, va = strided_like(a_np, torch.float32, (3, 40), 1024, offset=5)      # transposed-ish, gaps
    tb = torch.from_numpy(b_np).cuda()
    got = ops.add(ta, tb).cpu().numpy()
    np.testing.assert_array_equal(got, port.binary("add", va, b_np, oracle.F32))
    out = torch.empty((14, 9), device="cuda").t()                            # column-major output
    ops.mul(ta, tb, out=out)
    np.testing.assert_array_equal(out.cpu().numpy(), a_np * b_np)


def test_negative_strides_through_the_c_abi(port):
    """torch has no negative strides, VibeTensor views do: build the descriptors by hand."""
    import ctypes
    from vibetensor_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(19)
    a_np = rng.standard_normal((6, 10), dtype=np.float32)
    b_np = rng.standard_normal((6, 10), dtype=np.float32)
    ta, tb = torch.from_numpy(a_np).cuda(), torch.from_numpy(b_np).cuda()
    out = torch.zeros((6, 10), device="cuda")

    def d(t, shape, strides, off):
        keep = ((ctypes.c_int64 * 2)(*shape), (ctypes.c_int64 * 2)(*strides))
        s = _lib.VbtTensor(t.data_ptr() + 4 * off, _lib.F32, 2, keep[0], keep[1])
        s._keep = keep
        return s
    # b read reversed along both dims, out written with rows reversed
    db = d(tb, (6, 10), (-10, -1), 59)
    da = d(ta, (6, 10), (10, 1), 0)
    do = d(out, (6, 10), (-10, 1), 50)
    _lib.check(L.vbt_b200_binary(0, ctypes.byref(do), ctypes.byref(da), ctypes.byref(db),
                                 _lib.stream_ptr(out)))
    want = a_np + b_np[::-1, ::-1]
    np.testing.assert_array_equal(out.cpu().numpy()[::-1], want)


def test_exhaustive_small_shapes_vs_oracle(ops, port):
    """All stride patterns (dense, broadcast 0, gapped, reversed) over small ranks: every
    offset the kernel computes is checked against the oracle's odometer."""
    rng = np.random.default_rng(18)
    sizes = [1, 2, 3, 5, 33]
    for trial in range(60):
        nd = int(rng.integers(1, 5))
        shape = tuple(int(rng.choice(sizes)) for _ in range(nd))
        bshape = tuple(s if rng.random() < 0.6 else 1 for s in shape)
        a_np = rng.standard_normal(shape, dtype=np.float32)
        b_np = rng.standard_normal(bshape, dtype=np.float32)
        ta = torch.from_numpy(a_np).cuda()
        if rng.random() < 0.5 and nd >= 2:
            perm = list(rng.permutation(nd))
            ta = torch.from_numpy(np.ascontiguousarray(a_np.transpose(perm))).cuda().permute(
                *np.argsort(perm).tolist())
        tb = torch.from_numpy(b_np).cuda()
        got = ops.add(ta, tb).cpu().numpy()
        np.testing.assert_array_equal(got, a_np + b_np, err_msg=f"{shape} {bshape}")


def test_empty_and_scalar(ops):
    e = torch.empty((0, 4), device="cuda")
    assert ops.add(e, e).shape == (0, 4)
    s = torch.tensor(3.0, device="cuda")
    assert ops.mul(s, s).item() == 9.0
    assert ops.relu(torch.tensor(-1.0, device="cuda")).item() == 0.0


def test_misaligned_and_ragged_flat(ops):
    x = torch.arange(1003, dtype=torch.float32, device="cuda")
    for off in (0, 1, 3):
        v = x[off:]
        np.testing.assert_array_equal(ops.add(v, v).cpu().numpy(), 2 * v.cpu().numpy())
    xb = torch.arange(517, dtype=torch.float32, device="cuda").bfloat16()
    assert torch.equal(ops.add(xb[1:], xb[1:]), xb[1:] + xb[1:])


def test_copy_contiguous(ops):
    x = torch.arange(2 * 3 * 5, dtype=torch.float32, device="cuda").reshape(2, 3, 5).permute(2, 0, 1)
    assert torch.equal(ops.contiguous(x), x.contiguous())
    xi = torch.arange(30, dtype=torch.int64, device="cuda").reshape(5, 6).t()
    assert torch.equal(ops.contiguous(xi), xi.contiguous())


def test_overlap_is_rejected(ops):
    x = torch.zeros(16, device="cuda")
    with pytest.raises(ValueError, match="overlap"):
        ops.add(x[:8], x[:8], out=torch.as_strided(x, (8,), (0,)))
    with pytest.raises(ValueError, match="partially overlaps"):
        ops.add(x[:8], x[:8], out=x[4:12])
    ops.add(x[:8], x[:8], out=x[:8])  # exact in-place is fine


def test_large_dim_over_2_31_elements_linearity(ops):
    """> 2^31 output elements in one call (64-bit offsets): a[65536,1] + b[1,32769] in bf16,
    checked on sampled positions and by a checksum that is linear in the inputs."""
    n0, n1 = 65536, 32769
    a = torch.arange(n0, device="cuda", dtype=torch.float32).remainder(7).bfloat16().reshape(n0, 1)
    b = torch.arange(n1, device="cuda", dtype=torch.float32).remainder(5).bfloat16().reshape(1, n1)
    out = ops.add(a, b)
    assert out.numel() > 2 ** 31
    for (i, j) in [(0, 0), (n0 - 1, n1 - 1), (40000, 32768), (65535, 1), (12345, 23456)]:
        assert out[i, j].item() == float((i % 7) + (j % 5))
    # row sums: sum_j (a_i + b_j) = n1*a_i + sum(b); exact in fp32 for these small integers
    rs = out[::4096].float().sum(1).cpu().numpy()
    ai = (np.arange(n0)[::4096] % 7).astype(np.float64)
    np.testing.assert_array_equal(rs, n1 * ai + float((np.arange(n1) % 5).sum()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.bool])
@pytest.mark.parametrize("shape", [(100, 70), (33, 1000), (16, 16), (4, 50, 37), (3, 2, 64, 48), (128, 192),
                                   (68, 132), (2, 260, 64), (520, 1032), (1028, 260)])
def test_transposed_operands_use_the_tiled_transpose_path(ops, port, dtype, shape):
    """contiguous() of a transposed view, an op between a tensor and its transpose, where()
    into a transposed output: inputs contiguous along another dim than the output."""
    rng = np.random.default_rng(41)
    if dtype == torch.bool:
        x = rng.integers(0, 2, shape).astype(np.uint8)
    else:
        x = rand_storage(rng, shape, dtype)
    t = from_np(x, dtype)
    xt = np.swapaxes(x, -1, -2)
    tt = t.transpose(-1, -2)
    got = to_np(ops.contiguous(tt))
    np.testing.assert_array_equal(got, np.ascontiguousarray(xt))
    if dtype in (torch.float32, torch.bfloat16, torch.int64):
        y = rand_storage(rng, xt.shape, dtype)
        ty = from_np(y, dtype)
        got = to_np(ops.add(ty, tt))                       # dense + transposed
        np.testing.assert_array_equal(got, port.binary("add", y, xt, CODE[dtype]))
        out = torch.empty(shape, dtype=dtype, device="cuda").transpose(-1, -2)
        cond = rng.integers(0, 2, xt.shape).astype(np.uint8)
        ops.where(from_np(cond, torch.bool), ty, tt, out=out)   # transposed output and operand
        np.testing.assert_array_equal(to_np(out), port.where(cond, y, xt, CODE[dtype]))
        # a transposed condition, two dense operands: one of them rides in the free staging slot
        c2 = rng.integers(0, 2, shape).astype(np.uint8)
        y2 = rand_storage(rng, xt.shape, dtype)
        got = to_np(ops.where(from_np(c2, torch.bool).transpose(-1, -2), ty, from_np(y2, dtype)))
        np.testing.assert_array_equal(got, port.where(np.swapaxes(c2, -1, -2), y, y2, CODE[dtype]))
        got = to_np(ops.mul(tt, ty))                        # transposed * dense, the other way round
        np.testing.assert_array_equal(got, port.binary("mul", xt, y, CODE[dtype]))
    if len(shape) == 2 and min(shape) >= 16:
        assert ops.ti_plan(torch.empty(xt.shape, dtype=dtype, device="cuda"), tt)[2] == 3


@pytest.mark.parametrize("cdt", [torch.complex64, torch.complex128])
def test_complex_add_mul_and_copy(ops, port, cdt):
    """Complex64 / Complex128 take vt::add, vt::mul (src/vbt/ops/cuda_elementwise.cu:162-190,
    :3169-3188) and strided copies; every other op rejects them.  Bit-exact against the oracle's
    separately rounded products: contiguous, broadcast, a transposed view, a ragged strided view."""
    rng = np.random.default_rng(61)
    ndt = np.complex64 if cdt == torch.complex64 else np.complex128
    mk = lambda shape: (rng.standard_normal(shape) + 1j * rng.standard_normal(shape)).astype(ndt)  # noqa: E731
    a, b = mk((37, 65)), mk((37, 65))
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    for name in ("add", "mul"):
        got = ops.binary(name, ta, tb).cpu().numpy()
        np.testing.assert_array_equal(got, port.complex_binary(name, a, b), err_msg=name)
        # broadcast row and column operands
        r, c = mk((1, 65)), mk((37, 1))
        got = ops.binary(name, torch.from_numpy(r).cuda(), torch.from_numpy(c).cuda()).cpu().numpy()
        np.testing.assert_array_equal(got, port.complex_binary(name, r, c), err_msg=name + " broadcast")
        # one operand transposed, output a strided slice of a larger buffer
        sq = mk((48, 48))
        tsq = torch.from_numpy(sq).cuda()
        big = torch.zeros((48, 100), dtype=cdt, device="cuda")
        ops.binary(name, tsq, tsq.t(), out=big[:, 3:99:2])
        np.testing.assert_array_equal(big[:, 3:99:2].cpu().numpy(), port.complex_binary(name, sq, sq.T), err_msg=name + " strided")
        assert not big[:, 4:99:2].any() and not big[:, :3].any()
    np.testing.assert_array_equal(ops.contiguous(ta.t()).cpu().numpy(), a.T)
    np.testing.assert_array_equal(ops.contiguous(ta[::3, 1::2]).cpu().numpy(), a[::3, 1::2])
    for name in ("sub", "div", "maximum", "eq"):
        with pytest.raises(ValueError, match="unsupported dtype"):
            ops.binary(name, ta, tb)
    with pytest.raises(ValueError, match="dtype mismatch"):
        ops.binary("add", ta, tb.to(torch.complex128 if cdt == torch.complex64 else torch.complex64))


@pytest.mark.parametrize("dtype", FLOATS)
def test_polygamma(ops, port, dtype):
    """vt::polygamma(n, x) (cuda_elementwise.cu:1288-1330, :3853-3876): order 2 against the
    oracle's restatement of the same recurrence + asymptotic series, NaN at poles and for every
    other order, the scalar-tensor rule for n, a strided x."""
    rng = np.random.default_rng(62)
    x = 6 * rng.standard_normal((33, 70), dtype=np.float32)
    x.flat[:10] = [1.0, 0.5, 2.0, 10.0, 25.0, 0.0, -1.0, -2.0, -0.5, -3.25]
    xs = oracle.to_storage(x, CODE[dtype])
    tx = from_np(xs, dtype)
    two = torch.tensor([2.0], device="cuda").to(dtype)
    got = to_np(ops.polygamma(two, tx))
    want = port.polygamma(2.0, xs, CODE[dtype])
    g, w = as_f32(got, dtype), as_f32(want, dtype)
    np.testing.assert_array_equal(np.isnan(g), np.isnan(w))
    fin = np.isfinite(w)
    if dtype == torch.float32:
        np.testing.assert_allclose(g[fin], w[fin], rtol=1e-6, atol=0)
        assert abs(g.flat[0] - (-2.4041138063)) < 1e-6     # psi''(1) = -2 zeta(3)
    else:
        np.testing.assert_array_equal(got[fin], want[fin])   # the double result rounds once to the storage type
    assert np.isnan(g.flat[5]) and np.isnan(g.flat[6]) and np.isnan(g.flat[7]) and np.isfinite(g.flat[8])
    for order in (0.0, 1.0, 3.0):
        n = torch.tensor([order], device="cuda").to(dtype)
        assert np.isnan(as_f32(to_np(ops.polygamma(n, tx)), dtype)).all()
    view = tx.t()[::2]
    got_v = to_np(ops.polygamma(two.reshape(1, 1), view))
    np.testing.assert_array_equal(got_v, np.ascontiguousarray(got.T[::2]))
    with pytest.raises(ValueError, match="expected n to be a scalar tensor"):
        ops.polygamma(torch.zeros(2, device="cuda").to(dtype), tx)
