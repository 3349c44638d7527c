"""CPU-only checks of the C ABI: the library loads, exports every declared symbol, and its
host-side logic (iteration planner, shape inference, argument validation, error text)
behaves like the reference's TensorIterator / dispatch helpers.  No kernel is launched."""
import ctypes
import os
import re

import pytest
import torch

from vibetensor_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    if not os.path.exists(_lib.LIB_PATH):
        from vibetensor_b200 import build
        build.build()
    return _lib.lib()


def fake(shape, strides, dtype=_lib.F32, ptr=0x10000):
    """A descriptor with a made-up device address: enough for host-side planning."""
    t = _lib.VbtTensor()
    keep = ((ctypes.c_int64 * max(len(shape), 1))(*shape), (ctypes.c_int64 * max(len(shape), 1))(*strides))
    t.data, t.dtype, t.ndim, t.sizes, t.strides = ptr, dtype, len(shape), keep[0], keep[1]
    t._keep = keep
    return t


def dense(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return list(reversed(st))


def plan(L, *tensors):
    arr = (ctypes.POINTER(_lib.VbtTensor) * len(tensors))(*[ctypes.pointer(t) for t in tensors])
    shape = (ctypes.c_int64 * 25)()
    strides = (ctypes.c_int64 * (25 * len(tensors)))()
    nd, kern, pieces = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    rc = L.vbt_b200_ti_plan(arr, len(tensors), shape, strides, ctypes.byref(nd), ctypes.byref(kern),
                            ctypes.byref(pieces))
    if rc:
        raise ValueError(L.vbt_b200_last_error().decode())
    n = nd.value
    return list(shape[:n]), [list(strides[k * 25:k * 25 + n]) for k in range(len(tensors))], kern.value


def test_every_declared_symbol_is_exported(L):
    hdr = open(os.path.join(ROOT, "include", "vbt_b200.h")).read()
    declared = set(re.findall(r"VBT_B200_API\s+[\w\s\*]+?\b(vbt_b200_\w+)\s*\(", hdr))
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(L, name), f"{name} declared in include/vbt_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert L.vbt_b200_compiled_arch() == 100


def test_plan_config3_orders_dims_by_output_stride(L):
    # out = base[64,1024,512,128].transpose(1,3): sizes [64,128,512,1024]
    out = fake([64, 128, 512, 1024], [67108864, 1, 128, 65536], _lib.BF16)
    a = fake([64, 1, 512, 1], [512, 512, 1, 1], _lib.BF16, 1 << 40)
    b = fake([1, 128, 1, 1024], [131072, 1024, 1024, 1], _lib.BF16, 2 << 40)
    c = fake([64, 128, 1, 1024], [131072, 1024, 1024, 1], _lib.BF16, 3 << 40)
    shape, strides, kern = plan(L, out, a, b, c)
    assert shape == [128, 512, 1024, 64]            # d1, d2, d3, n0: output memory order
    assert strides[0] == [1, 128, 65536, 67108864]
    assert strides[1] == [0, 1, 0, 512]             # a varies with d2 and n0 only
    assert strides[2] == [1024, 0, 1, 0]
    assert strides[3] == [1024, 0, 1, 131072]
    assert kern == 1                                # vector kernel along the output's inner dim


def test_plan_coalesces_and_drops_size1(L):
    out = fake([4, 1, 8, 16], dense([4, 1, 8, 16]))
    a = fake([4, 1, 8, 16], dense([4, 1, 8, 16]), ptr=0x20000)
    shape, strides, kern = plan(L, out, a)
    assert shape == [512] and strides == [[1], [1]] and kern == 0
    b = fake([16], [1], ptr=0x30000)                # broadcast over the leading dims
    shape, strides, kern = plan(L, out, a, b)
    assert shape == [16, 32] and strides[2] == [1, 0] and kern == 1
    s = fake([], [], ptr=0x30000)                   # 0-d operand
    shape, strides, kern = plan(L, out, a, s)
    assert shape == [512] and strides[2] == [0] and kern == 0


def test_plan_matches_reference_broadcast_offsets(L, port):
    # tests/cpp/tensor_iter_cuda_meta_test.cc:353-400: out/a [2,256], b [256]
    out = fake([2, 256], [256, 1])
    a = fake([2, 256], [256, 1], ptr=0x20000)
    b = fake([256], [1], ptr=0x30000)
    shape, strides, _ = plan(L, out, a, b)
    for li in range(512):
        r, c = divmod(li, 256)
        assert port.offset_elems(li, shape, strides[1]) == r * 256 + c
        assert port.offset_elems(li, shape, strides[2]) == c


def test_plan_negative_and_permuted_output(L):
    out = fake([3, 5], [-5, 1], ptr=0x10000 + 4 * 10)   # rows walked backwards
    a = fake([3, 5], [5, 1], ptr=0x20000)
    shape, strides, _ = plan(L, out, a)
    assert shape == [5, 3] and strides[0] == [1, 5] and strides[1] == [1, -5]
    out = fake([3, 5], [1, 3])                           # column-major output
    shape, strides, _ = plan(L, out, a)
    assert shape == [3, 5] and strides[0] == [1, 3] and strides[1] == [5, 1]


def test_plan_errors(L):
    with pytest.raises(ValueError, match="25D"):
        plan(L, fake([1] * 26, [1] * 26), fake([1] * 26, [1] * 26))
    with pytest.raises(ValueError, match="cannot be broadcast"):
        plan(L, fake([4], [1]), fake([3], [1]), fake([4], [1]))
    with pytest.raises(ValueError, match="internal overlap"):
        plan(L, fake([4, 4], [1, 1]), fake([4, 4], [4, 1], ptr=0x90000))
    with pytest.raises(ValueError, match="partially overlaps"):
        plan(L, fake([8], [1], ptr=0x10010), fake([8], [1], ptr=0x10000))


def test_status_codes_and_messages_without_a_gpu(L):
    a, b = fake([4], [1]), fake([4], [1], _lib.BF16)
    assert L.vbt_b200_binary(0, ctypes.byref(a), ctypes.byref(a), ctypes.byref(b), None) == 1
    assert L.vbt_b200_last_error() == b"vt::add: dtype mismatch"
    i64 = fake([4], [1], _lib.I64)
    assert L.vbt_b200_binary(3, ctypes.byref(i64), ctypes.byref(i64), ctypes.byref(i64), None) == 1
    assert L.vbt_b200_unary(4, ctypes.byref(i64), ctypes.byref(i64), None) == 1
    assert b"floating tensor expected" in L.vbt_b200_last_error()
    assert L.vbt_b200_unary(99, ctypes.byref(a), ctypes.byref(a), None) == 1
    cond = fake([4], [1], _lib.F32)
    assert L.vbt_b200_where(ctypes.byref(a), ctypes.byref(cond), ctypes.byref(a), ctypes.byref(a), None) == 1
    # reductions
    x = fake([3, 0], [1, 1])
    o = fake([3], [1])
    assert L.vbt_b200_reduce(2, ctypes.byref(o), None, ctypes.byref(x), _lib.i64_array([1]), 1, 0, None, 0, None) == 2
    assert L.vbt_b200_last_error() == b"amax: empty"
    xi = fake([3, 4], [4, 1], _lib.I64)
    assert L.vbt_b200_reduce(1, ctypes.byref(o), None, ctypes.byref(xi), _lib.i64_array([1]), 1, 0, None, 0, None) == 1
    assert L.vbt_b200_last_error() == b"mean: expected dtype=float32"
    x2 = fake([3, 4], [4, 1])
    assert L.vbt_b200_reduce(0, ctypes.byref(o), None, ctypes.byref(x2), _lib.i64_array([5]), 1, 0, None, 0, None) == 1
    assert L.vbt_b200_last_error() == b"sum: dim out of range"
    # indexing
    idxf = fake([2], [1], _lib.F32)
    tab = fake([4, 3], [3, 1])
    out = fake([2, 3], [3, 1])
    assert L.vbt_b200_index_rows(ctypes.byref(out), ctypes.byref(tab), ctypes.byref(idxf), 0, None, None) == 1
    assert b"Int32 and Int64" in L.vbt_b200_last_error()


def test_reduce_shape_and_workspace(L):
    x = fake([5, 7, 9], dense([5, 7, 9]))
    out = (ctypes.c_int64 * 25)()
    nd = ctypes.c_int32()
    assert L.vbt_b200_reduce_shape(ctypes.byref(x), _lib.i64_array([1]), 1, 0, out, ctypes.byref(nd)) == 0
    assert list(out[:nd.value]) == [5, 9]
    assert L.vbt_b200_reduce_shape(ctypes.byref(x), _lib.i64_array([-1, 0]), 2, 1, out, ctypes.byref(nd)) == 0
    assert list(out[:nd.value]) == [1, 7, 1]
    assert L.vbt_b200_reduce_shape(ctypes.byref(x), _lib.i64_array([]), 0, 0, out, ctypes.byref(nd)) == 0
    assert nd.value == 0
    # [2^32] -> scalar needs partials + a ticket; [4096,4096] sum(-1) needs nothing
    big = fake([1 << 32], [1])
    assert L.vbt_b200_reduce_workspace_bytes(0, ctypes.byref(big), _lib.i64_array([]), 0) > 0
    sq = fake([4096, 4096], [4096, 1])
    assert L.vbt_b200_reduce_workspace_bytes(0, ctypes.byref(sq), _lib.i64_array([1]), 1) == 0
    assert L.vbt_b200_reduce_workspace_bytes(1, ctypes.byref(sq), _lib.i64_array([0]), 1) > 0
    col = fake([1 << 20, 4096], [4096, 1], _lib.BF16)
    assert L.vbt_b200_reduce_workspace_bytes(0, ctypes.byref(col), _lib.i64_array([0]), 1) > 0


def test_broadcast_shape(L):
    a, b = fake([64, 1, 512, 1], [512, 512, 1, 1]), fake([128, 1, 1024], [1024, 1024, 1])
    arr = (ctypes.POINTER(_lib.VbtTensor) * 2)(ctypes.pointer(a), ctypes.pointer(b))
    out = (ctypes.c_int64 * 25)()
    nd = ctypes.c_int32()
    assert L.vbt_b200_broadcast_shape(arr, 2, out, ctypes.byref(nd)) == 0
    assert list(out[:nd.value]) == [64, 128, 512, 1024]


def test_product_has_no_cpu_path():
    from vibetensor_b200 import kernels, ops
    with pytest.raises(ValueError, match="no CPU path"):
        ops.add(torch.ones(3), torch.ones(3))
    with pytest.raises(RuntimeError, match="CUDA"):
        kernels.softmax(torch.ones(3, 3))
    src = open(os.path.join(ROOT, "vibetensor_b200", "ops.py")).read() + \
        open(os.path.join(ROOT, "vibetensor_b200", "kernels.py")).read() + \
        open(os.path.join(ROOT, "vibetensor_b200", "fabric.py")).read()
    assert "oracle" not in src


def test_null_data_and_bad_policy_are_rejected_before_any_launch(L):
    """A descriptor with elements but no data pointer (a failed or empty allocation passed through
    a binding) must come back as INVALID_ARGUMENT from every family -- a kernel given a null base
    would fault on the device -- and so must an unknown index policy."""
    null = lambda shape, dt=_lib.F32: fake(shape, dense(shape), dt, ptr=0)  # noqa: E731
    x, o = fake([3, 4], [4, 1]), fake([3], [1])
    da = _lib.i64_array([1])
    for args in ((ctypes.byref(null([3])), None, ctypes.byref(x)), (ctypes.byref(o), None, ctypes.byref(null([3, 4])))):
        assert L.vbt_b200_reduce(0, args[0], args[1], args[2], da, 1, 0, None, 0, None) == 1
        assert b"null data pointer" in L.vbt_b200_last_error()
    assert L.vbt_b200_reduce_noalloc(0, ctypes.byref(null([3])), None, ctypes.byref(x), da, 1, 0, None) == 1
    assert L.vbt_b200_reduce_partial(0, ctypes.byref(o), ctypes.byref(null([3, 4])), da, 1, 0, None, 0, 0, None) == 1
    oi = fake([3], [1], _lib.I64)
    assert L.vbt_b200_reduce(5, ctypes.byref(o), ctypes.byref(null([3], _lib.I64)), ctypes.byref(x), da, 1, 0, None, 0,
                             None) == 1
    assert L.vbt_b200_reduce(5, ctypes.byref(o), ctypes.byref(oi), ctypes.byref(null([3, 4])), da, 1, 0, None, 0, None) == 1
    # zero elements need no pointer
    e, eo = null([0, 4]), null([0])
    assert L.vbt_b200_reduce(0, ctypes.byref(eo), None, ctypes.byref(e), da, 1, 0, None, 0, None) == 0
    tab, idx, out = fake([4, 3], [3, 1]), fake([2], [1], _lib.I64), fake([2, 3], [3, 1])
    for t_, i_, o_ in ((null([4, 3]), idx, out), (tab, null([2], _lib.I64), out), (tab, idx, null([2, 3]))):
        assert L.vbt_b200_index_rows(ctypes.byref(o_), ctypes.byref(t_), ctypes.byref(i_), 0, None, None) == 1
        assert b"null data pointer" in L.vbt_b200_last_error()
        assert L.vbt_b200_index_put_rows(ctypes.byref(t_), ctypes.byref(i_), ctypes.byref(o_), 1, 0, None, None) == 1
        assert L.vbt_b200_index_put_rows_sorted(ctypes.byref(t_), ctypes.byref(i_), ctypes.byref(o_), 0, None, None, 0,
                                                None) == 1
    src, od = fake([5, 4], [4, 1]), fake([5, 2], [2, 1])
    for s_, i_, o_ in ((null([5, 4]), idx, od), (src, null([2], _lib.I64), od), (src, idx, null([5, 2]))):
        assert L.vbt_b200_index_lastdim(ctypes.byref(o_), ctypes.byref(s_), ctypes.byref(i_), 0, None, None) == 1
        assert b"null data pointer" in L.vbt_b200_last_error()
    for pol in (-1, 3, 99):
        assert L.vbt_b200_index_lastdim(ctypes.byref(od), ctypes.byref(src), ctypes.byref(idx), pol, None, None) == 1
        assert b"unknown index policy" in L.vbt_b200_last_error()
        assert L.vbt_b200_index_put_lastdim(ctypes.byref(src), ctypes.byref(idx), ctypes.byref(od), 0, pol, None, None) == 1
        assert L.vbt_b200_index_rows(ctypes.byref(out), ctypes.byref(tab), ctypes.byref(idx), pol, None, None) == 1
    # a mask descriptor without sizes is rejected on the host, not dereferenced
    bad_mask = _lib.VbtTensor()
    bad_mask.data, bad_mask.dtype, bad_mask.ndim = 0x10000, _lib.BOOL, 1
    cnt = ctypes.c_uint64()
    assert L.vbt_b200_mask_select(ctypes.byref(bad_mask), None, 0, ctypes.byref(cnt), None, 0, None) == 1
    # fabric: shape / dtype rules come first and carry the reference's prefix
    a, b = fake([4, 4], [4, 1]), fake([4, 5], [5, 1])
    mode = ctypes.c_int32()
    assert L.vbt_b200_fabric_binary(0, ctypes.byref(a), ctypes.byref(a), ctypes.byref(b), 0, 0, 1, None, 0,
                                    ctypes.byref(mode), None) == 2
    assert L.vbt_b200_last_error() == b"[Fabric] vt::fabric_add: requires equal shapes"
    c = fake([4, 4], [4, 1], _lib.BF16)
    assert L.vbt_b200_fabric_binary(2, ctypes.byref(a), ctypes.byref(a), ctypes.byref(c), 0, 0, 1, None, 0,
                                    ctypes.byref(mode), None) == 2
    assert L.vbt_b200_last_error() == b"[Fabric] vt::fabric_mul: requires equal dtypes"


def test_launch_info_and_counters_are_host_side_state(L):
    info = _lib.LaunchInfo()
    L.vbt_b200_reset_last_launch_info()
    assert L.vbt_b200_last_launch_info(ctypes.byref(info)) == 0
    assert info.family == 0 and info.launches == 0
    L.vbt_b200_reset_launch_counts()
    assert _lib.launch_counts() == {name: 0 for name in _lib.FAMILIES}
    assert L.vbt_b200_last_launch_info(None) == 1


def test_polygamma_and_complex_argument_rules_without_a_gpu(L):
    """vt::polygamma's argument checks carry the reference's messages
    (src/vbt/ops/cuda_elementwise.cu:3853-3872); complex tensors are taken by vt::add / vt::mul
    only (:3169-3188) -- everything is decided before a launch."""
    x, o = fake([3, 4], [4, 1]), fake([3, 4], [4, 1])
    n1, n2 = fake([1], [1]), fake([2], [1])
    assert L.vbt_b200_polygamma(ctypes.byref(o), ctypes.byref(n2), ctypes.byref(x), None) == 1
    assert b"vt::polygamma: expected n to be a scalar tensor" in L.vbt_b200_last_error()
    ni = fake([1], [1], _lib.I64)
    assert L.vbt_b200_polygamma(ctypes.byref(o), ctypes.byref(ni), ctypes.byref(x), None) == 1
    assert b"vt::polygamma: expected n to have floating dtype" in L.vbt_b200_last_error()
    nh = fake([1], [1], _lib.F16)
    assert L.vbt_b200_polygamma(ctypes.byref(o), ctypes.byref(nh), ctypes.byref(x), None) == 1
    assert b"vt::polygamma: dtype mismatch" in L.vbt_b200_last_error()
    assert L.vbt_b200_polygamma(ctypes.byref(o), None, ctypes.byref(x), None) == 1
    e = fake([0, 4], [4, 1])
    assert L.vbt_b200_polygamma(ctypes.byref(e), ctypes.byref(n1), ctypes.byref(e), None) == 0  # nothing to do
    ca, co = fake([3, 4], [4, 1], _lib.C64), fake([3, 4], [4, 1], _lib.C64)
    for op in range(_lib.lib().vbt_b200_binary_op_count() if hasattr(_lib.lib(), "vbt_b200_binary_op_count") else 14):
        if op in (0, 2):
            continue
        assert L.vbt_b200_binary(op, ctypes.byref(co), ctypes.byref(ca), ctypes.byref(ca), None) == 1, op
        assert b"unsupported dtype" in L.vbt_b200_last_error()
    cb = fake([3, 4], [4, 1], _lib.C128)
    assert L.vbt_b200_binary(0, ctypes.byref(co), ctypes.byref(ca), ctypes.byref(cb), None) == 1
    assert b"vt::add: dtype mismatch" in L.vbt_b200_last_error()
    assert L.vbt_b200_binary(2, ctypes.byref(cb), ctypes.byref(ca), ctypes.byref(ca), None) == 1
    assert b"vt::mul: output dtype mismatch" in L.vbt_b200_last_error()
    assert L.vbt_b200_unary(0, ctypes.byref(co), ctypes.byref(ca), None) == 1   # no complex unary ops


def test_scatter_add_engine_choice_follows_the_measured_crossovers():
    """ops.index_put_rows_(accumulate=True, deterministic=None): integer tables group from 2^19
    updates on, float32 from 2^21, 16-bit tables never (the grouping kernels do not take them)."""
    import torch
    from vibetensor_b200 import ops
    assert not ops.grouping_engine_pays(torch.int64, (1 << 19) - 1)
    assert ops.grouping_engine_pays(torch.int64, 1 << 19) and ops.grouping_engine_pays(torch.int32, 1 << 22)
    assert not ops.grouping_engine_pays(torch.float32, 1 << 20)
    assert ops.grouping_engine_pays(torch.float32, 1 << 21)
    assert not ops.grouping_engine_pays(torch.bfloat16, 1 << 24) and not ops.grouping_engine_pays(torch.float16, 1 << 24)
