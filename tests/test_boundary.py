"""The reference-facing boundary as built code: the plugin for the stable plugin C ABI
(boundary/vbt_b200_plugin.c) loaded by a test double of the plugin host (boundary/test_host.c),
and the in-tree binding (boundary/vbt_b200_glue.cc) compiled against the reference's headers.

Host-only tests: ABI handshake, registration table, the "vt::add is ignored" quirk, ops the host
has no schema for, status / message mapping, the output-shape rule, symbols of the glue object.
GPU tests: every registered kernel called through the host double and compared with the oracle.

The artefacts are built by boundary/build.sh where a reference checkout is present (its headers
are needed); the built files travel to machines without one.
"""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle
from tests.util import CODE, as_f32, from_np, to_np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "boundary", "_build")
PLUGIN = os.path.join(BUILD, "libvbt_b200_plugin.so")
HOST = os.path.join(BUILD, "libvbt_test_host.so")
GLUE = os.path.join(BUILD, "vbt_b200_glue.o")
OK, INVALID_ARG, UNSUPPORTED, NOT_FOUND, INTERNAL, ABI_MISMATCH = 0, 1, 2, 3, 4, 5
KDL_INT, KDL_FLOAT, KDL_BFLOAT, KDL_BOOL = 0, 2, 4, 6
DL = {torch.float32: (KDL_FLOAT, 32), torch.float16: (KDL_FLOAT, 16), torch.bfloat16: (KDL_BFLOAT, 16),
      torch.int64: (KDL_INT, 64), torch.int32: (KDL_INT, 32), torch.bool: (KDL_BOOL, 8)}

# plugin op name -> oracle op name, where they differ (aliases the reference registers on one functor)
ALIAS = {"celu": "elu", "conj_physical": "positive", "true_divide": "div", "clamp_min": "maximum",
         "clamp_max": "minimum", "float_power": "pow", "special_xlog1py": "xlog1py",
         "bitwise_left_shift": "lshift", "bitwise_right_shift": "rshift", "clip": "clamp"}
INT_OPS = {"bitwise_and", "bitwise_or", "bitwise_xor", "lshift", "rshift", "gcd", "lcm", "bitwise_not"}


def _ensure_built():
    ref = os.environ.get("VBT_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    have = all(os.path.exists(p) for p in (PLUGIN, HOST, GLUE))
    if os.path.isfile(os.path.join(ref, "include", "vbt", "plugin", "vbt_plugin.h")):
        srcs = [os.path.join(ROOT, "boundary", f) for f in ("vbt_b200_plugin.c", "test_host.c", "vbt_b200_glue.cc",
                                                            "build.sh")]
        stale = have and max(os.path.getmtime(s) for s in srcs) > min(os.path.getmtime(p) for p in (PLUGIN, HOST, GLUE))
        if not have or stale:
            subprocess.run(["bash", os.path.join(ROOT, "boundary", "build.sh"), ref], check=True,
                           stdout=subprocess.DEVNULL)
        return True
    return have


@pytest.fixture(scope="module")
def host():
    if not _ensure_built():
        pytest.skip("boundary/_build is not built and there is no reference checkout to build it against")
    h = ctypes.CDLL(HOST)
    h.th_last_error.restype = ctypes.c_char_p
    h.th_kernel_name.restype = ctypes.c_char_p
    h.th_load_plugin.argtypes = [ctypes.c_char_p, ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint32),
                                 ctypes.POINTER(ctypes.c_char_p)]
    h.th_make_tensor.restype = ctypes.c_void_p
    h.th_make_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    h.th_free_tensor.argtypes = [ctypes.c_void_p]
    h.th_tensor_data.restype = ctypes.c_void_p
    h.th_tensor_data.argtypes = [ctypes.c_void_p]
    h.th_tensor_ndim.argtypes = [ctypes.c_void_p]
    h.th_tensor_size.restype = ctypes.c_int64
    h.th_tensor_size.argtypes = [ctypes.c_void_p, ctypes.c_int]
    h.th_call.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                          ctypes.POINTER(ctypes.c_void_p)]
    h.th_set_schemas.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.c_int]
    h.th_set_stream.argtypes = [ctypes.c_uint64]
    h.th_plugin_symbol.restype = ctypes.c_void_p
    h.th_plugin_symbol.argtypes = [ctypes.c_char_p]
    return h


def _load(h, minor=4):
    abi = ctypes.c_uint32()
    name = ctypes.c_char_p()
    st = h.th_load_plugin(PLUGIN.encode(), minor, ctypes.byref(abi), ctypes.byref(name))
    return st, abi.value, name.value


def _names(h):
    return [h.th_kernel_name(i).decode() for i in range(h.th_num_kernels())]


ALLOC_FN = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int32)


class Tensors:
    """vt_tensor handles of the host double over torch (or fake) memory, freed on exit."""

    def __init__(self, h):
        self.h, self.handles, self.keep = h, [], []

    def make(self, data_ptr, dtype, shape, strides, device_type=2, device_id=0):
        code, bits = DL[dtype]
        nd = len(shape)
        sizes = (ctypes.c_int64 * max(nd, 1))(*shape)
        st = (ctypes.c_int64 * max(nd, 1))(*strides)
        t = self.h.th_make_tensor(ctypes.c_void_p(data_ptr), code, bits, device_type, device_id, nd, sizes, st)
        assert t
        self.handles.append(t)
        return t

    def of(self, t: torch.Tensor):
        self.keep.append(t)
        return self.make(t.data_ptr(), t.dtype, tuple(t.shape), tuple(t.stride()), 2, t.device.index or 0)

    def close(self):
        for t in self.handles:
            self.h.th_free_tensor(t)
        self.handles.clear()


def _call(h, name, handles):
    args = (ctypes.c_void_p * len(handles))(*handles)
    out = ctypes.c_void_p()
    st = h.th_call(name.encode(), args, len(handles), ctypes.byref(out))
    return st, out.value


# ------------------------------------------------------------------------------------------
# host-only
# ------------------------------------------------------------------------------------------
def test_abi_handshake_and_registration_table(host):
    st, abi, name = _load(host)
    assert st == OK, host.th_last_error()
    assert abi == (1 << 16) | 4                      # VBT_PLUGIN_ABI_ENCODE(1, 4)
    assert b"vbt_b200" in name
    names = _names(host)
    assert "vt::add" not in names and host.th_ignored_add() == 1   # the loader drops vt::add silently
    for must in ("vt::mul", "vt::sub", "vt::div", "vt::relu", "vt::neg", "vt::abs", "vt::reciprocal", "vt::where",
                 "vt::clamp", "vt::addcmul", "vt::maximum", "vt::pow", "vt::bitwise_and", "vt::masked_fill"):
        assert must in names, must
    # comparisons / predicates need a BOOL output the host cannot allocate "like" an input
    for absent in ("vt::eq", "vt::gt", "vt::isnan", "vt::logical_and", "vt::sum"):
        assert absent not in names
    assert len(names) == len(set(names)) >= 100
    reg = ctypes.CFUNCTYPE(ctypes.c_int)(host.th_plugin_symbol(b"vbt_b200_plugin_registered"))
    assert reg() == len(names) + 1                   # + the ignored vt::add
    # arity: binary ops arrive as vt_kernel2_fn, the others boxed
    ar = {host.th_kernel_name(i).decode(): host.th_kernel_arity(i) for i in range(host.th_num_kernels())}
    assert ar["vt::mul"] == 2 and ar["vt::relu"] == -1 and ar["vt::where"] == -1


def test_plugin_minor_newer_than_host_is_an_abi_mismatch(host):
    st, abi, _ = _load(host, minor=3)
    assert st == ABI_MISMATCH and abi == (1 << 16) | 4
    assert host.th_num_kernels() == 0
    assert _load(host, minor=5)[0] == OK             # an older plugin on a newer host loads


def test_ops_without_a_schema_are_skipped_not_fatal(host):
    """The dispatcher only knows the ops its build defines (the default build: relu, add, mul, sub,
    div, abs, neg, reciprocal, ...; src/vbt/ops/default_kernels.cc:1046-1110)."""
    have = [b"vt::relu", b"vt::add", b"vt::mul", b"vt::sub", b"vt::div", b"vt::abs", b"vt::neg", b"vt::reciprocal"]
    arr = (ctypes.c_char_p * len(have))(*have)
    host.th_set_schemas(arr, len(have))
    try:
        st, _, _ = _load(host)
        assert st == OK, host.th_last_error()
        assert sorted(_names(host)) == sorted(n.decode() for n in have if n != b"vt::add")
        skipped = ctypes.CFUNCTYPE(ctypes.c_int)(host.th_plugin_symbol(b"vbt_b200_plugin_skipped"))
        assert skipped() > 90
    finally:
        host.th_set_schemas(None, 0)


def test_status_and_message_mapping_without_a_gpu(host):
    """Validation failures come back as a vt_status with the library's message in the host's
    thread-local error slot, before anything is launched; the host drops the output the kernel
    had created.  Pointers here are fake: no kernel runs."""
    assert _load(host)[0] == OK
    fake = np.zeros(4096, np.uint8)
    allocs = []

    @ALLOC_FN
    def alloc(nbytes, device):
        allocs.append(nbytes)
        return fake.ctypes.data

    host.th_set_allocator(alloc)
    ts = Tensors(host)
    try:
        a = ts.make(fake.ctypes.data, torch.float32, (3, 4), (4, 1))
        b64 = ts.make(fake.ctypes.data, torch.int64, (3, 4), (4, 1))
        st, out = _call(host, "vt::mul", [a, b64])
        assert st == INVALID_ARG and out is None
        assert b"vt::mul: dtype mismatch" in host.th_last_error()
        assert allocs == [48]                               # the output was allocated like `a`, then dropped
        # integer division is rejected as in the reference (cuda_elementwise.cu:2889-2891)
        st, _ = _call(host, "vt::div", [b64, b64])
        assert st == INVALID_ARG and b"vt::div" in host.th_last_error()
        # result shape [3,4] from [3,1] x [1,4]: like neither input -> the host cannot allocate it
        c = ts.make(fake.ctypes.data, torch.float32, (3, 1), (1, 1))
        d = ts.make(fake.ctypes.data, torch.float32, (1, 4), (4, 1))
        st, _ = _call(host, "vt::mul", [c, d])
        assert st == UNSUPPORTED and b"allocate an output like an input" in host.th_last_error()
        # shapes that do not broadcast
        e = ts.make(fake.ctypes.data, torch.float32, (5,), (1,))
        st, _ = _call(host, "vt::sub", [a, e])
        assert st == INVALID_ARG and b"broadcast" in host.th_last_error()
        # CPU tensors are refused; wrong arity through the boxed entry
        cpu = ts.make(fake.ctypes.data, torch.float32, (3, 4), (4, 1), device_type=1)
        st, _ = _call(host, "vt::relu", [cpu])
        assert st == INVALID_ARG and b"CUDA" in host.th_last_error()
        st, _ = _call(host, "vt::relu", [a, a])
        assert st == INVALID_ARG
        st, _ = _call(host, "vt::nosuch", [a])
        assert st == NOT_FOUND
        # a zero-element op succeeds without a launch and returns an output like its input
        z = ts.make(0, torch.float32, (0, 4), (4, 1))
        st, out = _call(host, "vt::neg", [z])
        assert st == OK and out is not None and host.th_tensor_ndim(out) == 2
        host.th_free_tensor(out)
    finally:
        ts.close()
        host.th_set_allocator(ALLOC_FN(0))


def test_glue_object_defines_the_reference_symbols():
    if not _ensure_built():
        pytest.skip("boundary/_build is not built")
    out = subprocess.run(["nm", "-g", "--defined-only", GLUE], capture_output=True, text=True, check=True).stdout
    syms = {line.split()[-1] for line in out.splitlines() if line.strip()}
    for s in ("vbt_cuda_add_impl", "vbt_cuda_mul_impl", "vbt_cuda_gt_impl", "vbt_cuda_relu_impl", "vbt_cuda_where_impl",
              "vbt_cuda_masked_fill_impl", "vbt_cuda_clamp_impl", "vbt_cuda_addcmul_impl", "vbt_cuda_isnan_impl",
              "vbt_cuda_sum_impl", "vbt_cuda_prod_impl", "vbt_cuda_min_impl", "vbt_cuda_max_impl", "vbt_cuda_mean_impl",
              "vbt_register_cuda_elementwise_kernels"):
        assert s in syms, s
    assert len([s for s in syms if s.startswith("vbt_cuda_") and s.endswith("_impl")]) >= 120
    # everything it needs from this repository is the C ABI
    und = subprocess.run(["nm", "-g", "--undefined-only", GLUE], capture_output=True, text=True, check=True).stdout
    used = {line.split()[-1] for line in und.splitlines() if "vbt_b200_" in line}
    assert {"vbt_b200_binary", "vbt_b200_unary", "vbt_b200_ternary", "vbt_b200_where", "vbt_b200_reduce",
            "vbt_b200_reduce_shape", "vbt_b200_reduce_workspace_bytes", "vbt_b200_broadcast_shape",
            "vbt_b200_binary_scalar", "vbt_b200_last_error"} <= used


# ------------------------------------------------------------------------------------------
# GPU: every registered kernel through the host double, against the oracle
# ------------------------------------------------------------------------------------------
def _compare(name, got_np, want_np, dtype):
    if dtype in (torch.int64, torch.int32, torch.bool):
        np.testing.assert_array_equal(got_np, want_np, err_msg=name)
        return
    g, w = as_f32(got_np, dtype), as_f32(want_np, dtype)
    np.testing.assert_array_equal(np.isnan(g), np.isnan(w), err_msg=name)
    fin = np.isfinite(w)
    np.testing.assert_array_equal(g[~fin & ~np.isnan(w)], w[~fin & ~np.isnan(w)], err_msg=name)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    np.testing.assert_allclose(g[fin], w[fin], rtol=tol, atol=1e-6 if dtype == torch.float32 else tol, err_msg=name)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_every_registered_kernel_against_the_oracle(host, port, dtype):
    assert _load(host)[0] == OK
    keep = []

    @ALLOC_FN
    def alloc(nbytes, device):
        buf = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{device}")
        keep.append(buf)
        return buf.data_ptr()

    host.th_set_allocator(alloc)
    host.th_set_stream(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(41)
    shape = (33, 130)
    code = CODE[dtype]

    def fl(lo=0.1, hi=0.9):
        return oracle.to_storage((lo + (hi - lo) * rng.random(shape)).astype(np.float32), code)

    ts = Tensors(host)
    checked = 0
    try:
        for i in range(host.th_num_kernels()):
            fq = host.th_kernel_name(i).decode()
            name = ALIAS.get(fq[4:], fq[4:])
            arity = 1 if name in oracle.UNARY else 2 if name in oracle.BINARY else 3
            op_dtype = dtype
            if name in INT_OPS:
                if dtype != torch.float32:
                    continue
                op_dtype = torch.int64
                ins = [rng.integers(0 if name in ("lshift", "rshift") else -1000, 40 if name in ("lshift", "rshift")
                                    else 1000, shape).astype(np.int64) for _ in range(arity)]
            elif name == "where" or name == "masked_fill":
                ins = None
            elif name == "polygamma":
                ins = "polygamma"
            elif name == "nan_to_num" and dtype != torch.float32:
                continue
            elif name == "acosh":
                ins = [fl(1.1, 3.0)]
            elif name == "ldexp":
                ins = [fl(), oracle.to_storage(rng.integers(-3, 4, shape).astype(np.float32), code)]
            elif name == "clamp":
                ins = [fl(0.0, 1.0), fl(0.2, 0.4), fl(0.6, 0.8)]
            else:
                ins = [fl() for _ in range(arity)]
                # the second operand of a binary op broadcasts INTO the first one's shape
                if arity == 2:
                    ins[1] = np.ascontiguousarray(ins[1][:1])
            if ins is None:
                cond = (rng.random(shape) < 0.5).astype(np.uint8)
                x, y = fl(), fl()
                tc, tx, ty = from_np(cond, torch.bool), from_np(x, dtype), from_np(y, dtype)
                if name == "where":
                    st, out = _call(host, fq, [ts.of(tc), ts.of(tx), ts.of(ty)])
                    want = port.where(cond, x, y, code)
                else:
                    st, out = _call(host, fq, [ts.of(tx), ts.of(tc), ts.of(ty)])   # (self, mask, value)
                    want = port.where(cond, y, x, code)
            elif ins == "polygamma":   # (n, x): n a one-element tensor, the result is like x
                x = oracle.to_storage((8 * rng.random(shape) - 2).astype(np.float32), code)
                two = oracle.to_storage(np.array([2.0], np.float32), code)
                tens = [from_np(two, dtype), from_np(x, dtype)]
                st, out = _call(host, fq, [ts.of(t) for t in tens])
                want = port.polygamma(2.0, x, code)
            else:
                tens = [from_np(a, op_dtype) for a in ins]
                st, out = _call(host, fq, [ts.of(t) for t in tens])
                c = CODE[op_dtype]
                want = (port.unary(name, ins[0], c) if arity == 1 else
                        port.binary(name, ins[0], ins[1], c) if arity == 2 else
                        port.ternary(name, ins[0], ins[1], ins[2], c))
            assert st == OK, (fq, host.th_last_error())
            assert [host.th_tensor_size(out, d) for d in range(host.th_tensor_ndim(out))] == list(shape), fq
            torch.cuda.synchronize()
            nbytes = int(np.prod(shape)) * torch.empty((), dtype=op_dtype).element_size()
            raw = next(b for b in keep if b.data_ptr() == host.th_tensor_data(out))
            got = to_np(raw[:nbytes].view(op_dtype).reshape(shape))
            _compare(fq, got, want.reshape(shape), op_dtype)
            host.th_free_tensor(out)
            checked += 1
    finally:
        ts.close()
        host.th_set_allocator(ALLOC_FN(0))
    assert checked >= (100 if dtype == torch.float32 else 90)
