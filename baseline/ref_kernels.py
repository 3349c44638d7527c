"""Loader for the reference's own torch-tensor Triton kernels (baseline/_ref, installed by
baseline/install_ref.sh).  Not part of the product: used to generate golden vectors and to
time the reference's kernels beside ours.

The reference's ``vibe_kernels.common.alloc`` imports ``vibetensor._C`` (its compiled core, which
cannot be built without its third-party submodules) at module load, but only touches it for
VibeTensor tensors; torch tensors go through ``Tensor.new_empty``.  An empty stand-in module
named ``vibetensor`` is therefore enough to run the reference's kernels, unmodified, on torch
tensors.
"""
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.isdir(os.path.join(REF_ROOT, "vibe_kernels"))


def load():
    """Returns a namespace with softmax, log_softmax, rmsnorm_fn (the autograd Function),
    gather, scatter_add -- the reference's torch-tensor entry points
    (vibe_kernels/softmax/impl/triton_impl.py:212-225, rmsnorm/impl/triton_impl.py:176-280,
    indexing/kernel.py:109-410)."""
    if not available():
        raise RuntimeError("baseline/_ref/vibe_kernels is missing: run baseline/install_ref.sh <reference checkout>")
    if "vibetensor" not in sys.modules:
        stub = types.ModuleType("vibetensor")
        stub._C = types.SimpleNamespace()
        stub.__path__ = []
        sys.modules["vibetensor"] = stub
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    from vibe_kernels.indexing import kernel as ik
    from vibe_kernels.rmsnorm.impl import triton_impl as rn
    from vibe_kernels.softmax.impl import triton_impl as sm
    return types.SimpleNamespace(softmax=sm.softmax, log_softmax=sm.log_softmax, rmsnorm_fn=rn._RMSNormFn,
                                 gather=ik.gather, scatter_add=ik.scatter_add)
