"""vibetensor_b200: the vt:: data-parallel op path of VibeTensor on B200 (sm_100a).

``ops``      elementwise / broadcast, dim reductions, indexing (vt:: operator surface)
``kernels``  softmax, log_softmax, rmsnorm, gather, scatter_add (vibe_kernels surface)
``fabric``   row-sharded tensors across ranks: local kernels + NCCL combine

All compute runs in libvbt_b200.so through its C ABI (include/vbt_b200.h); importing a
submodule that computes fails loudly if that library has not been built.
"""
from . import _lib  # noqa: F401

__all__ = ["ops", "kernels", "fabric", "build"]
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("ops", "kernels", "fabric", "build"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
