"""Shared fixtures.  Tests that need a B200 carry @pytest.mark.gpu; everything else runs on
CPU (oracle pins, host planning logic, symbol export, gloo multi-rank logic)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device in this container")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    import oracle
    if not oracle.have_ref():
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    return oracle.ref()


def pytest_terminal_summary(terminalreporter):
    """Worst observed error of every tolerance check that recorded one (error / scale, bound)."""
    try:
        from tests.util import WORST
    except Exception:  # pragma: no cover
        return
    if not WORST:
        return
    terminalreporter.write_line("worst observed error / scale per tolerance check (bound):")
    for label in sorted(WORST):
        err, bound = WORST[label]
        terminalreporter.write_line(f"  {label}: {err:.3e} ({bound:.0e})")
