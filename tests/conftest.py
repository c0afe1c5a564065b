import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def engine():
    """One engine handle on cuda:0 for the whole session."""
    from sddmm_gpu_b200 import api
    h = api.Handle(0)
    yield h
    h.close()


def pytest_terminal_summary(terminalreporter):
    """How the checked nonzeros split by conditioning (see tests/helpers.py)."""
    try:
        from helpers import parity_stats as st
    except Exception:
        return
    if st["checked"]:
        terminalreporter.write_line(
            f"parity: {st['checked']} nonzeros checked against the oracle; {st['well_conditioned']} well-conditioned "
            f"(plain 1e-4 relative asserted), {st['between_1e-3_and_1e-2']} with 1e-3 A <= |ref| < 1e-2 A and "
            f"{st['below_1e-3']} below 1e-3 A (magnitude-scaled bound only)")
