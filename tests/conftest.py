"""Shared pytest configuration: the `gpu` marker, package loading and a per-session GPU context."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN = REPO / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def ctx(pkg):
    """One library context on cuda:0 for the whole session. Fails (never skips) when the CUDA library
    cannot be used: GPU tests must not pass on a fallback."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    c = pkg.Context(0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def stream():
    """A non-default torch stream; its raw handle is what the C ABI receives."""
    import torch
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    return st
