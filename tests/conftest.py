"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; everything
else runs on a CPU-only machine."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def dev(pkg):
    """The sm_100a device behind the C ABI.  Fails (does not skip) when the CUDA
    path cannot be brought up: a GPU test must never pass on a fallback."""
    d = pkg.hal.CudaSm100Device(0)
    yield d
    d.close()
