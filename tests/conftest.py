"""Shared pytest setup: the ``gpu`` marker and import paths."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200, sm_100a)")


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return ROOT / "tests" / "golden"


@pytest.fixture(scope="session")
def mx():
    """The product package; GPU tests fail loudly when the native library is absent."""
    import mxfp6_sm120_b200 as package

    package.load_library()
    return package
