"""Shared pytest set-up: the ``gpu`` marker, the repository root on ``sys.path`` and a clean runtime after each test
(as the reference's conftest resets configuration and pool; reference: tests/conftest.py:8-13)."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(autouse=True)
def _reset_runtime():
    yield
    import miles_ext_kernels_b200 as package

    package.configure()
    if "torch" in sys.modules:
        package.release()
