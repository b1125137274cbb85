"""pytest configuration: registers the ``gpu`` marker and puts the repository
root on ``sys.path`` so ``tritonkv_b200`` and the ``oracle`` checker import."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
