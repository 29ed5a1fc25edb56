import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs through the C ABI on cuda:0)")


@pytest.fixture(scope="session")
def gpu():
    """One library context on cuda:0 for the GPU tests (C ABI, no torch)."""
    from qwen_metal_b200 import abi
    ctx = abi.Gpu()
    yield ctx
    ctx.close()
