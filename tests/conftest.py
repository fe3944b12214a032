import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import pyasc_b200  # noqa: E402,F401  (makes `asc` / `asc2` importable)
from asc.runtime import config  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_addoption(parser: pytest.Parser):
    # same options as the reference's asc2 conftest (python/test/asc2/conftest.py:27-33), CUDA by default
    parser.addoption("--backend", type=config.Backend, default=config.Backend.CUDA, help="Runtime backend")
    parser.addoption("--platform", type=config.Platform, default=config.Platform.B200, help="Runtime platform")
    parser.addoption("--device", type=int, default=0, help="Device ID")


@pytest.fixture
def backend(request: pytest.FixtureRequest):
    return request.config.getoption("--backend")


@pytest.fixture
def platform(request: pytest.FixtureRequest):
    return request.config.getoption("--platform")


@pytest.fixture
def device_id(request: pytest.FixtureRequest):
    return request.config.getoption("--device")


@pytest.fixture
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")
