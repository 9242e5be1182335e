"""Shared pytest setup: registers the `gpu` marker and exposes the package and the oracle."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    """The host-side package, with libixk.so built if it is not there yet."""
    mod = entry.load_package()
    if not os.path.exists(mod.library_path()):
        entry.build()
    mod.load_library()
    return mod


@pytest.fixture(scope="session")
def orc():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def cuda(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu but no CUDA device is visible")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_clean(request, pkg):
    """After every GPU test: no bounded device-side wait may have given up."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        assert pkg.device_status() == 0
