import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def library():
    """The C-ABI library, built on demand; a missing library is an error, never a skip."""
    from cudabackend_b200 import api, build
    if not os.path.exists(api.library_path()):
        build.build()
    return api.load()


@pytest.fixture(scope="session")
def device_count(library):
    from cudabackend_b200 import api
    return api.number_of_devices()


@pytest.fixture()
def ctx(library, device_count):
    """A context with its own stream on device 0."""
    from cudabackend_b200 import api
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    context = api.Context(0)
    yield context
    context.synchronize()
    assert context.last_device_status() == 0, "a tensor-core kernel reported a bounded wait that ran out"
    context.destroy()
