"""pytest configuration: the `gpu` marker, import paths for the oracle, and the in-tree build of the library."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    """The allocation-free entry point's tests run last: a run that stops at the first failure (-x) has then already
    run every other test."""
    last = [it for it in items if it.fspath.basename == "test_no_alloc.py"]
    if last:
        items[:] = [it for it in items if it.fspath.basename != "test_no_alloc.py"] + last


@pytest.fixture(scope="session")
def built_library():
    """Path of libops_tensor_b200.so; builds it with nvcc when a source is newer (no GPU needed for that)."""
    from ops_tensor_b200 import build
    if build.LIB_PATH.exists() and not build.needs_build():
        return build.LIB_PATH
    try:
        return build.build()
    except RuntimeError as exc:          # no nvcc on this machine: use the shipped binary if there is one
        if build.LIB_PATH.exists():
            return build.LIB_PATH
        pytest.fail(str(exc))


@pytest.fixture(scope="session")
def cuda_device(built_library):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
