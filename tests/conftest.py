import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return graft.load_package()


@pytest.fixture(scope="session")
def po():
    return graft.load_oracle()


@pytest.fixture(scope="session")
def orc(po):
    return po.Oracle()


@pytest.fixture(scope="session")
def ref(po):
    """The reference's own compiled CPU path (default flags), or skip."""
    if not po.Ref.available():
        pytest.skip("oracle/_ref/libsiref.so not built (reference tree absent)")
    return po.Ref()


@pytest.fixture(scope="session")
def ref_strict(po):
    if not po.Ref.available(strict=True):
        pytest.skip("oracle/_ref/libsiref_nofma.so not built (reference tree absent)")
    return po.Ref(strict=True)


@pytest.fixture(scope="session")
def be(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return pkg.make_cuda_backend(0)
