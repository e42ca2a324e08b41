import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle binding (builds liboracle.so on first use)."""
    from oracle import oracle as mod
    mod.build()
    return mod


@pytest.fixture(scope="session")
def bk():
    """The Python access layer of the C-ABI library (raises if the library is not built)."""
    import __graft_entry__ as entry
    pkg = entry.load_package()
    pkg.lib()
    return pkg


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu was started without a CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
