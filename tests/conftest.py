import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def ph():
    """The product package (phobos-lang_b200/), loaded under an importable name."""
    import __graft_entry__ as entry
    return entry.load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def dev(ph):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ph.lib()
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
