import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc

    orc.build()
    return orc


@pytest.fixture(scope="session")
def df8():
    """The product library, built in-tree if needed. Fails loudly when it cannot be loaded."""
    import deepfuse_b200 as pkg
    from deepfuse_b200 import build as builder

    if not (pkg.LIB_DIR / "libdf8.so").exists():
        builder.build_all()
    pkg.lib()
    return pkg


@pytest.fixture(scope="session")
def cuda():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
