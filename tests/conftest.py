import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """The C oracle; built on demand (gcc) when the shared object is not there yet."""
    import subprocess

    from oracle import exl3_oracle as O

    if not (O.HERE / "libexl3_oracle.so").exists():
        subprocess.check_call(["make", "-C", str(O.HERE), "oracle"])
    return O.COracle()


@pytest.fixture(scope="session")
def gpu():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
