import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import q35oracle

    q35oracle.lib()
    return q35oracle


@pytest.fixture(scope="session")
def engine():
    """The product library; built on demand where nvcc exists, else the prebuilt file must be present."""
    import shutil

    import qwen35x_b200
    from qwen35x_b200 import build as b

    if shutil.which("nvcc"):
        b.build()
    qwen35x_b200.lib()
    return qwen35x_b200
