import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("PYTHONPATH", str(ROOT))
if str(ROOT) not in os.environ["PYTHONPATH"].split(os.pathsep):
    os.environ["PYTHONPATH"] = str(ROOT) + os.pathsep + os.environ["PYTHONPATH"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")


@pytest.fixture(autouse=True)
def _fresh_mesh():
    from olmax_b200.parallel import set_mesh

    set_mesh(None)
    yield
    set_mesh(None)
