import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def library():
    """The in-tree CUDA library, built on demand (nvcc cross-compiles without a GPU)."""
    from tilemega_b200.build import build_library
    return build_library()


@pytest.fixture(scope="session")
def plan_dir():
    """Plan libraries of this test session: inside the package tree, removed afterwards."""
    from tilemega_b200.planbuild import PLAN_DIR, remove_plans
    folder = PLAN_DIR / f"pytest-{os.getpid()}"
    yield folder
    remove_plans(folder)
