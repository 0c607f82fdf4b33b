import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Build the C-ABI library (nvcc cross-compiles without a GPU) and the C oracle once."""
    from ternel_b200.build import build
    build()
    from oracle import c_oracle
    c_oracle.lib()


@pytest.fixture(scope="session")
def golden_cases():
    import numpy as np
    data = np.load(GOLDEN / "matmul_cases.npz")
    cases = {}
    for key in data.files:
        case, name = key.split("/")
        cases.setdefault(case, {})[name] = data[key]
    return cases
