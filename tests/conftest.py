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
    from ternel_b200.build import build, build_checked
    build()
    build_checked()
    from oracle import c_oracle
    c_oracle.lib()


@pytest.fixture(autouse=True)
def _no_bounds_violation(request):
    """Under the bounds-checking build (TERNEL_B200_LIBRARY points at it) every GPU test also asserts that no
    kernel tried to touch memory outside the extents its launcher knows."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from ternel_b200 import _native
    torch.cuda.synchronize()
    record = _native.bounds_record()
    if record is not None:
        assert record[0] == 0, (f"{record[0]} out-of-bounds access(es) skipped; first: code {record[1]}, "
                                f"index {record[2]}, limit {record[3]}")


@pytest.fixture(scope="session")
def golden_cases():
    import numpy as np
    data = np.load(GOLDEN / "matmul_cases.npz")
    cases = {}
    for key in data.files:
        case, name = key.split("/")
        cases.setdefault(case, {})[name] = data[key]
    return cases
