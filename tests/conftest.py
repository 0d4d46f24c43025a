import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The op registers through MagiCompiler when that package is importable.  The unit tests pin the
# package's own mirror of the decorator; the integration with a real checkout runs in a subprocess.
os.environ.setdefault("MAGI_SWIGLU_USE_MAGI_COMPILER", "0")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "swiglu_reference_eager.npz")
