import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    with np.load(ROOT / "tests" / "golden" / "bctx_golden.npz") as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def orc():
    from oracle import bcx_oracle

    bcx_oracle.build()
    return bcx_oracle


@pytest.fixture(scope="session")
def oracle_coder(orc):
    return orc.Coder("oracle")
