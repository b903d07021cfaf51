import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o

    o.build()
    return o


@pytest.fixture(scope="session")
def golden():
    import glob

    import numpy as np

    files = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz")))
    assert files, "tests/golden/*.npz missing (generate with tests/golden/make_golden.py)"
    return {os.path.basename(f)[:-4]: dict(np.load(f)) for f in files}


@pytest.fixture(scope="session")
def qm():
    """The product package; importing it loads libquadmul_b200.so or fails."""
    import quadmul_b200

    return quadmul_b200


@pytest.fixture()
def cuda_clean(qm):
    """Yields torch; afterwards checks that no kernel recorded a wait time-out."""
    import torch

    assert torch.cuda.is_available(), "gpu test run without a CUDA device"
    yield torch
    code, where = qm.device_status(clear=True)
    assert (code, where) == (0, 0), f"in-kernel wait expired: code={code} site={where & 0xFF} block={where >> 8}"
