from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def codebooks() -> dict[str, bytes]:
    """IQ codebooks from the committed fixture (generated from the reference by tests/golden/make_golden.py)."""
    with np.load(REPO / "tests" / "golden" / "iq_codebooks.npz") as z:
        return {k: z[k].tobytes() for k in z.files}
