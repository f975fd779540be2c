import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Vectors produced by the reference project (tests/golden/make_golden.py)."""

    def __init__(self):
        self._z = np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))

    def cases(self, prefix):
        names = sorted({k.split("/")[1] for k in self._z.files if k.startswith(prefix + "/")})
        return names

    def get(self, key, bf16=False):
        a = self._z[key]
        t = torch.from_numpy(a.copy())
        if a.dtype == np.uint16:
            t = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        return t


@pytest.fixture(scope="session")
def golden():
    return Golden()


@pytest.fixture(scope="session", autouse=True)
def _built_artifacts():
    """The kernel library and the C oracle must exist and be current: both builds compare
    modification times, so this costs nothing when they are up to date and never lets the
    tests run against a library older than its sources."""
    from newt_b200.csrc import build as kbuild
    from oracle import cport

    kbuild.build()
    cport.build()
