import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a) and the built native library")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Read-only view of tests/golden/pope_golden.npz (vectors produced by the reference itself)."""

    def __init__(self):
        self._z = np.load(os.path.join(ROOT, "tests", "golden", "pope_golden.npz"))

    def case(self, prefix):
        pre = prefix.rstrip("/") + "/"
        return {k[len(pre):]: torch.from_numpy(self._z[k]) for k in self._z.files if k.startswith(pre)}

    def tags(self, group):
        pre = group.rstrip("/") + "/"
        return sorted({k[len(pre):].split("/")[0] for k in self._z.files if k.startswith(pre)})


@pytest.fixture(scope="session")
def golden():
    return Golden()
