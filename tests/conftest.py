import os, sys, ast
import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


class GoldenCases:
    """Inputs and outputs of the unmodified reference (see tests/golden/make_golden.py)."""

    def __init__(self):
        path = os.path.join(ROOT, "tests", "golden", "converse2d_ref_cases.npz")
        self.z = np.load(path)
        self.meta = ast.literal_eval(str(self.z["meta"]))

    def __len__(self):
        return len(self.meta)

    def case(self, i):
        c = dict(self.meta[i])
        z = self.z
        return c, z[f"x{i}"], z[f"w{i}"], z[f"b{i}"], z[f"ref32_{i}"], z[f"ref64_{i}"]


@pytest.fixture(scope="session")
def golden():
    return GoldenCases()
