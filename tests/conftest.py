import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


def load_golden(name):
    """Load a fixture written by tests/golden/make_golden.py as a dict of torch tensors."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for key in z.files:
        a = z[key]
        if key.endswith("_bf16"):
            t = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
            out[key[:-5]] = t
        elif a.ndim == 0:
            out[key] = float(a)
        else:
            out[key] = torch.from_numpy(a.copy())
    return out
