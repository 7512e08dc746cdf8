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


def check_close(got, ref, tol, names, what=""):
    """Parity assertion of the GPU tests: for every tensor max|x - ref| <= tol * max|ref| (``tol``: one number or a
    dict by name).  The message lists, for ALL tensors, the error relative to max|ref| AND the maximum absolute error
    with max|ref| beside it, so a failure (or ``-rA``) shows both figures."""
    rows, bad = [], []
    for n, x, r in zip(names, got, ref):
        if r is None and x is None:
            continue
        assert x is not None and r is not None, f"{what}{n}: one side is None"
        x64, r64 = x.detach().double().cpu(), r.detach().double().cpu()
        assert x64.shape == r64.shape, f"{what}{n}: shape {tuple(x64.shape)} != {tuple(r64.shape)}"
        den = r64.abs().max().item() if r64.numel() else 0.0
        mabs = (x64 - r64).abs().max().item() if r64.numel() else 0.0
        rel = mabs / den if den > 0 else mabs
        t = tol[n] if isinstance(tol, dict) else tol
        rows.append(f"{n}: rel-to-max {rel:.2e} (tol {t:.0e}), max-abs {mabs:.3e} of max|ref| {den:.3e}")
        if not (rel < t):
            bad.append(n)
    report = what + "; ".join(rows)
    assert not bad, f"out of tolerance: {bad} | {report}"
    return report
