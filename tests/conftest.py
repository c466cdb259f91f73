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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name, dtype=None):
    z = np.load(os.path.join(GOLDEN, name))
    out = {}
    for key in z.files:
        if z[key].dtype.kind in "US":
            out[key] = str(z[key])
            continue
        t = torch.from_numpy(z[key])
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        out[key] = t
    return out


def rel_err(a, b):
    """max |a-b| / max |b|: the relative error used by every parity test."""
    a, b = a.double(), b.double()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()
