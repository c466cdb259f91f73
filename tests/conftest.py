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


def rel_err_rows(a, b, dim, start, length=128):
    """The same ratio restricted to ``length`` consecutive rows of dimension ``dim``: max |a-b| over the window
    divided by max |b| over the SAME window.  Rows late in a causal sequence are averages over thousands of
    values and far smaller than the first rows; the whole-tensor ratio is blind to errors of their size."""
    n = b.shape[dim]
    start = max(0, min(start, n - 1))
    length = min(length, n - start)
    return rel_err(a.narrow(dim, start, length), b.narrow(dim, start, length))


def worst_window_err(a, b, dim, length=128):
    """The largest ``rel_err_rows`` over three windows: the first rows, the middle and the last rows."""
    n = b.shape[dim]
    starts = sorted({0, max(0, n // 2), max(0, n - length)})
    return max(rel_err_rows(a, b, dim, s, length) for s in starts)


def _second_order_masks(d=16):
    """Index masks into the 273 Taylor features: constant, first order, second-order diagonal (i == j) and
    second-order off-diagonal terms (layout of TaylorExp.forward, linear_attention.py:69-75)."""
    idx = torch.arange(1 + d + d * d)
    g = idx - (1 + d)
    i, j = g // d, g % d
    second = idx >= 1 + d
    return {"const": idx == 0, "first": (idx >= 1) & (idx < 1 + d), "diag": second & (i == j), "offdiag": second & (i != j)}


def state_block_errs(state, ref):
    """Relative error of a ``[..., 273]`` state per feature block, each normalised by that block's own max |ref|:
    the second-order entries are an order of magnitude smaller than the constant column, so a wrong scale in one
    block hides inside a whole-tensor ratio."""
    return {name: rel_err(state[..., m], ref[..., m]) for name, m in _second_order_masks().items()}
