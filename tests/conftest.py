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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """A golden fixture as a dict of torch tensors (numpy scalars stay Python numbers)."""
    data = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for key in data.files:
        arr = data[key]
        out[key] = arr.item() if arr.ndim == 0 else torch.from_numpy(arr.copy())
    return out


def assert_close_rel_max(actual, expected, tol, what=""):
    """|a - e| <= tol * max|e| + tol * |e|: the reference tests' criterion (relative to the largest
    value of the tensor, so one fp16 ulp flip does not fail a big tensor)."""
    scale = expected.float().abs().max().clamp(min=1e-6).item()
    torch.testing.assert_close(actual.float(), expected.float(), rtol=tol, atol=tol * scale,
                               msg=lambda m: f"{what}: {m}")


def rel_norm(actual, expected):
    e = expected.double()
    return ((actual.double() - e).norm() / e.norm().clamp(min=1e-30)).item()
