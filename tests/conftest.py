"""Shared pytest configuration: the `gpu` marker, import paths, golden-vector loader."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "bi-mamba2_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

# make every operator call in the tests verify the library's device status word (bounded waits that ran out)
os.environ.setdefault("BISSD_CHECK_STATUS", "1")

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Return a dict of torch tensors (float64 for float arrays) from tests/golden/<name>.npz."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        if k == "meta":
            out[k] = [int(v) for v in a]
        elif k == "dt_limit":
            out[k] = (float(a[0]), float(a[1]))
        else:
            out[k] = torch.from_numpy(a.astype(np.float64))
    return out


GOLDEN_TRITON = ["triton_bi_plain", "triton_bi_full", "triton_bi_ragged_limit"]
GOLDEN_TORCHREF = ["torchref_small", "torchref_hdimD"]
