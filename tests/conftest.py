"""pytest configuration: the ``gpu`` marker, import paths, golden-file loader."""

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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Load a golden ``.npz`` and turn arrays back into torch tensors
    (int16 payloads are bf16 bit patterns, uint8 payloads are e4m3)."""
    z = np.load(os.path.join(GOLDEN, name), allow_pickle=False)
    out = {}
    for k in z.files:
        a = z[k]
        if a.dtype.kind in "US":
            out[k] = str(a)
            continue
        t = torch.from_numpy(np.ascontiguousarray(a))
        if a.dtype == np.int16:
            t = t.view(torch.bfloat16)
        elif a.dtype == np.uint8:
            t = t.view(torch.float8_e4m3fn)
        out[k] = t
    return out


def golden_files(prefix):
    return sorted(f for f in os.listdir(GOLDEN) if f.startswith(prefix) and f.endswith(".npz"))
