"""Shared pytest setup: markers, import paths, golden-vector loader."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
for p in (ROOT, os.path.join(ROOT, "attention_impl_b200", "dropin")):
    if p not in sys.path:
        sys.path.insert(0, p)


# the reference's own test files (fetched, not committed) are run by test_reference_suite_gpu.py in a
# child process, never collected into this suite
collect_ignore_glob = ["reference_suite/*"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


_DT = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32,
       "torch.float64": torch.float64, "torch.int32": torch.int32, "torch.int64": torch.int64}


def load_golden(tag):
    """Load ``tests/golden/<tag>.npz`` back into torch tensors (half stored as uint16 bits)."""
    z = np.load(os.path.join(GOLDEN, tag + ".npz"))
    out = {}
    for k in z.files:
        if k.startswith("dtype_"):
            continue
        dt = _DT[str(z["dtype_" + k])]
        a = z[k]
        if dt in (torch.float16, torch.bfloat16):
            out[k] = torch.from_numpy(a.view(np.int16).copy()).view(dt)
        else:
            out[k] = torch.from_numpy(np.array(a)).to(dt)
    return out


@pytest.fixture
def golden():
    return load_golden
