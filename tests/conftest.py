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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def load_golden(name):
    """Golden vectors written by the reference itself (tests/golden/make_golden.py)."""
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        out = {}
        for k in z.files:
            a = z[k]
            out[k] = torch.from_numpy(a) if a.shape != () else a.item()
        return out


@pytest.fixture(scope="session")
def golden():
    return load_golden


def reference_extension():
    """The reference's own compiled CPU extension, if it was built here
    (``make -C oracle ref``); None elsewhere."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "_fast_rnnt.so")):
        return None
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    try:
        import _fast_rnnt
        return _fast_rnnt
    except Exception:
        return None
