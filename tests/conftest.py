import glob
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _all_golden():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def golden_names():
    """Fixtures of the linear layer (quantizer + GEMM)."""
    return [n for n in _all_golden() if not n.startswith("next_")]


def next_golden_names():
    """Fixtures of the GEMM's optional next-layer quantisation (smooth_next)."""
    return [n for n in _all_golden() if n.startswith("next_")]


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        d = {k: z[k] for k in z.files}
    for k in ("M", "K", "N", "R", "exact"):
        if k in d:
            d[k] = int(d[k])
    d["dtype"] = str(d["dtype"])
    return d


@pytest.fixture(scope="session")
def lib_path():
    """Builds the CUDA library once per session if nvcc is here; the GPU box receives it prebuilt."""
    from svdquant_kernels_b200 import build as b
    if b.needs_build():
        b.build()
    return b.LIB_PATH
