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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz"))
                  if not os.path.basename(p).startswith("cfg"))


def load_golden(name):
    """Returns (x, params, y, meta) of one golden case as numpy / python objects."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    ndim, c, k, levels, stride, bias = (int(v) for v in z["meta"])
    params = {key[2:]: z[key] for key in z.files if key.startswith("p:")}
    meta = dict(ndim=ndim, C=c, K=k, L=levels, stride=stride, bias=bool(bias), dtype=str(z["dtype"]))
    return z["x"], params, z["y"], meta


def max_err(y, ref):
    """Normalised max error max|y-ref| / max|ref| (the parity measure used throughout)."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = max(float(np.abs(ref).max()), 1e-30)
    return float(np.abs(y - ref).max()) / den


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN_DIR
