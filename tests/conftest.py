"""pytest configuration: the ``gpu`` marker and shared helpers."""
import ast
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def golden_names():
    """Operator fixtures (tests/golden/make_golden.py); the step_* and splat_* files belong to
    make_step_golden.py and make_splat_golden.py."""
    return sorted(p.stem for p in GOLDEN_DIR.glob("*.npz") if not p.stem.startswith(("step_", "splat_")))


def load_golden(name):
    """Returns (meta dict, dict of arrays) of one fixture written by tests/golden/make_golden.py."""
    blob = np.load(GOLDEN_DIR / f"{name}.npz")
    meta = ast.literal_eval(str(blob["meta"]))
    return meta, {k: blob[k] for k in blob.files if k != "meta"}


def assert_close(actual, expected, rtol, atol_scale, what=""):
    """|a - e| <= rtol * |e| + atol_scale * max|e| elementwise."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} vs {expected.shape}"
    scale = float(np.max(np.abs(expected))) if expected.size else 0.0
    err = np.abs(actual - expected)
    tol = rtol * np.abs(expected) + atol_scale * scale
    bad = err > tol
    if bad.any():
        k = int(np.argmax(err - tol))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.size} elements out of tolerance; worst |err|={err.flat[k]:.3e} "
            f"expected={expected.flat[k]:.6e} scale={scale:.3e} (rtol={rtol}, atol={atol_scale}*scale)")


@pytest.fixture(scope="session")
def native():
    """The loaded CUDA library wrapper; GPU tests fail loudly if it is missing."""
    from npa_b200 import _native
    return _native
