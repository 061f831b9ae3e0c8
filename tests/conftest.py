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


# The stated fp32 bar of every floating-point operator: elementwise
# |out - truth| <= PARITY_RTOL * |truth| + PARITY_ATOL * max|truth|, truth = the fp64 evaluation.
PARITY_RTOL = 1e-5
PARITY_ATOL = 1e-6
# Largest ratio (error of the float build of the C oracle) / (error of the reference's own fp32
# run, torch_sph.py on float tensors) over every tensor of every fixture; pinned by
# tests/test_oracle_golden.py.  Where no stored fp32 output of the reference exists, the float
# oracle stands in for it and its error is divided by this ratio first.
FP32_PROXY_RATIO = 1.7


def assert_parity(actual, truth, ref32, what="", proxy=False):
    """The parity gate of the floating-point operators.

    Passes when ``|actual - truth| <= 1e-5 |truth| + 1e-6 max|truth|`` holds elementwise, or when
    the largest error of ``actual`` is no worse than twice the largest error of the reference's own
    fp32 evaluation ``ref32`` of the same tensor against the same fp64 ``truth``.  ``proxy=True``
    says ``ref32`` came from the float build of the C oracle instead of the reference itself; its
    error is then scaled down by FP32_PROXY_RATIO, so the clause never allows more than twice the
    reference's fp32 error.
    """
    actual = np.asarray(actual, dtype=np.float64)
    truth = np.asarray(truth, dtype=np.float64)
    assert actual.shape == truth.shape, f"{what}: shape {actual.shape} vs {truth.shape}"
    if truth.size == 0:
        return
    scale = float(np.max(np.abs(truth)))
    err = np.abs(actual - truth)
    tol = PARITY_RTOL * np.abs(truth) + PARITY_ATOL * scale
    bad = err > tol
    if not bad.any():
        return
    worst = float(err.max())
    ref_err = None
    if ref32 is not None:
        ref_err = float(np.max(np.abs(np.asarray(ref32, dtype=np.float64) - truth)))
        if proxy:
            ref_err /= FP32_PROXY_RATIO
        if worst <= 2.0 * ref_err:
            return
    k = int(np.argmax(err - tol))
    raise AssertionError(
        f"{what}: {int(bad.sum())}/{bad.size} elements outside 1e-5 rel / 1e-6 abs (worst |err|={err.flat[k]:.3e} "
        f"at truth={truth.flat[k]:.6e}, scale={scale:.3e}) and max |err|={worst:.3e} exceeds twice the "
        f"reference's fp32 error ({'n/a' if ref_err is None else format(ref_err, '.3e')})")


@pytest.fixture(scope="session")
def native():
    """The loaded CUDA library wrapper; GPU tests fail loudly if it is missing."""
    from npa_b200 import _native
    return _native
