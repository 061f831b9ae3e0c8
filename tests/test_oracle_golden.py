"""Pins the C oracle (oracle/sph_oracle.c) to the reference's own operators.

The fixtures were produced by importing the reference's sphops/torch_sph.py
(tests/golden/make_golden.py).  The oracle accumulates in double, so it must
agree with the fp64 run to rounding, and with the fp32 run to fp32 accuracy.
"""
import numpy as np
import pytest

import oracle
from conftest import FP32_PROXY_RATIO, GOLDEN_DIR, assert_close, assert_parity, golden_names, load_golden

FWD = ["rho", "rho_grad", "blur", "grad", "moment"]


def _inputs(meta, arr):
    box = [g * meta["eps"] for g in meta["grid"]] if meta["periodic"] else None
    kw = dict(mass=arr.get("in_mass"), s=arr["in_s"], rho_in=arr["in_rho_in"],
              periodic=meta["periodic"], box_size=box)
    return arr["in_x"], kw


@pytest.mark.parametrize("name", golden_names())
def test_forward_matches_reference(name):
    meta, arr = load_golden(name)
    x, kw = _inputs(meta, arr)
    out = oracle.forward(x, meta["eps"], meta["dim"], want=("count", *FWD), **kw)
    # count is evaluated with the reference's fp32 arithmetic: exact
    np.testing.assert_array_equal(out["count"], arr["f32_count"])
    for k in FWD:
        assert_close(out[k], arr[f"f64_{k}"], rtol=1e-9, atol_scale=1e-11, what=f"{name}:{k} vs fp64")
        assert_close(out[k], arr[f"f32_{k}"], rtol=1e-4, atol_scale=2e-6, what=f"{name}:{k} vs fp32")


@pytest.mark.parametrize("name", golden_names())
@pytest.mark.parametrize("op,up", [("density", "g_rho"), ("rho_grad", "g_rho_grad"), ("blur", "g_blur"),
                                   ("grad", "g_grad"), ("moment", "g_moment")])
def test_backward_matches_reference_autograd(name, op, up):
    meta, arr = load_golden(name)
    x, kw = _inputs(meta, arr)
    dx, ds, drho = oracle.backward(x, meta["eps"], meta["dim"], **kw, **{up: arr[f"in_{up}"]})
    assert_close(dx, arr[f"f64_bw_{op}_dx"], rtol=1e-8, atol_scale=1e-10, what=f"{name}:{op} dx")
    if f"f64_bw_{op}_ds" in arr:
        assert_close(ds, arr[f"f64_bw_{op}_ds"], rtol=1e-8, atol_scale=1e-10, what=f"{name}:{op} ds")
    if f"f64_bw_{op}_drho" in arr:
        assert_close(drho, arr[f"f64_bw_{op}_drho"], rtol=1e-8, atol_scale=1e-10, what=f"{name}:{op} drho")


@pytest.mark.parametrize("name", golden_names())
def test_chained_backward_matches_reference_autograd(name):
    """rho = density(x) feeding blur and gradient: two oracle calls composed as autograd does."""
    meta, arr = load_golden(name)
    x, kw = _inputs(meta, arr)
    kw = dict(kw)
    # the chain differentiates through the density the operators were fed, i.e. torch's own rho;
    # the fixture's chain used rho computed in the run's dtype, so feed the fp64 truth rounded once
    kw["rho_in"] = arr["f64_rho"].astype(np.float32)
    dx1, ds, drho = oracle.backward(x, meta["eps"], meta["dim"], **kw,
                                    g_blur=arr["in_g_blur"], g_grad=arr["in_g_grad"])
    g_rho_total = (arr["in_g_rho"].astype(np.float64) + drho).astype(np.float32)
    kw2 = dict(kw, s=None, rho_in=None)
    dx2, _, _ = oracle.backward(x, meta["eps"], meta["dim"], **kw2, g_rho=g_rho_total,
                                g_rho_grad=arr["in_g_rho_grad"])
    # rho rounded to fp32 and the fp32 hand-over of drho bound the agreement: the parity gate with
    # the reference's own fp32 chain as the yardstick
    assert_parity(dx1 + dx2, arr["f64_chain_dx"], arr["f32_chain_dx"], what=f"{name}: chain dx")
    assert_parity(ds, arr["f64_chain_ds"], arr["f32_chain_ds"], what=f"{name}: chain ds")


@pytest.mark.parametrize("name", golden_names())
def test_float_build_tracks_the_reference_fp32_error(name):
    """The float build of the oracle (precision="f32") stands in for the reference's fp32 run in the
    parity gate of cases that have no stored fp32 output.  On every fixture tensor its error against
    the fp64 truth must stay within FP32_PROXY_RATIO of torch_sph's own fp32 error (so dividing by
    that ratio never overstates what the reference itself achieves), and it must not be a double
    evaluation in disguise (error above a tenth of the reference's)."""
    meta, arr = load_golden(name)
    x, kw = _inputs(meta, arr)
    got = oracle.forward(x, meta["eps"], meta["dim"], want=tuple(FWD), precision="f32", **kw)
    for op, up in [("density", "g_rho"), ("rho_grad", "g_rho_grad"), ("blur", "g_blur"), ("grad", "g_grad"),
                   ("moment", "g_moment")]:
        dx, ds, drho = oracle.backward(x, meta["eps"], meta["dim"], precision="f32", **kw, **{up: arr[f"in_{up}"]})
        got[f"bw_{op}_dx"], got[f"bw_{op}_ds"], got[f"bw_{op}_drho"] = dx, ds, drho
    checked = 0
    for k, v in got.items():
        if f"f64_{k}" not in arr:
            continue
        truth = arr[f"f64_{k}"]
        mine = np.abs(v - truth).max()
        theirs = np.abs(arr[f"f32_{k}"].astype(np.float64) - truth).max()
        assert mine <= FP32_PROXY_RATIO * theirs, (name, k, mine, theirs)
        assert mine >= 0.1 * theirs, (name, k, mine, theirs)
        checked += 1
    assert checked == 15


def test_safe_inverse_identity_fallback():
    rng = np.random.default_rng(0)
    for dim in (2, 3):
        a = rng.standard_normal((50, dim, dim)).astype(np.float32)
        m = a @ a.transpose(0, 2, 1) + 0.5 * np.eye(dim, dtype=np.float32)
        m[0] = 0.0  # singular -> identity
        inv = oracle.safe_inv_sym_mat(m, 1e-3)
        np.testing.assert_array_equal(inv[0], np.eye(dim, dtype=np.float32))
        np.testing.assert_allclose(inv[1:] @ m[1:], np.broadcast_to(np.eye(dim), (49, dim, dim)), atol=2e-4)


STEP_CASES = ["step_d2", "step_d3", "step_d2_all"]


@pytest.mark.parametrize("name", STEP_CASES)
def test_step_oracle_matches_reference_step_euler(name):
    """oracle/step.py against NPA.forward + step_euler of the reference (fixtures made by
    tests/golden/make_step_golden.py): new positions / states bit for bit, dL/dy to 1e-6."""
    from oracle import step as step_oracle
    g = np.load(GOLDEN_DIR / f"{name}.npz")
    dim, eps, alpha, dt = int(g["dim"]), float(g["eps"]), float(g["alpha"]), float(g["dt"])
    x, s = step_oracle.step_forward(g["y"], g["x_bin"], g["s_bin"], g["mask"], dim, eps, alpha, dt)
    np.testing.assert_array_equal(s, g["s_new"])
    np.testing.assert_allclose(x, g["x_new"], rtol=0, atol=2e-7 * np.abs(g["x_new"]).max())
    g_y = step_oracle.step_backward(g["y"], g["mask"], dim, eps, alpha, dt, g["up_x"], g["up_s"])
    np.testing.assert_allclose(g_y, g["g_y"], rtol=1e-5, atol=1e-6 * np.abs(g["g_y"]).max())
    # gradients with respect to the binned inputs are the upstream gradients themselves
    np.testing.assert_array_equal(g["g_x_bin"], g["up_x"])
    np.testing.assert_array_equal(g["g_s_bin"], g["up_s"])


SPLAT_CASES = ["splat_default_small", "splat_plain_yup", "splat_wide_box"]


@pytest.mark.parametrize("name", SPLAT_CASES)
def test_splat_oracle_matches_reference_splatting(name):
    """oracle/splat.py against the reference's splat_particles_batch run in float64 (fixtures made by
    tests/golden/make_splat_golden.py): image and both gradients to 1e-9."""
    import ast
    from oracle import splat as splat_oracle
    g = np.load(GOLDEN_DIR / f"{name}.npz")
    meta = ast.literal_eval(str(g["meta"]))
    for b in range(meta["B"]):
        x, c = g["x"][b].astype(np.float64), g["color"][b].astype(np.float64)
        out = splat_oracle.splat_forward(x, c, **meta["kw"])
        scale = np.abs(g["out_f64"][b]).max()
        np.testing.assert_allclose(out, g["out_f64"][b], rtol=1e-9, atol=1e-12 * scale)
        g_x, g_c = splat_oracle.splat_backward(x, c, g["up"][b], **meta["kw"])
        np.testing.assert_allclose(g_x, g["g_x_f64"][b], rtol=1e-8, atol=1e-10 * np.abs(g["g_x_f64"][b]).max())
        want_c = g["g_color_f64"][b]
        np.testing.assert_allclose(g_c, want_c[:, -3:], rtol=1e-9, atol=1e-12 * np.abs(want_c).max())
        assert not want_c[:, :-3].any()   # only the last three colour channels are rendered
