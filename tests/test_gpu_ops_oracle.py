"""Forward / backward parity of the CUDA operators with the C oracle on seeded inputs.

Covers both dimensions, both boundaries, both hash orders, masses, channel counts that take
every dispatch path (vector widths, lanes per particle, feature chunking), crowded cells that
split into several work items, and the benchmark shapes at sizes the oracle finishes in seconds.
"""
import numpy as np
import pytest
import torch

from conftest import assert_close, assert_parity
from helpers import ATOL_SCALE, RTOL, make_grid, np64, oracle_backward, oracle_forward
from npa_b200.workloads import CONFIGS, Workload, make_inputs, scaled

pytestmark = pytest.mark.gpu

GEOMS = [
    Workload("o_2d_clamped", dim=2, B=2, N=1500, C=16, eps=0.06, grid_size=(18, 18)),
    Workload("o_2d_periodic", dim=2, B=2, N=1200, C=16, eps=0.07, grid_size=(14, 15), boundary="periodic"),
    Workload("o_2d_morton", dim=2, B=1, N=1500, C=8, eps=1 / 16, grid_size=(16, 16), mode="particle",
             boundary="periodic"),
    Workload("o_3d_clamped", dim=3, B=2, N=3000, C=32, eps=0.13, grid_size=(8, 8, 8)),
    Workload("o_3d_periodic", dim=3, B=1, N=3000, C=16, eps=0.125, grid_size=(8, 8, 8), boundary="periodic"),
    Workload("o_3d_morton", dim=3, B=1, N=2500, C=12, eps=0.125, grid_size=(8, 8, 8), mode="particle"),
    Workload("o_3d_small_periodic", dim=3, B=1, N=400, C=4, eps=0.3, grid_size=(3, 2, 4), boundary="periodic"),
]
CHANNELS = [1, 3, 4, 8, 12, 20, 33, 64, 132, 160]


def _prepare(w, seed=0, with_mass=False, crowd=True):
    from npa_b200 import sphops as sph
    x, s, ups = make_inputs(w, seed)
    if w.boundary == "periodic":
        x[..., : w.dim] *= torch.tensor([g * w.eps for g in w.grid_size[: w.dim]])
    else:
        x[..., : w.dim] *= torch.tensor([(g - 2) * w.eps for g in w.grid_size[: w.dim]])
    if crowd:
        x[:, : w.N // 6, : w.dim] *= 0.15      # crowded cells -> several work items per cell
        x[:, 3] = x[:, 2]                       # coincident pair
    g = torch.Generator().manual_seed(seed + 1)
    mass = (torch.rand(w.B, w.N, generator=g) + 0.5) if with_mass else None
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    if mass is None:
        xb, sb = sph.bin_particles(x.cuda(), s.cuda(), snap)
        mb = None
    else:
        xb, sb, mb = sph.bin_particles(x.cuda(), s.cuda(), snap, mass.cuda())
    return sph, snap, xb, sb, mb, {k: v.cuda() for k, v in ups.items()}


def _check_all(w, with_mass, seed=0):
    sph, snap, xb, sb, mb, ups = _prepare(w, seed, with_mass)
    dim = w.dim
    rho = sph.density(xb, snap, mb)
    names = ("rho", "rho_grad", "blur", "grad", "moment")
    ref = oracle_forward(xb, w, ("count", *names), s=sb, mass=mb, rho_in=rho)
    # the float build of the oracle sizes the "twice the reference's fp32 error" clause of the gate
    ref32 = oracle_forward(xb, w, names, s=sb, mass=mb, rho_in=rho, precision="f32")
    np.testing.assert_array_equal(sph.count(xb, snap).cpu().numpy(), ref["count"])
    got = {"rho": rho, "rho_grad": sph.density_gradient(xb, snap, mb), "blur": sph.blur(xb, rho, sb, snap, mb),
           "grad": sph.gradient(xb, rho, sb, snap, mb), "moment": sph.moment_matrix(xb, rho, snap, mb)}
    for k in names:
        assert_parity(np64(got[k]), ref[k], ref32[k], f"{w.name}: {k}", proxy=True)

    g = torch.Generator().manual_seed(seed + 2)
    g_moment = torch.randn(w.B, w.N, dim, dim, generator=g).cuda()
    specs = {
        "density": (lambda xr, sr, rr: sph.density(xr, snap, mb), dict(g_rho=ups["g_rho"])),
        "rho_grad": (lambda xr, sr, rr: sph.density_gradient(xr, snap, mb), dict(g_rho_grad=ups["g_rho_grad"])),
        "blur": (lambda xr, sr, rr: sph.blur(xr, rr, sr, snap, mb), dict(g_blur=ups["g_blur"])),
        "grad": (lambda xr, sr, rr: sph.gradient(xr, rr, sr, snap, mb), dict(g_grad=ups["g_grad"])),
        "moment": (lambda xr, sr, rr: sph.moment_matrix(xr, rr, snap, mb), dict(g_moment=g_moment)),
    }
    for op, (fn, up) in specs.items():
        xr, sr, rr = (t.clone().requires_grad_(True) for t in (xb, sb, rho))
        fn(xr, sr, rr).backward(next(iter(up.values())))
        dx, ds, dr = oracle_backward(xb, w, s=sb, mass=mb, rho_in=rho, **up)
        dx32, ds32, dr32 = oracle_backward(xb, w, s=sb, mass=mb, rho_in=rho, precision="f32", **up)
        assert_parity(np64(xr.grad)[..., :dim], dx, dx32, f"{w.name}:{op} dx", proxy=True)
        if op in ("blur", "grad"):
            assert_parity(np64(sr.grad), ds, ds32, f"{w.name}:{op} ds", proxy=True)
        if op in ("blur", "grad", "moment"):
            assert_parity(np64(rr.grad), dr, dr32, f"{w.name}:{op} drho", proxy=True)


@pytest.mark.parametrize("w", GEOMS, ids=lambda w: w.name)
@pytest.mark.parametrize("with_mass", [False, True], ids=["unit_mass", "mass"])
def test_every_operator_every_geometry(w, with_mass):
    _check_all(w, with_mass)


@pytest.mark.parametrize("C", CHANNELS)
def test_feature_operators_channel_counts(C):
    """Blur / gradient forward, full backward and features-only backward for every dispatch path."""
    w = Workload(f"c{C}", dim=3 if C % 2 == 0 else 2, B=1, N=900, C=C, eps=0.2,
                 grid_size=(6, 6, 6) if C % 2 == 0 else (6, 6))
    sph, snap, xb, sb, mb, ups = _prepare(w, seed=C, with_mass=C % 3 == 0)
    rho = sph.density(xb, snap, mb)
    ref = oracle_forward(xb, w, ("blur", "grad"), s=sb, mass=mb, rho_in=rho)
    assert_close(np64(sph.blur(xb, rho, sb, snap, mb)), ref["blur"], RTOL, ATOL_SCALE, f"C={C}: blur")
    assert_close(np64(sph.gradient(xb, rho, sb, snap, mb)), ref["grad"], RTOL, ATOL_SCALE, f"C={C}: grad")
    dx, ds, dr = oracle_backward(xb, w, s=sb, mass=mb, rho_in=rho, g_blur=ups["g_blur"], g_grad=ups["g_grad"])
    # full backward of both operators
    xr, sr, rr = (t.clone().requires_grad_(True) for t in (xb, sb, rho))
    torch.autograd.backward([sph.blur(xr, rr, sr, snap, mb), sph.gradient(xr, rr, sr, snap, mb)],
                            [ups["g_blur"], ups["g_grad"]])
    assert_close(np64(xr.grad)[..., : w.dim], dx, RTOL, ATOL_SCALE, f"C={C}: dx")
    assert_close(np64(sr.grad), ds, RTOL, ATOL_SCALE, f"C={C}: ds")
    assert_close(np64(rr.grad), dr, RTOL, ATOL_SCALE, f"C={C}: drho")
    # features-only backward (positions and density detached, as NPA trains by default)
    sr2 = sb.clone().requires_grad_(True)
    torch.autograd.backward([sph.blur(xb, rho, sr2, snap, mb), sph.gradient(xb, rho, sr2, snap, mb)],
                            [ups["g_blur"], ups["g_grad"]])
    assert_close(np64(sr2.grad), ds, RTOL, ATOL_SCALE, f"C={C}: ds (features only)")
    # fused features-only backward
    sr3 = sb.clone().requires_grad_(True)
    _, blur_f, grad_f, _ = sph.perceive(xb, sr3, snap, mb)
    torch.autograd.backward([blur_f, grad_f], [ups["g_blur"], ups["g_grad"]])
    assert_close(np64(sr3.grad), ds, RTOL, ATOL_SCALE, f"C={C}: ds (fused, features only)")


def _oracle_chain(xb, sb, rho, w, ups, precision):
    """Forward and chained backward of the perception step with the oracle: rho feeds blur and gradient,
    their density gradient joins the upstream of the density (two gather passes, as autograd composes them)."""
    fw = oracle_forward(xb, w, ("rho", "rho_grad", "blur", "grad"), s=sb, rho_in=rho, precision=precision)
    dx1, ds, drho = oracle_backward(xb, w, s=sb, rho_in=rho, g_blur=ups["g_blur"], g_grad=ups["g_grad"],
                                    precision=precision)
    g_total = (np64(ups["g_rho"]) + drho).astype(np.float32)
    dx2, _, _ = oracle_backward(xb, w, g_rho=torch.from_numpy(g_total), g_rho_grad=ups["g_rho_grad"],
                                precision=precision)
    return fw, ds, dx1 + dx2


@pytest.mark.parametrize("name,B", [("cfg1_2d_growing", 1), ("cfg2_2d_texture_blobs", 1),
                                    ("cfg3_2d_pointmnist_strokes", 16), ("cfg4_3d_splat", 1),
                                    ("cfg5_3d_rollout", 1)])
def test_benchmark_shapes_fused_chain(name, B):
    """The fused perception step on every benchmark shape (one or a few systems at full particle count,
    the 262,144-particle periodic rollout shape included) against the oracle chain."""
    from npa_b200 import sphops as sph
    w = scaled(CONFIGS[name], B=B)
    x, s, ups = make_inputs(w, seed=21)
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    xb, sb = sph.bin_particles(x.cuda(), s.cuda(), snap)
    ups = {k: v.cuda() for k, v in ups.items()}
    xr, sr = xb.clone().requires_grad_(True), sb.clone().requires_grad_(True)
    rho, blur, grad, dg = sph.perceive(xr, sr, snap)
    fw, ds, dx = _oracle_chain(xb, sb, rho, w, ups, "f64")
    fw32, ds32, dx32 = _oracle_chain(xb, sb, rho, w, ups, "f32")
    for k, t in (("rho", rho), ("rho_grad", dg), ("blur", blur), ("grad", grad)):
        assert_parity(np64(t), fw[k], fw32[k], f"{name}: {k}", proxy=True)
    torch.autograd.backward([rho, blur, grad, dg], [ups["g_rho"], ups["g_blur"], ups["g_grad"], ups["g_rho_grad"]])
    assert_parity(np64(sr.grad), ds, ds32, f"{name}: chain ds", proxy=True)
    assert_parity(np64(xr.grad)[..., : w.dim], dx, dx32, f"{name}: chain dx", proxy=True)


def test_safe_inverse_and_gradient_hybrid():
    import oracle
    from npa_b200 import sphops as sph
    w = Workload("hyb", dim=3, B=1, N=2000, C=8, eps=0.15, grid_size=(8, 8, 8))
    sph_, snap, xb, sb, mb, ups = _prepare(w, seed=4)
    rho = sph.density(xb, snap)
    M = sph.moment_matrix(xb, rho, snap)
    Minv = sph.safe_inv_sym_mat(M, rtol=1e-3)
    # same closed form; the GPU contracts products into FMAs, so agreement is to rounding
    ref = oracle.safe_inv_sym_mat(M.cpu().numpy(), 1e-3)
    np.testing.assert_allclose(Minv.cpu().numpy(), ref, rtol=1e-4, atol=1e-5 * np.abs(ref).max())
    M2 = M[..., :2, :2].contiguous()
    M2[0, :7] = 0.0                        # singular matrices take the identity branch
    inv2 = sph.safe_inv_sym_mat(M2, rtol=1e-3).cpu().numpy()
    ref2 = oracle.safe_inv_sym_mat(M2.cpu().numpy(), 1e-3)
    np.testing.assert_array_equal(inv2[0, :7], np.broadcast_to(np.eye(2, dtype=np.float32), (7, 2, 2)))
    np.testing.assert_allclose(inv2, ref2, rtol=1e-4, atol=1e-5 * np.abs(ref2).max())
    sr = sb.clone().requires_grad_(True)
    hyb = sph.gradient_hybrid(xb, rho, sr, snap)
    raw = sph.gradient(xb, rho, sb, snap)
    assert torch.allclose(hyb, raw @ Minv, rtol=1e-5, atol=1e-5 * float(raw.abs().max()))
    hyb.backward(ups["g_grad"])
    sr2 = sb.clone().requires_grad_(True)
    sph.gradient(xb, rho, sr2, snap).backward(ups["g_grad"])
    assert torch.equal(sr.grad, sr2.grad)   # the correction is detached: gradient of the raw operator
