"""The cell-tile streaming engine (bulk-copy staging of neighbour cells in shared memory) against
the gather kernels and the oracle, through the C ABI.

The engine is an alternative implementation of the fused blur + gradient sweeps, switched per
direction with ``npa_tile_tuning``.  Every case runs the same call twice, engine off and on, on
poison-filled outputs, and checks that the engine really ran (results differ in the last bits or
the status word was consulted), that no bounded wait ran out, and that both agree to rounding;
one case is also held to the oracle with the parity gate.
"""
import numpy as np
import pytest
import torch

from conftest import assert_parity
from helpers import make_grid, np64, oracle_backward, oracle_forward
from npa_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu

CASES = [
    # name, workload, tuning (rows_per_stage, particles_per_tile, stages, consumer_warps, cells_per_tile), with_mass
    ("d3_clamped_c32_multichunk", Workload("t1", dim=3, B=2, N=6000, C=32, eps=0.12, grid_size=(10, 10, 10)),
     (64, 16, 2, 8, 2), False),
    ("d3_periodic_c16", Workload("t2", dim=3, B=2, N=5000, C=16, eps=0.125, grid_size=(8, 8, 8), boundary="periodic"),
     (0, 0, 0, 0, 0), True),
    ("d3_periodic_small_axes", Workload("t3", dim=3, B=1, N=600, C=8, eps=0.3, grid_size=(3, 2, 4),
                                        boundary="periodic"), (0, 0, 0, 16, 3), False),
    ("d2_clamped_c64_crowded", Workload("t4", dim=2, B=2, N=4000, C=64, eps=0.06, grid_size=(18, 18),
                                        max_particles_per_block=64), (96, 8, 3, 16, 1), True),
    ("d2_periodic_c128", Workload("t5", dim=2, B=1, N=3000, C=128, eps=0.07, grid_size=(14, 15), boundary="periodic"),
     (0, 0, 2, 8, 4), False),
    ("d3_clamped_c4_24warps", Workload("t6", dim=3, B=1, N=3000, C=4, eps=0.13, grid_size=(8, 8, 8)),
     (128, 32, 4, 24, 2), False),
]


@pytest.fixture(autouse=True)
def _engine_off_afterwards():
    from npa_b200 import _native as n
    yield
    n.tile_tuning(False, enabled=False)
    n.tile_tuning(True, enabled=False)


def _setup(w, with_mass, seed=0):
    from npa_b200 import sphops as sph
    x, s, ups = make_inputs(w, seed)
    scale = [(g if w.boundary == "periodic" else g - 2) * w.eps for g in w.grid_size[: w.dim]]
    x[..., : w.dim] *= torch.tensor(scale)
    x[:, : w.N // 5, : w.dim] *= 0.2   # crowded cells: several work items per cell, tiles longer than a stage
    mass = (torch.rand(w.B, w.N, generator=torch.Generator().manual_seed(seed + 1)) + 0.5) if with_mass else None
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    if mass is None:
        xb, sb = sph.bin_particles(x.cuda(), s.cuda(), snap)
        mb = None
    else:
        xb, sb, mb = sph.bin_particles(x.cuda(), s.cuda(), snap, mass.cuda())
    rho = sph.density(xb, snap, mb)
    return grid, snap, xb, sb, mb, rho, {k: v.cuda() for k, v in ups.items()}


def _sweeps(grid, snap, xb, sb, mb, rho, ups, moment):
    """Fused forward (+ moment), full backward and features-only backward through the native layer."""
    hg = grid.hashgrid
    B, N, C = sb.shape
    D = grid.dim
    nan = float("nan")
    blur = torch.full((B, N, C), nan, device="cuda")
    grad = torch.full((B, N, C, D), nan, device="cuda")
    mom = torch.full((B, N, D, D), nan, device="cuda") if moment else None
    hg.blur_gradient_forward(xb, rho, mb, sb, blur, grad, snap.bin_offsets, snap.block_info, moment_matrix_out=mom)
    gx, gs, gr = torch.full_like(xb, nan), torch.full_like(sb, nan), torch.full_like(rho, nan)
    hg.blur_gradient_backward(xb, rho, mb, sb, ups["g_blur"], ups["g_grad"], gx, gs, gr, snap.bin_offsets,
                              snap.block_info)
    gs2 = torch.full_like(sb, nan)
    hg.blur_gradient_backward(xb, rho, mb, sb, ups["g_blur"], ups["g_grad"], None, gs2, None, snap.bin_offsets,
                              snap.block_info)
    out = {"blur": blur, "grad": grad, "grad_x": gx, "grad_s": gs, "grad_rho": gr, "grad_s_features_only": gs2}
    if moment:
        out["moment"] = mom
    return out


@pytest.mark.parametrize("name,w,tuning,with_mass", CASES, ids=[c[0] for c in CASES])
def test_engine_matches_gather_kernels(name, w, tuning, with_mass):
    from npa_b200 import _native as n
    args = _setup(w, with_mass)
    n.tile_tuning(False, enabled=False)
    n.tile_tuning(True, enabled=False)
    ref = _sweeps(*args, moment=True)
    rows, tp, stages, warps, cells = tuning
    n.tile_tuning(False, True, rows, tp, stages, warps, cells)
    n.tile_tuning(True, True, rows, tp, stages, 8 if warps == 24 else warps, cells)
    got = _sweeps(*args, moment=True)
    torch.cuda.synchronize()
    assert n.tile_status() == 0, "a bounded wait of the engine ran out"
    differs = False
    for k in ref:
        a, b = got[k].double(), ref[k].double()
        assert torch.isfinite(a).all(), f"{name}: {k} has unwritten or non-finite entries"
        scale = float(b.abs().max())
        err = float((a - b).abs().max())
        # two fp32 evaluations of the same sums in different orders
        assert err <= 2e-6 * scale, f"{name}: {k} differs from the gather kernels by {err:.3e} (scale {scale:.3e})"
        differs = differs or err > 0.0
    assert differs, "identical bits everywhere: the engine did not take the call"


def test_engine_against_oracle():
    from npa_b200 import _native as n
    w = Workload("t_oracle", dim=3, B=1, N=8000, C=32, eps=0.11, grid_size=(12, 12, 12))
    grid, snap, xb, sb, mb, rho, ups = _setup(w, with_mass=False, seed=3)
    n.tile_tuning(False, True, 0, 0, 0, 0, 0)
    n.tile_tuning(True, True, 0, 0, 0, 0, 0)
    got = _sweeps(grid, snap, xb, sb, mb, rho, ups, moment=False)
    torch.cuda.synchronize()
    assert n.tile_status() == 0
    want = oracle_forward(xb, w, ("blur", "grad"), s=sb, rho_in=rho)
    want32 = oracle_forward(xb, w, ("blur", "grad"), s=sb, rho_in=rho, precision="f32")
    for k in ("blur", "grad"):
        assert_parity(np64(got[k]), want[k], want32[k], f"engine: {k}", proxy=True)
    dx, ds, dr = oracle_backward(xb, w, s=sb, rho_in=rho, g_blur=ups["g_blur"], g_grad=ups["g_grad"])
    dx32, ds32, dr32 = oracle_backward(xb, w, s=sb, rho_in=rho, g_blur=ups["g_blur"], g_grad=ups["g_grad"],
                                       precision="f32")
    assert_parity(np64(got["grad_x"])[..., :3], dx, dx32, "engine: grad_x", proxy=True)
    assert float(got["grad_x"][..., 3].abs().max()) == 0.0
    assert_parity(np64(got["grad_s"]), ds, ds32, "engine: grad_s", proxy=True)
    assert_parity(np64(got["grad_s_features_only"]), ds, ds32, "engine: grad_s (features only)", proxy=True)
    assert_parity(np64(got["grad_rho"]), dr, dr32, "engine: grad_rho", proxy=True)


def test_packed_perception_on_the_engine():
    """perceive_features (blur + gradient + moment + packed epilogue in one sweep) gives the same rows."""
    from npa_b200 import _native as n, sphops as sph
    w = Workload("t_pack", dim=3, B=2, N=5000, C=16, eps=0.12, grid_size=(10, 10, 10))
    grid, snap, xb, sb, mb, rho, ups = _setup(w, with_mass=False, seed=5)
    z_ref = sph.perceive_features(xb, sb, snap, 0.1)
    n.tile_tuning(False, True, 0, 0, 0, 0, 0)
    z = sph.perceive_features(xb, sb, snap, 0.1)
    torch.cuda.synchronize()
    assert n.tile_status() == 0
    assert not torch.equal(z, z_ref)
    scale = float(z_ref.abs().max())
    assert float((z - z_ref).abs().max()) <= 1e-5 * scale


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier that nothing completes returns after its limit with the time-out code; the
    context stays usable (no trap, no fault, no endless loop)."""
    from npa_b200 import _native as n
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rc = n.lib.npa_tile_wait_selftest(2000, n.ptr(res), n.current_stream())
    n.check(rc)
    torch.cuda.synchronize()
    assert int(res.item()) == 1
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
