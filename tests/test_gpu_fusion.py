"""Sibling-output fusion behind the per-operator API (enable_fusion) and the call sequence of the
reference's NPA.perceive (models/npa.py:87-137) on top of it."""
import pytest
import torch

from helpers import make_grid
from npa_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture
def fusion():
    from npa_b200 import sphops as sph
    sph.enable_fusion(True)
    yield sph
    sph.enable_fusion(False)


def _log_normalize(v):
    n = v.norm(dim=-1, keepdim=True)
    return torch.log(1.0 + n) * torch.nn.functional.normalize(v, dim=-1)


def npa_perceive(sph, x, s, grid, eps0=0.1, stopgrad_pos=True):
    """The operator calls and glue of NPA.perceive, written against the public sphops API."""
    B, N, C = s.shape
    with torch.no_grad():
        snap = grid.instantiate(x)
    x_bin, s_bin = sph.bin_particles(x, s, snap)
    xp = x_bin.detach() if stopgrad_pos else x_bin
    rho = sph.density(xp, snap)
    blur_s = sph.blur(xp, rho, s_bin, snap)
    grad_s = sph.gradient_hybrid(xp, rho, s_bin, snap)
    coef = grid.eps / eps0
    grad_s = _log_normalize(grad_s * coef)
    grad_rho = sph.density_gradient(xp, snap) * (coef ** (1 + grid.dim)) / N
    z = torch.cat([s_bin, blur_s, grad_s.view(B, N, -1), _log_normalize(grad_rho)], dim=-1)
    return z, snap


@pytest.mark.parametrize("dim,boundary,stopgrad", [(3, "clamped", True), (3, "clamped", False),
                                                   (2, "periodic", True), (2, "periodic", False)])
def test_npa_perceive_sequence_fused_equals_unfused(fusion, dim, boundary, stopgrad):
    sph = fusion
    w = Workload("fuse", dim=dim, B=2, N=3000, C=16, eps=0.12 if dim == 3 else 0.05,
                 grid_size=(10, 10, 10) if dim == 3 else (20, 20), boundary=boundary)
    x, s, _ = make_inputs(w, seed=3)
    x[..., :dim] *= 0.95 * w.grid_size[0] * w.eps
    grid = make_grid(sph, w)
    g = torch.Generator().manual_seed(1)
    up = torch.randn(w.B, w.N, 2 * w.C + w.C * dim + dim, generator=g).cuda()
    results = []
    for fused in (True, False):
        sph.enable_fusion(fused)
        xr, sr = x.cuda().requires_grad_(True), s.cuda().requires_grad_(True)
        z, snap = npa_perceive(sph, xr, sr, grid, stopgrad_pos=stopgrad)
        if fused:
            assert not snap.parked, f"unclaimed parked outputs: {list(snap.parked)}"
        z.backward(up)
        results.append((z.detach(), sr.grad, xr.grad))
    (zf, gsf, gxf), (zu, gsu, gxu) = results
    # the fused sweep sums the moment matrix in a different order: equal to rounding, not bit-identical
    assert torch.allclose(zf, zu, rtol=1e-4, atol=1e-5 * float(zu.abs().max()))
    scale = gsu.abs().max()
    assert torch.allclose(gsf, gsu, rtol=1e-4, atol=1e-5 * float(scale))
    if stopgrad:
        assert gxf is None or float(gxf.abs().max()) == 0.0
    else:
        assert torch.allclose(gxf, gxu, rtol=1e-4, atol=1e-5 * float(gxu.abs().max()))


@pytest.fixture
def per_particle_density_sweep():
    """The density-only sweep shares candidates between the particles of a tile and sums in another order
    than the per-particle sweep the fused call (density + density gradient) runs: with the shared sweep
    switched off a claimed output is bit-identical to the operator's own launch."""
    from npa_b200 import _native as n
    n.check(n.lib.npa_scalar_sweep_tuning(0))
    yield
    n.check(n.lib.npa_scalar_sweep_tuning(3))


def test_parked_outputs_are_only_claimed_by_the_same_inputs(fusion, per_particle_density_sweep):
    sph = fusion
    w = Workload("park", dim=2, B=1, N=1500, C=8, eps=0.06, grid_size=(18, 18))
    x, s, _ = make_inputs(w, seed=5)
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    xb, sb = sph.bin_particles(x.cuda(), s.cuda(), snap)
    sph.enable_fusion(False)
    ref_dg = sph.density_gradient(xb, snap)
    ref_rho = sph.density(xb, snap)
    ref_grad = sph.gradient(xb, ref_rho, sb, snap)
    ref_grad2 = sph.gradient(xb, ref_rho, 2.0 * sb, snap)
    ref_m = sph.moment_matrix(xb, ref_rho, snap)
    sph.enable_fusion(True)

    rho = sph.density(xb, snap)
    assert torch.equal(rho, ref_rho) and "density_gradient" in snap.parked
    # a different tensor object (even with the same storage) does not claim the parked output
    other = sph.density_gradient(xb.detach(), snap)
    assert torch.equal(other, ref_dg) and "density_gradient" in snap.parked
    assert torch.equal(sph.density_gradient(xb, snap), ref_dg) and "density_gradient" not in snap.parked

    sph.blur(xb, rho, sb, snap)
    s2 = 2.0 * sb
    assert torch.equal(sph.gradient(xb, rho, s2, snap), ref_grad2)        # other features: own kernel
    assert "gradient" in snap.parked
    with torch.no_grad():
        m = sph.moment_matrix(xb, rho, snap)                               # claimed (no autograd wanted)
        assert torch.allclose(m, ref_m, rtol=1e-5, atol=1e-6 * float(ref_m.abs().max()))
    assert "moment_matrix" not in snap.parked
    assert torch.equal(sph.gradient(xb, rho, sb, snap), ref_grad) and "gradient" not in snap.parked

    # an in-place change of an input after parking invalidates the parked sibling
    sph.blur(xb, rho, sb, snap)
    sb.mul_(2.0)
    assert torch.equal(sph.gradient(xb, rho, sb, snap), ref_grad2)
    # a differentiable moment matrix is computed by its own node, not taken from the parking lot
    sph.blur(xb, rho, sb, snap)
    rr = rho.clone().requires_grad_(True)
    m = sph.moment_matrix(xb, rr, snap)
    assert m.requires_grad


def test_fused_moment_equals_single_operator():
    from npa_b200 import sphops as sph
    for dim, grid_size, eps in ((2, (16, 16), 0.07), (3, (8, 8, 8), 0.14)):
        w = Workload("mom", dim=dim, B=2, N=2500, C=12, eps=eps, grid_size=grid_size)
        x, s, _ = make_inputs(w, seed=8)
        grid = make_grid(sph, w)
        snap = grid.instantiate(x.cuda())
        xb, sb = sph.bin_particles(x.cuda(), s.cuda(), snap)
        rho = sph.density(xb, snap)
        blur, grad, mom = sph.BlurGradient.apply(xb, sb, rho, None, snap)
        assert torch.equal(blur, sph.blur(xb, rho, sb, snap))
        assert torch.equal(grad, sph.gradient(xb, rho, sb, snap))
        ref = sph.moment_matrix(xb, rho, snap)
        assert torch.allclose(mom, ref, rtol=1e-5, atol=1e-6 * float(ref.abs().max()))


@pytest.mark.parametrize("dim,boundary,C,stopgrad,log_norm", [
    (3, "clamped", 16, True, True), (3, "clamped", 32, False, True), (2, "periodic", 16, True, True),
    (2, "clamped", 6, False, True), (2, "clamped", 16, False, False), (3, "periodic", 5, True, True),
    (2, "clamped", 64, False, True), (2, "clamped", 132, True, True)])
def test_packed_perception_equals_the_operator_sequence(dim, boundary, C, stopgrad, log_norm):
    """perceive_features (two sweeps + fused epilogue) against the per-operator calls + torch glue."""
    from npa_b200 import sphops as sph
    sph.enable_fusion(False)
    w = Workload("pack", dim=dim, B=2, N=2500, C=C, eps=0.12 if dim == 3 else 0.05,
                 grid_size=(10, 10, 10) if dim == 3 else (20, 20), boundary=boundary)
    x, s, _ = make_inputs(w, seed=11)
    x[..., :dim] *= 0.95 * w.grid_size[0] * w.eps
    x[:, 7] = x[:, 6]                       # a coincident pair
    x[:, -1, :dim] = 0.49 * w.grid_size[0] * w.eps   # an isolated particle: singular moment matrix -> identity
    grid = make_grid(sph, w)
    eps0 = 0.07
    up = torch.randn(w.B, w.N, 2 * C + C * dim + dim, generator=torch.Generator().manual_seed(2)).cuda()

    def reference(xr, sr):
        snap = grid.instantiate(xr.detach())
        x_bin, s_bin = sph.bin_particles(xr, sr, snap)
        xp = x_bin.detach() if stopgrad else x_bin
        rho = sph.density(xp, snap)
        blur_s = sph.blur(xp, rho, s_bin, snap)
        g = sph.gradient_hybrid(xp, rho, s_bin, snap) * (grid.eps / eps0)
        dg = sph.density_gradient(xp, snap) * ((grid.eps / eps0) ** (1 + dim)) / w.N
        if log_norm:
            g, dg = _log_normalize(g), _log_normalize(dg)
        return torch.cat([s_bin, blur_s, g.view(w.B, w.N, -1), dg], dim=-1)

    def packed(xr, sr):
        snap = grid.instantiate(xr.detach())
        x_bin, s_bin = sph.bin_particles(xr, sr, snap)
        xp = x_bin.detach() if stopgrad else x_bin
        return sph.perceive_features(xp, s_bin, snap, eps0, log_norm_grad=log_norm, log_norm_density_grad=log_norm)

    outs = []
    for fn in (reference, packed):
        xr, sr = x.cuda().requires_grad_(True), s.cuda().requires_grad_(True)
        z = fn(xr, sr)
        z.backward(up)
        outs.append((z.detach(), sr.grad, xr.grad))
    (zr, gsr, gxr), (zp, gsp, gxp) = outs
    assert zp.shape == zr.shape
    assert torch.allclose(zp, zr, rtol=1e-4, atol=1e-5 * float(zr.abs().max()))
    assert torch.allclose(gsp, gsr, rtol=1e-4, atol=1e-5 * float(gsr.abs().max()))
    if stopgrad:
        assert gxp is None or float(gxp.abs().max()) == 0.0
    else:
        assert torch.allclose(gxp, gxr, rtol=1e-4, atol=2e-5 * float(gxr.abs().max()))
    with torch.no_grad():                   # inference path keeps no tensor for backward
        assert torch.equal(packed(x.cuda(), s.cuda()), zp)


def test_unclaimed_parked_outputs_do_not_accumulate(fusion):
    """A caller that uses only density + blur never claims the parked gradient / moment matrix / density
    gradient.  They are dropped at the next instantiate(), and the weakly held input keys keep nothing alive:
    device memory stays flat over many steps, also while older snapshots are kept (a BPTT rollout)."""
    sph = fusion
    w = Workload("park", dim=3, B=2, N=4000, C=16, eps=0.12, grid_size=(10, 10, 10))
    x, s, _ = make_inputs(w, seed=9)
    x, s = x.cuda(), s.cuda()
    grid = make_grid(sph, w)
    kept = []

    def step():
        snap = grid.instantiate(x)
        xb, sb = sph.bin_particles(x, s, snap)
        rho = sph.density(xb, snap)
        out = sph.blur(xb, rho, sb, snap)
        kept.append(snap)          # snapshots of every step stay alive, their parked outputs must not
        return float(out.sum())

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    snapshots_only = sum(t.numel() * t.element_size() for sn in kept[-1:] for t in (sn.bin_offsets, sn.permutation, sn.block_info))
    base = torch.cuda.memory_allocated()
    for _ in range(10):
        step()
    torch.cuda.synchronize()
    grown = torch.cuda.memory_allocated() - base
    # ten more snapshots (offsets, permutation, work list) and nothing else
    assert grown <= 10 * snapshots_only + (1 << 20), f"device memory grew by {grown} bytes over ten steps"
    assert all(not sn.parked for sn in kept[:-1])
