"""Size-independent properties of the CUDA path at the benchmark's full sizes."""
import numpy as np
import pytest
import torch

from helpers import make_grid
from npa_b200.workloads import CONFIGS, HEADLINE, make_inputs, scaled

pytestmark = pytest.mark.gpu


def _run(w, seed=0):
    from npa_b200 import sphops as sph
    x, s, ups = make_inputs(w, seed)
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    xb, sb = sph.bin_particles(x.cuda(), s.cuda(), snap)
    return sph, snap, xb, sb, {k: v.cuda() for k, v in ups.items()}


@pytest.mark.parametrize("name", [HEADLINE, "cfg2_2d_texture_blobs", "cfg3_2d_pointmnist_strokes"])
def test_full_size_invariants(name):
    w = CONFIGS[name]
    sph, snap, xb, sb, ups = _run(w)
    xr, sr = xb.clone().requires_grad_(True), sb.clone().requires_grad_(True)
    rho, blur, grad, dg = sph.perceive(xr, sr, snap)
    for t in (rho, blur, grad, dg):
        assert torch.isfinite(t).all()
    # (1) the neighbour relation is symmetric: sum_i count_i == number of ordered pairs == sum over
    #     pairs seen from j; a constant feature is reproduced: blur of ones == sum_j v_j W_ij, and the
    #     gradient of a constant feature field is exactly zero.
    ones = torch.ones_like(sb[..., :4]).contiguous()
    assert float(sph.gradient(xb, rho, ones, snap).abs().max()) == 0.0
    # (2) linearity in the features
    a = sph.blur(xb, rho, sb, snap)
    b = sph.blur(xb, rho, 2.0 * sb, snap)
    assert torch.allclose(b, 2.0 * a, rtol=1e-6, atol=0.0)
    # (3) translation invariance: forces sum to zero over each system
    torch.autograd.backward([rho, blur, grad, dg], [ups["g_rho"], ups["g_blur"], ups["g_grad"], ups["g_rho_grad"]])
    gx = xr.grad[..., : w.dim].double()
    total = gx.sum(dim=1).abs().max().item()
    scale = gx.abs().sum(dim=1).max().item()
    assert total <= 2e-5 * scale, (total, scale)
    # (4) adjointness of blur in the features: <g, blur(s)> == <blur^T g, s> with blur^T g = ds
    lhs = (ups["g_blur"].double() * blur.detach().double()).sum() + (ups["g_grad"].double() * grad.detach().double()).sum()
    rhs = (sr.grad.double() * sb.double()).sum()
    assert abs(lhs.item() - rhs.item()) <= 1e-5 * max(abs(lhs.item()), abs(rhs.item()), 1.0) + 1e-6 * (
        ups["g_grad"].double().abs() * grad.detach().double().abs()).sum().item()
    # (5) determinism: a second run is bit-identical
    xr2, sr2 = xb.clone().requires_grad_(True), sb.clone().requires_grad_(True)
    out2 = sph.perceive(xr2, sr2, snap)
    torch.autograd.backward(list(out2), [ups["g_rho"], ups["g_blur"], ups["g_grad"], ups["g_rho_grad"]])
    assert torch.equal(out2[1], blur) and torch.equal(out2[2], grad)
    assert torch.equal(xr2.grad, xr.grad) and torch.equal(sr2.grad, sr.grad)


def test_count_symmetry_full_size():
    """sum_i count_i counts ordered pairs, so it is even after removing the N self pairs per system."""
    w = CONFIGS[HEADLINE]
    sph, snap, xb, sb, ups = _run(w, seed=1)
    cnt = sph.count(xb, snap)
    per_system = cnt.double().sum(dim=1) - w.N
    assert torch.all(per_system % 2 == 0)
    assert cnt.min().item() >= 1.0


def test_rollout_periodic_shard():
    """A few steps of the periodic rollout at one GPU's share: outputs stay finite, every output slot is
    written (poisoned buffers), and re-binning after a move keeps the particle multiset."""
    from npa_b200 import sphops as sph
    from npa_b200.workloads import smooth_velocity
    w = scaled(CONFIGS["cfg5_3d_rollout"], B=2)
    x, s, ups = make_inputs(w, 2)
    x, s = x.cuda(), s.cuda()
    grid = make_grid(sph, w)
    checksum = s.double().sum().item()
    for step in range(3):
        snap = grid.instantiate(x)
        xb, sb = sph.bin_particles(x, s, snap)
        rho, blur, grad = sph.perceive(xb, sb, snap, with_density_gradient=False)
        assert torch.isfinite(rho).all() and torch.isfinite(blur).all() and torch.isfinite(grad).all()
        assert rho.min().item() > 0.0
        moved = xb + 0.002 * smooth_velocity(xb, 3, seed=step)
        x = torch.cat([grid.wrap_positions(moved), torch.zeros_like(moved[..., :1])], dim=-1).contiguous()
        s = sb
        assert abs(s.double().sum().item() - checksum) < 1e-6 * max(1.0, abs(checksum))
