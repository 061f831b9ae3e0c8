"""The multi-step perception rollout (npa_b200.rollout) against the same loop written with the public
sphops API and autograd."""
import pytest
import torch

from npa_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("w", [
    Workload("r3", dim=3, B=2, N=3000, C=16, eps=0.125, grid_size=(8, 8, 8), boundary="periodic"),
    Workload("r2", dim=2, B=3, N=1500, C=8, eps=0.08, grid_size=(14, 14)),
], ids=lambda w: w.name)
def test_rollout_matches_the_public_api_loop(w):
    from npa_b200 import sphops as sph
    from npa_b200.rollout import PerceptionRollout, VelocityField
    steps, dt = 4, 0.004
    x0, s0, ups = make_inputs(w, seed=2)
    box = torch.tensor([g * w.eps for g in w.grid_size[: w.dim]])
    x0[..., : w.dim] *= box * (1.0 if w.boundary == "periodic" else 0.8)
    x0, s0 = x0.cuda(), s0.cuda()
    ups = {k: v.cuda() for k, v in ups.items()}
    grid = sph.HashGrid(dim=w.dim, boundary=w.boundary, mode="grid", grid_size=w.grid_size, eps=w.eps,
                        num_particles=w.N, batch_size=w.B, max_particles_per_block=32)
    vel = VelocityField(w.dim, x0.device, seed=4)
    roll = PerceptionRollout(grid, w.C, steps, dt, vel)
    x, s = x0.clone(), s0.clone()
    gx, gs = roll.run(x, s, ups)
    rho, blur, grad = roll.rho.clone(), roll.blur.clone(), roll.grad.clone()

    # the same loop with the public API: instantiate, bin, perceive, move, wrap; backward through the last step
    xr, sr = x0.clone(), s0.clone()
    for k in range(steps):
        last = k == steps - 1
        if last:
            xr.requires_grad_(True)
            sr.requires_grad_(True)
        snap = grid.instantiate(xr.detach())
        xb, sb = sph.bin_particles(xr, sr, snap)
        r, bl, gr = sph.perceive(xb, sb, snap, with_density_gradient=False)
        if not last:
            xn = xb[..., : w.dim] + dt * vel(xb)
            if w.boundary == "periodic":
                xn = grid.wrap_positions(xn)
            xr = xb.clone()
            xr[..., : w.dim] = xn
            sr = sb
    assert torch.equal(x, xr.detach()), "positions entering the last step differ"
    assert torch.equal(s, sr.detach())
    assert torch.equal(rho, r) and torch.equal(blur, bl) and torch.equal(grad, gr)
    torch.autograd.backward([r, bl, gr], [ups["g_rho"], ups["g_blur"], ups["g_grad"]])
    assert torch.equal(gx, xr.grad), "gradient with respect to the positions of the last step differs"
    assert torch.equal(gs, sr.grad)
