"""The fused Euler update (npa_step_update_forward / backward, sphops.step_update) against the
fixtures made by the reference's NPA.forward + step_euler, against the numpy oracle on larger
seeded inputs, and against torch autograd at the limiter's singular point."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from helpers import make_grid
from npa_b200.workloads import CONFIGS, Workload

pytestmark = pytest.mark.gpu

RTOL, ATOL_SCALE = 1e-5, 1e-6  # fp32 against fp64 truth, as for the operators


def _close(got, want, name):
    want = np.asarray(want, dtype=np.float64)
    got = got.detach().cpu().numpy().astype(np.float64)
    tol = RTOL * np.abs(want) + ATOL_SCALE * max(np.abs(want).max(), 1e-30)
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{name}: {int(bad.sum())} of {bad.size} outside tolerance, worst {np.abs(got - want).max():.3e}"


def _grid_for(sph, dim, B, N, eps, boundary="clamped"):
    w = Workload("step", dim=dim, B=B, N=N, C=4, eps=eps, grid_size=(8,) * dim, boundary=boundary)
    grid = make_grid(sph, w)
    P = 2 if dim == 2 else 4
    snap = grid.instantiate(torch.zeros(B, N, P, device="cuda"))
    return grid, snap


@pytest.mark.parametrize("name", ["step_d2", "step_d3", "step_d2_all"])
def test_fixture_of_reference_step_euler(name):
    from npa_b200 import sphops as sph
    g = np.load(GOLDEN_DIR / f"{name}.npz")
    dim, eps, alpha, dt = int(g["dim"]), float(g["eps"]), float(g["alpha"]), float(g["dt"])
    B, N = g["y"].shape[:2]
    _, snap = _grid_for(sph, dim, B, N, eps)
    t = lambda k: torch.from_numpy(g[k]).cuda()
    y, xb, sb = t("y").requires_grad_(True), t("x_bin").requires_grad_(True), t("s_bin").requires_grad_(True)
    x_new, s_new = sph.step_update(y, xb, sb, snap, alpha, dt, update_mask=t("mask").reshape(B, N, 1))
    # same fp32 operations in the same order as the reference: the state is bit-identical, the
    # position differs at most by the rounding of the norm
    assert torch.equal(s_new.cpu(), torch.from_numpy(g["s_new"]))
    assert float((x_new.cpu() - torch.from_numpy(g["x_new"])).abs().max()) <= 2e-7 * float(np.abs(g["x_new"]).max())
    torch.autograd.backward([x_new, s_new], [t("up_x"), t("up_s")])
    _close(y.grad, g["g_y"], "g_y")
    assert torch.equal(xb.grad.cpu(), torch.from_numpy(g["g_x_bin"]))
    assert torch.equal(sb.grad.cpu(), torch.from_numpy(g["g_s_bin"]))


@pytest.mark.parametrize("dim,C,boundary", [(2, 16, "clamped"), (3, 32, "clamped"), (3, 5, "periodic"), (2, 7, "periodic")])
def test_seeded_inputs_against_oracle(dim, C, boundary):
    from npa_b200 import sphops as sph
    from oracle import step as step_oracle
    B, N, eps, alpha, dt = 3, 2000, 0.07, 1.3, 0.5
    P = 2 if dim == 2 else 4
    grid, snap = _grid_for(sph, dim, B, N, eps, boundary)
    g = torch.Generator().manual_seed(21)
    y = torch.randn(B, N, dim + C, generator=g) * 2.0
    xb = (torch.rand(B, N, P, generator=g) - 0.5) * 8 * eps * 1.5  # some positions outside the periodic box
    sb = torch.randn(B, N, C, generator=g)
    mask = (torch.rand(B, N, generator=g) < 0.5).float()
    up_x, up_s = torch.randn(B, N, P, generator=g), torch.randn(B, N, C, generator=g)
    wrap = boundary == "periodic"
    box = [8 * eps] * dim if wrap else None
    want_x, want_s = step_oracle.step_forward(y.numpy(), xb.numpy(), sb.numpy(), mask.numpy(), dim, eps, alpha, dt, box)
    yc = y.cuda().requires_grad_(True)
    x_new, s_new = sph.step_update(yc, xb.cuda(), sb.cuda(), snap, alpha, dt, update_mask=mask.cuda(), wrap=wrap)
    assert torch.equal(s_new.cpu(), torch.from_numpy(want_s))
    # wrapped coordinates may land on either end of the box when they hit the seam: compare modulo L
    diff = (x_new.cpu() - torch.from_numpy(want_x))[..., :dim].abs()
    if wrap:
        diff = torch.minimum(diff, (diff - 8 * eps).abs())
    assert float(diff.max()) <= 1e-6 * 8 * eps * 1.5
    if dim == 3:
        assert torch.equal(x_new[..., 3].cpu(), xb[..., 3])
    torch.autograd.backward([x_new, s_new], [up_x.cuda(), up_s.cuda()])
    want_g = step_oracle.step_backward(y.numpy(), mask.numpy(), dim, eps, alpha, dt, up_x.numpy(), up_s.numpy())
    _close(yc.grad, want_g, "g_y")
    # the wrap matches HashGrid.wrap_positions of the same grid
    if wrap:
        ref = grid.wrap_positions(torch.from_numpy(step_oracle.step_forward(
            y.numpy(), xb.numpy(), sb.numpy(), mask.numpy(), dim, eps, alpha, dt)[0]).cuda())
        d2 = (x_new[..., :dim] - ref).abs()
        d2 = torch.minimum(d2, (d2 - 8 * eps).abs())
        assert float(d2.max()) <= 1e-6 * 8 * eps * 1.5


def test_zero_displacement_and_no_mask_against_torch_autograd():
    """|dx| = 0 is the singular point of the limiter: forward gives no motion, backward k * g (torch's
    norm backward contributes zero there).  Also the mask-free path and a NULL upstream."""
    from npa_b200 import sphops as sph
    dim, C, B, N, eps, alpha, dt = 2, 4, 1, 64, 0.1, 1.5, 1.0
    _, snap = _grid_for(sph, dim, B, N, eps)
    g = torch.Generator().manual_seed(3)
    y = torch.randn(B, N, dim + C, generator=g)
    y[0, :8, :dim] = 0.0
    xb, sb = torch.randn(B, N, 2, generator=g), torch.randn(B, N, C, generator=g)
    up_x = torch.randn(B, N, 2, generator=g)

    yt = y.clone().double().requires_grad_(True)
    dx = alpha * yt[..., :dim] * eps / (1.0 + yt[..., :dim].norm(dim=-1, keepdim=True))
    xt = xb.double() + dt * dx
    xt.backward(up_x.double())

    yc = y.cuda().requires_grad_(True)
    x_new, s_new = sph.step_update(yc, xb.cuda(), sb.cuda(), snap, alpha, dt)
    assert torch.equal(x_new[0, :8].cpu(), xb[0, :8])
    _close(x_new, xt.detach().numpy(), "x_new")
    x_new.backward(up_x.cuda())  # s_new gets no upstream gradient
    _close(yc.grad, yt.grad.numpy(), "g_y")
    assert float(yc.grad[..., dim:].abs().max()) == 0.0


def test_full_size_properties():
    """Headline size: particles with mask 0 keep position and state bit for bit; no particle moves
    further than dt * alpha * eps; the gradient of masked particles is zero."""
    from npa_b200 import sphops as sph
    w = CONFIGS["cfg4_3d_splat"]
    grid = make_grid(sph, w)
    B, N, C, dim = w.B, w.N, w.C, w.dim
    g = torch.Generator(device="cuda").manual_seed(8)
    xb = (torch.rand(B, N, 4, generator=g, device="cuda") - 0.5) * 2
    sb = torch.randn(B, N, C, generator=g, device="cuda")
    y = (torch.randn(B, N, dim + C, generator=g, device="cuda") * 5).requires_grad_(True)
    mask = (torch.rand(B, N, generator=g, device="cuda") < 0.5).float()
    snap = grid.instantiate(xb)
    alpha, dt = 1.0, 1.0
    x_new, s_new = sph.step_update(y, xb, sb, snap, alpha, dt, update_mask=mask)
    still = mask == 0
    assert torch.equal(x_new[still], xb[still]) and torch.equal(s_new[still], sb[still])
    moved = (x_new - xb)[..., :dim].norm(dim=-1)
    assert float(moved.max()) <= dt * alpha * w.eps * (1 + 1e-5)
    assert torch.equal(x_new[..., 3], xb[..., 3])
    (x_new.sum() + s_new.sum()).backward()
    assert float(y.grad[still].abs().max()) == 0.0
    assert torch.isfinite(y.grad).all()


class _TinyNPA(torch.nn.Module):
    """The attributes of the reference's NPA module (models/npa.py:14-75) that a step reads."""

    def __init__(self, dim, C, hidden=32, eps0=0.1, alpha=1.0):
        super().__init__()
        self.spatial_dims, self.state_dims = dim, C
        self.register_buffer("eps0", torch.tensor([eps0]))
        self.register_buffer("alpha", torch.tensor([alpha]))
        self.state_grad = self.density_grad = self.log_norm_grad = self.log_norm_density_grad = True
        self.stopgrad_pos, self.stopgrad_state = True, False
        self.model = torch.nn.Sequential(torch.nn.Linear(2 * C + C * dim + dim, hidden), torch.nn.ReLU(),
                                         torch.nn.Linear(hidden, dim + C, bias=False))


def _reference_like_step(sph, model, x, s, grid, dt, update_prob):
    """NPA.forward + step_euler written operator by operator with torch glue (models/npa.py:87-203)."""
    from test_gpu_fusion import npa_perceive
    B, N, C = s.shape
    D = model.spatial_dims
    with torch.no_grad():
        snap = grid.instantiate(x)
    z, snap = npa_perceive(sph, x, s, grid, eps0=float(model.eps0), stopgrad_pos=True)
    x_bin, s_bin = sph.bin_particles(x, s, snap)
    y = model.model(z)
    dx = y[..., :D]
    dx = model.alpha * dx * grid.eps / (1.0 + dx.norm(dim=-1, keepdim=True))
    ds = y[..., D:]
    mask = (torch.rand(B, N, 1, device=x.device) < update_prob).float()
    if D != x.shape[-1]:
        dx = torch.cat([dx, torch.zeros(B, N, 1, device=x.device)], dim=-1).contiguous()
    return x_bin + dt * dx * mask, s_bin + dt * ds * mask


@pytest.mark.parametrize("dim", [2, 3])
def test_step_euler_equals_the_operator_sequence(dim):
    from npa_b200 import sphops as sph
    from npa_b200.stepping import step_euler
    from npa_b200.workloads import make_inputs
    w = Workload("se", dim=dim, B=2, N=3000, C=16, eps=0.12 if dim == 3 else 0.05,
                 grid_size=(10, 10, 10) if dim == 3 else (20, 20), boundary="clamped")
    x, s, _ = make_inputs(w, seed=4)
    x[..., :dim] *= 0.95 * w.grid_size[0] * w.eps
    grid = make_grid(sph, w)
    torch.manual_seed(0)
    model = _TinyNPA(dim, w.C).cuda()
    with torch.no_grad():
        for p in model.model.parameters():
            p.mul_(5.0)
    g = torch.Generator().manual_seed(2)
    up_x = torch.randn(w.B, w.N, x.shape[-1], generator=g).cuda()
    up_s = torch.randn(w.B, w.N, w.C, generator=g).cuda()
    results = []
    for fused in (True, False):
        model.zero_grad()
        xr, sr = x.cuda().requires_grad_(True), s.cuda().requires_grad_(True)
        torch.manual_seed(99)
        if fused:
            x_new, s_new, stats = step_euler(model, xr, sr, grid, dt=0.5, update_prob=0.5, intermediate=True)
            assert stats["dx_norm"].item() > 0
        else:
            x_new, s_new = _reference_like_step(sph, model, xr, sr, grid, 0.5, 0.5)
        torch.autograd.backward([x_new, s_new], [up_x, up_s])
        results.append([x_new.detach(), s_new.detach(), xr.grad, sr.grad] + [p.grad.clone() for p in model.parameters()])
    for a, b in zip(*results):
        scale = float(b.abs().max())
        assert float((a - b).abs().max()) <= 2e-5 * scale + 1e-30, (a.shape, float((a - b).abs().max()), scale)


def test_step_euler_makes_no_host_synchronisation_after_the_first_step():
    """eps0 / alpha of the model are device buffers; the step reads them once and caches the floats, so a
    training loop does not stall its launch queue on a device-to-host copy every step (the reference keeps
    them on the device and never synchronises in step_euler)."""
    from npa_b200 import sphops as sph
    from npa_b200.stepping import step_euler

    class Model(torch.nn.Module):
        def __init__(self, dim, C):
            super().__init__()
            self.spatial_dims, self.state_dims = dim, C
            self.register_buffer("eps0", torch.tensor([0.1]))
            self.register_buffer("alpha", torch.tensor([1.0]))
            width = 2 * C + C * dim + dim
            self.model = torch.nn.Sequential(torch.nn.Linear(width, 128), torch.nn.ReLU(),
                                             torch.nn.Linear(128, dim + C, bias=False))

    dim, C = 2, 16
    model = Model(dim, C).cuda()
    grid = sph.HashGrid(dim=dim, boundary="periodic", mode="grid", grid_size=(10, 10), eps=0.2, num_particles=2048,
                        batch_size=2, max_particles_per_block=32)
    g = torch.Generator().manual_seed(0)
    x = ((torch.rand(2, 2048, dim, generator=g) - 0.5) * 2.0).cuda()
    s = torch.randn(2, 2048, C, generator=g).cuda()
    step_euler(model, x, s, grid, update_prob=1.0)      # first step: reads the buffers, sizes the launches
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        x1, s1, _ = step_euler(model, x, s, grid, update_prob=1.0)
        x2, s2, _ = step_euler(model, x1, s1, grid, update_prob=1.0)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    assert torch.isfinite(x2).all() and torch.isfinite(s2).all()
    model.alpha.mul_(0.5)                               # an in-place change of the buffer is picked up
    x3, _, _ = step_euler(model, x, s, grid, update_prob=1.0)
    assert not torch.equal(x3, x1)
