"""The double-buffered host pipeline gives the same results as copy -> step -> copy run serially."""
import pytest
import torch

from helpers import make_grid
from npa_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu


def test_pipeline_matches_serial_execution():
    from npa_b200 import sphops as sph
    from npa_b200.pipeline import HostStepPipeline
    w = Workload("pipe", dim=3, B=2, N=4000, C=16, eps=0.12, grid_size=(10, 10, 10))
    grid = make_grid(sph, w)
    batches = []
    for k in range(5):
        x, s, ups = make_inputs(w, seed=k)
        batches.append((x.pin_memory(), s.pin_memory()))
    g_blur = torch.randn(w.B, w.N, w.C, device="cuda")

    def step(inp):
        x, s = inp
        xr, sr = x.detach().requires_grad_(True), s.detach().requires_grad_(True)
        snap = grid.instantiate(xr.detach())
        xb, sb = sph.bin_particles(xr, sr, snap)
        rho, blur, grad = sph.perceive(xb, sb, snap, with_density_gradient=False)
        torch.autograd.backward([blur, rho], [g_blur, torch.ones_like(rho)])
        return xr.grad, sr.grad

    serial = []
    for x, s in batches:
        gx, gs = step((x.cuda(), s.cuda()))
        serial.append((gx.cpu(), gs.cpu()))
    got = {}
    pipe = HostStepPipeline(step, batches[0], serial[0], depth=2)
    n = pipe.run(batches, lambda i, outs: got.__setitem__(i, [o.clone() for o in outs]))
    assert n == len(batches) and sorted(got) == list(range(len(batches)))
    for i, (gx, gs) in enumerate(serial):
        assert torch.equal(got[i][0], gx) and torch.equal(got[i][1], gs)
