"""A forward perception step recorded in a CUDA graph replays to the same result as the eager calls."""
import pytest
import torch

from helpers import make_grid
from npa_b200.workloads import CONFIGS, make_inputs, scaled

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,B", [("cfg1_2d_growing", 1), ("cfg3_2d_pointmnist_strokes", 32)])
def test_graphed_step_equals_eager(name, B):
    from npa_b200 import sphops as sph
    from npa_b200.graphs import GraphedPerception
    w = scaled(CONFIGS[name], B=B)
    grid = make_grid(sph, w)
    graphed = GraphedPerception(grid, w.C, eps0=0.1)
    for seed in (1, 2):                      # replay twice with different inputs
        x, s, _ = make_inputs(w, seed=seed)
        x, s = x.cuda(), s.cuda()
        z, xb, sb = graphed(x, s)
        with torch.no_grad():
            snap = grid.instantiate(x)
            xb_e, sb_e = sph.bin_particles(x, s, snap)
            z_e = sph.perceive_features(xb_e, sb_e, snap, 0.1)
        assert torch.equal(graphed.snapshot.permutation, snap.permutation)
        assert torch.equal(xb, xb_e) and torch.equal(sb, sb_e)
        assert torch.equal(z, z_e)


def test_graphed_euler_rollout_equals_eager():
    """Eight graphed steps of a small periodic system give the positions and states of eight eager
    steps (update_prob = 1: no random mask, so the two runs are comparable)."""
    from npa_b200 import sphops as sph
    from npa_b200.graphs import GraphedEulerStep
    from npa_b200.stepping import step_euler
    from npa_b200.workloads import Workload
    from test_gpu_step_update import _TinyNPA
    w = Workload("roll", dim=2, B=16, N=512, C=16, eps=0.06, grid_size=(16, 16), boundary="periodic")
    grid = make_grid(sph, w)
    torch.manual_seed(5)
    model = _TinyNPA(2, w.C).cuda()
    x, s, _ = make_inputs(w, seed=3)
    x, s = x.cuda(), s.cuda()
    graphed = GraphedEulerStep(model, grid, w.C, dt=1.0, update_prob=1.0, wrap=True)
    xg, sg = graphed.rollout(x, s, 8)
    with torch.no_grad():
        xe, se = x, s
        for _ in range(8):
            xe, se, _ = step_euler(model, xe, se, grid, dt=1.0, update_prob=1.0, wrap=True)
    assert torch.allclose(xg, xe, rtol=0, atol=1e-6) and torch.allclose(sg, se, rtol=1e-5, atol=1e-5)
    assert float(xg.abs().max()) <= 0.5 * 16 * 0.06 + 1e-6  # wrapped into the box
