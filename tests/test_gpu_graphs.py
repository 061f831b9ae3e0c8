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
