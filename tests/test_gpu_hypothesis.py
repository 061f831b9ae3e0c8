"""Randomised geometry: binning stays bit-exact and the neighbour count stays exact (clamped grids)
against the oracles for arbitrary dimensions, grid sizes, particle counts and work-item sizes."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

from helpers import make_grid, oracle_binning, oracle_forward
from npa_b200.workloads import Workload

pytestmark = pytest.mark.gpu


@st.composite
def geometries(draw):
    dim = draw(st.sampled_from([2, 3]))
    mode = draw(st.sampled_from(["grid", "grid", "particle"]))
    boundary = draw(st.sampled_from(["clamped", "periodic"]))
    if mode == "particle":
        size = draw(st.sampled_from([2, 4, 8, 16]))
        grid = (size,) * dim
    else:
        grid = tuple(draw(st.integers(1, 12)) for _ in range(dim))
    eps = draw(st.sampled_from([0.05, 0.1, 0.125, 0.2, 1.0 / 3.0]))
    B = draw(st.integers(1, 3))
    N = draw(st.integers(1, 700))
    mpb = draw(st.sampled_from([1, 3, 32, 64]))
    seed = draw(st.integers(0, 2 ** 16))
    spread = draw(st.sampled_from([0.3, 1.0, 1.7]))   # fraction of the box the particles cover (may exceed it)
    return Workload("hyp", dim=dim, B=B, N=N, C=4, eps=eps, grid_size=grid, boundary=boundary, mode=mode,
                    max_particles_per_block=mpb), seed, spread


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(geometries())
def test_binning_and_count_on_random_geometries(case):
    from npa_b200 import sphops as sph
    w, seed, spread = case
    g = torch.Generator().manual_seed(seed)
    box = torch.tensor([n * w.eps for n in w.grid_size[: w.dim]])
    x = torch.zeros(w.B, w.N, w.P)
    x[..., : w.dim] = (torch.rand(w.B, w.N, w.dim, generator=g) - 0.5) * box * spread
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    perm, offsets, info = oracle_binning(x, w)
    np.testing.assert_array_equal(snap.permutation.cpu().numpy(), perm)
    np.testing.assert_array_equal(snap.bin_offsets.cpu().numpy(), offsets)
    np.testing.assert_array_equal(snap.block_info.cpu().numpy(), info)
    # neighbour count: exact whenever the grid sees every neighbour (particles inside a clamped grid,
    # or any periodic grid whose box is at least two cut-off radii wide)
    inside = spread <= 1.0 if w.boundary == "clamped" else min(w.grid_size[: w.dim]) >= 2
    if inside:
        xb, _ = sph.bin_particles(x.cuda(), torch.zeros(w.B, w.N, 4, device="cuda"), snap)
        ref = oracle_forward(xb, w, ("count",))["count"]
        got = sph.count(xb, snap).cpu().numpy()
        if w.boundary == "clamped":
            np.testing.assert_array_equal(got, ref)
        else:
            # a wrapped displacement is rounded differently from torch's remainder: pairs within one
            # ulp of the cut-off may flip
            assert np.abs(got - ref).max() <= 1.0 and (got != ref).mean() < 0.01
