"""Bit-exact parity of the GPU binning (through the sphops API / C ABI) with the numpy oracle."""
import numpy as np
import pytest
import torch

from helpers import make_grid, oracle_binning
from npa_b200.workloads import CONFIGS, Workload, make_positions, scaled

pytestmark = pytest.mark.gpu

CASES = [
    Workload("b_2d_clamped", dim=2, B=3, N=1000, C=4, eps=0.1, grid_size=(10, 12)),
    Workload("b_2d_periodic_odd", dim=2, B=2, N=777, C=4, eps=0.09, grid_size=(11, 13), boundary="periodic"),
    Workload("b_2d_morton", dim=2, B=2, N=2048, C=4, eps=1 / 16, grid_size=(16, 16), mode="particle",
             boundary="periodic"),
    Workload("b_3d_clamped", dim=3, B=2, N=3000, C=4, eps=0.15, grid_size=(8, 6, 10)),
    Workload("b_3d_periodic", dim=3, B=2, N=4096, C=4, eps=0.125, grid_size=(8, 8, 8), boundary="periodic"),
    Workload("b_3d_morton_clamped", dim=3, B=1, N=5000, C=4, eps=0.125, grid_size=(8, 8, 8), mode="particle"),
    Workload("b_tiny_mpb", dim=2, B=2, N=300, C=4, eps=0.25, grid_size=(4, 4), max_particles_per_block=7),
    Workload("b_big_table", dim=3, B=2, N=20000, C=4, eps=1 / 24, grid_size=(24, 24, 24)),  # > shared-histogram limit
]


def _check(sph, w, x_cpu):
    grid = make_grid(sph, w)
    snap = grid.instantiate(x_cpu.cuda())
    perm, offsets, info = oracle_binning(x_cpu, w)
    np.testing.assert_array_equal(snap.bin_offsets.cpu().numpy(), offsets, err_msg=f"{w.name}: bin_offsets")
    np.testing.assert_array_equal(snap.permutation.cpu().numpy(), perm, err_msg=f"{w.name}: permutation")
    np.testing.assert_array_equal(snap.block_info.cpu().numpy(), info, err_msg=f"{w.name}: block_info")
    return snap


@pytest.mark.parametrize("w", CASES, ids=lambda w: w.name)
def test_binning_bit_exact(w):
    from npa_b200 import sphops as sph
    g = torch.Generator().manual_seed(11)
    scale = 1.4 if w.boundary == "periodic" else 1.1          # some particles outside the domain
    x = (torch.rand(w.B, w.N, w.P, generator=g) - 0.5) * scale
    x[:, 5] = x[:, 4]                                          # coincident particles
    x[:, : w.N // 4] *= 0.2                                    # crowd a few cells beyond MPB
    _check(sph, w, x)


def test_binning_all_in_one_cell_and_empty_cells():
    from npa_b200 import sphops as sph
    w = Workload("one_cell", dim=2, B=2, N=513, C=4, eps=0.1, grid_size=(8, 8), max_particles_per_block=32)
    x = torch.full((w.B, w.N, 2), 0.013)
    snap = _check(sph, w, x)
    # stable order inside the single occupied cell: the permutation is the identity
    assert torch.equal(snap.permutation.cpu(), torch.arange(w.N, dtype=torch.int32).expand(w.B, -1))


@pytest.mark.parametrize("N", [65536, 300000])
def test_binning_collapsed_system_is_ranked_in_linear_time(N):
    """Every particle of a large system in one cell (a diverged rollout, or particles clamped into an
    edge cell), next to a system with a few crowded cells: bit-exact and stable, and the grid build
    stays far from the quadratic per-cell scan (which needs N^2 / 2 comparisons: seconds at this size)."""
    import time
    from npa_b200 import sphops as sph
    w = Workload("collapsed", dim=3, B=2, N=N, C=4, eps=0.1, grid_size=(12, 12, 12), max_particles_per_block=64)
    g = torch.Generator().manual_seed(2)
    x = torch.zeros(w.B, w.N, 4)
    x[0, :, :3] = 0.031 + 0.01 * torch.rand(w.N, 3, generator=g)            # one cell holds the whole system
    x[1, :, :3] = (torch.rand(w.N, 3, generator=g) - 0.5) * 1.1
    x[1, : w.N // 2, :3] = x[1, : w.N // 2, :3] * 0.05                        # half the system in a handful of cells
    snap = _check(sph, w, x)
    assert torch.equal(snap.permutation[0].cpu(), torch.arange(w.N, dtype=torch.int32))
    grid = make_grid(sph, w)
    xc = x.cuda()
    grid.instantiate(xc)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(5):
        grid.instantiate(xc)
    torch.cuda.synchronize()
    per_build = (time.perf_counter() - t0) / 5
    assert per_build < 5e-3, f"grid build of a collapsed system took {per_build * 1e3:.2f} ms"


def test_binning_is_deterministic_and_reusable():
    from npa_b200 import sphops as sph
    w = scaled(CONFIGS["cfg2_2d_texture_blobs"], B=2, N=8192)
    x = make_positions(w, seed=3).cuda()
    grid = make_grid(sph, w)
    a = grid.instantiate(x)
    b = grid.instantiate(x)          # same grid object, scratch reused
    assert torch.equal(a.permutation, b.permutation)
    assert torch.equal(a.bin_offsets, b.bin_offsets)
    assert torch.equal(a.block_info, b.block_info)


@pytest.mark.parametrize("name", ["cfg1_2d_growing", "cfg2_2d_texture_blobs", "cfg3_2d_pointmnist_strokes",
                                  "cfg4_3d_splat"])
def test_binning_benchmark_shapes(name):
    from npa_b200 import sphops as sph
    w = CONFIGS[name]
    _check(sph, w, make_positions(w, seed=5))


def test_binning_rollout_shape_one_gpu_shard():
    """The 3D periodic rollout configuration at the size one of eight GPUs holds (8 systems)."""
    from npa_b200 import sphops as sph
    w = scaled(CONFIGS["cfg5_3d_rollout"], B=2)
    _check(sph, w, make_positions(w, seed=6))


def test_bin_unbin_round_trip_and_gradients():
    from npa_b200 import sphops as sph
    w = Workload("rt", dim=3, B=2, N=1500, C=7, eps=0.2, grid_size=(6, 6, 6))
    g = torch.Generator().manual_seed(2)
    x = ((torch.rand(w.B, w.N, 4, generator=g) - 0.5)).cuda()
    s = torch.randn(w.B, w.N, w.C, generator=g).cuda()
    m = (torch.rand(w.B, w.N, generator=g) + 0.1).cuda()
    grid = make_grid(sph, w)
    snap = grid.instantiate(x)
    xr, sr, mr = x.clone().requires_grad_(True), s.clone().requires_grad_(True), m.clone().requires_grad_(True)
    xb, sb, mb = sph.bin_particles(xr, sr, snap, mr)
    perm = snap.permutation.long()
    # forward: out[perm[i]] = in[i]
    exp = torch.empty_like(s)
    exp.scatter_(1, perm.unsqueeze(-1).expand(-1, -1, w.C), s)
    assert torch.equal(sb.detach(), exp)
    x0, s0, m0 = sph.unbin_particles(xb.detach(), sb.detach(), snap, mb.detach())
    assert torch.equal(x0, x) and torch.equal(s0, s) and torch.equal(m0, m)
    # backward of a permutation is the inverse permutation of the upstream gradient
    gx, gs, gm = torch.randn_like(xb), torch.randn_like(sb), torch.randn_like(mb)
    torch.autograd.backward([xb, sb, mb], [gx, gs, gm])
    assert torch.equal(sr.grad, torch.gather(gs, 1, perm.unsqueeze(-1).expand(-1, -1, w.C)))
    assert torch.equal(xr.grad, torch.gather(gx, 1, perm.unsqueeze(-1).expand(-1, -1, 4)))
    assert torch.equal(mr.grad, torch.gather(gm, 1, perm))
    # mass=None returns two tensors
    assert len(sph.bin_particles(x, s, snap)) == 2


def test_cells_are_contiguous_and_sorted():
    """Size-independent property: binned particles are sorted by cell hash and offsets delimit them."""
    from npa_b200 import sphops as sph
    from oracle.binning import cell_ids
    w = CONFIGS["cfg4_3d_splat"]
    x = make_positions(w, seed=9)
    grid = make_grid(sph, w)
    snap = grid.instantiate(x.cuda())
    xb, _ = sph.bin_particles(x.cuda(), torch.zeros(w.B, w.N, 4, device="cuda"), snap)
    ids = cell_ids(xb.cpu().numpy(), w.dim, w.grid_size, w.eps, False, False)
    assert (np.diff(ids, axis=1) >= 0).all()
    off = snap.bin_offsets.cpu().numpy().astype(np.int64)
    cells = grid.num_cells
    for b in range(w.B):
        counts = np.bincount(ids[b], minlength=cells)
        np.testing.assert_array_equal(np.diff(off[b * cells:(b + 1) * cells + 1]), counts)
    assert off[-1] == w.B * w.N
