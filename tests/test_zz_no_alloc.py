"""The allocation-free binning entry point, ``npa_grid_build_static``.

Some hosts own every byte of device memory themselves (fixed arenas set up at start-up) and do
not allow a plugin to call cudaMalloc; for them the library carries its binning work arrays in a
fixed built-in device array.  This test calls that entry point through the C ABI and checks, on
two calls in a row (the array keeps the previous call's contents), that its three outputs are
bit-identical to those of ``npa_grid_build`` with caller-provided scratch.  The file name makes
pytest collect it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build_both(n, desc, x, scratch_bytes, cells, max_blocks, B, N):
    dev = x.device
    outs = []
    for static in (False, True):
        perm = torch.full((B, N), -1, dtype=torch.int32, device=dev)
        offs = torch.full((B * cells + 1,), -1, dtype=torch.int32, device=dev)
        info = torch.full((max_blocks, 4), -1, dtype=torch.int32, device=dev)
        stream = n.current_stream()
        if static:
            rc = n.lib.npa_grid_build_static(ctypes.byref(desc), n.ptr(x), n.ptr(perm), n.ptr(offs), n.ptr(info),
                                             stream)
        else:
            scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
            rc = n.lib.npa_grid_build(ctypes.byref(desc), n.ptr(x), n.ptr(perm), n.ptr(offs), n.ptr(info),
                                      n.ptr(scratch), scratch_bytes, stream)
        assert rc == n.NPA_OK, n.last_error()
        torch.cuda.synchronize()
        outs.append((perm, offs, info))
    return outs


def test_static_scratch_build_matches_scratch_build_twice():
    from npa_b200 import _native as n
    B, N = 3, 20000
    desc = n.make_grid(3, "clamped", "grid", (16, 16, 16), 1.0 / 16, B, N, 32)
    ref = ctypes.byref(desc)
    cells, max_blocks = int(n.lib.npa_grid_num_cells(ref)), int(n.lib.npa_grid_max_blocks(ref))
    need = int(n.lib.npa_grid_scratch_bytes(ref))
    assert need <= 8 << 20
    g = torch.Generator().manual_seed(17)
    for call in range(2):                              # second call: different positions, stale array contents
        x = (torch.rand(B, N, 4, generator=g) - 0.5).cuda()
        (p0, o0, i0), (p1, o1, i1) = _build_both(n, desc, x, need, cells, max_blocks, B, N)
        assert torch.equal(p0, p1), f"call {call}: permutation differs"
        assert torch.equal(o0, o1), f"call {call}: bin_offsets differ"
        assert torch.equal(i0, i1), f"call {call}: block_info differs"
        assert int(o1[-1]) == B * N and int(p1.min()) >= 0


def test_static_scratch_build_rejects_large_grids():
    from npa_b200 import _native as n
    desc = n.make_grid(3, "periodic", "grid", (32, 32, 32), 1.0 / 32, 8, 262144, 32)
    assert int(n.lib.npa_grid_scratch_bytes(ctypes.byref(desc))) > 8 << 20
    rc = n.lib.npa_grid_build_static(ctypes.byref(desc), None, None, None, None, None)
    assert rc == n.NPA_ERR_SCRATCH_TOO_SMALL
    assert "built-in array holds" in n.last_error()


def test_static_scratch_through_the_grid_object():
    from npa_b200 import sphops as sph
    grid = sph.HashGrid(dim=2, boundary="periodic", mode="grid", grid_size=(20, 20), eps=0.05,
                        num_particles=4096, batch_size=2, max_particles_per_block=32)
    x = (torch.rand(2, 4096, 2, generator=torch.Generator().manual_seed(3)) - 0.5).cuda()
    snap = grid.instantiate(x)
    perm, offs, info = (torch.empty_like(snap.permutation), torch.empty_like(snap.bin_offsets),
                        torch.empty_like(snap.block_info))
    grid.hashgrid.initialize_static(x, perm, offs, info)
    assert torch.equal(perm, snap.permutation) and torch.equal(offs, snap.bin_offsets)
    assert torch.equal(info, snap.block_info)
