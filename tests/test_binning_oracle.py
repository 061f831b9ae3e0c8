"""Properties of the numpy binning oracle (it has no reference CPU code to be pinned to, so it is
checked against brute-force definitions on small inputs)."""
import numpy as np
import pytest

from oracle import binning as ob


@pytest.mark.parametrize("dim,grid,periodic,morton", [(2, (5, 7), False, False), (2, (8, 8), True, True),
                                                      (3, (4, 3, 5), True, False), (3, (4, 4, 4), False, True)])
def test_oracle_definitions(dim, grid, periodic, morton):
    rng = np.random.default_rng(3)
    B, N, eps, mpb = 2, 300, 0.21, 8
    x = ((rng.random((B, N, dim if dim == 2 else 4)) - 0.5) * 1.6).astype(np.float32)
    ids = ob.cell_ids(x, dim, grid, eps, periodic, morton)
    cells = int(np.prod(grid))
    assert ids.min() >= 0 and ids.max() < cells
    # brute-force cell coordinates
    inv = np.float32(1.0) / np.float32(eps)
    for b in range(B):
        for i in range(0, N, 37):
            c = [int(np.floor(x[b, i, d] * inv)) + grid[d] // 2 for d in range(dim)]
            c = [ci % grid[d] if periodic else min(max(ci, 0), grid[d] - 1) for d, ci in enumerate(c)]
            if morton:
                h = 0
                for bit in range(10):
                    for d in range(dim):
                        h |= ((c[d] >> bit) & 1) << (bit * dim + d)
            else:
                h = c[-1]
                for d in range(dim - 2, -1, -1):
                    h = h * grid[d] + c[d]
            assert ids[b, i] == h
    perm, off, info = ob.bin_particles(x, dim, grid, eps, periodic, morton, mpb)
    assert off[-1] == B * N and off[0] == 0 and (np.diff(off) >= 0).all()
    for b in range(B):
        assert sorted(perm[b]) == list(range(N))                       # a permutation
        inv_perm = np.argsort(perm[b])
        assert (np.diff(ids[b][inv_perm]) >= 0).all()                  # sorted by cell
        same = np.diff(ids[b][inv_perm]) == 0
        assert (np.diff(inv_perm)[same] > 0).all()                     # stable inside a cell
        for c in range(cells):
            lo, hi = off[b * cells + c] - b * N, off[b * cells + c + 1] - b * N
            assert (ids[b][inv_perm[lo:hi]] == c).all()
    rows = info[info[:, 2] > 0]
    assert (info[len(rows):] == 0).all()
    counts = np.diff(off)
    assert rows[:, 2].sum() == B * N and (rows[:, 2] <= mpb).all()
    assert (np.diff(rows[:, 0]) >= 0).all()
    for cell, o, c, sys_ in rows[:: 11]:
        assert 0 <= o < counts[cell] and c == min(mpb, counts[cell] - o) and sys_ == cell // cells
    assert info.shape[0] == B * min(N, cells + (N + mpb - 1) // mpb)
