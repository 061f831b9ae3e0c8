"""TEST INFRASTRUCTURE -- numpy restatement of the reference's uniform-grid binning.

The reference has no CPU code for binning (``torch_sph.bin_particles`` only
applies a permutation it is handed, sphops/torch_sph.py:55-94), so this follows
the CUDA source:

* cell coordinate ``floor(x * (1/eps)) + G/2`` in fp32, then clamp or positive
  modulo (sphops/utils.cuh:394-440);
* linear hash ``(z*Gy + y)*Gx + x`` or Morton bit interleave
  (sphops/utils.cuh:442-453, 481-524);
* ``bin_offsets`` = exclusive scan of the per-cell counts over all systems,
  length ``B*cells + 1`` (sphops/sph_cuda.cu:1961-1967);
* ``permutation[b, i]`` = slot of particle i inside system b = cell start + rank
  (sphops/sph_cuda.cu:81-83), where rank is taken in original particle order
  (stable): the reference's rank is atomic arrival order and therefore not
  reproducible, so the stable order is the definition parity is checked against;
* ``block_info`` rows ``(global cell, offset, count, system)`` per chunk of at
  most ``max_particles_per_block`` particles of a non-empty cell, in cell order
  (sphops/sph_cuda.cu:169-206), zero rows after the last item.
"""
from __future__ import annotations

import numpy as np


def _dilate(v: np.ndarray, dim: int) -> np.ndarray:
    v = v.astype(np.uint32) & np.uint32(0x3FF)
    if dim == 2:
        v = (v | (v << np.uint32(16))) & np.uint32(0x0000FFFF)
        v = (v | (v << np.uint32(8))) & np.uint32(0x00FF00FF)
        v = (v | (v << np.uint32(4))) & np.uint32(0x0F0F0F0F)
        v = (v | (v << np.uint32(2))) & np.uint32(0x33333333)
        v = (v | (v << np.uint32(1))) & np.uint32(0x55555555)
    else:
        v = (v | (v << np.uint32(16))) & np.uint32(0x030000FF)
        v = (v | (v << np.uint32(8))) & np.uint32(0x0300F00F)
        v = (v | (v << np.uint32(4))) & np.uint32(0x030C30C3)
        v = (v | (v << np.uint32(2))) & np.uint32(0x09249249)
    return v


def cell_ids(x: np.ndarray, dim: int, grid_size, eps: float, periodic: bool, morton: bool) -> np.ndarray:
    """Hash of the cell of every particle, ``[B, N]`` int64."""
    x = np.asarray(x, dtype=np.float32)
    inv_eps = np.float32(1.0) / np.float32(eps)
    coords = []
    for d in range(dim):
        g = int(grid_size[d])
        c = np.floor(x[..., d] * inv_eps).astype(np.int64) + g // 2
        c = np.mod(c, g) if periodic else np.clip(c, 0, g - 1)
        coords.append(c)
    if morton:
        h = _dilate(coords[0], dim)
        for d in range(1, dim):
            h = h | (_dilate(coords[d], dim) << np.uint32(d))
        return h.astype(np.int64)
    h = coords[dim - 1]
    for d in range(dim - 2, -1, -1):
        h = h * int(grid_size[d]) + coords[d]
    return h


def bin_particles(x: np.ndarray, dim: int, grid_size, eps: float, periodic: bool, morton: bool,
                  max_particles_per_block: int):
    """Returns ``(permutation [B,N] int32, bin_offsets [B*cells+1] int32, block_info [max_blocks,4] int32)``."""
    B, N = x.shape[:2]
    cells = int(np.prod([int(g) for g in grid_size[:dim]]))
    ids = cell_ids(x, dim, grid_size, eps, periodic, morton)
    counts = np.zeros(B * cells, dtype=np.int64)
    perm = np.empty((B, N), dtype=np.int32)
    for b in range(B):
        order = np.argsort(ids[b], kind="stable")           # slot -> particle
        perm[b, order] = np.arange(N, dtype=np.int32)        # particle -> slot
        counts[b * cells:(b + 1) * cells] = np.bincount(ids[b], minlength=cells)
    offsets = np.zeros(B * cells + 1, dtype=np.int64)
    np.cumsum(counts, out=offsets[1:])
    mpb = int(max_particles_per_block)
    max_blocks = B * min(N, cells + (N + mpb - 1) // mpb)
    info = np.zeros((max_blocks, 4), dtype=np.int32)
    nblk = (counts + mpb - 1) // mpb                        # work items per cell
    first_row = np.concatenate([[0], np.cumsum(nblk)[:-1]])
    cell_of_row = np.repeat(np.arange(B * cells), nblk)
    total = cell_of_row.size
    off = (np.arange(total) - first_row[cell_of_row]) * mpb
    info[:total, 0] = cell_of_row
    info[:total, 1] = off
    info[:total, 2] = np.minimum(mpb, counts[cell_of_row] - off)
    info[:total, 3] = cell_of_row // cells
    return perm, offsets.astype(np.int32), info
