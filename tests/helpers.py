"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from oracle import binning as obin

# Tolerance of the strict GPU-vs-oracle comparisons: elementwise
# |gpu - truth| <= RTOL * |truth| + ATOL_SCALE * max|truth|, truth = the fp64 oracle.  Where a case
# can exceed it for reasons every fp32 evaluation shares (periodic wraps round at the magnitude of
# the box; chained gradients cancel), the tests use conftest.assert_parity, which also accepts an
# error no worse than twice the reference's own fp32 error on the same tensor.
RTOL = 1e-5
ATOL_SCALE = 1e-6


def make_grid(sph, w, B=None, N=None, device="cuda"):
    return sph.HashGrid(dim=w.dim, boundary=w.boundary, mode=w.mode, grid_size=w.grid_size, eps=w.eps,
                        num_particles=w.N if N is None else N, batch_size=w.B if B is None else B,
                        max_particles_per_block=w.max_particles_per_block)


def box_of(w):
    return [g * w.eps for g in w.grid_size[:w.dim]] if w.boundary == "periodic" else None


def oracle_binning(x_cpu, w):
    return obin.bin_particles(x_cpu.numpy(), w.dim, w.grid_size, w.eps, w.boundary == "periodic",
                              w.mode == "particle", w.max_particles_per_block)


def oracle_forward(x_bin, w, want, s=None, mass=None, rho_in=None, precision="f64"):
    cpu = lambda t: None if t is None else t.detach().cpu().numpy()
    return oracle.forward(cpu(x_bin), w.eps, w.dim, mass=cpu(mass), s=cpu(s), rho_in=cpu(rho_in),
                          periodic=w.boundary == "periodic", box_size=box_of(w), want=want, precision=precision)


def oracle_backward(x_bin, w, s=None, mass=None, rho_in=None, precision="f64", **ups):
    cpu = lambda t: None if t is None else t.detach().cpu().numpy()
    return oracle.backward(cpu(x_bin), w.eps, w.dim, mass=cpu(mass), s=cpu(s), rho_in=cpu(rho_in),
                           periodic=w.boundary == "periodic", box_size=box_of(w), precision=precision,
                           **{k: cpu(v) for k, v in ups.items()})


def np64(t):
    return t.detach().cpu().numpy().astype(np.float64)
