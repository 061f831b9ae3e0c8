"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from oracle import binning as obin

# Tolerance of every GPU-vs-oracle comparison of a floating-point operator: elementwise
# |gpu - truth| <= RTOL * |truth| + ATOL_SCALE * max|truth|, truth = the fp64 oracle.
# 1e-5 relative / 1e-6 absolute (on tensors normalised to unit scale) is the stated fp32 bar.
RTOL = 1e-5
ATOL_SCALE = 1e-6
# Periodic grids: the box length g * eps is not representable in fp32 and particles outside the
# primary box go through a general minimum-image wrap that rounds at the magnitude of the box, so
# every fp32 implementation carries ~1e-7 * L absolute error in wrapped displacements, amplified
# by cancellation in the gradient sums.  The reference's own fp32 run (torch_sph) misses the
# clamped tolerance by up to 13x on the periodic fixtures (measured when they were generated);
# the kernels are held to 2e-5 relative / 4e-6 absolute there.
RTOL_PERIODIC = 2e-5
ATOL_SCALE_PERIODIC = 4e-6


def tolerance(periodic):
    return (RTOL_PERIODIC, ATOL_SCALE_PERIODIC) if periodic else (RTOL, ATOL_SCALE)


def make_grid(sph, w, B=None, N=None, device="cuda"):
    return sph.HashGrid(dim=w.dim, boundary=w.boundary, mode=w.mode, grid_size=w.grid_size, eps=w.eps,
                        num_particles=w.N if N is None else N, batch_size=w.B if B is None else B,
                        max_particles_per_block=w.max_particles_per_block)


def box_of(w):
    return [g * w.eps for g in w.grid_size[:w.dim]] if w.boundary == "periodic" else None


def oracle_binning(x_cpu, w):
    return obin.bin_particles(x_cpu.numpy(), w.dim, w.grid_size, w.eps, w.boundary == "periodic",
                              w.mode == "particle", w.max_particles_per_block)


def oracle_forward(x_bin, w, want, s=None, mass=None, rho_in=None):
    cpu = lambda t: None if t is None else t.detach().cpu().numpy()
    return oracle.forward(cpu(x_bin), w.eps, w.dim, mass=cpu(mass), s=cpu(s), rho_in=cpu(rho_in),
                          periodic=w.boundary == "periodic", box_size=box_of(w), want=want)


def oracle_backward(x_bin, w, s=None, mass=None, rho_in=None, **ups):
    cpu = lambda t: None if t is None else t.detach().cpu().numpy()
    return oracle.backward(cpu(x_bin), w.eps, w.dim, mass=cpu(mass), s=cpu(s), rho_in=cpu(rho_in),
                           periodic=w.boundary == "periodic", box_size=box_of(w),
                           **{k: cpu(v) for k, v in ups.items()})


def np64(t):
    return t.detach().cpu().numpy().astype(np.float64)
