"""Multi-step rollout of the perception path over a shard of independent particle systems.

The loop a trainer runs per epoch (train.py:225-238 and models/npa.py:168-204 of the reference):
every step re-bins the particles, runs the perception forward (density sweep, blur + gradient
sweep) on the particles in cell order, and moves them; the positions are wrapped into the periodic
box; the backward pass runs through the final step only.  Here the per-particle update is a
prescribed smooth velocity field instead of the model's MLP, so that the loop exercises exactly the
perception path: grid build, reorder, the two forward sweeps, and for the last step the two backward
sweeps and the inverse reorder.

Everything is launched through the native layer (ctypes -> C ABI) on the current stream with
buffers allocated once; a rollout makes no host synchronisation.
"""
from __future__ import annotations

import math

import torch

from . import sphops as sph


class VelocityField:
    """Seeded smooth velocity field: a sum of low-frequency sine modes of amplitude ~1 (the same field
    as ``workloads.smooth_velocity``), with its parameters resident on the device."""

    def __init__(self, dim: int, device, seed: int = 0, modes: int = 8):
        g = torch.Generator().manual_seed(seed)
        k = torch.randint(1, 4, (modes, dim), generator=g).float() * (2.0 * math.pi)
        phase = torch.rand(modes, generator=g) * (2.0 * math.pi)
        amp = torch.randn(modes, dim, generator=g) / math.sqrt(modes)
        self.dim = dim
        self.k_t = k.t().contiguous().to(device)      # [dim, modes]
        self.phase = phase.to(device)
        self.amp = amp.to(device)                     # [modes, dim]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        arg = x[..., : self.dim] @ self.k_t + self.phase
        return torch.sin(arg) @ self.amp


class PerceptionRollout:
    """``steps`` perception steps over ``B`` systems of ``N`` particles, backward through the last one.

    ``x`` is ``[B, N, P]`` (P = 2, or 4 in 3D), ``s`` is ``[B, N, C]``; both are overwritten by the
    particles in the cell order of the last step.  ``upstream`` holds the gradients of the last
    step's outputs (``g_rho [B,N]``, ``g_blur [B,N,C]``, ``g_grad [B,N,C,D]``).  ``list_slots`` is the row
    length of the neighbour lists (one count + up to ``list_slots - 1`` neighbours, at most 513); particles
    with more neighbours fall back to the cell search.
    """

    def __init__(self, grid: "sph.HashGrid", channels: int, steps: int, dt: float, velocity: VelocityField,
                 list_slots: int = 128):
        self.grid, self.hg = grid, grid.hashgrid
        self.steps, self.dt, self.velocity = int(steps), float(dt), velocity
        B, N, D = grid.batch_size, grid.num_particles, grid.dim
        P = 2 if D == 2 else 4
        dev = velocity.amp.device
        i32 = dict(dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.perm = torch.empty(B, N, **i32)
        self.offs = torch.empty(B * grid.num_cells + 1, **i32)
        self.info = torch.empty(self.hg.max_blocks, 4, **i32)
        self.x_bin = torch.empty(B, N, P, **f32)
        self.s_bin = torch.empty(B, N, channels, **f32)
        self.rho = torch.empty(B, N, **f32)
        self.blur = torch.empty(B, N, channels, **f32)
        self.grad = torch.empty(B, N, channels, D, **f32)
        self.grad_x = torch.empty(B, N, P, **f32)
        self.grad_s = torch.empty(B, N, channels, **f32)
        self.grad_rho = torch.empty(B, N, **f32)
        self.grad_x_in = torch.empty(B, N, P, **f32)
        self.grad_s_in = torch.empty(B, N, channels, **f32)
        self.pairs = torch.empty(B, N, list_slots, **i32)  # neighbour lists of the current step, shared by its sweeps
        self.half_box = None
        if grid.boundary == "periodic":
            self.box = torch.tensor([g * grid.eps for g in grid.grid_size[:D]], **f32)
            self.half_box = 0.5 * self.box
        # kernels of this library per rollout: 7 grid build + reorder + 2 sweeps per step, and for the
        # last step 2 backward sweeps + the inverse reorder
        self.launches = self.steps * 10 + 3

    def _forward(self, x, s, last):
        hg = self.hg
        hg.initialize(x, self.perm, self.offs, self.info)
        hg.bin_particles(x, s, None, self.perm, self.x_bin, self.s_bin, None)
        # the density sweep records the neighbour lists in every step: writing them costs 15 % of that sweep, and
        # the blur + gradient sweep that reads them takes less than half the time of one that searches the cells
        # itself (cfg5's shape, 3D periodic: 1.05 + 1.09 ms against 0.91 + 2.42 ms per million particles)
        hg.perception_forward(self.x_bin, None, None, self.rho, None, None, None, None, None, self.offs, self.info,
                              pair_cache=self.pairs)
        hg.blur_gradient_forward(self.x_bin, self.rho, None, self.s_bin, self.blur, self.grad, self.offs, self.info,
                                 pair_cache=self.pairs, pair_cache_valid=True)

    def _move(self, x, s):
        """x <- wrap(x_bin + dt * v(x_bin)), s <- s_bin: the particles continue in cell order."""
        D = self.grid.dim
        xn = self.x_bin[..., :D] + self.dt * self.velocity(self.x_bin)
        if self.half_box is not None:
            xn = torch.remainder(xn + self.half_box, self.box) - self.half_box
        x[..., :D] = xn
        s.copy_(self.s_bin)

    def run(self, x, s, upstream):
        """One rollout; returns ``(grad_x, grad_s)`` with respect to the inputs of the final step."""
        for k in range(self.steps):
            last = k == self.steps - 1
            self._forward(x, s, last)
            if not last:
                self._move(x, s)
        hg = self.hg
        hg.blur_gradient_backward(self.x_bin, self.rho, None, self.s_bin, upstream["g_blur"], upstream["g_grad"],
                                  self.grad_x, self.grad_s, self.grad_rho, self.offs, self.info, pair_cache=self.pairs)
        hg.density_chain_backward(self.x_bin, None, upstream["g_rho"], self.grad_rho, None, self.grad_x, True,
                                  self.offs, self.info, pair_cache=self.pairs)
        # gradients back in the particle order the final step received (Permute.backward, sph.py:127-184)
        hg.backward_bin_particles(self.grad_x, self.grad_s, None, self.perm, self.grad_x_in, self.grad_s_in, None)
        return self.grad_x_in, self.grad_s_in
