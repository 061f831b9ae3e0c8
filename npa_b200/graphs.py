"""CUDA-graph capture of a forward perception step.

For small particle systems a step is bound by kernel launches (a grid build is six launches, the
reorder and the two sweeps four more), not by the kernels.  Every entry point of the C ABI is
capture-safe once warmed up (no allocation, no synchronisation, launches on the stream it is
given), so a whole step -- grid build, reorder into cell order, packed perception -- can be
recorded once and replayed with one launch.  Forward only: use it for rollouts and inference
(``torch.no_grad``); training steps go through autograd as usual.
"""
from __future__ import annotations

import torch

from . import sphops as sph


class GraphedPerception:
    """``z, x_bin, s_bin = graphed(x, s)`` with the work recorded in a CUDA graph.

    ``grid`` fixes batch size, particle count and geometry; ``channels`` the feature count.
    Inputs are copied into static buffers and the returned tensors are static as well: they are
    overwritten by the next call, so consume (or clone) them first.  ``snapshot`` gives the
    static snapshot tensors (permutation, bin_offsets, block_info) of the last call.
    """

    def __init__(self, grid: sph.HashGrid, channels: int, eps0: float, device=None, log_norm_grad: bool = True,
                 log_norm_density_grad: bool = True, warmup: int = 3):
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        B, N, P = grid.batch_size, grid.num_particles, (2 if grid.dim == 2 else 4)
        self.grid = grid
        self.x = torch.zeros(B, N, P, device=dev)
        self.s = torch.zeros(B, N, channels, device=dev)
        # spread the placeholder positions so that the warm-up does not put every particle in one cell
        span = torch.tensor([g * grid.eps for g in grid.grid_size[:grid.dim]], device=dev)
        self.x[..., :grid.dim] = (torch.rand(B, N, grid.dim, device=dev) - 0.5) * span * 0.9

        def step():
            snap = grid.instantiate(self.x)
            x_bin, s_bin = sph.bin_particles(self.x, self.s, snap)
            z = sph.perceive_features(x_bin, s_bin, snap, eps0, log_norm_grad=log_norm_grad,
                                      log_norm_density_grad=log_norm_density_grad)
            return z, x_bin, s_bin, snap

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(max(1, warmup)):   # allocates the grid scratch, sizes the persistent launches
                step()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.z, self.x_bin, self.s_bin, self.snapshot = step()

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, s: torch.Tensor):
        self.x.copy_(x, non_blocking=True)
        self.s.copy_(s, non_blocking=True)
        self.graph.replay()
        return self.z, self.x_bin, self.s_bin


class GraphedEulerStep:
    """A whole forward Euler step of an NPA model -- grid build, reorder, packed perception, the
    model's MLP, the fused update (and the periodic wrap) -- recorded in one CUDA graph.

    For rollouts and inference (no autograd): ``x, s = graphed(x, s)`` advances the particles by one
    step; the returned tensors are static buffers in cell order, overwritten by the next call, and
    may be passed straight back in (a rollout copies them into the input buffers on the device).
    The update mask of the reference's ``step_euler`` (models/npa.py:189-191) is drawn inside the
    graph with torch's CUDA generator, which torch keeps consistent across replays.
    """

    def __init__(self, model, grid: sph.HashGrid, channels: int, dt: float = 1.0, update_prob: float = 0.5,
                 wrap: bool = False, device=None, warmup: int = 3):
        from .stepping import frozen_view, step_euler
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        B, N, P = grid.batch_size, grid.num_particles, (2 if grid.dim == 2 else 4)
        model = frozen_view(model)  # eps0 / alpha as host numbers: reading a device buffer would synchronise
        self.x = torch.zeros(B, N, P, device=dev)
        self.s = torch.zeros(B, N, channels, device=dev)
        span = torch.tensor([g * grid.eps for g in grid.grid_size[:grid.dim]], device=dev)
        self.x[..., :grid.dim] = (torch.rand(B, N, grid.dim, device=dev) - 0.5) * span * 0.9

        def step():
            x_new, s_new, _ = step_euler(model, self.x, self.s, grid, dt=dt, update_prob=update_prob, wrap=wrap)
            return x_new, s_new

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                step()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.x_new, self.s_new = step()

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, s: torch.Tensor):
        self.x.copy_(x, non_blocking=True)
        self.s.copy_(s, non_blocking=True)
        self.graph.replay()
        return self.x_new, self.s_new

    @torch.no_grad()
    def rollout(self, x: torch.Tensor, s: torch.Tensor, steps: int):
        """``steps`` consecutive steps; returns clones of the final positions and states."""
        for _ in range(steps):
            x, s = self(x, s)
        return x.clone(), s.clone()
