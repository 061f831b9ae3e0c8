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
