"""Seeded synthetic particle systems with the shapes of the benchmark configurations.

No dataset is involved anywhere on this path: positions, features and upstream
gradients are drawn from a seeded CPU generator (so a CPU oracle and the GPU see
identical bits) with the shapes, sizes and value distributions the five
benchmark configurations describe.  Grids are centred on the origin (cell =
floor(x / eps) + G/2), so samplers that draw in [0, 1]^D subtract 0.5.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class Workload:
    name: str
    dim: int
    B: int
    N: int
    C: int
    eps: float
    grid_size: tuple
    boundary: str = "clamped"
    mode: str = "grid"
    max_particles_per_block: int = 32
    sampler: str = "uniform"
    extra: dict = field(default_factory=dict)

    @property
    def P(self) -> int:
        return 2 if self.dim == 2 else 4


def _pad3(x):
    """[B, N, 3] -> [B, N, 4] with w = 0 (3D positions are stored 4 wide)."""
    return torch.cat([x, torch.zeros_like(x[..., :1])], dim=-1).contiguous()


def _uniform_square(B, N, g):
    return torch.rand(B, N, 2, generator=g) - 0.5


def _blobs(B, N, g, centres=64, sigma=0.04):
    c = torch.rand(B, centres, 2, generator=g)
    pick = torch.randint(0, centres, (B, N), generator=g)
    x = torch.gather(c, 1, pick.unsqueeze(-1).expand(-1, -1, 2)) + sigma * torch.randn(B, N, 2, generator=g)
    return x.clamp_(0.0, 1.0) - 0.5


def _strokes(B, N, g, jitter=0.01):
    """3-6 random polyline strokes of 2-4 segments per system, points uniform in arclength."""
    out = torch.empty(B, N, 2)
    for b in range(B):
        n_strokes = int(torch.randint(3, 7, (1,), generator=g))
        segs = []
        for _ in range(n_strokes):
            n_seg = int(torch.randint(2, 5, (1,), generator=g))
            pts = torch.rand(n_seg + 1, 2, generator=g)
            segs += [(pts[k], pts[k + 1]) for k in range(n_seg)]
        a = torch.stack([p for p, _ in segs])
        bb = torch.stack([q for _, q in segs])
        length = (bb - a).norm(dim=-1)
        cum = torch.cumsum(length, 0)
        t = torch.rand(N, generator=g) * cum[-1]
        k = torch.searchsorted(cum, t).clamp_(max=len(segs) - 1)
        start = cum[k] - length[k]
        u = ((t - start) / length[k].clamp_min(1e-9)).unsqueeze(-1)
        out[b] = a[k] + u * (bb[k] - a[k])
    out += jitter * torch.randn(B, N, 2, generator=g)
    return out.clamp_(0.0, 1.0) - 0.5


def _ball_with_shell(B, N, g, shell_fraction=0.1, shell_lo=0.98):
    direction = torch.nn.functional.normalize(torch.randn(B, N, 3, generator=g), dim=-1)
    radius = torch.rand(B, N, generator=g) ** (1.0 / 3.0)
    n_shell = int(round(N * shell_fraction))
    radius[:, :n_shell] = shell_lo + (1.0 - shell_lo) * torch.rand(B, n_shell, generator=g)
    perm = torch.stack([torch.randperm(N, generator=g) for _ in range(B)])
    x = direction * radius.unsqueeze(-1)
    return torch.gather(x, 1, perm.unsqueeze(-1).expand(-1, -1, 3))


def _uniform_cube(B, N, g):
    return torch.rand(B, N, 3, generator=g) - 0.5


def make_positions(w: Workload, seed: int = 0) -> torch.Tensor:
    """CPU fp32 positions ``[B, N, P]`` of workload ``w``."""
    g = torch.Generator().manual_seed(seed)
    if w.sampler == "uniform":
        x = _uniform_square(w.B, w.N, g) if w.dim == 2 else _uniform_cube(w.B, w.N, g)
    elif w.sampler == "blobs":
        x = _blobs(w.B, w.N, g)
    elif w.sampler == "strokes":
        x = _strokes(w.B, w.N, g)
    elif w.sampler == "ball_shell":
        x = _ball_with_shell(w.B, w.N, g)
    else:
        raise ValueError(f"unknown sampler {w.sampler!r}")
    x = x.float()
    return _pad3(x) if w.dim == 3 else x.contiguous()


def make_inputs(w: Workload, seed: int = 0):
    """Positions, features and N(0,1) upstream gradients for every output, all on the CPU."""
    x = make_positions(w, seed)
    g = torch.Generator().manual_seed(seed + 7919)
    s = torch.randn(w.B, w.N, w.C, generator=g)
    ups = {
        "g_rho": torch.randn(w.B, w.N, generator=g),
        "g_blur": torch.randn(w.B, w.N, w.C, generator=g),
        "g_grad": torch.randn(w.B, w.N, w.C, w.dim, generator=g),
        "g_rho_grad": torch.randn(w.B, w.N, w.dim, generator=g),
    }
    return x, s, ups


def smooth_velocity(x: torch.Tensor, dim: int, seed: int = 0, modes: int = 8) -> torch.Tensor:
    """Seeded smooth velocity field (sum of low-frequency sine modes, amplitude ~1) at positions x."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randint(1, 4, (modes, dim), generator=g).float() * (2.0 * math.pi)
    phase = torch.rand(modes, generator=g) * (2.0 * math.pi)
    amp = torch.randn(modes, dim, generator=g) / math.sqrt(modes)
    k, phase, amp = k.to(x.device), phase.to(x.device), amp.to(x.device)
    arg = torch.einsum("...d,md->...m", x[..., :dim], k) + phase
    v = torch.einsum("...m,md->...d", torch.sin(arg), amp)
    if x.shape[-1] > dim:
        v = torch.cat([v, torch.zeros_like(v[..., :1])], dim=-1)
    return v


def _h_for_neighbours_3d_ball(N, neighbours, fill=0.9):
    # interior number density n = fill * N / (4 pi / 3); neighbours = n * (4 pi / 3) h^3
    return (neighbours / (fill * N)) ** (1.0 / 3.0)


# The five benchmark configurations (shapes, value distributions and smoothing radii).
CONFIGS = {
    "cfg1_2d_growing": Workload("cfg1_2d_growing", dim=2, B=1, N=4096, C=16, eps=0.05, grid_size=(20, 20)),
    "cfg2_2d_texture_blobs": Workload("cfg2_2d_texture_blobs", dim=2, B=8, N=16384, C=32, eps=0.025,
                                      grid_size=(40, 40), sampler="blobs"),
    "cfg3_2d_pointmnist_strokes": Workload("cfg3_2d_pointmnist_strokes", dim=2, B=256, N=512, C=16, eps=0.06,
                                           grid_size=(18, 18), sampler="strokes", max_particles_per_block=64),
    "cfg4_3d_splat": Workload("cfg4_3d_splat", dim=3, B=4, N=65536, C=32,
                              eps=round(_h_for_neighbours_3d_ball(65536, 40.0), 4), grid_size=(24, 24, 24),
                              sampler="ball_shell"),
    "cfg5_3d_rollout": Workload("cfg5_3d_rollout", dim=3, B=64, N=262144, C=16, eps=1.0 / 32.0,
                                grid_size=(32, 32, 32), boundary="periodic",
                                extra={"steps": 64, "dt": 0.002}),
}

HEADLINE = "cfg4_3d_splat"


def scaled(w: Workload, **overrides) -> Workload:
    """Copy of ``w`` with some fields replaced (smaller B / N for parity tests)."""
    d = dict(w.__dict__)
    d.update(overrides)
    return Workload(**d)
