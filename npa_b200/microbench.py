"""Timings of the kernels around the perception path: the fused Euler update and the splat renderer.

    python -m npa_b200.microbench step_update [--workload cfg4_3d_splat]
    python -m npa_b200.microbench splat [--systems 8 --particles 4096]
    python -m npa_b200.microbench euler_step [--workload cfg4_3d_splat]

Each prints one JSON line.  CUDA events on torch's current stream; inputs rotate over several
buffer sets larger than L2 so that consecutive launches do not find their inputs cached.  The
"torch" figures time the same mathematics written with torch tensor operations (elementwise glue
for the update; index tensors + ``scatter_add_`` for the splat), on the same device.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from . import sphops as sph
from . import splatting
from .workloads import CONFIGS


def _time(fn, sets, reps):
    for _ in range(3):  # warm-up: kernels, launch sizes, and the caching allocator's pools
        for t in sets:
            fn(t)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        for t in sets:
            fn(t)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * len(sets))  # ms per call


def bench_step_update(args):
    w = CONFIGS[args.workload]
    B, N, C, D = w.B, w.N, w.C, w.dim
    P = 2 if D == 2 else 4
    grid = sph.HashGrid(dim=D, boundary=w.boundary, mode=w.mode, grid_size=w.grid_size, eps=w.eps, num_particles=N,
                        batch_size=B, max_particles_per_block=w.max_particles_per_block)
    hg = grid.hashgrid
    per_set = B * N * 4 * (2 * (D + C) + 2 * P + 2 * C + 1)
    n_sets = max(2, math.ceil(300e6 / per_set))  # > 126 MB of L2 between two uses of a buffer
    dev = "cuda"
    sets = [dict(y=torch.randn(B, N, D + C, device=dev), x=torch.randn(B, N, P, device=dev),
                 s=torch.randn(B, N, C, device=dev), m=(torch.rand(B, N, device=dev) < 0.5).float(),
                 xo=torch.empty(B, N, P, device=dev), so=torch.empty(B, N, C, device=dev),
                 gy=torch.empty(B, N, D + C, device=dev)) for _ in range(n_sets)]

    def forward(t):
        hg.step_update_forward(t["y"], t["x"], t["s"], t["m"], 1.0, 1.0, False, t["xo"], t["so"])

    def backward(t):
        hg.step_update_backward(t["y"], t["m"], C, 1.0, 1.0, t["xo"], t["so"], t["gy"])

    def torch_forward(t):  # NPA.forward's limiter + step_euler's update as torch operations
        y, mask = t["y"], t["m"].unsqueeze(-1)
        dx = y[..., :D]
        dx = 1.0 * dx * w.eps / (1.0 + dx.norm(dim=-1, keepdim=True))
        if D != P:
            dx = torch.cat([dx, torch.zeros(B, N, 1, device=dev)], dim=-1).contiguous()
        return t["x"] + 1.0 * dx * mask, t["s"] + 1.0 * y[..., D:] * mask

    fwd_bytes = B * N * (4 * (D + C) + 8 * P + 8 * C + 4)
    bwd_bytes = B * N * (8 * (D + C) + 4 * P + 4 * C + 4)
    reps = max(3, args.reps // n_sets)
    f, b, t = _time(forward, sets, reps), _time(backward, sets, reps), _time(torch_forward, sets, reps)
    return {"kernel": "step_update", "workload": w.name, "particles": B * N, "buffer_sets": n_sets,
            "forward_us": f * 1e3, "forward_gbs": fwd_bytes / (f * 1e-3) / 1e9, "forward_bytes": fwd_bytes,
            "backward_us": b * 1e3, "backward_gbs": bwd_bytes / (b * 1e-3) / 1e9, "backward_bytes": bwd_bytes,
            "torch_forward_us": t * 1e3}


def _torch_scatter_splat(x, color, img_size=256, sigma=2.0, lo=-1.0, hi=1.0, pixel_size=2.0 / 128.0):
    """One system, normalised mode, with torch index tensors and scatter_add_ (for timing only)."""
    dev = x.device
    p = (x - lo) / (hi - lo) * (img_size - 1)
    sig = sigma * img_size * pixel_size / (hi - lo)
    r = max(1, math.ceil(5 * sig))
    side = 2 * r + 1
    offs = torch.arange(-r, r + 1, device=dev)
    yy, xx = torch.meshgrid(offs, offs, indexing="ij")
    dx, dy = xx.reshape(-1), yy.reshape(-1)
    base = torch.floor(p)
    frac = p - base
    xi = base[:, 0].long()[:, None] + dx[None]
    yi = base[:, 1].long()[:, None] + dy[None]
    mask = (xi >= 0) & (xi < img_size) & (yi >= 0) & (yi < img_size)
    g = torch.exp(-((dx[None] - frac[:, 0:1]) ** 2 + (dy[None] - frac[:, 1:2]) ** 2) / (2 * sig * sig))
    g = g / (1e-8 + g.sum(-1, keepdim=True)) * (img_size * pixel_size / (hi - lo)) ** 2
    flat, wgt = (yi * img_size + xi)[mask], g[mask]
    c = color[:, None, :].expand(-1, side * side, -1)[mask, :]
    dens = torch.zeros(img_size * img_size, 1, device=dev)
    rgb = torch.zeros(img_size * img_size, 3, device=dev)
    dens.scatter_add_(0, flat[:, None], wgt[:, None])
    rgb.scatter_add_(0, flat[:, None].expand(-1, 3), c * wgt[:, None])
    return torch.cat([rgb, dens], 1).view(img_size, img_size, 4)


def bench_splat(args):
    B, n, img = args.systems, args.particles, 256
    dev = "cuda"
    sets = [dict(x=(torch.rand(B, n, 2, device=dev) - 0.5) * 1.6, c=torch.rand(B, n, 3, device=dev),
                 up=torch.randn(B, img, img, 4, device=dev)) for _ in range(3)]

    def fwd(t):
        return splatting.splat_particles_batch(t["x"], t["c"])

    def fwd_bwd(t):
        x, c = t["x"].clone().requires_grad_(True), t["c"].clone().requires_grad_(True)
        splatting.splat_particles_batch(x, c).backward(t["up"])

    def torch_fwd(t):
        return torch.stack([_torch_scatter_splat(t["x"][b], t["c"][b]) for b in range(B)])

    def torch_fwd_bwd(t):
        x, c = t["x"].clone().requires_grad_(True), t["c"].clone().requires_grad_(True)
        torch.stack([_torch_scatter_splat(x[b], c[b]) for b in range(B)]).backward(t["up"])

    diff = float((fwd(sets[0]) - torch_fwd(sets[0])).abs().max())
    reps = max(2, args.reps // 10)
    return {"kernel": "splat", "systems": B, "particles_per_system": n, "img_size": img, "patch": 41,
            "forward_ms": _time(fwd, sets, reps), "forward_backward_ms": _time(fwd_bwd, sets, reps),
            "torch_forward_ms": _time(torch_fwd, sets, 1), "torch_forward_backward_ms": _time(torch_fwd_bwd, sets, 1),
            "max_abs_difference_to_torch": diff}


class _Model(torch.nn.Module):
    """An NPA-shaped module (models/npa.py:14-75): the attributes a step reads and the 2-layer MLP."""

    def __init__(self, dim, C, hidden=128, eps0=0.1, alpha=1.0):
        super().__init__()
        self.spatial_dims, self.state_dims = dim, C
        self.eps0, self.alpha = eps0, alpha
        self.state_grad = self.density_grad = self.log_norm_grad = self.log_norm_density_grad = True
        self.stopgrad_pos, self.stopgrad_state = True, False
        self.model = torch.nn.Sequential(torch.nn.Linear(2 * C + C * dim + dim, hidden), torch.nn.ReLU(),
                                         torch.nn.Linear(hidden, dim + C, bias=False))


def bench_euler_step(args):
    """One training step of an NPA model: step_euler forward (grid build, reorder, packed perception,
    MLP, fused update) + backward to the MLP weights and the input states, and the share of the MLP
    (torch / cuBLAS fp32) in it."""
    from .stepping import step_euler
    from .workloads import make_inputs
    w = CONFIGS[args.workload]
    B, N, C, D = w.B, w.N, w.C, w.dim
    grid = sph.HashGrid(dim=D, boundary=w.boundary, mode=w.mode, grid_size=w.grid_size, eps=w.eps, num_particles=N,
                        batch_size=B, max_particles_per_block=w.max_particles_per_block)
    torch.manual_seed(0)
    model = _Model(D, C).cuda()
    x, s, _ = make_inputs(w, seed=0)
    x, s = x.cuda(), s.cuda()
    up_x, up_s = torch.randn_like(x), torch.randn_like(s)
    z = torch.randn(B, N, 2 * C + C * D + D, device="cuda")
    up_y = torch.randn(B, N, D + C, device="cuda")

    def full(_):
        model.zero_grad(set_to_none=True)
        sr = s.clone().requires_grad_(True)
        x_new, s_new, _ = step_euler(model, x, sr, grid, dt=1.0, update_prob=0.5)
        torch.autograd.backward([x_new, s_new], [up_x, up_s])

    def mlp_only(_):
        model.zero_grad(set_to_none=True)
        zr = z.clone().requires_grad_(True)
        model.model(zr).backward(up_y)

    def mlp_fused(_):
        from .mlp import apply_mlp
        model.zero_grad(set_to_none=True)
        zr = z.clone().requires_grad_(True)
        apply_mlp(model.model, zr).backward(up_y)

    def forward_only(_):
        with torch.no_grad():
            step_euler(model, x, s, grid, dt=1.0, update_prob=0.5)

    reps = max(5, args.reps)
    return {"kernel": "euler_step", "workload": w.name, "particles": B * N, "mlp": [2 * C + C * D + D, 128, D + C],
            "train_step_ms": _time(full, [None], reps), "forward_only_ms": _time(forward_only, [None], reps),
            "mlp_forward_backward_ms": _time(mlp_fused, [None], reps),
            "torch_mlp_forward_backward_ms": _time(mlp_only, [None], reps)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["step_update", "splat", "euler_step"])
    ap.add_argument("--workload", default="cfg4_3d_splat")
    ap.add_argument("--systems", type=int, default=8)
    ap.add_argument("--particles", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=30)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise RuntimeError("npa_b200.microbench needs a CUDA device: the kernels have no CPU fallback")
    out = {"step_update": bench_step_update, "splat": bench_splat, "euler_step": bench_euler_step}[args.what](args)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
