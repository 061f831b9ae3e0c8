"""Generates tests/golden/step_*.npz by running the reference's own NPA.forward and step_euler.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_step_golden.py [/path/to/reference]

``models/npa.py`` imports the CUDA-backed ``sphops`` package at module level; the perception
operators are not what these fixtures pin, so a placeholder module satisfies the import and
``NPA.perceive`` is replaced by a function that returns given tensors ``(z, x_bin, s_bin)``.
Everything after perception -- the MLP, the displacement limiter of ``NPA.forward``
(models/npa.py:139-153) and the update of ``step_euler`` (models/npa.py:168-204) -- is the
reference's code, run in fp32 on the CPU with autograd for the backward.  Each fixture stores the
MLP output ``y``, the update mask the reference drew (re-drawn here from the same seed), the new
positions and states, and the gradients of a seeded linear loss with respect to ``y``'s inputs.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = {
    # name: spatial dims, B, N, C, eps, alpha, dt, update_prob
    "step_d2": dict(dim=2, B=2, N=96, C=16, eps=0.05, alpha=1.0, dt=1.0, update_prob=0.5),
    "step_d3": dict(dim=3, B=1, N=128, C=8, eps=0.0879, alpha=0.7, dt=0.5, update_prob=0.75),
    "step_d2_all": dict(dim=2, B=1, N=64, C=4, eps=0.1, alpha=2.0, dt=1.0, update_prob=1.0),
}


def load_reference_npa(ref_root: Path):
    names = ["blur", "gradient", "moment_matrix", "density_gradient", "density", "gradient_hybrid",
             "bin_particles", "unbin_particles", "HashGrid"]
    placeholder = types.ModuleType("sphops")
    for n in names:
        setattr(placeholder, n, None)
    saved = sys.modules.get("sphops")
    sys.modules["sphops"] = placeholder
    try:
        spec = importlib.util.spec_from_file_location("ref_models_npa", ref_root / "models" / "npa.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        if saved is None:
            del sys.modules["sphops"]
        else:
            sys.modules["sphops"] = saved
    return mod


class _Grid:
    def __init__(self, eps):
        self.eps = eps


def run_case(ref, cfg, seed):
    dim, B, N, C = cfg["dim"], cfg["B"], cfg["N"], cfg["C"]
    P = 2 if dim == 2 else 4
    g = torch.Generator().manual_seed(seed)
    model = ref.NPA(spatial_dims=dim, state_dims=C, hidden_dims=32, alpha=cfg["alpha"])
    with torch.no_grad():  # larger weights than the 0.1-gain init so that |dx| is not tiny
        for p in model.model.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.3)
    z = torch.randn(B, N, model.perception_dim, generator=g).requires_grad_(True)
    x_bin = torch.randn(B, N, P, generator=g)
    if dim == 3:
        x_bin[..., 3] = torch.randn(B, N, generator=g)  # the padding column must be carried over
    s_bin = torch.randn(B, N, C, generator=g)
    x_bin.requires_grad_(True)
    s_bin.requires_grad_(True)
    model.perceive = lambda x, s, grid: (z, x_bin, s_bin, None)
    y = model.model(z)

    torch.manual_seed(seed + 7)  # step_euler draws its mask from the global generator
    x_new, s_new, _ = ref.step_euler(model, x_bin, s_bin, _Grid(cfg["eps"]), dt=cfg["dt"],
                                     update_prob=cfg["update_prob"])
    torch.manual_seed(seed + 7)
    mask = (torch.rand(B, N, 1) < cfg["update_prob"]).float() if cfg["update_prob"] < 1.0 else torch.ones(B, N, 1)

    up_x = torch.randn(x_new.shape, generator=g)
    up_s = torch.randn(s_new.shape, generator=g)
    torch.autograd.backward([x_new, s_new], [up_x, up_s], inputs=[z, x_bin, s_bin] + list(model.model.parameters()))
    # dL/dy, recomputed by pushing the same upstream through the reference's tail only
    y2 = y.detach().clone().requires_grad_(True)
    model2_dx = y2[..., :dim]
    eps = cfg["eps"]
    dx = model.alpha * model2_dx * eps / (1.0 + model2_dx.norm(dim=-1, keepdim=True))
    if dim != P:
        dx = torch.cat([dx, torch.zeros(B, N, 1)], dim=-1)
    xs = x_bin.detach() + cfg["dt"] * dx * mask
    ss = s_bin.detach() + cfg["dt"] * y2[..., dim:] * mask
    assert torch.equal(xs, x_new.detach()) and torch.equal(ss, s_new.detach()), "tail restatement differs"
    torch.autograd.backward([xs, ss], [up_x, up_s])
    return dict(
        dim=np.int64(dim), eps=np.float64(eps), alpha=np.float64(cfg["alpha"]), dt=np.float64(cfg["dt"]),
        y=y.detach().numpy(), x_bin=x_bin.detach().numpy(), s_bin=s_bin.detach().numpy(),
        mask=mask.reshape(B, N).numpy(), x_new=x_new.detach().numpy(), s_new=s_new.detach().numpy(),
        up_x=up_x.numpy(), up_s=up_s.numpy(), g_y=y2.grad.numpy(), g_x_bin=x_bin.grad.numpy(),
        g_s_bin=s_bin.grad.numpy(), g_z=z.grad.numpy(),
    )


def main():
    ref_root = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE.parents[2] / "reference"
    ref = load_reference_npa(ref_root)
    for k, (name, cfg) in enumerate(CASES.items()):
        out = run_case(ref, cfg, seed=300 + k)
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(name, {n: v.shape for n, v in out.items() if hasattr(v, "shape") and v.ndim})


if __name__ == "__main__":
    main()
