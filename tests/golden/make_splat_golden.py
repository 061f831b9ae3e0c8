"""Generates tests/golden/splat_*.npz by running the reference's own ``utils/splatting.py``.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_splat_golden.py [/path/to/reference]

``splat_particles`` is pure torch; it runs here on the CPU in float64 ("truth") and float32 ("as
the reference runs"), forward and autograd backward with a seeded upstream image.  Cases cover both
normalisation modes, the y flip, particles whose patch leaves the image, particles entirely
outside, and a batch.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = {
    # name: B, N, colour channels, kwargs of splat_particles
    "splat_default_small": dict(B=1, N=60, D=3, kw=dict(img_size=48, sigma=1.0, pixel_size=2.0 / 48.0)),
    "splat_plain_yup": dict(B=2, N=40, D=5, kw=dict(img_size=32, sigma=1.5, normalize_color=False, y_up=True)),
    "splat_wide_box": dict(B=1, N=80, D=4, kw=dict(img_size=40, sigma=2.0, lo=-2.0, hi=1.5, pixel_size=3.5 / 40.0, y_up=True)),
}


def load_reference(ref_root: Path):
    spec = importlib.util.spec_from_file_location("ref_splatting", ref_root / "utils" / "splatting.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_case(ref, cfg, seed):
    g = torch.Generator().manual_seed(seed)
    B, N, D, kw = cfg["B"], cfg["N"], cfg["D"], cfg["kw"]
    lo, hi = kw.get("lo", -1.0), kw.get("hi", 1.0)
    x = lo + (hi - lo) * (torch.rand(B, N, 2, generator=g, dtype=torch.float64) * 1.3 - 0.15)  # some outside
    x[:, 0] = hi + 10.0            # far outside: touches no pixel
    x[:, 1] = lo                   # exactly on the corner pixel
    color = torch.rand(B, N, D, generator=g, dtype=torch.float64)
    up = torch.randn(B, kw["img_size"], kw["img_size"], 4, generator=g, dtype=torch.float64)
    out = {"x": x.float().numpy(), "color": color.float().numpy(), "up": up.float().numpy(),
           "meta": repr(dict(B=B, N=N, D=D, kw=kw))}
    for tag, dt in (("f64", torch.float64), ("f32", torch.float32)):
        xs = x.float().to(dt).requires_grad_(True)       # both precisions see the same fp32 inputs
        cs = color.float().to(dt).requires_grad_(True)
        img = ref.splat_particles_batch(xs, cs, **kw)
        img.backward(up.float().to(dt))
        out[f"out_{tag}"] = img.detach().numpy()
        out[f"g_x_{tag}"] = xs.grad.numpy()
        out[f"g_color_{tag}"] = cs.grad.numpy()
    return out


def main():
    ref_root = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE.parents[2] / "reference"
    ref = load_reference(ref_root)
    for k, (name, cfg) in enumerate(CASES.items()):
        out = run_case(ref, cfg, seed=500 + k)
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(name, out["out_f64"].shape, float(np.abs(out["out_f64"]).max()),
              "fp32 vs fp64 worst", float(np.abs(out["out_f32"] - out["out_f64"]).max()))


if __name__ == "__main__":
    main()
