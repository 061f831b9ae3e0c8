"""Generates tests/golden/*.npz by running the reference's own pure-torch operators.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_golden.py [/path/to/reference]

For each small seeded case it stores the inputs (fp32) and the outputs of
``sphops/torch_sph.py`` in fp64 ("truth") and fp32 ("as the reference runs"),
forward and autograd backward, operator by operator, plus the chained backward
rho = density(x); blur(x, rho, s); gradient(x, rho, s); density_gradient(x).
The committed fixtures pin the C oracle (tests/test_oracle_golden.py) and are
compared with the CUDA kernels directly (tests/test_gpu_golden.py).
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = {
    # name: dim, B, N, C, eps, grid, periodic, with_mass, position sampler
    "d2_clamped_mass": dict(dim=2, B=2, N=192, C=8, eps=0.1, grid=(16, 16), periodic=False, mass=True, spread="rand", scale=0.4),
    "d2_periodic": dict(dim=2, B=2, N=160, C=6, eps=0.15, grid=(8, 6), periodic=True, mass=False, spread="randn", scale=0.3),
    "d3_clamped": dict(dim=3, B=1, N=256, C=4, eps=0.4, grid=(6, 6, 6), periodic=False, mass=False, spread="rand", scale=1.0),
    "d3_periodic_mass": dict(dim=3, B=2, N=200, C=5, eps=0.3, grid=(6, 5, 4), periodic=True, mass=True, spread="randn", scale=0.6),
}


def load_torch_sph(ref_root: Path):
    spec = importlib.util.spec_from_file_location("ref_torch_sph", ref_root / "sphops" / "torch_sph.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_inputs(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    dim, B, N, C = cfg["dim"], cfg["B"], cfg["N"], cfg["C"]
    if cfg["spread"] == "rand":
        x = (torch.rand(B, N, dim, generator=g) - 0.5) * 2.0 * cfg["scale"]
    else:
        x = torch.randn(B, N, dim, generator=g) * cfg["scale"]
    # a few coincident particles exercise the d == 0 branches
    x[:, 1] = x[:, 0]
    x[:, N // 2] = x[:, N // 2 - 1]
    s = torch.randn(B, N, C, generator=g)
    mass = torch.rand(B, N, generator=g) + 0.5 if cfg["mass"] else None
    ups = dict(
        g_rho=torch.randn(B, N, generator=g),
        g_rho_grad=torch.randn(B, N, dim, generator=g),
        g_blur=torch.randn(B, N, C, generator=g),
        g_grad=torch.randn(B, N, C, dim, generator=g),
        g_moment=torch.randn(B, N, dim, dim, generator=g),
    )
    return x, s, mass, ups


def run_case(ts, cfg, seed, dtype):
    x32, s32, m32, ups32 = make_inputs(cfg, seed)
    dim, eps, periodic = cfg["dim"], cfg["eps"], cfg["periodic"]
    box = [g * eps for g in cfg["grid"]] if periodic else None
    cast = lambda t: None if t is None else t.to(dtype)
    x, s, mass = cast(x32), cast(s32), cast(m32)
    ups = {k: cast(v) for k, v in ups32.items()}
    out = {}
    with torch.no_grad():
        rho = ts.density(x, eps, mass, periodic, box)
        # the density every rho-consuming operator is fed: the fp32-rounded value, so that fp64
        # truth and the kernels see the same input bits
        rho_in32 = ts.density(x32, eps, m32, periodic, box).float()
        rho_in = rho_in32.to(dtype)
        out["count"] = ts.count(x, eps, periodic, box)
        out["rho"] = rho
        out["rho_grad"] = ts.density_gradient(x, eps, mass, periodic, box)
        out["blur"] = ts.blur(x, rho_in, s, eps, mass, periodic, box)
        out["grad"] = ts.gradient(x, rho_in, s, eps, mass, periodic, box)
        out["moment"] = ts.moment_matrix(x, rho_in, eps, mass, periodic, box)

    def grads(fn, needs):
        xr = x.clone().requires_grad_(True)
        sr = s.clone().requires_grad_("s" in needs)
        rr = rho_in.clone().requires_grad_("rho" in needs)
        y, up = fn(xr, sr, rr)
        y.backward(up)
        return (xr.grad, sr.grad if "s" in needs else None, rr.grad if "rho" in needs else None)

    bw = {
        "density": grads(lambda xr, sr, rr: (ts.density(xr, eps, mass, periodic, box), ups["g_rho"]), ""),
        "rho_grad": grads(lambda xr, sr, rr: (ts.density_gradient(xr, eps, mass, periodic, box), ups["g_rho_grad"]), ""),
        "blur": grads(lambda xr, sr, rr: (ts.blur(xr, rr, sr, eps, mass, periodic, box), ups["g_blur"]), "s rho"),
        "grad": grads(lambda xr, sr, rr: (ts.gradient(xr, rr, sr, eps, mass, periodic, box), ups["g_grad"]), "s rho"),
        "moment": grads(lambda xr, sr, rr: (ts.moment_matrix(xr, rr, eps, mass, periodic, box), ups["g_moment"]), "rho"),
    }
    for name, (dx, ds, dr) in bw.items():
        out[f"bw_{name}_dx"] = dx
        if ds is not None:
            out[f"bw_{name}_ds"] = ds
        if dr is not None:
            out[f"bw_{name}_drho"] = dr

    # chained backward: rho flows from density into blur and gradient
    xr = x.clone().requires_grad_(True)
    sr = s.clone().requires_grad_(True)
    rho_c = ts.density(xr, eps, mass, periodic, box)
    loss = (rho_c * ups["g_rho"]).sum()
    loss = loss + (ts.blur(xr, rho_c, sr, eps, mass, periodic, box) * ups["g_blur"]).sum()
    loss = loss + (ts.gradient(xr, rho_c, sr, eps, mass, periodic, box) * ups["g_grad"]).sum()
    loss = loss + (ts.density_gradient(xr, eps, mass, periodic, box) * ups["g_rho_grad"]).sum()
    loss.backward()
    out["chain_dx"] = xr.grad
    out["chain_ds"] = sr.grad

    inputs = dict(x=x32, s=s32, rho_in=rho_in32, **ups32)
    if m32 is not None:
        inputs["mass"] = m32
    return inputs, {k: v.detach() for k, v in out.items()}


def main():
    # default: a sibling directory "reference" of this repository
    ref_root = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE.parents[2] / "reference"
    ts = load_torch_sph(ref_root)
    torch.set_num_threads(8)
    for idx, (name, cfg) in enumerate(CASES.items()):
        seed = 1234 + idx
        inputs, out64 = run_case(ts, cfg, seed, torch.float64)
        _, out32 = run_case(ts, cfg, seed, torch.float32)
        blob = {f"in_{k}": v.numpy() for k, v in inputs.items()}
        blob.update({f"f64_{k}": v.numpy().astype(np.float64) for k, v in out64.items()})
        blob.update({f"f32_{k}": v.numpy().astype(np.float32) for k, v in out32.items()})
        meta = dict(cfg)
        meta["grid"] = list(cfg["grid"])
        blob["meta"] = np.array(repr(meta))
        np.savez_compressed(HERE / f"{name}.npz", **blob)
        print(name, {k: tuple(v.shape) for k, v in out64.items() if k in ("rho", "grad")},
              "mean count", float(out64["count"].mean()))


if __name__ == "__main__":
    main()
