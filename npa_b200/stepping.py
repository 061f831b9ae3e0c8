"""One Euler step of an NPA model on the fused kernels.

``step_euler`` has the contract of the reference's ``step_euler`` (models/npa.py:168-204) and
works on the reference's ``NPA`` module unchanged (it reads ``model.model``, ``alpha``, ``eps0``,
``spatial_dims`` and the perception flags), but runs

    grid build -> reorder -> packed perception (two neighbour sweeps) -> model.model (torch GEMMs,
    weight gradients by one fused kernel)
    -> fused limiter + update (+ wrap)

instead of five neighbour sweeps and ~25 elementwise torch kernels.  Values and gradients are
those of ``NPA.forward`` followed by the reference's update (tests/test_gpu_step_update.py).
"""
from __future__ import annotations

import math

import torch

from . import sphops as sph
from .mlp import apply_mlp


def _scalar(v) -> float:
    return float(v.item()) if isinstance(v, torch.Tensor) else float(v)


def _buffer_scalar(model, name) -> float:
    """``model.<name>`` (a one-element buffer such as ``eps0`` or ``alpha``) as a Python float, read from
    the device once and cached on the module until the buffer is modified in place or replaced: a step
    then makes no device-to-host copy (the reference keeps these as device tensors and never syncs)."""
    v = getattr(model, name)
    if not isinstance(v, torch.Tensor):
        return float(v)
    cache = model.__dict__.setdefault("_npa_b200_scalars", {})
    hit = cache.get(name)
    if hit is not None and hit[0] is v and hit[1] == v._version:
        return hit[2]
    value = float(v.item())
    cache[name] = (v, v._version, value)
    return value


class _FrozenView:
    """The attributes of an NPA module that a step reads, with ``eps0`` and ``alpha`` as Python floats."""

    def __init__(self, model):
        self.model = model.model
        self.eps0, self.alpha = _scalar(model.eps0), _scalar(model.alpha)
        self.spatial_dims = model.spatial_dims
        for flag, default in (("state_grad", True), ("density_grad", True), ("log_norm_grad", True),
                              ("log_norm_density_grad", True), ("stopgrad_pos", True), ("stopgrad_state", False)):
            setattr(self, flag, getattr(model, flag, default))
        self.last_snapshot = None


def frozen_view(model):
    """A stand-in for ``model`` whose scalar buffers were read once: ``step_euler`` on it makes no
    device-to-host copy, which a step recorded in a CUDA graph must not."""
    return model if isinstance(model, _FrozenView) else _FrozenView(model)


def perceive(model, x, s, grid):
    """``NPA.perceive`` (models/npa.py:87-137) on the packed perception call; returns
    ``(z, x_bin, s_bin, snapshot)`` like the reference."""
    if not (getattr(model, "state_grad", True) and getattr(model, "density_grad", True)):
        raise NotImplementedError("the packed perception covers state_grad=True, density_grad=True "
                                  "(every shipped configuration); use the per-operator API otherwise")
    with torch.no_grad():
        snapshot = grid.instantiate(x)
    x_bin, s_bin = sph.bin_particles(x, s, snapshot)
    x_perceive = x_bin.detach() if getattr(model, "stopgrad_pos", True) else x_bin
    s_perceive = s_bin.detach() if getattr(model, "stopgrad_state", False) else s_bin
    z = sph.perceive_features(x_perceive, s_perceive, snapshot, _buffer_scalar(model, "eps0"),
                              log_norm_grad=getattr(model, "log_norm_grad", True),
                              log_norm_density_grad=getattr(model, "log_norm_density_grad", True))
    return z, x_bin, s_bin, snapshot


def step_euler(model, x, s, grid, dt=1.0, update_prob=0.5, intermediate=False, noise_std=0.0, wrap=False):
    """``x, s, stats`` after one step; the particles come back in cell order, as in the reference.

    ``wrap=True`` additionally applies ``grid.wrap_positions`` (the reference's trainers call it
    after the rollout, train.py:238); the 3D padding column is kept either way.
    """
    B, N, C = s.shape
    z, x_bin, s_bin, snapshot = perceive(model, x, s, grid)
    model.last_snapshot = snapshot
    y = apply_mlp(model.model, z)  # (B, N, dim + C); torch GEMMs, fused weight-gradient kernel in the backward

    stats = None
    if intermediate:
        d = y[..., : model.spatial_dims]
        dx = _buffer_scalar(model, "alpha") * d * grid.eps / (1.0 + d.norm(dim=-1, keepdim=True))
        stats = {"dx_norm": dx.norm(dim=-1).mean()}

    update_mask = None
    if update_prob < 1.0:
        update_mask = (torch.rand(B, N, 1, device=x.device) < update_prob).float()
    x_new, s_new = sph.step_update(y, x_bin, s_bin, snapshot, _buffer_scalar(model, "alpha"), dt, update_mask, wrap)
    if noise_std > 0:
        noise = torch.randn_like(x_new) * noise_std * math.sqrt(dt)
        x_new = x_new + (noise * update_mask if update_mask is not None else noise)
    return x_new, s_new, stats
