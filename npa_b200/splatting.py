"""Differentiable Gaussian splatting of particles into images on the B200 kernels.

Same functions, arguments and defaults as the reference's ``utils/splatting.py`` (``splat_particles``
:6-100, ``splat_particles_batch`` :103-110, ``splat_particles_sections`` :113-117), which render the
particles for its splat loss (losses/splat_loss.py:71-86).  The forward is a per-pixel gather and the
backward a per-particle gather (``csrc/splat.cu``): no [N, (2r+1)^2] intermediates, no atomics,
deterministic sums.  CUDA tensors only; there is no CPU fallback.
"""
from __future__ import annotations

import math

import torch

from . import _native as N

_lib = N.lib


def _derived(img_size, sigma, lo, hi, normalize_color, pixel_size):
    """sigma in pixels, patch radius and colour scale exactly as utils/splatting.py:43-46,75-77."""
    scale = 1.0
    if normalize_color:
        sigma = sigma * img_size * pixel_size / (hi - lo)
        scale = (img_size * pixel_size / (hi - lo)) ** 2.0
    radius = max(1, math.ceil(5 * float(sigma)))
    return float(sigma), int(radius), float(scale)


class _Splat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, color, img_size, sigma_pix, radius, lo, hi, y_up, normalize, scale):
        B, n = x.shape[0], x.shape[1]
        out = torch.empty(B, img_size, img_size, 4, dtype=torch.float32, device=x.device)
        scratch = torch.empty(B, n, dtype=torch.float32, device=x.device) if normalize else None
        with torch.cuda.device(x.device):
            N.check(_lib.npa_splat_forward(N.ptr(x), N.ptr(color), B, n, img_size, sigma_pix, radius, lo, hi,
                                           1 if y_up else 0, 1 if normalize else 0, scale, N.ptr(scratch), N.ptr(out),
                                           N.current_stream()))
        ctx.save_for_backward(x, color)
        ctx.consts = (img_size, sigma_pix, radius, lo, hi, y_up, normalize, scale)
        return out

    @staticmethod
    def backward(ctx, g_out):
        x, color = ctx.saved_tensors
        img_size, sigma_pix, radius, lo, hi, y_up, normalize, scale = ctx.consts
        need_x, need_c = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not (need_x or need_c):
            return (None,) * 10
        g_out = g_out.contiguous()
        g_x = torch.empty_like(x) if need_x else None
        g_c = torch.empty_like(color) if need_c else None
        with torch.cuda.device(x.device):
            N.check(_lib.npa_splat_backward(N.ptr(x), N.ptr(color), N.ptr(g_out), x.shape[0], x.shape[1], img_size,
                                            sigma_pix, radius, lo, hi, 1 if y_up else 0, 1 if normalize else 0, scale,
                                            N.ptr(g_x), N.ptr(g_c), N.current_stream()))
        return (g_x, g_c) + (None,) * 8


def _check(x, color):
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32):
        raise TypeError("x must be a float32 CUDA tensor")
    if not (isinstance(color, torch.Tensor) and color.is_cuda and color.dtype == torch.float32):
        raise TypeError("color must be a float32 CUDA tensor")
    if x.shape[-1] != 2 or color.shape[-1] < 3 or x.shape[:-1] != color.shape[:-1]:
        raise RuntimeError(f"x must have shape (..., N, 2) and color (..., N, >=3), got {tuple(x.shape)} and {tuple(color.shape)}")


def splat_particles_batch(x, color, img_size=256, sigma=2.0, lo=-1.0, hi=1.0, normalize_color=True, y_up=False,
                          pixel_size=2.0 / 128.0):
    """``x [B, N, 2]``, ``color [B, N, >=3]`` (the last three channels are r, g, b) ->
    ``[B, img_size, img_size, 4]`` with channels ``(r, g, b, density)``; one launch for the batch."""
    _check(x, color)
    sigma_pix, radius, scale = _derived(img_size, sigma, lo, hi, normalize_color, pixel_size)
    return _Splat.apply(x.contiguous(), color[..., -3:].contiguous(), int(img_size), sigma_pix, radius, float(lo),
                        float(hi), bool(y_up), bool(normalize_color), scale)


def splat_particles(x, color, img_size=256, sigma=2.0, lo=-1.0, hi=1.0, normalize_color=True, y_up=False,
                    pixel_size=2.0 / 128.0):
    """``x [N, 2]``, ``color [N, >=3]`` -> ``[img_size, img_size, 4]``."""
    return splat_particles_batch(x[None], color[None], img_size, sigma, lo, hi, normalize_color, y_up, pixel_size)[0]


def splat_particles_sections(x, color, sections, **kwargs):
    """Images of consecutive sections of a flat particle list (utils/splatting.py:113-117)."""
    xx, cc = torch.split(x, sections, dim=0), torch.split(color, sections, dim=0)
    return torch.stack([splat_particles(bx, bc, **kwargs) for bx, bc in zip(xx, cc)], dim=0)
