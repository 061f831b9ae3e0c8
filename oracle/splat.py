"""CPU restatement (numpy, float64) of the reference's Gaussian particle splatting and its
gradients.  Test infrastructure only: nothing of the product imports it.

Follows ``splat_particles`` (utils/splatting.py:6-100): pixel position
``p = (x - lo) / (hi - lo) * (img - 1)`` (:33, y flipped at :36), sigma converted to pixels and the
patch radius ``max(1, ceil(5 sigma))`` (:43-46), ``base = floor(p)``, ``frac = p - base`` (:55-58),
weights ``exp(-((dx - frac_x)^2 + (dy - frac_y)^2) / (2 sigma^2))`` over the (2r+1)^2 patch (:70-72),
normalised by ``1e-8 +`` their sum over the whole patch and scaled (:75-77), masked to the image
(:65-67) and scatter-added as ``[sum c w | sum w]`` (:91-99).  ``floor`` passes no gradient.
Pinned against fixtures produced by the reference's own code in float64
(tests/golden/make_splat_golden.py, tests/test_oracle_golden.py).
"""
import math

import numpy as np


def derived(img_size, sigma, lo, hi, normalize_color, pixel_size):
    scale = 1.0
    if normalize_color:
        sigma = sigma * img_size * pixel_size / (hi - lo)
        scale = (img_size * pixel_size / (hi - lo)) ** 2.0
    return float(sigma), max(1, math.ceil(5 * float(sigma))), float(scale)


def _patch(x, img_size, sigma, lo, hi, normalize_color, y_up, pixel_size):
    x = np.asarray(x, dtype=np.float64)
    sig, r, scale = derived(img_size, sigma, lo, hi, normalize_color, pixel_size)
    p = (x - lo) / (hi - lo) * (img_size - 1)
    if y_up:
        p = np.stack([p[:, 0], (img_size - 1) - p[:, 1]], axis=1)
    base = np.floor(p)
    frac = p - base
    offs = np.arange(-r, r + 1)
    tx = offs[None, :] - frac[:, 0:1]            # [N, P]
    ty = offs[None, :] - frac[:, 1:2]
    gx = np.exp(-tx ** 2 / (2 * sig * sig))
    gy = np.exp(-ty ** 2 / (2 * sig * sig))
    px = base[:, 0].astype(np.int64)[:, None] + offs[None, :]
    py = base[:, 1].astype(np.int64)[:, None] + offs[None, :]
    vx = (px >= 0) & (px < img_size)
    vy = (py >= 0) & (py < img_size)
    return sig, scale, tx, ty, gx, gy, px, py, vx, vy


def splat_forward(x, color, img_size=256, sigma=2.0, lo=-1.0, hi=1.0, normalize_color=True, y_up=False,
                  pixel_size=2.0 / 128.0):
    """``x [N,2]``, ``color [N,>=3]`` -> ``[img, img, 4]`` float64."""
    c = np.asarray(color, dtype=np.float64)[:, -3:]
    sig, scale, tx, ty, gx, gy, px, py, vx, vy = _patch(x, img_size, sigma, lo, hi, normalize_color, y_up, pixel_size)
    out = np.zeros((img_size, img_size, 4))
    for n in range(len(c)):
        w = gy[n][:, None] * gx[n][None, :]       # [P(dy), P(dx)]
        if normalize_color:
            w = w / (1e-8 + w.sum()) * scale
        ys, xs = py[n][vy[n]], px[n][vx[n]]
        if len(ys) == 0 or len(xs) == 0:
            continue
        wv = w[np.ix_(vy[n], vx[n])]
        out[np.ix_(ys, xs, [3])] += wv[:, :, None]
        out[np.ix_(ys, xs, [0, 1, 2])] += wv[:, :, None] * c[n][None, None, :]
    return out


def splat_backward(x, color, g_out, img_size=256, sigma=2.0, lo=-1.0, hi=1.0, normalize_color=True, y_up=False,
                   pixel_size=2.0 / 128.0):
    """Gradients ``(g_x [N,2], g_color [N,3])`` of ``sum(out * g_out)``."""
    c = np.asarray(color, dtype=np.float64)[:, -3:]
    g_out = np.asarray(g_out, dtype=np.float64)
    sig, scale, tx, ty, gx, gy, px, py, vx, vy = _patch(x, img_size, sigma, lo, hi, normalize_color, y_up, pixel_size)
    g_x, g_c = np.zeros((len(c), 2)), np.zeros((len(c), 3))
    chain = (img_size - 1) / (hi - lo)
    for n in range(len(c)):
        g = gy[n][:, None] * gx[n][None, :]
        ys, xs = py[n][vy[n]], px[n][vx[n]]
        d = np.zeros(g.shape + (4,))
        if len(ys) and len(xs):
            d[np.ix_(vy[n], vx[n])] = g_out[np.ix_(ys, xs)]
        A = d[..., :3] @ c[n] + d[..., 3]          # dL/dw per patch pixel (0 outside the image)
        TX, TY = np.broadcast_to(tx[n][None, :], g.shape), np.broadcast_to(ty[n][:, None], g.shape)
        a0, ax, ay = (A * g).sum(), (A * g * TX).sum(), (A * g * TY).sum()
        s = 1.0
        if normalize_color:
            S = g.sum()
            inv = 1.0 / (1e-8 + S)
            s = scale * inv
            ax -= a0 * inv * (g * TX).sum()
            ay -= a0 * inv * (g * TY).sum()
        g_c[n] = s * (g[..., None] * d[..., :3]).sum(axis=(0, 1))
        g_x[n] = [s * ax / sig ** 2 * chain, (-1.0 if y_up else 1.0) * s * ay / sig ** 2 * chain]
    return g_x, g_c
