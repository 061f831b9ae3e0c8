"""CPU restatement (numpy) of the Euler update after perception and the MLP.  Test infrastructure
only: nothing of the product imports it.

Follows the reference line by line:
  * displacement limiter of ``NPA.forward`` (models/npa.py:145-149):
    ``dx = alpha * dx * eps / (1 + |dx|)``;
  * ``step_euler`` (models/npa.py:183-203): zero padding of a 3D displacement to 4 columns,
    ``x = x_bin + dt * dx * mask``, ``s = s_bin + dt * ds * mask``;
  * optional ``HashGrid.wrap_positions`` (sphops/sph.py:107-123):
    ``remainder(x + L/2, L) - L/2`` on the first ``dim`` columns.
Pinned against fixtures produced by the reference's own code (tests/golden/step_*.npz,
tests/test_oracle_golden.py).
"""
import numpy as np


def step_forward(y, x_bin, s_bin, mask, dim, eps, alpha, dt, box=None):
    """fp32 arithmetic in the reference's order.  ``mask`` [B,N] of 0/1 or None."""
    f = np.float32
    y, x_bin, s_bin = (np.asarray(t, dtype=f) for t in (y, x_bin, s_bin))
    m = np.ones(y.shape[:2], dtype=f) if mask is None else np.asarray(mask, dtype=f)
    m = m[..., None]
    dx = y[..., :dim]
    norm = np.sqrt(np.sum(dx * dx, axis=-1, keepdims=True, dtype=f)).astype(f)
    lim = ((f(alpha) * dx) * f(eps)) / (f(1.0) + norm)
    if x_bin.shape[-1] != dim:
        lim = np.concatenate([lim, np.zeros(lim.shape[:2] + (1,), dtype=f)], axis=-1)
    x = x_bin + (f(dt) * lim) * m
    s = s_bin + (f(dt) * y[..., dim:]) * m
    if box is not None:
        for d in range(dim):
            L = f(box[d])
            x[..., d] = np.mod(x[..., d] + f(0.5) * L, L) - f(0.5) * L
    return x.astype(f), s.astype(f)


def step_backward(y, mask, dim, eps, alpha, dt, g_x, g_s):
    """dL/dy in float64 (truth for the fp32 kernel).  d limiter / d dx = k [ I/(1+n) - dx dx^T / (n (1+n)^2) ]."""
    y = np.asarray(y, dtype=np.float64)
    m = np.ones(y.shape[:2]) if mask is None else np.asarray(mask, dtype=np.float64)
    m = m[..., None]
    g_y = np.zeros_like(y)
    g_y[..., dim:] = dt * m * np.asarray(g_s, dtype=np.float64)
    u = y[..., :dim]
    gx = np.asarray(g_x, dtype=np.float64)[..., :dim]
    n = np.sqrt(np.sum(u * u, axis=-1, keepdims=True))
    inv = 1.0 / (1.0 + n)
    proj = np.sum(u * gx, axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        second = np.where(n > 0, u * proj * inv * inv / n, 0.0)
    g_y[..., :dim] = alpha * eps * dt * m * (gx * inv - second)
    return g_y
