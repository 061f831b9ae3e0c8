"""Gaussian particle splatting (npa_splat_forward / backward, npa_b200.splatting) against fixtures
produced by the reference's utils/splatting.py, against the float64 oracle on larger seeded inputs,
and through size-independent properties at the sizes the reference's trainers use."""
import ast

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR

pytestmark = pytest.mark.gpu

# fp32 against float64 truth.  The pixel position p = (x - lo) / (hi - lo) * (img - 1) carries an fp32
# rounding of ~img * 6e-8 pixels into every weight of a particle, so the bound is relative to the
# largest value of the tensor; the reference's own fp32 run is held to the same bound below.
RTOL, ATOL_SCALE = 1e-5, 5e-6


def _close(got, want, name, ref32=None):
    want = np.asarray(want, dtype=np.float64)
    got = got.detach().cpu().numpy().astype(np.float64)
    scale = max(np.abs(want).max(), 1e-30)
    tol = RTOL * np.abs(want) + ATOL_SCALE * scale
    err = np.abs(got - want)
    assert (err <= tol).all(), f"{name}: worst {err.max():.3e} at scale {scale:.3e}"
    if ref32 is not None:  # not worse than twice what the reference's fp32 run loses (plus a floor)
        ref_err = np.abs(np.asarray(ref32, dtype=np.float64) - want).max()
        assert err.max() <= 2 * ref_err + 1e-6 * scale, f"{name}: {err.max():.3e} vs reference fp32 {ref_err:.3e}"


@pytest.mark.parametrize("name", ["splat_default_small", "splat_plain_yup", "splat_wide_box"])
def test_fixture_of_reference_splatting(name):
    from npa_b200 import splatting
    g = np.load(GOLDEN_DIR / f"{name}.npz")
    meta = ast.literal_eval(str(g["meta"]))
    x = torch.from_numpy(g["x"]).cuda().requires_grad_(True)
    c = torch.from_numpy(g["color"]).cuda().requires_grad_(True)
    out = splatting.splat_particles_batch(x, c, **meta["kw"])
    assert out.shape == g["out_f64"].shape
    _close(out, g["out_f64"], "image", g["out_f32"])
    out.backward(torch.from_numpy(g["up"]).cuda())
    _close(x.grad, g["g_x_f64"], "g_x", g["g_x_f32"])
    _close(c.grad, g["g_color_f64"], "g_color", g["g_color_f32"])
    # single-system call and the list-of-sections call of the reference's API
    one = splatting.splat_particles(x[0].detach(), c[0].detach(), **meta["kw"])
    assert torch.equal(one, out[0].detach())
    n = x.shape[1]
    sec = splatting.splat_particles_sections(x.detach().reshape(-1, 2), c.detach().reshape(-1, c.shape[-1]),
                                             [n] * x.shape[0], **meta["kw"])
    assert torch.equal(sec, out.detach())


@pytest.mark.parametrize("normalize,y_up,img,sigma", [(True, False, 64, 1.0), (False, True, 50, 2.5), (True, True, 33, 0.5)])
def test_seeded_inputs_against_oracle(normalize, y_up, img, sigma):
    from npa_b200 import splatting
    from oracle import splat as splat_oracle
    g = torch.Generator().manual_seed(31)
    B, n = 2, 700
    kw = dict(img_size=img, sigma=sigma, lo=-1.0, hi=1.0, normalize_color=normalize, y_up=y_up, pixel_size=2.0 / img)
    x = (torch.rand(B, n, 2, generator=g) * 2.4 - 1.2)       # a margin of particles outside the image
    c = torch.rand(B, n, 3, generator=g)
    up = torch.randn(B, img, img, 4, generator=g)
    xc, cc = x.cuda().requires_grad_(True), c.cuda().requires_grad_(True)
    out = splatting.splat_particles_batch(xc, cc, **kw)
    out.backward(up.cuda())
    for b in range(B):
        want = splat_oracle.splat_forward(x[b].numpy(), c[b].numpy(), **kw)
        _close(out[b], want, "image")
        g_x, g_c = splat_oracle.splat_backward(x[b].numpy(), c[b].numpy(), up[b].numpy(), **kw)
        _close(xc.grad[b], g_x, "g_x")
        _close(cc.grad[b], g_c, "g_color")


def test_trainer_size_properties_and_determinism():
    """img 256, sigma 2 (patch 41 x 41), 8 systems of 4,096 particles -- the reference's growing /
    texture setting.  Particles well inside the image deposit exactly norm_scale of density each and
    their colour times that; two runs give identical bits; an empty region stays zero."""
    from npa_b200 import splatting
    g = torch.Generator(device="cuda").manual_seed(4)
    B, n, img = 8, 4096, 256
    x = (torch.rand(B, n, 2, generator=g, device="cuda") - 0.5) * 1.0      # inside [-0.5, 0.5]: patches stay inside
    c = torch.rand(B, n, 3, generator=g, device="cuda")
    xr, cr = x.clone().requires_grad_(True), c.clone().requires_grad_(True)
    out = splatting.splat_particles_batch(xr, cr)
    again = splatting.splat_particles_batch(x, c)
    assert torch.equal(out.detach(), again)
    scale = (img * (2.0 / 128.0) / 2.0) ** 2
    dens = out[..., 3].sum(dim=(1, 2)).double()
    assert torch.allclose(dens, torch.full_like(dens, n * scale), rtol=2e-5)
    rgb = out[..., :3].sum(dim=(1, 2)).double()
    assert torch.allclose(rgb, c.double().sum(dim=1) * scale, rtol=2e-5)
    assert float(out[:, :20, :20].abs().max()) == 0.0            # no particle reaches the corner
    # the total density does not depend on the positions, so its gradient with respect to x vanishes
    out[..., 3].sum().backward()
    assert float(xr.grad.abs().max()) <= 1e-3 * scale * 255 / 2
    assert float(cr.grad.abs().max()) == 0.0


def test_argument_errors():
    from npa_b200 import splatting
    x = torch.zeros(1, 8, 2, device="cuda")
    c = torch.zeros(1, 8, 3, device="cuda")
    with pytest.raises(TypeError):
        splatting.splat_particles_batch(x.cpu(), c)
    with pytest.raises(RuntimeError):
        splatting.splat_particles_batch(x, c[:, :4])
    with pytest.raises(ValueError):          # patch radius beyond what the kernels support
        splatting.splat_particles_batch(x, c, img_size=64, sigma=20.0, normalize_color=False)
