"""The reference's own ``models/npa.py``, unmodified, running on the GPU on top of this package.

A copy of the reference checkout is expected under ``baseline/_ref/`` (kept out of the history; the
tests skip when it is absent).  ``npa_b200.install_as_sphops()`` makes ``from sphops import ...``
resolve to the B200 implementation, the file is loaded from disk exactly as it is, and its
``NPA.perceive`` / ``NPA.forward`` / ``step_euler`` (models/npa.py:87-204) are run forward and
backward.  What they produce is compared with the fused path of this package
(``npa_b200.stepping``: packed perception, fused update) on the same inputs and the same weights.
"""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REF_ROOT = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
REF_NPA = REF_ROOT / "models" / "npa.py"

CASES = {
    "d2_periodic": dict(dim=2, boundary="periodic", grid=(10, 10), eps=0.2, N=4096, B=2, C=16),
    "d3_clamped": dict(dim=3, boundary="clamped", grid=(12, 12, 12), eps=0.2, N=6000, B=2, C=16),
}


@pytest.fixture(scope="module")
def ref_npa():
    if not REF_NPA.exists():
        pytest.skip("no copy of the reference under baseline/_ref")
    import npa_b200
    saved = {k: sys.modules.get(k) for k in ("sphops", "sphops.sph", "sphops.sph_cuda")}
    npa_b200.install_as_sphops()
    spec = importlib.util.spec_from_file_location("reference_models_npa", REF_NPA)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    yield mod
    for k, v in saved.items():
        if v is None:
            sys.modules.pop(k, None)
        else:
            sys.modules[k] = v


def _inputs(c, seed):
    g = torch.Generator().manual_seed(seed)
    dim = c["dim"]
    half = [0.5 * n * c["eps"] for n in c["grid"]]
    span = torch.tensor(half) * (2.0 if c["boundary"] == "periodic" else 1.6)
    x = (torch.rand(c["B"], c["N"], dim, generator=g) - 0.5) * span
    if dim == 3:
        x = torch.cat([x, torch.zeros(c["B"], c["N"], 1)], dim=-1)
    s = 0.5 * torch.randn(c["B"], c["N"], c["C"], generator=g)
    return x.cuda().contiguous(), s.cuda().contiguous()


def _grid(c):
    from npa_b200 import sphops as sph
    return sph.HashGrid(dim=c["dim"], boundary=c["boundary"], mode="grid", grid_size=c["grid"], eps=c["eps"],
                        num_particles=c["N"], batch_size=c["B"], max_particles_per_block=32)


def _close(a, b, what, rtol=2e-5, atol=2e-6):
    """Two fp32 evaluations of the same formulas (operator by operator with torch glue, and fused).  Each
    side is held to 1e-5 relative / 1e-6 of the tensor's scale against the fp64 truth elsewhere
    (tests/test_gpu_ops_oracle.py, tests/test_gpu_fusion.py), so the two may differ from one another by
    twice that: 2e-5 relative / 2e-6 of the scale, elementwise."""
    a, b = a.detach().double(), b.detach().double()
    scale = float(b.abs().max())
    err = (a - b).abs()
    bad = err > rtol * b.abs() + atol * scale
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} of {bad.numel()} differ, worst {float(err.max()):.3e} (scale {scale:.3e})"


@pytest.mark.parametrize("case", sorted(CASES))
@pytest.mark.parametrize("stopgrad_pos", [True, False], ids=["stopgrad_pos", "grad_pos"])
def test_perceive_of_the_reference_model(ref_npa, case, stopgrad_pos):
    """``NPA.perceive`` of the reference on the per-operator API against the packed perception call."""
    from npa_b200 import stepping
    c = CASES[case]
    torch.manual_seed(3)
    model = ref_npa.NPA(spatial_dims=c["dim"], state_dims=c["C"], hidden_dims=128, eps0=0.1,
                        stopgrad_pos=stopgrad_pos).cuda()
    grid = _grid(c)
    x, s = _inputs(c, seed=11)
    xr, sr = x.clone().requires_grad_(True), s.clone().requires_grad_(True)
    z_ref, xb_ref, sb_ref, snap = model.perceive(xr, sr, grid)
    xf, sf = x.clone().requires_grad_(True), s.clone().requires_grad_(True)
    z, xb, sb, _ = stepping.perceive(model, xf, sf, grid)
    assert torch.equal(xb, xb_ref) and torch.equal(sb, sb_ref)
    assert z.shape == z_ref.shape == (c["B"], c["N"], model.perception_dim)
    _close(z, z_ref, f"{case}: z")
    up = torch.randn(z.shape, generator=torch.Generator().manual_seed(5)).cuda()
    z_ref.backward(up)
    z.backward(up)
    _close(sf.grad, sr.grad, f"{case}: dL/ds")
    if stopgrad_pos:
        assert xr.grad is None or float(xr.grad.abs().max()) == 0.0
    else:
        _close(xf.grad, xr.grad, f"{case}: dL/dx")


@pytest.mark.parametrize("case", sorted(CASES))
@pytest.mark.parametrize("stopgrad_pos", [True, False], ids=["stopgrad_pos", "grad_pos"])
def test_two_euler_steps_of_the_reference_model(ref_npa, case, stopgrad_pos):
    """Two ``step_euler`` steps of the reference file, forward and backward, against two steps of
    ``npa_b200.stepping.step_euler`` with the same weights, the same random update masks and the same
    upstream gradients: positions, states, and the gradients of the MLP weights and the input states."""
    from npa_b200 import stepping
    c = CASES[case]
    torch.manual_seed(7)
    model = ref_npa.NPA(spatial_dims=c["dim"], state_dims=c["C"], hidden_dims=128, eps0=0.1, alpha=1.0,
                        stopgrad_pos=stopgrad_pos).cuda()
    grid = _grid(c)
    x0, s0 = _inputs(c, seed=23)
    g = torch.Generator().manual_seed(9)
    up_x = torch.randn(x0.shape, generator=g).cuda()
    up_s = torch.randn(s0.shape, generator=g).cuda()
    if c["dim"] == 3:
        up_x[..., 3] = 0.0

    def rollout(step_fn):
        model.zero_grad(set_to_none=True)
        torch.manual_seed(101)  # the update masks of both rollouts come from the same stream of draws
        x, s = x0.clone(), s0.clone().requires_grad_(True)
        s_in = s
        for _ in range(2):
            x, s, _ = step_fn(model, x, s, grid, dt=1.0, update_prob=0.5)
        ((x * up_x).sum() + (s * up_s).sum()).backward()
        grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
        return x.detach(), s.detach(), s_in.grad.clone(), grads

    x_ref, s_ref, ds_ref, g_ref = rollout(ref_npa.step_euler)
    x_new, s_new, ds_new, g_new = rollout(stepping.step_euler)
    _close(x_new, x_ref, f"{case}: positions after two steps")
    _close(s_new, s_ref, f"{case}: states after two steps")
    _close(ds_new, ds_ref, f"{case}: dL/ds0")
    assert set(g_new) == set(g_ref) and g_ref
    for name in g_ref:
        _close(g_new[name], g_ref[name], f"{case}: grad of {name}")
