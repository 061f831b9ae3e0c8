"""The adaptation MLP on the tensor-core linear kernels (three TF32 MMAs per product:
npa_linear_tcgen05 with the accumulators in tensor memory, and npa_linear_tf32x3 on mma.sync) and the
fused weight-gradient kernel (npa_mlp_weight_grad) against torch: values and gradients held to
float64 truth about as tightly as torch's own float32 run.  Every test runs once per engine."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["tcgen05", "mma.sync"])
def engine(request, monkeypatch):
    import npa_b200.mlp as mlp
    monkeypatch.setattr(mlp, "TENSOR_ENGINE", request.param)
    yield request.param
    if request.param == "tcgen05":   # no bounded wait of the kernel ever gave up
        from npa_b200 import _native as n
        status = ctypes.c_uint32(0)
        n.check(n.lib.npa_linear_tcgen05_status(ctypes.byref(status), 1))
        assert status.value == 0, f"linear_umma_kernel reported status {status.value}"


def _mlp(k, o, hidden=128, seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(k, hidden), torch.nn.ReLU(), torch.nn.Linear(hidden, o, bias=False)).cuda()


@pytest.mark.parametrize("rows,k,o", [(1000, 66, 18), (4096 + 7, 163, 35), (31, 176, 48), (2048, 5, 1), (65536 * 4, 163, 35)])
def test_gradients_match_float64_truth(rows, k, o):
    from npa_b200.mlp import apply_mlp, supported
    mlp = _mlp(k, o)
    assert supported(mlp)
    g = torch.Generator(device="cuda").manual_seed(1)
    shape = (2, rows // 2, k) if rows % 2 == 0 else (rows, k)
    z = torch.randn(*shape, generator=g, device="cuda")
    up = torch.randn(*shape[:-1], o, generator=g, device="cuda")

    def run(fn, module, dtype):
        module.zero_grad(set_to_none=True)
        zr = z.detach().clone().to(dtype).requires_grad_(True)
        y = fn(module, zr)
        y.backward(up.to(dtype))
        return [y.detach(), zr.grad] + [p.grad.clone() for p in module.parameters()]

    ours = run(apply_mlp, mlp, torch.float32)
    theirs = run(lambda m, t: m(t), mlp, torch.float32)
    truth = run(lambda m, t: m(t), _mlp(k, o).double(), torch.float64)
    names = ["y", "g_z", "g_W1", "g_b1", "g_W2"]
    for name, a, b, t in zip(names, ours, theirs, truth):
        scale = float(t.abs().max())
        err_ours = float((a.double() - t).abs().max())
        err_torch = float((b.double() - t).abs().max())
        # the split-precision products drop a term of 2^-22 per product: allow a few fp32 roundings more
        assert err_ours <= 4 * err_torch + 4e-6 * scale, (name, err_ours, err_torch, scale)
        print(f"{name}: error {err_ours:.3e} (torch fp32 {err_torch:.3e}) at scale {scale:.3e}")


def test_two_runs_are_bit_identical_and_unsupported_shapes_fall_back():
    from npa_b200.mlp import apply_mlp, supported
    mlp = _mlp(66, 18)
    z = torch.randn(3, 5000, 66, device="cuda")
    up = torch.randn(3, 5000, 18, device="cuda")
    grads = []
    for _ in range(2):
        mlp.zero_grad(set_to_none=True)
        apply_mlp(mlp, z.clone().requires_grad_(True)).backward(up)
        grads.append([p.grad.clone() for p in mlp.parameters()])
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    wide = _mlp(66, 18, hidden=64)
    assert not supported(wide)
    zr = z.clone().requires_grad_(True)
    apply_mlp(wide, zr).backward(up)      # plain module call
    assert zr.grad is not None and wide[0].weight.grad is not None
    big = _mlp(200, 18)
    assert not supported(big)


@pytest.mark.parametrize("rows,k,n,out_by_in,relu,bias", [(1000, 163, 128, True, True, True), (777, 128, 35, True, False, False),
                                                          (4096, 35, 128, False, False, False), (130, 128, 163, False, False, False),
                                                          (64, 176, 128, True, True, True), (5, 3, 1, True, False, True),
                                                          (128 * 148 * 2 + 77, 163, 128, True, True, True),
                                                          (40000, 128, 163, False, False, False), (300, 200, 256, True, False, True)])
def test_linear_kernel_against_float64(rows, k, n, out_by_in, relu, bias, engine):
    """The linear kernel alone, both weight layouts, odd sizes, partial tiles, more tiles than CTAs."""
    from npa_b200.mlp import _linear
    if engine == "mma.sync" and max(k, n) > 176:
        pytest.skip("the mma.sync kernel holds the whole weight matrix in shared memory: up to 176 x 176")
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(rows, k, generator=g, device="cuda")
    w = torch.randn((n, k) if out_by_in else (k, n), generator=g, device="cuda")
    b = torch.randn(n, generator=g, device="cuda") if bias else None
    got = _linear(a, w, b, relu, out_by_in)
    want = a.double() @ (w.double().t() if out_by_in else w.double())
    if bias:
        want = want + b.double()
    if relu:
        want = want.relu()
    plain = (a @ (w.t() if out_by_in else w)) + (b if bias else 0)
    plain = plain.relu() if relu else plain
    scale = float(want.abs().max())
    err, err_torch = float((got.double() - want).abs().max()), float((plain.double() - want).abs().max())
    assert err <= 4 * err_torch + 4e-6 * scale, (err, err_torch, scale)


def test_gated_linear_is_the_relu_backward():
    from npa_b200.mlp import _linear
    g = torch.Generator(device="cuda").manual_seed(3)
    dy = torch.randn(3000, 35, generator=g, device="cuda")
    w2 = torch.randn(35, 128, generator=g, device="cuda")
    h = torch.randn(3000, 128, generator=g, device="cuda").relu()
    want = torch.where(h > 0, dy.double() @ w2.double(), torch.zeros((), dtype=torch.float64, device="cuda"))
    for force in (True, False):
        got = _linear(dy, w2, None, False, False, gate=h, force_tensor=force)
        assert float((got.double() - want).abs().max()) <= 4e-6 * float(want.abs().max())
        assert torch.equal(got == 0, want == 0) or float(((got == 0) != (want == 0)).float().mean()) < 1e-6


def test_a_wait_that_runs_out_ends_the_tcgen05_kernel_roles_cleanly(engine):
    """The bounded waits of linear_umma_kernel: a wait on an mbarrier that nothing completes gives up after
    its limit and raises the leave flag; a second role waiting elsewhere leaves through the flag; the
    context stays usable (no trap, no fault, no endless loop)."""
    if engine != "tcgen05":
        pytest.skip("the mma.sync kernel has no mbarrier waits")
    from npa_b200 import _native as n
    res = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    n.check(n.lib.npa_linear_tcgen05_wait_selftest(2000, n.ptr(res), n.current_stream()))
    torch.cuda.synchronize()
    assert res.tolist() == [1, 1]
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
