"""The per-particle adaptation MLP of an NPA model: tensor-core linear layers, fused weight gradients.

The reference's MLP (models/npa.py:63-75) is ``Linear(in, hidden) -> ReLU -> Linear(hidden, out,
bias=False)`` applied to every particle.  Its two forward GEMMs and the two input-gradient GEMMs
run on the tensor cores at fp32 accuracy (three TF32 MMAs per product on split operands, bias and
ReLU in the epilogue): ``npa_linear_tcgen05`` (tcgen05.mma, accumulators in tensor memory) by
default, ``npa_linear_tf32x3`` (``mma.sync``) when ``TENSOR_ENGINE = "mma.sync"``; the gradients of
the weights -- three reductions over all ``B * N`` rows, half of the MLP's forward + backward time
in torch -- come from one kernel: ``npa_mlp_weight_grad_tcgen05`` (the same tensor cores,
accumulation chains of 128 rows added in fp32) by default, the CUDA-core ``npa_mlp_weight_grad`` with
the other engine.  ``apply_mlp(module, z)`` returns ``module(z)`` computed
this way when ``module`` has the reference's structure and a hidden width of 128, and plain
``module(z)`` otherwise.
"""
from __future__ import annotations

import torch

from . import _native as N

_lib = N.lib
HIDDEN = 128
MAX_IN, MAX_OUT = 176, 48
MAX_IN_TCGEN05 = 175  # the tcgen05 weight-gradient kernel appends a column of ones to z: in + 1 <= 176
MIN_TENSOR_DIM = 64   # narrower products go to the library
TENSOR_ENGINE = "tcgen05"   # or "mma.sync": which kernel runs the wide products
FUSED_HIDDEN_GRAD = True    # dh = (dy W2) with the ReLU mask in one pass on the CUDA cores
FUSED_FORWARD = True        # tcgen05 engine: both layers of the forward in one kernel (h kept in tensor memory)
GATED_DH_ON_TENSOR_CORES = False  # dh = (dy W2) gated by h in one tensor-core kernel: measured slower (1.42 vs 1.35 ms per MLP pass) than the thin library GEMM + a mask pass


def _linear(a, w, bias, relu, w_is_out_by_in, gate=None, force_tensor=False):
    """``a @ w.T`` (``w`` is [out, in], as in F.linear) or ``a @ w`` (``w`` is [in, out]) with optional
    bias and ReLU on the tensor cores (three TF32 MMAs per product, fp32 accuracy); with ``gate`` the
    result is zeroed where ``gate <= 0`` (the backward of the ReLU that produced ``gate``)."""
    m, k = a.shape
    n = w.shape[0] if w_is_out_by_in else w.shape[1]
    if min(k, n) < MIN_TENSOR_DIM and not force_tensor:
        # thin products (35 output or input columns) are bound by memory and launch latency, not by
        # arithmetic: the library's fp32 kernels are faster there
        wt = w.t() if w_is_out_by_in else w
        c = torch.addmm(bias, a, wt) if bias is not None else a @ wt
        if gate is not None:
            c = torch.ops.aten.threshold_backward(c, gate, 0.0)
        return c.relu_() if relu else c
    stride_out, stride_in = (w.stride(0), w.stride(1)) if w_is_out_by_in else (w.stride(1), w.stride(0))
    c = torch.empty(m, n, dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        if TENSOR_ENGINE == "tcgen05":
            nbytes = _lib.npa_linear_tcgen05_scratch_bytes(k, n)
            scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=a.device)  # weight image, private to the call
            N.check(_lib.npa_linear_tcgen05(N.ptr(a), N.ptr(w), N.ptr(bias), N.ptr(gate), N.ptr(c), m, k, n, stride_out,
                                            stride_in, 1 if relu else 0, N.ptr(scratch), nbytes, N.current_stream()))
        else:
            N.check(_lib.npa_linear_tf32x3(N.ptr(a), N.ptr(w), N.ptr(bias), N.ptr(gate), N.ptr(c), m, k, n, stride_out,
                                           stride_in, 1 if relu else 0, N.current_stream()))
    return c


class _AdaptationMLP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, w1, b1, w2):
        rows = z.reshape(-1, z.shape[-1])
        m, k, o = rows.shape[0], rows.shape[1], w2.shape[0]
        if TENSOR_ENGINE == "tcgen05" and FUSED_FORWARD and o <= MAX_OUT:
            # both layers in one kernel: h stays in tensor memory between them (it is also stored for the backward)
            h = torch.empty(m, HIDDEN, dtype=torch.float32, device=rows.device)
            y = torch.empty(m, o, dtype=torch.float32, device=rows.device)
            nbytes = _lib.npa_mlp_forward_tcgen05_scratch_bytes(k, o)
            scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=rows.device)
            with torch.cuda.device(rows.device):
                N.check(_lib.npa_mlp_forward_tcgen05(N.ptr(rows), N.ptr(w1), N.ptr(b1), N.ptr(w2), N.ptr(h), N.ptr(y), m, k, o,
                                                     w1.stride(0), w1.stride(1), w2.stride(0), w2.stride(1), N.ptr(scratch), nbytes,
                                                     N.current_stream()))
        else:
            h = _linear(rows, w1, b1, True, True)
            y = _linear(h, w2, None, False, True)
        ctx.save_for_backward(rows, h, w1, w2)
        ctx.z_shape = z.shape
        return y.reshape(*z.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, g_y):
        rows, h, w1, w2 = ctx.saved_tensors
        need_z, need_w1, need_b1, need_w2 = ctx.needs_input_grad
        dy = g_y.reshape(-1, g_y.shape[-1]).contiguous()
        if FUSED_HIDDEN_GRAD and w2.shape[0] <= MAX_OUT:
            # dh = (dy W2) masked by h > 0 in one pass (fp32, CUDA cores) instead of a thin GEMM plus a masking pass
            dh = torch.empty_like(h)
            with torch.cuda.device(h.device):
                N.check(_lib.npa_mlp_hidden_grad(N.ptr(dy), N.ptr(w2), N.ptr(h), N.ptr(dh), dy.shape[0], HIDDEN, w2.shape[0],
                                                 w2.stride(0), w2.stride(1), N.current_stream()))
        else:
            dh = _linear(dy, w2, None, False, False, gate=h, force_tensor=GATED_DH_ON_TENSOR_CORES)  # ReLU mask from h
        g_z = _linear(dh, w1, None, False, False).reshape(ctx.z_shape) if need_z else None
        g_w1 = g_b1 = g_w2 = None
        if need_w1 or need_b1 or need_w2:
            m, k, o = rows.shape[0], rows.shape[1], w2.shape[0]
            g_w1, g_b1, g_w2 = torch.empty_like(w1), torch.empty(HIDDEN, dtype=w1.dtype, device=w1.device), torch.empty_like(w2)
            on_tcgen05 = TENSOR_ENGINE == "tcgen05" and k <= MAX_IN_TCGEN05
            sizer, kernel = ((_lib.npa_mlp_weight_grad_tcgen05_scratch_floats, _lib.npa_mlp_weight_grad_tcgen05) if on_tcgen05
                             else (_lib.npa_mlp_weight_grad_scratch_floats, _lib.npa_mlp_weight_grad))
            n_scratch = sizer(m, k, o)
            scratch = torch.empty(n_scratch, dtype=torch.float32, device=rows.device)
            with torch.cuda.device(rows.device):
                N.check(kernel(N.ptr(rows), N.ptr(dh), N.ptr(h), N.ptr(dy), m, k, HIDDEN, o, N.ptr(scratch), n_scratch,
                               N.ptr(g_w1), N.ptr(g_w2), N.ptr(g_b1), N.current_stream()))
        return g_z, (g_w1 if need_w1 else None), (g_b1 if need_b1 else None), (g_w2 if need_w2 else None)


def supported(module) -> bool:
    """True for ``Sequential(Linear(in, 128), ReLU, Linear(128, out, bias=False))`` in float32 on a
    CUDA device with ``in <= 176`` and ``out <= 48`` -- the shape of the reference's adaptation MLP."""
    if not (isinstance(module, torch.nn.Sequential) and len(module) == 3):
        return False
    l1, act, l2 = module[0], module[1], module[2]
    if not (isinstance(l1, torch.nn.Linear) and isinstance(act, torch.nn.ReLU) and isinstance(l2, torch.nn.Linear)):
        return False
    if l1.bias is None or l2.bias is not None or l1.out_features != HIDDEN or l2.in_features != HIDDEN:
        return False
    if l1.in_features > MAX_IN or l2.out_features > MAX_OUT:
        return False
    return l1.weight.is_cuda and l1.weight.dtype == torch.float32 and l2.weight.dtype == torch.float32


def apply_mlp(module, z):
    """``module(z)``; with the fused weight-gradient backward when ``supported(module)``."""
    if not (supported(module) and z.is_cuda and z.dtype == torch.float32):
        return module(z)
    return _AdaptationMLP.apply(z.contiguous(), module[0].weight, module[0].bias, module[2].weight)
