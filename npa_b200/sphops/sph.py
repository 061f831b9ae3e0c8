"""The ``sphops`` operator API on top of the B200 kernels.

Same public names, signatures, defaults and autograd behaviour as the
reference's ``sphops/sph.py`` (HashGrid :42-123, Permute :127-184,
unbin_particles :187-198, Count :201-229, Density :232-267, Blur :270-321,
Gradient :324-376, DensityGradient :379-413, MomentMatrix :416-464,
safe_inv_sym_mat :467-471, gradient_hybrid :474-484), so ``models/npa.py`` and
the trainers of the reference run unchanged on it.  Two additions that the
reference does not have: :func:`perceive`, the fused forward/backward of the
whole perception step, and the ``device`` argument of :class:`HashGrid`.

Semantics kept from the reference: default mass is 1.0 per particle; ``rho`` is
a density and the operators form ``mass / rho`` themselves; 3D positions are
``[B, N, 4]`` with an ignored fourth column whose gradient is 0; gradients of
inputs that do not require grad are returned as ``None``.
"""
from __future__ import annotations

import math
import weakref
from dataclasses import dataclass, field

import torch

from . import sph_cuda


def _default_mass(x, mass):
    if mass is None:
        B, N, _ = x.shape
        return x.new_full((B, N), 1.0)
    if mass.dim() == 3 and mass.shape[-1] == 1:
        return mass.squeeze(-1)
    return mass


_GRID_CLASSES = {
    (2, "periodic", "grid"): "HashGrid2DPeriodic",
    (3, "periodic", "grid"): "HashGrid3DPeriodic",
    (2, "clamped", "grid"): "HashGrid2DBox",
    (3, "clamped", "grid"): "HashGrid3DBox",
    (2, "periodic", "particle"): "VHashGrid2DPeriodic",
    (3, "periodic", "particle"): "VHashGrid3DPeriodic",
    (2, "clamped", "particle"): "VHashGrid2DBox",
    (3, "clamped", "particle"): "VHashGrid3DBox",
}


def get_hashgrid_cls(dim, boundary, mode):
    return getattr(sph_cuda, _GRID_CLASSES[(dim, boundary, mode)])


@dataclass
class HashGridSnapshot:
    """Result of one binning pass; every tensor a later operator needs lives here."""

    grid: object
    bin_offsets: torch.Tensor
    permutation: torch.Tensor
    block_info: torch.Tensor
    dim: int
    # outputs computed ahead of their call by a fused sweep (see enable_fusion); not part of the
    # reference's dataclass, defaulted so positional construction still works
    parked: dict = field(default_factory=dict, repr=False, compare=False)


class HashGrid:
    """Uniform grid over ``[-G*eps/2, G*eps/2)`` per axis, cell size = cut-off ``eps``.

    ``mode="grid"`` orders cells linearly, ``mode="particle"`` along a Morton
    curve (power-of-two sizes only); both run the same kernels here.
    ``max_particles_per_block`` bounds the particles of one work item.
    """

    def __init__(self, dim=2, boundary="periodic", mode="grid", grid_size=(16, 16), eps=0.1,
                 num_particles=4096, batch_size=8, max_particles_per_block=64, device=None):
        self.dim = dim
        self.boundary = boundary
        self.mode = mode
        self.grid_size = grid_size
        self.eps = eps
        self.num_particles = num_particles
        self.batch_size = batch_size
        self.max_particles_per_block = max_particles_per_block
        if mode == "particle":
            for size in grid_size:
                assert (size & (size - 1)) == 0, "grid_size must be a power of 2"
        self.num_cells = math.prod(grid_size)
        self.hashgrid_cls = get_hashgrid_cls(dim, boundary, mode)
        self.hashgrid = self.hashgrid_cls(*grid_size, eps, num_particles, batch_size, max_particles_per_block)
        self.device = torch.device("cuda") if device is None else torch.device(device)
        self._last_snapshot = None

    def instantiate(self, x):
        """Bin positions ``x [B, N, P]`` and return the snapshot the operators take."""
        B, N, _ = x.shape
        dev = x.device if x.is_cuda else self.device
        permutation = torch.empty(B, N, dtype=torch.int32, device=dev)
        bin_offsets = torch.empty(B * self.num_cells + 1, dtype=torch.int32, device=dev)
        block_info = torch.empty(self.hashgrid.max_blocks, 4, dtype=torch.int32, device=dev)
        self.hashgrid.initialize(x, permutation, bin_offsets, block_info)
        # outputs a fused sweep parked on the previous snapshot and nobody claimed are dropped now: they would
        # otherwise live (with the autograd graph they hang on) for as long as that snapshot does
        previous = self._last_snapshot() if self._last_snapshot is not None else None
        if previous is not None:
            previous.parked.clear()
        snapshot = HashGridSnapshot(grid=self.hashgrid, bin_offsets=bin_offsets, permutation=permutation,
                                    block_info=block_info, dim=self.dim)
        self._last_snapshot = weakref.ref(snapshot)
        return snapshot

    def wrap_positions(self, x):
        """Periodic: map each of the ``dim`` coordinates into ``[-L/2, L/2)``; clamped: identity."""
        if self.boundary != "periodic":
            return x
        cols = []
        for d in range(self.dim):
            L = torch.tensor(self.grid_size[d] * self.eps, device=x.device)
            cols.append(torch.remainder(x[..., d] + 0.5 * L, L) - 0.5 * L)
        return torch.stack(cols, dim=-1)


# ---------------------------------------------------------------------------------------------
# Operator fusion behind the per-operator API.
#
# NPA.perceive (models/npa.py:105-126) calls density, blur, moment_matrix, gradient and
# density_gradient one after the other with the SAME tensor objects; each is a full sweep over the
# neighbour cells in the reference.  With fusion enabled, density() also computes the density
# gradient and blur() also computes the feature gradient and the moment matrix, in the same sweep,
# and parks the extra outputs on the snapshot; the later call returns the parked tensor when it
# is made with the very same input objects (identity and version), otherwise it runs its own
# kernel as usual.  Five sweeps become two, and autograd sees one node per sweep, so the backward
# is fused too.  Off by default: a caller that only wants blur would pay for the gradient.
# ---------------------------------------------------------------------------------------------
_FUSION = {"enabled": False}
# Columns of the neighbour-list cache the fused forward passes write for their backward pass
# (row = count, j_0, j_1, ...; particles with more neighbours are searched again); 0 = off.
_PAIR_CACHE = {"columns": 128}


def set_pair_cache(columns=128):
    """Size of the per-particle neighbour list the fused forward sweeps keep for their backward
    (4 * columns bytes per particle while the autograd graph is alive); 0 disables it."""
    columns = int(columns)
    if columns != 0 and not 2 <= columns <= 513:
        raise ValueError("columns must be 0 or between 2 and 513")
    _PAIR_CACHE["columns"] = columns


def _new_pair_cache(s_bin, wanted):
    K = _PAIR_CACHE["columns"]
    if not wanted or K == 0:
        return None
    B, N = s_bin.shape[:2]
    return torch.empty(B, N, K, dtype=torch.int32, device=s_bin.device)


def enable_fusion(flag=True):
    """Turn speculative sibling-output fusion of the per-operator API on or off (process wide)."""
    _FUSION["enabled"] = bool(flag)


def fusion_enabled():
    return _FUSION["enabled"]


def _key(*tensors):
    """Identity + version of the input tensor objects (None allowed), held weakly: a parked output never
    keeps its inputs alive, and an input that has died can never match again."""
    return tuple((None if t is None else weakref.ref(t), None if t is None else t._version) for t in tensors)


def _same(key, *tensors):
    return len(key) == len(tensors) and all(
        (t is None and kt is None) or (t is not None and kt is not None and kt() is t and kv == t._version)
        for (kt, kv), t in zip(key, tensors))


def _park(snapshot, name, key, value):
    snapshot.parked[name] = (key, value)


def _claim(snapshot, name, *tensors):
    entry = snapshot.parked.get(name)
    if entry is None or not _same(entry[0], *tensors):
        return None
    del snapshot.parked[name]
    return entry[1]


class DensityPair(torch.autograd.Function):
    """density and density_gradient of the same positions in one sweep."""

    @staticmethod
    def forward(ctx, x_bin, mass, snapshot, pairs=None):
        B, N = x_bin.shape[:2]
        rho = torch.empty(B, N, dtype=torch.float32, device=x_bin.device)
        rho_grad = torch.empty(B, N, snapshot.dim, dtype=torch.float32, device=x_bin.device)
        snapshot.grid.perception_forward(x_bin, mass, None, rho, None, rho_grad, None, None, None,
                                         snapshot.bin_offsets, snapshot.block_info, pair_cache=pairs)
        ctx.save_for_backward(x_bin, *([] if mass is None else [mass]))
        ctx.pairs = pairs
        ctx.has_mass = mass is not None
        ctx.snapshot = snapshot
        ctx.dLdx = x_bin.requires_grad
        return rho, rho_grad

    @staticmethod
    def backward(ctx, g_rho, g_rho_grad):
        if not ctx.dLdx or (g_rho is None and g_rho_grad is None):
            return None, None, None, None
        saved = ctx.saved_tensors
        x_bin, mass = saved[0], (saved[1] if ctx.has_mass else None)
        snap = ctx.snapshot
        grad_x = torch.empty_like(x_bin)
        cont = lambda t: None if t is None else t.contiguous()
        snap.grid.density_chain_backward(x_bin, mass, cont(g_rho), None, cont(g_rho_grad), grad_x, False,
                                         snap.bin_offsets, snap.block_info, pair_cache=ctx.pairs)
        return grad_x, None, None, None


class BlurGradient(torch.autograd.Function):
    """blur, feature gradient and (not differentiated) moment matrix in one sweep."""

    @staticmethod
    def forward(ctx, x_bin, s_bin, rho, mass, snapshot, pairs=None):
        B, N, C = s_bin.shape
        dev, dim = x_bin.device, snapshot.dim
        s_blur = torch.empty_like(s_bin)
        s_grad = torch.empty(B, N, C, dim, dtype=torch.float32, device=dev)
        moment = torch.empty(B, N, dim, dim, dtype=torch.float32, device=dev)
        valid = pairs is not None          # lists recorded by the density sweep of the same positions
        if pairs is None:
            pairs = _new_pair_cache(s_bin, x_bin.requires_grad or s_bin.requires_grad or rho.requires_grad)
        snapshot.grid.blur_gradient_forward(x_bin, rho, mass, s_bin, s_blur, s_grad, snapshot.bin_offsets,
                                            snapshot.block_info, moment, pair_cache=pairs, pair_cache_valid=valid)
        ctx.save_for_backward(x_bin, s_bin, rho, *([] if mass is None else [mass]))
        ctx.pairs = pairs
        ctx.has_mass = mass is not None
        ctx.snapshot = snapshot
        ctx.needs = (x_bin.requires_grad, s_bin.requires_grad, rho.requires_grad)
        ctx.mark_non_differentiable(moment)
        return s_blur, s_grad, moment

    @staticmethod
    def backward(ctx, g_blur, g_grad, _g_moment):
        saved = ctx.saved_tensors
        x_bin, s_bin, rho = saved[:3]
        mass = saved[3] if ctx.has_mass else None
        dLdx, dLds, dLdrho = ctx.needs
        if (g_blur is None and g_grad is None) or not (dLdx or dLds or dLdrho):
            return None, None, None, None, None, None
        snap = ctx.snapshot
        cont = lambda t: None if t is None else t.contiguous()
        grad_x = torch.empty_like(x_bin) if dLdx else None
        grad_s = torch.empty_like(s_bin) if dLds else None
        grad_rho = torch.empty_like(rho) if dLdrho else None
        snap.grid.blur_gradient_backward(x_bin, rho, mass, s_bin, cont(g_blur), cont(g_grad), grad_x, grad_s,
                                         grad_rho, snap.bin_offsets, snap.block_info, pair_cache=ctx.pairs)
        return grad_x, grad_s, grad_rho, None, None, None


def _zeros_like_shape(shape, dtype, device):
    return torch.zeros(shape, dtype=dtype, device=device)


class Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, s, mass, snapshot):
        x_bin, s_bin, mass_bin = torch.empty_like(x), torch.empty_like(s), torch.empty_like(mass)
        snapshot.grid.bin_particles(x, s, mass, snapshot.permutation, x_bin, s_bin, mass_bin)
        ctx.snapshot = snapshot
        ctx.meta = (x.shape, s.shape, mass.shape, x.dtype, x.device)
        ctx.needs = (x.requires_grad, s.requires_grad, mass.requires_grad)
        return x_bin, s_bin, mass_bin

    @staticmethod
    def backward(ctx, g_x, g_s, g_m):
        xs, ss, ms, dtype, device = ctx.meta
        g_x = _zeros_like_shape(xs, dtype, device) if g_x is None else g_x.contiguous()
        g_s = _zeros_like_shape(ss, dtype, device) if g_s is None else g_s.contiguous()
        g_m = _zeros_like_shape(ms, dtype, device) if g_m is None else g_m.contiguous()
        o_x, o_s, o_m = torch.empty_like(g_x), torch.empty_like(g_s), torch.empty_like(g_m)
        snap = ctx.snapshot
        snap.grid.backward_bin_particles(g_x, g_s, g_m, snap.permutation, o_x, o_s, o_m)
        nx, ns, nm = ctx.needs
        return (o_x if nx else None, o_s if ns else None, o_m if nm else None, None)


def bin_particles(x, s, snapshot, mass=None):
    no_mass = mass is None
    out = Permute.apply(x, s, _default_mass(x, mass), snapshot)
    return out[:2] if no_mass else out


def unbin_particles(x_bin, s_bin, snapshot, mass_bin=None):
    no_mass = mass_bin is None
    mass_bin = _default_mass(x_bin, mass_bin)
    x, s, mass = torch.empty_like(x_bin), torch.empty_like(s_bin), torch.empty_like(mass_bin)
    snapshot.grid.backward_bin_particles(x_bin, s_bin, mass_bin, snapshot.permutation, x, s, mass)
    return (x, s) if no_mass else (x, s, mass)


class Count(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_bin, snapshot):
        out = torch.empty(x_bin.shape[:-1], dtype=torch.float32, device=x_bin.device)
        snapshot.grid.count_forward(x_bin, out, snapshot.bin_offsets, snapshot.block_info)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        # a neighbour count is piecewise constant in the positions
        return None, None


def count(x_bin, snapshot):
    return Count.apply(x_bin, snapshot)


class Density(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_bin, mass, snapshot):
        rho = torch.empty(x_bin.shape[:-1], dtype=torch.float32, device=x_bin.device)
        snapshot.grid.density_forward(x_bin, mass, rho, snapshot.bin_offsets, snapshot.block_info)
        ctx.save_for_backward(x_bin, mass)
        ctx.snapshot = snapshot
        ctx.dLdx = x_bin.requires_grad
        return rho

    @staticmethod
    def backward(ctx, grad_output):
        if not ctx.dLdx:
            return None, None, None
        x_bin, mass = ctx.saved_tensors
        snap = ctx.snapshot
        grad_x = torch.empty_like(x_bin)
        snap.grid.density_backward(x_bin, mass, grad_output.contiguous(), grad_x, snap.bin_offsets,
                                   snap.block_info, True)
        return grad_x, None, None


def density(x_bin, snapshot, mass=None):
    if _FUSION["enabled"]:
        pairs = _new_pair_cache(x_bin, True)
        rho, rho_grad = DensityPair.apply(x_bin, None if mass is None else _default_mass(x_bin, mass), snapshot,
                                          pairs)
        _park(snapshot, "density_gradient", _key(x_bin, mass), rho_grad)
        if pairs is not None:
            _park(snapshot, "pair_cache", _key(x_bin), pairs)   # the lists depend on the positions only
        return rho
    return Density.apply(x_bin, _default_mass(x_bin, mass), snapshot)


class _FeatureOp(torch.autograd.Function):
    """Shared autograd plumbing of Blur and Gradient (inputs x_bin, s_bin, rho, mass, snapshot)."""

    @staticmethod
    def _forward(ctx, fwd_name, out_tail, x_bin, s_bin, rho, mass, snapshot):
        out = torch.empty(*s_bin.shape, *out_tail, dtype=torch.float32, device=x_bin.device)
        getattr(snapshot.grid, fwd_name)(x_bin, rho, mass, s_bin, out, snapshot.bin_offsets, snapshot.block_info)
        ctx.save_for_backward(x_bin, s_bin, rho, mass)
        ctx.snapshot = snapshot
        ctx.needs = (x_bin.requires_grad, s_bin.requires_grad, rho.requires_grad)
        return out

    @staticmethod
    def _backward(ctx, bwd_name, grad_output):
        x_bin, s_bin, rho, mass = ctx.saved_tensors
        snap = ctx.snapshot
        dLdx, dLds, dLdrho = ctx.needs
        grad_x, grad_s, grad_rho = torch.empty_like(x_bin), torch.empty_like(s_bin), torch.empty_like(rho)
        getattr(snap.grid, bwd_name)(x_bin, rho, mass, s_bin, grad_output.contiguous(), grad_x, grad_s, grad_rho,
                                     snap.bin_offsets, snap.block_info, dLdx, dLds, dLdrho)
        return (grad_x if dLdx else None, grad_s if dLds else None, grad_rho if dLdrho else None, None, None)


class Blur(_FeatureOp):
    @staticmethod
    def forward(ctx, x_bin, s_bin, rho, mass, snapshot):
        return _FeatureOp._forward(ctx, "blur_forward", (), x_bin, s_bin, rho, mass, snapshot)

    @staticmethod
    def backward(ctx, grad_output):
        return _FeatureOp._backward(ctx, "blur_backward", grad_output)


def blur(x_bin, rho, s_bin, snapshot, mass=None):
    if _FUSION["enabled"]:
        s_blur, s_grad, moment = BlurGradient.apply(
            x_bin, s_bin, rho, None if mass is None else _default_mass(x_bin, mass), snapshot,
            _claim(snapshot, "pair_cache", x_bin))
        _park(snapshot, "gradient", _key(x_bin, rho, s_bin, mass), s_grad)
        _park(snapshot, "moment_matrix", _key(x_bin, rho, mass), moment)
        return s_blur
    return Blur.apply(x_bin, s_bin, rho, _default_mass(x_bin, mass), snapshot)


class Gradient(_FeatureOp):
    @staticmethod
    def forward(ctx, x_bin, s_bin, rho, mass, snapshot):
        return _FeatureOp._forward(ctx, "gradient_forward", (snapshot.dim,), x_bin, s_bin, rho, mass, snapshot)

    @staticmethod
    def backward(ctx, grad_output):
        return _FeatureOp._backward(ctx, "gradient_backward", grad_output)


def gradient(x_bin, rho, s_bin, snapshot, mass=None):
    parked = _claim(snapshot, "gradient", x_bin, rho, s_bin, mass)
    if parked is not None:
        return parked
    return Gradient.apply(x_bin, s_bin, rho, _default_mass(x_bin, mass), snapshot)


class DensityGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_bin, mass, snapshot):
        out = torch.empty(*x_bin.shape[:-1], snapshot.dim, dtype=torch.float32, device=x_bin.device)
        snapshot.grid.density_gradient_forward(x_bin, mass, out, snapshot.bin_offsets, snapshot.block_info)
        ctx.save_for_backward(x_bin, mass)
        ctx.snapshot = snapshot
        ctx.dLdx = x_bin.requires_grad
        return out

    @staticmethod
    def backward(ctx, grad_output):
        if not ctx.dLdx:
            return None, None, None
        x_bin, mass = ctx.saved_tensors
        snap = ctx.snapshot
        grad_x = torch.empty_like(x_bin)
        snap.grid.density_gradient_backward(x_bin, mass, grad_output.contiguous(), grad_x, snap.bin_offsets,
                                            snap.block_info, True)
        return grad_x, None, None


def density_gradient(x_bin, snapshot, mass=None):
    parked = _claim(snapshot, "density_gradient", x_bin, mass)
    if parked is not None:
        return parked
    return DensityGradient.apply(x_bin, _default_mass(x_bin, mass), snapshot)


class MomentMatrix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_bin, rho, mass, snapshot):
        dim = snapshot.dim
        out = torch.empty(*x_bin.shape[:-1], dim, dim, dtype=torch.float32, device=x_bin.device)
        snapshot.grid.moment_matrix_forward(x_bin, rho, mass, out, snapshot.bin_offsets, snapshot.block_info)
        ctx.save_for_backward(x_bin, rho, mass)
        ctx.snapshot = snapshot
        ctx.needs = (x_bin.requires_grad, rho.requires_grad)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        x_bin, rho, mass = ctx.saved_tensors
        snap = ctx.snapshot
        dLdx, dLdrho = ctx.needs
        grad_x, grad_rho = torch.empty_like(x_bin), torch.empty_like(rho)
        snap.grid.moment_matrix_backward(x_bin, rho, mass, grad_output.contiguous(), grad_x, grad_rho,
                                         snap.bin_offsets, snap.block_info, dLdx, dLdrho)
        return (grad_x if dLdx else None, grad_rho if dLdrho else None, None, None)


def moment_matrix(x_bin, rho, snapshot, mass=None):
    # the parked matrix carries no autograd history: usable when none is wanted (gradient_hybrid)
    if not (torch.is_grad_enabled() and (x_bin.requires_grad or rho.requires_grad)):
        parked = _claim(snapshot, "moment_matrix", x_bin, rho, mass)
        if parked is not None:
            return parked
    return MomentMatrix.apply(x_bin, rho, _default_mass(x_bin, mass), snapshot)


@torch.no_grad()
def safe_inv_sym_mat(M, rtol=1e-6):
    M_inv = torch.empty_like(M)
    sph_cuda.safe_inv_sym_mat(M, M_inv, rtol)
    return M_inv


def gradient_hybrid(x_bin, rho, s_bin, snapshot, mass=None):
    """Moment-corrected gradient: value ``raw @ inv(M)``, gradient of the raw SPH gradient."""
    with torch.no_grad():
        M = moment_matrix(x_bin, rho, snapshot, mass=mass)
        if snapshot.dim in (2, 3):
            L = safe_inv_sym_mat(M, rtol=1e-3)
        else:
            L = torch.linalg.pinv(M, hermitian=True, rtol=1e-3)
    raw = gradient(x_bin, rho, s_bin, snapshot, mass=mass)
    return raw + (raw @ L - raw).detach()


# ---------------------------------------------------------------------------------------------
# Fused perception step (extension; the reference issues one launch per operator).
# ---------------------------------------------------------------------------------------------
class Perception(torch.autograd.Function):
    """rho = density(x); blur(x, rho, s); gradient(x, rho, s); density_gradient(x) as one node.

    Forward runs two sweeps over the neighbour cells instead of four launches; backward runs the
    chained two-sweep backward, or the features-only variant when ``x_bin`` needs no gradient.
    """

    @staticmethod
    def forward(ctx, x_bin, s_bin, mass, snapshot, want_density_gradient):
        B, N, C = s_bin.shape
        dev, dim = x_bin.device, snapshot.dim
        rho = torch.empty(B, N, dtype=torch.float32, device=dev)
        s_blur = torch.empty_like(s_bin)
        s_grad = torch.empty(B, N, C, dim, dtype=torch.float32, device=dev)
        rho_grad = torch.empty(B, N, dim, dtype=torch.float32, device=dev) if want_density_gradient else None
        pairs = _new_pair_cache(s_bin, x_bin.requires_grad or s_bin.requires_grad)
        snapshot.grid.perception_forward(x_bin, mass, s_bin, rho, None, rho_grad, s_blur, s_grad, None,
                                         snapshot.bin_offsets, snapshot.block_info, pair_cache=pairs)
        ctx.pairs = pairs
        ctx.save_for_backward(x_bin, s_bin, rho, *([] if mass is None else [mass]))
        ctx.has_mass = mass is not None
        ctx.snapshot = snapshot
        ctx.needs = (x_bin.requires_grad, s_bin.requires_grad)
        ctx.want_dg = want_density_gradient
        if want_density_gradient:
            return rho, s_blur, s_grad, rho_grad
        return rho, s_blur, s_grad

    @staticmethod
    def backward(ctx, g_rho, g_blur, g_grad, g_rho_grad=None):
        saved = ctx.saved_tensors
        x_bin, s_bin, rho = saved[:3]
        mass = saved[3] if ctx.has_mass else None
        dLdx, dLds = ctx.needs
        snap = ctx.snapshot
        cont = lambda t: None if t is None else t.contiguous()
        grad_x = torch.empty_like(x_bin) if dLdx else None
        grad_s = torch.empty_like(s_bin) if dLds else None
        scratch = torch.empty_like(rho) if dLdx else None
        if dLdx or dLds:
            snap.grid.perception_backward(x_bin, mass, s_bin, rho, cont(g_rho) if dLdx else None, cont(g_blur),
                                          cont(g_grad), cont(g_rho_grad) if dLdx else None, grad_x, grad_s,
                                          scratch, snap.bin_offsets, snap.block_info, pair_cache=ctx.pairs)
        return grad_x, grad_s, None, None, None


def perceive(x_bin, s_bin, snapshot, mass=None, with_density_gradient=True):
    """Fused ``(rho, blur, gradient[, density_gradient])`` of binned particles.

    Equivalent to ``rho = density(x_bin, snapshot, mass)``, ``blur(x_bin, rho, s_bin, ...)``,
    ``gradient(x_bin, rho, s_bin, ...)`` and ``density_gradient(x_bin, ...)`` with gradients
    flowing through ``rho`` into ``x_bin``.
    """
    if mass is not None:
        mass = _default_mass(x_bin, mass)
    return Perception.apply(x_bin, s_bin, mass, snapshot, with_density_gradient)


class PerceiveFeatures(torch.autograd.Function):
    """The packed perception row of NPA.perceive (models/npa.py:87-137) as one autograd node."""

    @staticmethod
    def forward(ctx, x_bin, s_bin, mass, snapshot, coef, dg_scale, inv_tol, log_norm_grad, log_norm_dg):
        B, N, C = s_bin.shape
        dev, D = x_bin.device, snapshot.dim
        f32 = dict(dtype=torch.float32, device=dev)
        rho = torch.empty(B, N, **f32)
        rho_grad = torch.empty(B, N, D, **f32)
        z = torch.empty(B, N, 2 * C + C * D + D, **f32)
        keep = x_bin.requires_grad or s_bin.requires_grad
        vgrad = torch.empty(B, N, C, D, **f32) if keep else None
        pairs = _new_pair_cache(s_bin, keep)
        snapshot.grid.perceive_features_forward(x_bin, mass, s_bin, coef, dg_scale, inv_tol, log_norm_grad,
                                                log_norm_dg, rho, rho_grad, z, vgrad, snapshot.bin_offsets,
                                                snapshot.block_info, pair_cache=pairs)
        ctx.pairs = pairs
        if keep:
            ctx.save_for_backward(x_bin, s_bin, rho, rho_grad, vgrad, *([] if mass is None else [mass]))
        ctx.has_mass = mass is not None
        ctx.snapshot = snapshot
        ctx.consts = (coef, dg_scale, log_norm_grad, log_norm_dg)
        ctx.needs = (x_bin.requires_grad, s_bin.requires_grad)
        return z

    @staticmethod
    def backward(ctx, g_z):
        dLdx, dLds = ctx.needs
        if not (dLdx or dLds):
            return (None,) * 9
        saved = ctx.saved_tensors
        x_bin, s_bin, rho, rho_grad, vgrad = saved[:5]
        mass = saved[5] if ctx.has_mass else None
        coef, dg_scale, ln_g, ln_dg = ctx.consts
        snap = ctx.snapshot
        g_blur = torch.empty_like(s_bin)
        g_grad = torch.empty_like(vgrad)
        grad_x = torch.empty_like(x_bin) if dLdx else None
        grad_s = torch.empty_like(s_bin)
        g_rho_grad = torch.empty_like(rho_grad) if dLdx else None
        grad_rho = torch.empty_like(rho) if dLdx else None
        snap.grid.perceive_features_backward(x_bin, mass, s_bin, rho, rho_grad, vgrad, g_z.contiguous(), coef,
                                             dg_scale, ln_g, ln_dg, g_blur, g_grad, g_rho_grad, grad_rho, grad_x,
                                             grad_s, snap.bin_offsets, snap.block_info, pair_cache=ctx.pairs)
        return (grad_x, grad_s if dLds else None) + (None,) * 7


def perceive_features(x_bin, s_bin, snapshot, eps0, mass=None, log_norm_grad=True, log_norm_density_grad=True,
                      inv_rtol=1e-3):
    """The perception vector ``z [B, N, 2C + C*dim + dim]`` an NPA model feeds its MLP, in two sweeps.

    Same value and gradients as the body of ``NPA.perceive`` with its defaults (state and density
    gradients on): ``[s | blur(s) | LN(coef * gradient_hybrid(s)) | LN(coef^(1+dim)/N * density_gradient)]``
    with ``coef = eps / eps0`` and ``LN(w) = log(1+|w|) w/|w|`` (skipped when the flag is False).
    Pass ``x_bin.detach()`` to stop gradients into the positions, as NPA does by default.
    """
    if mass is not None:
        mass = _default_mass(x_bin, mass)
    B, N, C = s_bin.shape
    coef = float(snapshot.grid.eps) / float(eps0)
    dg_scale = coef ** (1 + snapshot.dim) / N
    if not ((C % 4 == 0 and C <= 128) or C <= 32):
        # wider feature rows than one warp pass covers: same result from the separate operators
        def _ln(v):
            return torch.log(1.0 + v.norm(dim=-1, keepdim=True)) * torch.nn.functional.normalize(v, dim=-1)
        rho = density(x_bin, snapshot, mass)
        s_blur = blur(x_bin, rho, s_bin, snapshot, mass)
        with torch.no_grad():
            L = safe_inv_sym_mat(moment_matrix(x_bin, rho, snapshot, mass), rtol=inv_rtol)
        raw = gradient(x_bin, rho, s_bin, snapshot, mass)
        g = (raw + (raw @ L - raw).detach()) * coef
        dg = density_gradient(x_bin, snapshot, mass) * dg_scale
        if log_norm_grad:
            g = _ln(g)
        if log_norm_density_grad:
            dg = _ln(dg)
        return torch.cat([s_bin, s_blur, g.reshape(B, N, -1), dg], dim=-1)
    return PerceiveFeatures.apply(x_bin, s_bin, mass, snapshot, coef, dg_scale, float(inv_rtol),
                                  bool(log_norm_grad), bool(log_norm_density_grad))


class StepUpdate(torch.autograd.Function):
    """The Euler update of step_euler (models/npa.py:183-203) with the displacement limiter of
    NPA.forward (models/npa.py:145-153) as one elementwise kernel and one autograd node."""

    @staticmethod
    def forward(ctx, y, x_bin, s_bin, mask, snapshot, alpha, dt, wrap):
        x_out, s_out = torch.empty_like(x_bin), torch.empty_like(s_bin)
        snapshot.grid.step_update_forward(y, x_bin, s_bin, mask, alpha, dt, wrap, x_out, s_out)
        ctx.save_for_backward(y, *([] if mask is None else [mask]))
        ctx.has_mask = mask is not None
        ctx.snapshot = snapshot
        ctx.consts = (s_bin.shape[2], alpha, dt)
        ctx.needs = (y.requires_grad, x_bin.requires_grad, s_bin.requires_grad)
        return x_out, s_out

    @staticmethod
    def backward(ctx, g_x, g_s):
        y = ctx.saved_tensors[0]
        mask = ctx.saved_tensors[1] if ctx.has_mask else None
        need_y, need_x, need_s = ctx.needs
        C, alpha, dt = ctx.consts
        g_x = g_x.contiguous() if g_x is not None else None
        g_s = g_s.contiguous() if g_s is not None else None
        g_y = None
        if need_y:
            g_y = torch.empty_like(y)
            ctx.snapshot.grid.step_update_backward(y, mask, C, alpha, dt, g_x, g_s, g_y)
        return g_y, (g_x if need_x else None), (g_s if need_s else None), None, None, None, None, None


def step_update(y, x_bin, s_bin, snapshot, alpha, dt=1.0, update_mask=None, wrap=False):
    """``(x, s)`` after one Euler step, from the MLP output ``y [B, N, dim + C]`` in cell order.

    ``dx = alpha * y[..., :dim] * eps / (1 + |y[..., :dim]|)``, ``x = x_bin + dt * dx * mask`` (the 3D
    padding column is carried over), ``s = s_bin + dt * y[..., dim:] * mask``; ``update_mask`` is the
    reference's ``(rand(B, N, 1) < update_prob).float()`` (or None); ``wrap=True`` also applies
    ``HashGrid.wrap_positions`` on a periodic grid (keeping the padding column).
    """
    if update_mask is not None:
        update_mask = update_mask.reshape(y.shape[0], y.shape[1]).to(torch.float32).contiguous()
    return StepUpdate.apply(y.contiguous(), x_bin.contiguous(), s_bin.contiguous(), update_mask, snapshot,
                            float(alpha), float(dt), bool(wrap))
