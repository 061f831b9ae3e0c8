"""Drop-in for the reference's native module ``sph_cuda``.

Exposes the same eight grid classes, the same fourteen methods with the same
argument order, and ``safe_inv_sym_mat`` (reference: sphops/sph_cuda.cu:3229-3441),
implemented over the C ABI of ``libnpa_b200.so``.  Outputs are caller-allocated
tensors written in place and nothing is returned, exactly like the nanobind
module, so the reference's own ``sphops/sph.py`` can run on top of this file
unchanged.

Argument checking follows nanobind's and the reference's behaviour: a tensor of
the wrong dtype, on the wrong device or non-contiguous is a ``TypeError``; a
wrong shape is a ``RuntimeError`` with the reference's wording
(sphops/utils.cuh:526-567).

Differences, all on purpose:
* kernels run on torch's current stream, not the legacy default stream;
* device scratch is a torch tensor owned by the grid object, and nothing a
  snapshot needs later lives in it, so snapshots of earlier steps stay valid
  while the same grid is re-instantiated (the reference reads its work-item
  count from per-grid scratch that the next ``initialize`` overwrites);
* ``max_blocks`` uses the block-per-cell formula in every mode, because the
  work list drives all kernels here.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as N

_lib = N.lib


def _shape_str(shape) -> str:
    return "(" + ", ".join(str(int(v)) for v in shape) + ")"


def _check(t, shape, name, dtype=torch.float32):
    """nanobind-style type check followed by the reference's shape check."""
    if not isinstance(t, torch.Tensor) or t.dtype != dtype or not t.is_cuda or not t.is_contiguous():
        what = type(t).__name__ if not isinstance(t, torch.Tensor) else (
            f"tensor(dtype={t.dtype}, device={t.device}, contiguous={t.is_contiguous()})")
        raise TypeError(
            f"{name}: incompatible function arguments; expected a contiguous CUDA tensor of dtype {dtype}, got {what}")
    if t.dim() != len(shape):
        raise RuntimeError(f"{name} must have {len(shape)} dimensions, got {t.dim()}")
    if tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name} must have shape {_shape_str(shape)}, got {_shape_str(t.shape)}")
    return t


class _HashGridBase:
    """One grid = geometry + lazily allocated device scratch for binning."""

    _dim = 2
    _boundary = "periodic"
    _mode = "grid"

    def __init__(self, *args):
        dim = self._dim
        if len(args) not in (dim + 3, dim + 4):
            raise TypeError(
                f"{type(self).__name__}(): incompatible function arguments; expected "
                f"({', '.join('grid_size_' + 'xyz'[d] for d in range(dim))}, eps, particle_count, batch_size"
                f"[, max_particles_per_block])")
        sizes = [int(a) for a in args[:dim]]
        eps = float(args[dim])
        particle_count, batch_size = int(args[dim + 1]), int(args[dim + 2])
        mpb = int(args[dim + 3]) if len(args) == dim + 4 else 64
        self._sizes = sizes
        self._desc = N.make_grid(dim, self._boundary, self._mode, sizes, eps, batch_size, particle_count, mpb)
        ref = ctypes.byref(self._desc)
        cells = _lib.npa_grid_num_cells(ref)
        if cells < 0:
            N.check(int(cells))
        self._cells = int(cells)
        self._max_blocks = int(_lib.npa_grid_max_blocks(ref))
        self._scratch_bytes = int(_lib.npa_grid_scratch_bytes(ref))
        self._scratch = None
        self._B, self._N, self._P = batch_size, particle_count, (2 if dim == 2 else 4)
        self._eps = eps
        self._mpb = mpb

    # ---- read-only properties of the nanobind classes ----------------------
    grid_size_x = property(lambda self: self._sizes[0])
    grid_size_y = property(lambda self: self._sizes[1])
    eps = property(lambda self: self._eps)
    particle_count = property(lambda self: self._N)
    batch_size = property(lambda self: self._B)
    max_blocks = property(lambda self: self._max_blocks)
    max_particles_per_block = property(lambda self: self._mpb)
    cell_count = property(lambda self: self._cells)

    # ---- helpers -------------------------------------------------------------
    def _ref(self):
        return ctypes.byref(self._desc)

    def _pos(self, t, name):
        return _check(t, (self._B, self._N, self._P), name)

    def _bn(self, t, name, *tail):
        return _check(t, (self._B, self._N, *tail), name)

    def _snap(self, bin_offsets, block_info):
        _check(bin_offsets, (self._B * self._cells + 1,), "bin_offsets", torch.int32)
        _check(block_info, (self._max_blocks, 4), "block_info", torch.int32)

    def _scratch_on(self, device):
        if self._scratch is None or self._scratch.device != device:
            self._scratch = torch.empty(self._scratch_bytes, dtype=torch.uint8, device=device)
        return self._scratch

    def _pairs(self, pair_cache):
        """(pointer, stride) of an optional neighbour-list cache ``[B, N, K]`` int32, 2 <= K <= 513."""
        if pair_cache is None:
            return None, 0
        K = pair_cache.shape[-1] if isinstance(pair_cache, torch.Tensor) and pair_cache.dim() == 3 else -1
        _check(pair_cache, (self._B, self._N, K), "pair_cache", torch.int32)
        if not 2 <= K <= 513:
            raise RuntimeError(f"pair_cache must have between 2 and 513 columns, got {K}")
        return N.ptr(pair_cache), K

    @staticmethod
    def _call(fn, tensor_for_device, *args):
        with torch.cuda.device(tensor_for_device.device):
            N.check(fn(*args, N.current_stream()))

    # ---- binning ---------------------------------------------------------------
    def initialize(self, positions, permutation, bin_offsets, block_info):
        self._pos(positions, "positions")
        _check(bin_offsets, (self._B * self._cells + 1,), "bin_offsets", torch.int32)
        _check(permutation, (self._B, self._N), "permutation", torch.int32)
        _check(block_info, (self._max_blocks, 4), "block_info", torch.int32)
        scratch = self._scratch_on(positions.device)
        self._call(_lib.npa_grid_build, positions, self._ref(), N.ptr(positions), N.ptr(permutation),
                   N.ptr(bin_offsets), N.ptr(block_info), N.ptr(scratch), self._scratch_bytes)

    def initialize_static(self, positions, permutation, bin_offsets, block_info):
        """``initialize`` without any scratch tensor: the work arrays are a fixed array inside the
        library (``npa_grid_build_static``).  For hosts that manage all device memory themselves and
        do not let this package allocate; raises ``RuntimeError`` when the grid needs more than the
        built-in array holds.  Calls on one device share that array, so keep them on one stream."""
        self._pos(positions, "positions")
        _check(bin_offsets, (self._B * self._cells + 1,), "bin_offsets", torch.int32)
        _check(permutation, (self._B, self._N), "permutation", torch.int32)
        _check(block_info, (self._max_blocks, 4), "block_info", torch.int32)
        self._call(_lib.npa_grid_build_static, positions, self._ref(), N.ptr(positions), N.ptr(permutation),
                   N.ptr(bin_offsets), N.ptr(block_info))

    def _permute(self, fn, xin, sin, min_, permutation, xout, sout, mout, names):
        C = sin.shape[2] if isinstance(sin, torch.Tensor) and sin.dim() == 3 else -1
        self._pos(xin, names[0])
        self._bn(sin, names[1], C)
        _check(permutation, (self._B, self._N), "permutation", torch.int32)
        self._pos(xout, names[3])
        self._bn(sout, names[4], C)
        if min_ is not None or mout is not None:  # extension: mass may be left out altogether
            self._bn(min_, names[2])
            self._bn(mout, names[5])
        if C == 0:
            sin = sout = None
        self._call(fn, xin, self._ref(), C, N.ptr(xin), N.ptr(sin), N.ptr(min_), N.ptr(permutation),
                   N.ptr(xout), N.ptr(sout), N.ptr(mout))

    def bin_particles(self, input_positions, input_state, input_mass, permutation,
                      output_positions, output_state, output_mass):
        self._permute(_lib.npa_bin_particles, input_positions, input_state, input_mass, permutation,
                      output_positions, output_state, output_mass,
                      ("input_positions", "input_state", "input_mass",
                       "output_positions", "output_state", "output_mass"))

    def backward_bin_particles(self, grad_output_positions, grad_output_state, grad_output_mass, permutation,
                               grad_input_positions, grad_input_state, grad_input_mass):
        self._permute(_lib.npa_unbin_particles, grad_output_positions, grad_output_state, grad_output_mass,
                      permutation, grad_input_positions, grad_input_state, grad_input_mass,
                      ("grad_output_positions", "grad_output_state", "grad_output_mass",
                       "grad_input_positions", "grad_input_state", "grad_input_mass"))

    # ---- forward operators -----------------------------------------------------
    def count_forward(self, binned_positions, count, bin_offsets, block_info):
        self._pos(binned_positions, "binned_positions")
        self._bn(count, "count")
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_count_forward, binned_positions, self._ref(), N.ptr(binned_positions), N.ptr(count),
                   N.ptr(bin_offsets), N.ptr(block_info))

    def density_forward(self, binned_positions, mass, rho, bin_offsets, block_info):
        self._pos(binned_positions, "binned_positions")
        self._bn(mass, "mass")
        self._bn(rho, "rho")
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_density_forward, binned_positions, self._ref(), N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(rho), N.ptr(bin_offsets), N.ptr(block_info))

    def blur_forward(self, binned_positions, rho, mass, state_in, state_out, bin_offsets, block_info):
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(mass, "mass")
        self._bn(state_in, "state_in", C)
        self._bn(state_out, "state_out", C)
        self._snap(bin_offsets, block_info)
        if C == 0:
            return
        self._call(_lib.npa_blur_forward, binned_positions, self._ref(), C, N.ptr(binned_positions), N.ptr(rho),
                   N.ptr(mass), N.ptr(state_in), N.ptr(state_out), N.ptr(bin_offsets), N.ptr(block_info))

    def gradient_forward(self, binned_positions, rho, mass, state_in, state_gradient_out, bin_offsets, block_info):
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(mass, "mass")
        self._bn(state_in, "state_in", C)
        self._bn(state_gradient_out, "state_gradient_out", C, self._dim)
        self._snap(bin_offsets, block_info)
        if C == 0:
            return
        self._call(_lib.npa_gradient_forward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(rho), N.ptr(mass), N.ptr(state_in), N.ptr(state_gradient_out), N.ptr(bin_offsets),
                   N.ptr(block_info))

    def density_gradient_forward(self, binned_positions, mass, density_gradient_out, bin_offsets, block_info):
        self._pos(binned_positions, "binned_positions")
        self._bn(mass, "mass")
        self._bn(density_gradient_out, "density_gradient_out", self._dim)
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_density_gradient_forward, binned_positions, self._ref(), N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(density_gradient_out), N.ptr(bin_offsets), N.ptr(block_info))

    def moment_matrix_forward(self, binned_positions, rho, mass, moment_matrix_out, bin_offsets, block_info):
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(mass, "mass")
        self._bn(moment_matrix_out, "moment_matrix_out", self._dim, self._dim)
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_moment_matrix_forward, binned_positions, self._ref(), N.ptr(binned_positions),
                   N.ptr(rho), N.ptr(mass), N.ptr(moment_matrix_out), N.ptr(bin_offsets), N.ptr(block_info))

    # ---- backward operators ----------------------------------------------------
    def density_backward(self, binned_positions, mass, dL_rho_out, grad_x, bin_offsets, block_info, dLdx=True):
        self._pos(binned_positions, "binned_positions")
        self._bn(mass, "mass")
        self._bn(dL_rho_out, "dL_rho_out")
        self._pos(grad_x, "grad_x")
        self._snap(bin_offsets, block_info)
        if not dLdx:
            return
        self._call(_lib.npa_density_backward, binned_positions, self._ref(), N.ptr(binned_positions), N.ptr(mass),
                   N.ptr(dL_rho_out), N.ptr(grad_x), N.ptr(bin_offsets), N.ptr(block_info))

    def _feature_backward(self, fn, up_name, binned_positions, rho, mass, state_in, upstream, grad_x, grad_s,
                          grad_rho, bin_offsets, block_info, dLdx, dLds, dLdrho, up_tail):
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(mass, "mass")
        self._bn(state_in, "state_in", C)
        self._bn(upstream, up_name, C, *up_tail)
        self._pos(grad_x, "grad_x")
        self._bn(grad_s, "grad_s", C)
        self._bn(grad_rho, "grad_rho")
        self._snap(bin_offsets, block_info)
        if C == 0 or not (dLdx or dLds or dLdrho):
            return
        self._call(fn, binned_positions, self._ref(), C, N.ptr(binned_positions), N.ptr(rho), N.ptr(mass),
                   N.ptr(state_in), N.ptr(upstream), N.ptr(grad_x if dLdx else None),
                   N.ptr(grad_s if dLds else None), N.ptr(grad_rho if dLdrho else None),
                   N.ptr(bin_offsets), N.ptr(block_info))

    def blur_backward(self, binned_positions, rho, mass, state_in, dL_blur_state_out, grad_x, grad_s, grad_rho,
                      bin_offsets, block_info, dLdx=True, dLds=True, dLdrho=True):
        self._feature_backward(_lib.npa_blur_backward, "dL_blur_state_out", binned_positions, rho, mass, state_in,
                               dL_blur_state_out, grad_x, grad_s, grad_rho, bin_offsets, block_info,
                               dLdx, dLds, dLdrho, ())

    def gradient_backward(self, binned_positions, rho, mass, state_in, dL_grad_state_out, grad_x, grad_s, grad_rho,
                          bin_offsets, block_info, dLdx=True, dLds=True, dLdrho=True):
        self._feature_backward(_lib.npa_gradient_backward, "dL_grad_state_out", binned_positions, rho, mass,
                               state_in, dL_grad_state_out, grad_x, grad_s, grad_rho, bin_offsets, block_info,
                               dLdx, dLds, dLdrho, (self._dim,))

    def density_gradient_backward(self, binned_positions, mass, dL_density_gradient_out, grad_x, bin_offsets,
                                  block_info, dLdx=True):
        self._pos(binned_positions, "binned_positions")
        self._bn(mass, "mass")
        self._bn(dL_density_gradient_out, "dL_density_gradient_out", self._dim)
        self._pos(grad_x, "grad_x")
        self._snap(bin_offsets, block_info)
        if not dLdx:
            return
        self._call(_lib.npa_density_gradient_backward, binned_positions, self._ref(), N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(dL_density_gradient_out), N.ptr(grad_x), N.ptr(bin_offsets),
                   N.ptr(block_info))

    def moment_matrix_backward(self, binned_positions, rho, mass, dL_moment_matrix_out, grad_x, grad_rho,
                               bin_offsets, block_info, dLdx=True, dLdrho=True):
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(mass, "mass")
        self._bn(dL_moment_matrix_out, "dL_moment_matrix_out", self._dim, self._dim)
        self._pos(grad_x, "grad_x")
        self._bn(grad_rho, "grad_rho")
        self._snap(bin_offsets, block_info)
        if not (dLdx or dLdrho):
            return
        self._call(_lib.npa_moment_matrix_backward, binned_positions, self._ref(), N.ptr(binned_positions),
                   N.ptr(rho), N.ptr(mass), N.ptr(dL_moment_matrix_out), N.ptr(grad_x if dLdx else None),
                   N.ptr(grad_rho if dLdrho else None), N.ptr(bin_offsets), N.ptr(block_info))

    # ---- fused sweeps (no counterpart in the reference module) ------------------
    def blur_gradient_forward(self, binned_positions, rho, mass, state_in, state_out, state_gradient_out,
                              bin_offsets, block_info, moment_matrix_out=None, pair_cache=None, pair_cache_valid=False):
        """blur and gradient in one launch; ``mass`` and either output may be None.  With
        ``moment_matrix_out`` (and both other outputs) the moment matrix rides the same sweep."""
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(state_in, "state_in", C)
        if mass is not None:
            self._bn(mass, "mass")
        if state_out is not None:
            self._bn(state_out, "state_out", C)
        if state_gradient_out is not None:
            self._bn(state_gradient_out, "state_gradient_out", C, self._dim)
        self._snap(bin_offsets, block_info)
        if moment_matrix_out is not None:
            self._bn(moment_matrix_out, "moment_matrix_out", self._dim, self._dim)
        if C == 0:
            return
        self._call(_lib.npa_blur_gradient_forward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(rho), N.ptr(mass), N.ptr(state_in), N.ptr(state_out), N.ptr(state_gradient_out),
                   N.ptr(moment_matrix_out), N.ptr(bin_offsets), N.ptr(block_info), *self._pairs(pair_cache),
                   1 if pair_cache_valid else 0)

    def blur_gradient_backward(self, binned_positions, rho, mass, state_in, dL_blur_state_out, dL_grad_state_out,
                               grad_x, grad_s, grad_rho, bin_offsets, block_info, pair_cache=None):
        """Backward of both feature operators in one launch; None outputs are not computed."""
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._bn(state_in, "state_in", C)
        if mass is not None:
            self._bn(mass, "mass")
        if dL_blur_state_out is not None:
            self._bn(dL_blur_state_out, "dL_blur_state_out", C)
        if dL_grad_state_out is not None:
            self._bn(dL_grad_state_out, "dL_grad_state_out", C, self._dim)
        if grad_x is not None:
            self._pos(grad_x, "grad_x")
        if grad_s is not None:
            self._bn(grad_s, "grad_s", C)
        if grad_rho is not None:
            self._bn(grad_rho, "grad_rho")
        self._snap(bin_offsets, block_info)
        if C == 0:
            return
        self._call(_lib.npa_blur_gradient_backward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(rho), N.ptr(mass), N.ptr(state_in), N.ptr(dL_blur_state_out), N.ptr(dL_grad_state_out),
                   N.ptr(grad_x), N.ptr(grad_s), N.ptr(grad_rho), N.ptr(bin_offsets), N.ptr(block_info),
                   *self._pairs(pair_cache))

    def density_chain_backward(self, binned_positions, mass, dL_rho_a, dL_rho_b, dL_density_gradient_out, grad_x,
                               accumulate, bin_offsets, block_info, pair_cache=None):
        """density (+ density gradient) backward; the two rho upstreams are summed."""
        self._pos(binned_positions, "binned_positions")
        if mass is not None:
            self._bn(mass, "mass")
        if dL_rho_a is not None:
            self._bn(dL_rho_a, "dL_rho_a")
        if dL_rho_b is not None:
            self._bn(dL_rho_b, "dL_rho_b")
        if dL_density_gradient_out is not None:
            self._bn(dL_density_gradient_out, "dL_density_gradient_out", self._dim)
        self._pos(grad_x, "grad_x")
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_density_chain_backward, binned_positions, self._ref(), N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(dL_rho_a), N.ptr(dL_rho_b), N.ptr(dL_density_gradient_out), N.ptr(grad_x),
                   1 if accumulate else 0, N.ptr(bin_offsets), N.ptr(block_info), *self._pairs(pair_cache))

    # ---- packed perception (no counterpart in the reference module) ------------
    def perceive_features_forward(self, binned_positions, mass, state_in, coef, dg_scale, inv_tol, log_norm_grad,
                                  log_norm_dg, rho, density_gradient_out, z, corrected_gradient_out, bin_offsets,
                                  block_info, pair_cache=None):
        """Two sweeps that write the packed perception row z; ``mass`` and ``corrected_gradient_out`` may be None."""
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        D = self._dim
        self._pos(binned_positions, "binned_positions")
        self._bn(state_in, "state_in", C)
        if mass is not None:
            self._bn(mass, "mass")
        self._bn(rho, "rho")
        self._bn(density_gradient_out, "density_gradient_out", D)
        self._bn(z, "z", 2 * C + C * D + D)
        if corrected_gradient_out is not None:
            self._bn(corrected_gradient_out, "corrected_gradient_out", C, D)
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_perceive_features_forward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(state_in), float(coef), float(dg_scale), float(inv_tol),
                   1 if log_norm_grad else 0, 1 if log_norm_dg else 0, N.ptr(rho), N.ptr(density_gradient_out),
                   N.ptr(z), N.ptr(corrected_gradient_out), N.ptr(bin_offsets), N.ptr(block_info),
                   *self._pairs(pair_cache))

    def perceive_features_backward(self, binned_positions, mass, state_in, rho, density_gradient, corrected_gradient,
                                   dL_dz, coef, dg_scale, log_norm_grad, log_norm_dg, g_blur_scratch, g_grad_scratch,
                                   g_rho_grad_scratch, grad_rho_scratch, grad_x, grad_s, bin_offsets, block_info, pair_cache=None):
        """Backward of ``perceive_features_forward``; ``grad_x`` (and its two scratch tensors) may be None."""
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        D = self._dim
        self._pos(binned_positions, "binned_positions")
        self._bn(state_in, "state_in", C)
        if mass is not None:
            self._bn(mass, "mass")
        self._bn(rho, "rho")
        self._bn(density_gradient, "density_gradient", D)
        self._bn(corrected_gradient, "corrected_gradient", C, D)
        self._bn(dL_dz, "dL_dz", 2 * C + C * D + D)
        self._bn(g_blur_scratch, "g_blur_scratch", C)
        self._bn(g_grad_scratch, "g_grad_scratch", C, D)
        if grad_x is not None:
            self._pos(grad_x, "grad_x")
            self._bn(g_rho_grad_scratch, "g_rho_grad_scratch", D)
            self._bn(grad_rho_scratch, "grad_rho_scratch")
        if grad_s is not None:
            self._bn(grad_s, "grad_s", C)
        self._snap(bin_offsets, block_info)
        self._call(_lib.npa_perceive_features_backward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(state_in), N.ptr(rho), N.ptr(density_gradient), N.ptr(corrected_gradient),
                   N.ptr(dL_dz), float(coef), float(dg_scale), 1 if log_norm_grad else 0, 1 if log_norm_dg else 0,
                   N.ptr(g_blur_scratch), N.ptr(g_grad_scratch), N.ptr(g_rho_grad_scratch), N.ptr(grad_rho_scratch),
                   N.ptr(grad_x), N.ptr(grad_s), N.ptr(bin_offsets), N.ptr(block_info), *self._pairs(pair_cache))

    # ---- Euler update after the MLP (no counterpart in the reference module) ----
    def step_update_forward(self, y, binned_positions, state_in, mask, alpha, dt, wrap, positions_out, state_out):
        """``x_out = x_bin + dt * limiter(y[..., :D]) * mask``, ``s_out = s_bin + dt * y[..., D:] * mask``
        (models/npa.py:145-153, 183-203); ``mask`` [B,N] of 0/1 or None."""
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._pos(binned_positions, "binned_positions")
        self._pos(positions_out, "positions_out")
        self._bn(state_in, "state_in", C)
        self._bn(state_out, "state_out", C)
        self._bn(y, "y", self._dim + C)
        if mask is not None:
            self._bn(mask, "mask")
        self._call(_lib.npa_step_update_forward, y, self._ref(), N.ptr(y), N.ptr(binned_positions), N.ptr(state_in),
                   N.ptr(mask), C, float(alpha), float(dt), 1 if wrap else 0, N.ptr(positions_out), N.ptr(state_out))

    def step_update_backward(self, y, mask, channels, alpha, dt, g_positions_out, g_state_out, g_y):
        """``dL/dy`` of ``step_update_forward``; either upstream gradient may be None (= zero)."""
        C = int(channels)
        self._bn(y, "y", self._dim + C)
        self._bn(g_y, "g_y", self._dim + C)
        if mask is not None:
            self._bn(mask, "mask")
        if g_positions_out is not None:
            self._pos(g_positions_out, "g_positions_out")
        if g_state_out is not None:
            self._bn(g_state_out, "g_state_out", C)
        self._call(_lib.npa_step_update_backward, y, self._ref(), N.ptr(y), N.ptr(mask), C, float(alpha), float(dt),
                   N.ptr(g_positions_out), N.ptr(g_state_out), N.ptr(g_y))

    # ---- fused perception (no counterpart in the reference module) -------------
    def perception_forward(self, binned_positions, mass, state_in, rho, count, density_gradient_out,
                           state_out, state_gradient_out, moment_matrix_out, bin_offsets, block_info, pair_cache=None):
        """rho is required; every other output and ``mass`` may be None."""
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._snap(bin_offsets, block_info)
        C = 0
        if state_out is not None or state_gradient_out is not None:
            C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
            self._bn(state_in, "state_in", C)
        if mass is not None:
            self._bn(mass, "mass")
        if count is not None:
            self._bn(count, "count")
        if density_gradient_out is not None:
            self._bn(density_gradient_out, "density_gradient_out", self._dim)
        if state_out is not None:
            self._bn(state_out, "state_out", C)
        if state_gradient_out is not None:
            self._bn(state_gradient_out, "state_gradient_out", C, self._dim)
        if moment_matrix_out is not None:
            self._bn(moment_matrix_out, "moment_matrix_out", self._dim, self._dim)
        self._call(_lib.npa_perception_forward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(state_in if C else None), N.ptr(rho), N.ptr(count),
                   N.ptr(density_gradient_out), N.ptr(state_out), N.ptr(state_gradient_out),
                   N.ptr(moment_matrix_out), N.ptr(bin_offsets), N.ptr(block_info), *self._pairs(pair_cache))

    def perception_backward(self, binned_positions, mass, state_in, rho, dL_rho_out, dL_blur_state_out,
                            dL_grad_state_out, dL_density_gradient_out, grad_x, grad_s, grad_rho_scratch,
                            bin_offsets, block_info, pair_cache=None):
        """Chained backward; upstreams, ``mass``, ``grad_x`` and ``grad_s`` may be None."""
        self._pos(binned_positions, "binned_positions")
        self._bn(rho, "rho")
        self._snap(bin_offsets, block_info)
        C = state_in.shape[2] if isinstance(state_in, torch.Tensor) and state_in.dim() == 3 else -1
        self._bn(state_in, "state_in", C)
        if mass is not None:
            self._bn(mass, "mass")
        if dL_rho_out is not None:
            self._bn(dL_rho_out, "dL_rho_out")
        if dL_blur_state_out is not None:
            self._bn(dL_blur_state_out, "dL_blur_state_out", C)
        if dL_grad_state_out is not None:
            self._bn(dL_grad_state_out, "dL_grad_state_out", C, self._dim)
        if dL_density_gradient_out is not None:
            self._bn(dL_density_gradient_out, "dL_density_gradient_out", self._dim)
        if grad_x is not None:
            self._pos(grad_x, "grad_x")
        if grad_s is not None:
            self._bn(grad_s, "grad_s", C)
        if grad_rho_scratch is not None:
            self._bn(grad_rho_scratch, "grad_rho_scratch")
        self._call(_lib.npa_perception_backward, binned_positions, self._ref(), C, N.ptr(binned_positions),
                   N.ptr(mass), N.ptr(state_in), N.ptr(rho), N.ptr(dL_rho_out), N.ptr(dL_blur_state_out),
                   N.ptr(dL_grad_state_out), N.ptr(dL_density_gradient_out), N.ptr(grad_x), N.ptr(grad_s),
                   N.ptr(grad_rho_scratch), N.ptr(bin_offsets), N.ptr(block_info), *self._pairs(pair_cache))


def _make(name, dim, boundary, mode):
    ns = {"_dim": dim, "_boundary": boundary, "_mode": mode, "__doc__": f"{dim}D {boundary} grid, {mode} hash order."}
    if dim == 3:
        ns["grid_size_z"] = property(lambda self: self._sizes[2])
    return type(name, (_HashGridBase,), ns)


HashGrid2DPeriodic = _make("HashGrid2DPeriodic", 2, "periodic", "grid")
HashGrid2DBox = _make("HashGrid2DBox", 2, "clamped", "grid")
VHashGrid2DPeriodic = _make("VHashGrid2DPeriodic", 2, "periodic", "particle")
VHashGrid2DBox = _make("VHashGrid2DBox", 2, "clamped", "particle")
HashGrid3DPeriodic = _make("HashGrid3DPeriodic", 3, "periodic", "grid")
HashGrid3DBox = _make("HashGrid3DBox", 3, "clamped", "grid")
VHashGrid3DPeriodic = _make("VHashGrid3DPeriodic", 3, "periodic", "particle")
VHashGrid3DBox = _make("VHashGrid3DBox", 3, "clamped", "particle")


def safe_inv_sym_mat(in_matrix, out_matrix, tol):
    """Inverse of ``[B, N, dim, dim]`` symmetric matrices, identity where ``|det| < tol``."""
    if not isinstance(in_matrix, torch.Tensor) or in_matrix.dim() != 4:
        raise TypeError("safe_inv_sym_mat: incompatible function arguments; expected a 4-D CUDA float tensor")
    B, n, dim = in_matrix.shape[0], in_matrix.shape[1], in_matrix.shape[2]
    if dim not in (2, 3):
        raise RuntimeError("safe_inverse only supports 2x2 or 3x3 matrices.")
    _check(in_matrix, (B, n, dim, dim), "in_matrix")
    _check(out_matrix, (B, n, dim, dim), "out_matrix")
    with torch.cuda.device(in_matrix.device):
        N.check(_lib.npa_safe_inv_sym_mat(dim, B * n, N.ptr(in_matrix), N.ptr(out_matrix), float(tol),
                                          N.current_stream()))
