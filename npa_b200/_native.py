"""ctypes binding of ``libnpa_b200.so`` (the C ABI in ``include/npa_b200.h``).

This is the whole Python <-> CUDA boundary: device pointers, sizes and a stream
go down, a status code comes back.  There is no CPU fallback: if the library is
missing or fails to load, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libnpa_b200.so"

ABI_VERSION = 1

NPA_OK = 0
NPA_ERR_INVALID_ARGUMENT = -1
NPA_ERR_UNSUPPORTED = -2
NPA_ERR_CUDA = -3
NPA_ERR_SCRATCH_TOO_SMALL = -4

BOUNDARY = {"clamped": 0, "periodic": 1}
HASH = {"grid": 0, "particle": 1}


class NpaGrid(ctypes.Structure):
    """Mirror of ``struct npa_grid``."""

    _fields_ = [
        ("dim", ctypes.c_int32),
        ("boundary", ctypes.c_int32),
        ("hash", ctypes.c_int32),
        ("grid", ctypes.c_int32 * 3),
        ("eps", ctypes.c_double),
        ("batch", ctypes.c_int32),
        ("particles", ctypes.c_int32),
        ("max_particles_per_block", ctypes.c_int32),
    ]


# name -> number of arguments after the grid pointer, for symbol / arity checks
_P = ctypes.c_void_p
_I32 = ctypes.c_int32
_I64 = ctypes.c_int64
SIGNATURES = {
    "npa_last_error": (ctypes.c_char_p, []),
    "npa_abi_version": (ctypes.c_int, []),
    "npa_grid_num_cells": (_I64, [_P]),
    "npa_grid_max_blocks": (_I64, [_P]),
    "npa_grid_scratch_bytes": (_I64, [_P]),
    "npa_grid_build": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _I64, _P]),
    "npa_grid_build_static": (ctypes.c_int, [_P, _P, _P, _P, _P, _P]),
    "npa_bin_particles": (ctypes.c_int, [_P, _I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_unbin_particles": (ctypes.c_int, [_P, _I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_count_forward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P]),
    "npa_density_forward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P]),
    "npa_blur_forward": (ctypes.c_int, [_P, _I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_gradient_forward": (ctypes.c_int, [_P, _I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_density_gradient_forward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P]),
    "npa_moment_matrix_forward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_density_backward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_blur_backward": (ctypes.c_int, [_P, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_gradient_backward": (ctypes.c_int, [_P, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_density_gradient_backward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_moment_matrix_backward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "npa_safe_inv_sym_mat": (ctypes.c_int, [_I32, _I64, _P, _P, ctypes.c_float, _P]),
    "npa_blur_gradient_forward": (ctypes.c_int, [_P, _I32] + [_P] * 9 + [_P, _I32, _I32, _P]),
    "npa_blur_gradient_backward": (ctypes.c_int, [_P, _I32] + [_P] * 11 + [_P, _I32, _P]),
    "npa_density_chain_backward": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _I32, _P, _P, _P, _I32, _P]),
    "npa_perceive_features_forward": (ctypes.c_int, [_P, _I32, _P, _P, _P, ctypes.c_float, ctypes.c_float,
                                                     ctypes.c_float, _I32, _I32, _P, _P, _P, _P, _P, _P, _P, _I32, _P]),
    "npa_perceive_features_backward": (ctypes.c_int, [_P, _I32] + [_P] * 7 + [ctypes.c_float, ctypes.c_float, _I32, _I32]
                                       + [_P] * 8 + [_P, _I32, _P]),
    "npa_perception_forward": (ctypes.c_int, [_P, _I32] + [_P] * 11 + [_P, _I32, _P]),
    "npa_perception_backward": (ctypes.c_int, [_P, _I32] + [_P] * 13 + [_P, _I32, _P]),
    "npa_step_update_forward": (ctypes.c_int, [_P] * 5 + [_I32, ctypes.c_float, ctypes.c_float, _I32, _P, _P, _P]),
    "npa_splat_forward": (ctypes.c_int, [_P, _P, _I32, _I32, _I32, ctypes.c_double, _I32, ctypes.c_double,
                                         ctypes.c_double, _I32, _I32, ctypes.c_double, _P, _P, _P]),
    "npa_splat_backward": (ctypes.c_int, [_P, _P, _P, _I32, _I32, _I32, ctypes.c_double, _I32, ctypes.c_double,
                                          ctypes.c_double, _I32, _I32, ctypes.c_double, _P, _P, _P]),
    "npa_mlp_weight_grad_scratch_floats": (ctypes.c_int64, [ctypes.c_int64, _I32, _I32]),
    "npa_mlp_weight_grad": (ctypes.c_int, [_P, _P, _P, _P, ctypes.c_int64, _I32, _I32, _I32, _P, ctypes.c_int64,
                                           _P, _P, _P, _P]),
    "npa_mlp_hidden_grad": (ctypes.c_int, [_P, _P, _P, _P, ctypes.c_int64, _I32, _I32, ctypes.c_int64, ctypes.c_int64, _P]),
    "npa_mlp_weight_grad_tcgen05": (ctypes.c_int, [_P, _P, _P, _P, ctypes.c_int64, _I32, _I32, _I32, _P, ctypes.c_int64,
                                                   _P, _P, _P, _P]),
    "npa_mlp_weight_grad_tcgen05_scratch_floats": (ctypes.c_int64, [ctypes.c_int64, _I32, _I32]),
    "npa_linear_tf32x3": (ctypes.c_int, [_P, _P, _P, _P, _P, ctypes.c_int64, _I32, _I32, ctypes.c_int64, ctypes.c_int64,
                                         _I32, _P]),
    "npa_linear_tcgen05": (ctypes.c_int, [_P, _P, _P, _P, _P, ctypes.c_int64, _I32, _I32, ctypes.c_int64, ctypes.c_int64,
                                          _I32, _P, ctypes.c_int64, _P]),
    "npa_mlp_forward_tcgen05": (ctypes.c_int, [_P] * 6 + [ctypes.c_int64, _I32, _I32] + [ctypes.c_int64] * 4 + [_P, ctypes.c_int64, _P]),
    "npa_mlp_forward_tcgen05_scratch_bytes": (ctypes.c_int64, [_I32, _I32]),
    "npa_linear_tcgen05_scratch_bytes": (ctypes.c_int64, [_I32, _I32]),
    "npa_linear_tcgen05_status": (ctypes.c_int, [_P, _I32]),
    "npa_linear_tcgen05_wait_selftest": (ctypes.c_int, [_I32, _P, _P]),
    "npa_step_update_backward": (ctypes.c_int, [_P] * 3 + [_I32, ctypes.c_float, ctypes.c_float, _P, _P, _P, _P]),
    "npa_tile_tuning": (ctypes.c_int, [_I32, _I32, _I32, _I32, _I32, _I32, _I32]),
    "npa_tile_status": (ctypes.c_int, [_P, _I32]),
    "npa_scalar_sweep_tuning": (ctypes.c_int, [_I32]),
    "npa_row_tickets_status": (ctypes.c_int, [_P, _I32]),
    "npa_tile_wait_selftest": (ctypes.c_int, [_I32, _P, _P]),
}


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA kernels first (python -m npa_b200.build). "
            "npa_b200 has no CPU fallback.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    got = lib.npa_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"libnpa_b200.so has ABI version {got}, this binding expects {ABI_VERSION}")
    return lib


lib = _load()


def last_error() -> str:
    return lib.npa_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Raise the Python exception the reference would have raised for this status."""
    if rc == NPA_OK:
        return
    msg = last_error()
    if rc == NPA_ERR_UNSUPPORTED:
        raise ValueError(msg)
    raise RuntimeError(msg)


def tile_tuning(backward: bool, enabled: bool = True, rows_per_stage: int = 0, particles_per_tile: int = 0,
                stages: int = 0, consumer_warps: int = 0, cells_per_tile: int = 0) -> None:
    """Process-wide switches of the cell-tile streaming engine (``npa_tile_tuning``)."""
    check(lib.npa_tile_tuning(int(bool(backward)), int(bool(enabled)), int(rows_per_stage),
                              int(particles_per_tile), int(stages), int(consumer_warps), int(cells_per_tile)))


def tile_status(reset: bool = True) -> int:
    """Status word of the engine's bounded waits (``npa_tile_status``); synchronises the device."""
    out = ctypes.c_int32(0)
    check(lib.npa_tile_status(ctypes.byref(out), int(bool(reset))))
    return int(out.value)


def row_tickets_nonzero(reset: bool = False) -> int:
    """Number of non-zero row-ticket words (``npa_row_tickets_status``); 0 when every sweep ended cleanly."""
    out = ctypes.c_int32(0)
    check(lib.npa_row_tickets_status(ctypes.byref(out), int(bool(reset))))
    return int(out.value)


def make_grid(dim, boundary, mode, grid_size, eps, batch, particles, mpb) -> NpaGrid:
    g = NpaGrid()
    g.dim = int(dim)
    g.boundary = BOUNDARY[boundary]
    g.hash = HASH[mode]
    sizes = list(grid_size) + [1, 1, 1]
    for d in range(3):
        g.grid[d] = int(sizes[d]) if d < dim else 1
    g.eps = float(eps)
    g.batch = int(batch)
    g.particles = int(particles)
    g.max_particles_per_block = int(mpb)
    return g


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def current_stream():
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
