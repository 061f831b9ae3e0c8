"""ctypes wrapper of the GPU comparator: the reference's own CUDA kernels (sphops/sph_cuda.cu),
compiled unmodified for sm_100 behind ``ref_driver.cu``.

``build()`` compiles ``baseline/_ref/libsph_cuda_ref.so`` from the copy of the reference under
``baseline/_ref`` (kept out of the history); ``ReferenceGrid`` mirrors the methods bench.py times.
Comparator only: nothing in ``npa_b200`` uses it.
"""
from __future__ import annotations

import ctypes
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_ROOT = HERE.parent / "_ref"
LIB_PATH = REF_ROOT / "libsph_cuda_ref.so"
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def build(force: bool = False) -> Path | None:
    """Compile the driver + the reference's translation unit (about two minutes); returns the library
    path, or None when no copy of the reference is present."""
    src = REF_ROOT / "sphops" / "sph_cuda.cu"
    if not src.exists():
        return None
    driver = HERE / "ref_driver.cu"
    newest = max(p.stat().st_mtime for p in (src, driver, HERE / "nanobind" / "nanobind.h", HERE / "nanobind" / "ndarray.h"))
    if LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= newest and not force:
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    # the reference's own flags (sphops/CMakeLists.txt:26): -O3 --use_fast_math; architecture: this GPU
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-I", str(HERE), "-I", str(src.parent), str(driver), "-o", str(LIB_PATH)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the reference kernels failed:\n{res.stderr[-4000:]}")
    return LIB_PATH


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.ref_last_error.restype = ctypes.c_char_p
        lib.ref_grid_create.restype = ctypes.c_void_p
        lib.ref_grid_create.argtypes = [ctypes.c_int] * 5 + [ctypes.c_float] + [ctypes.c_uint] * 3
        lib.ref_grid_destroy.argtypes = [ctypes.c_void_p]
        lib.ref_max_blocks.argtypes = [ctypes.c_void_p]
        P, I = ctypes.c_void_p, ctypes.c_int
        for name, args in {
            "ref_initialize": [P] * 5, "ref_bin_particles": [P] * 8 + [I], "ref_density_forward": [P] * 6,
            "ref_blur_forward": [P] * 6 + [I, P, P], "ref_gradient_forward": [P] * 6 + [I, P, P],
            "ref_density_backward": [P] * 7, "ref_blur_backward": [P] * 9 + [I, P, P],
            "ref_gradient_backward": [P] * 9 + [I, P, P],
        }.items():
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = args
        _lib = lib
    return _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


class ReferenceGrid:
    """One grid object of the reference (grid mode), driven with torch CUDA tensors.  The reference
    launches on the legacy default stream."""

    def __init__(self, dim, boundary, grid_size, eps, num_particles, batch_size, max_particles_per_block):
        self.lib = _load()
        g = list(grid_size) + [1, 1, 1]
        self.h = self.lib.ref_grid_create(dim, 1 if boundary == "periodic" else 0, g[0], g[1], g[2], float(eps),
                                          num_particles, batch_size, max_particles_per_block)
        if not self.h:
            raise RuntimeError(self.lib.ref_last_error().decode())
        self.max_blocks = self.lib.ref_max_blocks(self.h)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.ref_grid_destroy(self.h)
            self.h = None

    def _ok(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def initialize(self, x, perm, offs, info):
        self._ok(self.lib.ref_initialize(self.h, _p(x), _p(perm), _p(offs), _p(info)))

    def bin_particles(self, x, s, m, perm, xo, so, mo):
        self._ok(self.lib.ref_bin_particles(self.h, _p(x), _p(s), _p(m), _p(perm), _p(xo), _p(so), _p(mo), s.shape[-1]))

    def density_forward(self, x, m, rho, offs, info):
        self._ok(self.lib.ref_density_forward(self.h, _p(x), _p(m), _p(rho), _p(offs), _p(info)))

    def blur_forward(self, x, rho, m, s, out, offs, info):
        self._ok(self.lib.ref_blur_forward(self.h, _p(x), _p(rho), _p(m), _p(s), _p(out), s.shape[-1], _p(offs), _p(info)))

    def gradient_forward(self, x, rho, m, s, out, offs, info):
        self._ok(self.lib.ref_gradient_forward(self.h, _p(x), _p(rho), _p(m), _p(s), _p(out), s.shape[-1], _p(offs), _p(info)))

    def density_backward(self, x, m, g, gx, offs, info):
        self._ok(self.lib.ref_density_backward(self.h, _p(x), _p(m), _p(g), _p(gx), _p(offs), _p(info)))

    def blur_backward(self, x, rho, m, s, g, gx, gs, gr, offs, info):
        self._ok(self.lib.ref_blur_backward(self.h, _p(x), _p(rho), _p(m), _p(s), _p(g), _p(gx), _p(gs), _p(gr),
                                            s.shape[-1], _p(offs), _p(info)))

    def gradient_backward(self, x, rho, m, s, g, gx, gs, gr, offs, info):
        self._ok(self.lib.ref_gradient_backward(self.h, _p(x), _p(rho), _p(m), _p(s), _p(g), _p(gx), _p(gs), _p(gr),
                                                s.shape[-1], _p(offs), _p(info)))
