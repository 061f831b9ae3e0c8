"""TEST INFRASTRUCTURE -- CPU oracle for the npa_b200 kernels.

Nothing in the product (``npa_b200/``) imports this package.  It holds

* ``sph_oracle.c``: a C restatement (double accumulation, OpenMP over particles)
  of the reference's pure-torch operators ``sphops/torch_sph.py``, loaded here
  through ctypes (:func:`forward`, :func:`backward`, :func:`safe_inv_sym_mat`).
  The same file built with ``-DORACLE_FP32`` evaluates every sum in float
  (``precision="f32"``): the stand-in for the reference's own fp32 run where no
  stored fp32 output exists, used only to size the "no worse than twice the
  reference's fp32 error" clause of the parity gate;
* ``binning.py``: a numpy restatement of the reference's cell hashing and of a
  stable counting sort (:mod:`oracle.binning`).

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may use it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SRC = _DIR / "sph_oracle.c"
_LIB = _DIR / "libsph_oracle.so"
_LIB32 = _DIR / "libsph_oracle_f32.so"
_lib = None
_lib32 = None


class _Cfg(ctypes.Structure):
    _fields_ = [
        ("dim", ctypes.c_int32),
        ("pos_stride", ctypes.c_int32),
        ("periodic", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("particles", ctypes.c_int32),
        ("channels", ctypes.c_int32),
        ("h", ctypes.c_double),
        ("box", ctypes.c_double * 3),
    ]


def build(force: bool = False) -> Path:
    """Compile ``sph_oracle.c`` with gcc into ``oracle/libsph_oracle.so`` (double sums) and
    ``oracle/libsph_oracle_f32.so`` (float sums, no fused multiply-adds)."""
    for lib, extra in ((_LIB, []), (_LIB32, ["-DORACLE_FP32", "-ffp-contract=off"])):
        if force or not lib.exists() or lib.stat().st_mtime < _SRC.stat().st_mtime:
            cmd = ["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", *extra, "-o", str(lib), str(_SRC), "-lm"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"gcc failed on {_SRC.name}:\n{res.stderr}")
    return _LIB


def _open(path):
    lib = ctypes.CDLL(str(path))
    lib.oracle_forward.restype = ctypes.c_int
    lib.oracle_backward.restype = ctypes.c_int
    lib.oracle_num_threads.restype = ctypes.c_int
    return lib


def _load(precision: str = "f64"):
    global _lib, _lib32
    if precision not in ("f64", "f32"):
        raise ValueError(f"precision must be 'f64' or 'f32', got {precision!r}")
    if _lib is None:
        build()
        _lib = _open(_LIB)
        _lib32 = _open(_LIB32)
    return _lib if precision == "f64" else _lib32


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def set_threads(n: int) -> None:
    _load().oracle_set_threads(ctypes.c_int(int(n)))
    _load("f32").oracle_set_threads(ctypes.c_int(int(n)))


def _f32(a):
    return None if a is None else np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _cfg(x, dim, h, periodic, box_size, channels):
    B, N, P = x.shape
    c = _Cfg()
    c.dim, c.pos_stride, c.periodic = int(dim), int(P), int(bool(periodic))
    c.batch, c.particles, c.channels = int(B), int(N), int(channels)
    c.h = float(h)
    if periodic:
        box = np.broadcast_to(np.asarray(box_size, dtype=np.float64), (dim,))
        for d in range(dim):
            c.box[d] = float(box[d])
    return c


def forward(x, h, dim, *, mass=None, s=None, rho_in=None, periodic=False, box_size=None,
            want=("rho",), precision="f64"):
    """Run the C oracle forward.

    ``x`` is ``[B, N, P]`` (P >= dim; extra columns ignored), ``want`` names the
    outputs to compute out of ``count, rho, rho_grad, blur, grad, moment``.
    ``rho_in`` is the density handed to blur / grad / moment (their ``rho``
    argument).  ``precision="f32"`` runs the float build.  Returns a dict of numpy arrays
    (``count`` float32, others float64).
    """
    lib = _load(precision)
    x = _f32(x)
    B, N, _ = x.shape
    s = _f32(s)
    C = 0 if s is None else s.shape[-1]
    mass, rho_in = _f32(mass), _f32(rho_in)
    cfg = _cfg(x, dim, h, periodic, box_size, C)
    out = {}
    shapes = {"count": ((B, N), np.float32), "rho": ((B, N), np.float64),
              "rho_grad": ((B, N, dim), np.float64), "blur": ((B, N, C), np.float64),
              "grad": ((B, N, C, dim), np.float64), "moment": ((B, N, dim, dim), np.float64)}
    for k in want:
        shp, dt = shapes[k]
        out[k] = np.zeros(shp, dtype=dt)
    rc = lib.oracle_forward(ctypes.byref(cfg), _ptr(x), _ptr(mass), _ptr(s), _ptr(rho_in),
                            _ptr(out.get("count")), _ptr(out.get("rho")), _ptr(out.get("rho_grad")),
                            _ptr(out.get("blur")), _ptr(out.get("grad")), _ptr(out.get("moment")))
    if rc != 0:
        raise ValueError("oracle_forward: blur/grad/moment need rho_in (and s)")
    return out


def backward(x, h, dim, *, mass=None, s=None, rho_in=None, periodic=False, box_size=None,
             g_rho=None, g_rho_grad=None, g_blur=None, g_grad=None, g_moment=None, precision="f64"):
    """Run the C oracle backward (each operator differentiated independently, ``rho_in``
    treated as an input).  Returns ``dx [B,N,dim]``, ``ds [B,N,C]`` (or None) and ``drho [B,N]``."""
    lib = _load(precision)
    x = _f32(x)
    B, N, _ = x.shape
    s = _f32(s)
    C = 0 if s is None else s.shape[-1]
    mass, rho_in = _f32(mass), _f32(rho_in)
    ups = [_f32(g) for g in (g_rho, g_rho_grad, g_blur, g_grad, g_moment)]
    cfg = _cfg(x, dim, h, periodic, box_size, C)
    dx = np.zeros((B, N, dim), dtype=np.float64)
    ds = np.zeros((B, N, C), dtype=np.float64) if C else None
    drho = np.zeros((B, N), dtype=np.float64)
    rc = lib.oracle_backward(ctypes.byref(cfg), _ptr(x), _ptr(mass), _ptr(s), _ptr(rho_in),
                             *[_ptr(g) for g in ups], _ptr(dx), _ptr(ds), _ptr(drho))
    if rc != 0:
        raise ValueError("oracle_backward: feature / moment upstreams need rho_in (and s)")
    return dx, ds, drho


def safe_inv_sym_mat(m, tol):
    lib = _load()
    m = _f32(m)
    dim = m.shape[-1]
    out = np.empty_like(m)
    n = int(np.prod(m.shape[:-2]))
    lib.oracle_safe_inv_sym_mat(ctypes.c_int(dim), ctypes.c_long(n), _ptr(m), _ptr(out), ctypes.c_float(tol))
    return out
