"""In-tree build of the sm_100a kernel library ``libnpa_b200.so``.

``python -m npa_b200.build`` (or :func:`build`) compiles every ``csrc/*.cu`` with
nvcc for ``sm_100a`` (one object per translation unit, in parallel) and links
them into ``npa_b200/libnpa_b200.so`` next to this file.  nvcc cross-compiles,
so no GPU is needed to build.  Objects are rebuilt only when a source or header
is newer than the object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "_build"
LIB_PATH = PKG_DIR / "libnpa_b200.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the npa_b200 kernels cannot be built")
    return exe


def _headers_mtime() -> float:
    hdrs = list(SRC_DIR.glob("*.cuh")) + list(INCLUDE_DIR.glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose and (res.stdout or res.stderr):
        sys.stderr.write(f"--- {src.name}\n{res.stdout}{res.stderr}")
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    return obj


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link the library; returns its path."""
    OBJ_DIR.mkdir(exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    sources = sorted(SRC_DIR.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {SRC_DIR}")
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    workers = max(1, min(len(sources), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose or ptxas_info, extra), sources))
    if (not LIB_PATH.exists()) or any(o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "static", "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas-info" in sys.argv)
    print(path)
