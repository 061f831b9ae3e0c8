"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares, host-side
geometry validation, and the Python surface the reference's callers rely on.  No kernel is launched."""
import ast
import ctypes
import os
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "npa_b200.h"
# the reference checkout, when present: $NPA_REFERENCE_ROOT or a sibling directory "reference" of this repository
REFERENCE = Path(os.environ.get("NPA_REFERENCE_ROOT", ROOT.parent / "reference"))


def _declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(npa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from npa_b200 import _native
    names = _declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(_native.lib, n), f"{n} declared in include/npa_b200.h but not exported"
    # and the binding knows the arity of each of them
    assert set(names) == set(_native.SIGNATURES)
    assert _native.lib.npa_abi_version() == _native.ABI_VERSION


def test_geometry_queries_and_errors():
    from npa_b200 import _native as n
    g = n.make_grid(3, "clamped", "grid", (24, 24, 24), 0.0879, 4, 65536, 32)
    ref = ctypes.byref(g)
    assert n.lib.npa_grid_num_cells(ref) == 24 ** 3
    assert n.lib.npa_grid_max_blocks(ref) == 4 * min(65536, 24 ** 3 + 65536 // 32)
    assert n.lib.npa_grid_scratch_bytes(ref) > 4 * (2 * 4 * 24 ** 3 + 2 * 4 * 65536)
    bad = n.make_grid(4, "clamped", "grid", (8, 8, 8), 0.1, 1, 8, 32)
    assert n.lib.npa_grid_num_cells(ctypes.byref(bad)) == n.NPA_ERR_INVALID_ARGUMENT
    assert "dim must be 2 or 3" in n.last_error()
    neg = n.make_grid(2, "clamped", "grid", (8, 8), -1.0, 1, 8, 32)
    assert n.lib.npa_grid_num_cells(ctypes.byref(neg)) == n.NPA_ERR_INVALID_ARGUMENT
    morton = n.make_grid(2, "clamped", "particle", (12, 12), 0.1, 1, 8, 32)
    assert n.lib.npa_grid_num_cells(ctypes.byref(morton)) == n.NPA_ERR_UNSUPPORTED
    # NULL pointers are rejected before any launch
    rc = n.lib.npa_grid_build(ref, None, None, None, None, None, 0, None)
    assert rc == n.NPA_ERR_INVALID_ARGUMENT and "non-NULL" in n.last_error()
    rc = n.lib.npa_safe_inv_sym_mat(4, 1, None, None, 1e-3, None)
    assert rc == n.NPA_ERR_INVALID_ARGUMENT and "2x2 or 3x3" in n.last_error()


def test_hashgrid_host_side_contract():
    from npa_b200 import sphops as sph
    grid = sph.HashGrid(dim=2, boundary="clamped", mode="grid", grid_size=(16, 16), eps=0.1,
                        num_particles=512, batch_size=3, max_particles_per_block=32)
    assert (grid.dim, grid.boundary, grid.mode, grid.num_cells) == (2, "clamped", "grid", 256)
    assert grid.device == torch.device("cuda")
    hg = grid.hashgrid
    assert (hg.grid_size_x, hg.grid_size_y, hg.particle_count, hg.batch_size) == (16, 16, 512, 3)
    assert hg.max_blocks == 3 * min(512, 256 + 16) and hg.max_particles_per_block == 32
    assert abs(hg.eps - 0.1) < 1e-12
    with pytest.raises(AssertionError, match="power of 2"):
        sph.HashGrid(dim=2, mode="particle", grid_size=(12, 12))
    with pytest.raises(KeyError):
        sph.HashGrid(dim=2, boundary="mirror")
    # clamped wrap is the identity, periodic wrap maps into [-L/2, L/2) and drops the pad column
    x = torch.tensor([[[0.9, -0.9, 0.2, 0.0]]])
    assert sph.HashGrid(dim=3, boundary="clamped", grid_size=(4, 4, 4)).wrap_positions(x) is x
    per = sph.HashGrid(dim=3, boundary="periodic", grid_size=(4, 4, 4), eps=0.25)
    assert torch.allclose(per.wrap_positions(x), torch.tensor([[[-0.1, 0.1, 0.2]]]), atol=1e-6)


def test_argument_checks_mirror_the_reference_binding():
    """Wrong dtype / device / layout is a TypeError (nanobind), a wrong shape a RuntimeError with the
    reference's wording (sphops/utils.cuh:526-567).  CPU tensors never reach a kernel."""
    from npa_b200 import sphops as sph
    grid = sph.HashGrid(dim=2, boundary="clamped", mode="grid", grid_size=(8, 8), eps=0.1,
                        num_particles=16, batch_size=2)
    hg = grid.hashgrid
    with pytest.raises(TypeError, match="positions"):
        hg.initialize(torch.zeros(2, 16, 2), None, None, None)       # CPU tensor
    with pytest.raises(TypeError):
        hg.count_forward(torch.zeros(2, 16, 2, dtype=torch.float64), None, None, None)
    from npa_b200.sphops.sph_cuda import _check
    meta = torch.empty(2, 16, 3, device="meta")
    with pytest.raises(TypeError):
        _check(meta, (2, 16, 2), "positions")


@pytest.mark.skipif(not (REFERENCE / "sphops" / "sph.py").exists(), reason="reference checkout not present")
def test_python_surface_matches_the_reference():
    """Same public functions, argument names and defaults as the reference's sphops/sph.py and
    the same methods on the native grid classes as its nanobind module."""
    import inspect
    from npa_b200.sphops import sph as ours, sph_cuda

    tree = ast.parse((REFERENCE / "sphops" / "sph.py").read_text())
    funcs = {n.name: n for n in tree.body if isinstance(n, ast.FunctionDef)}
    classes = {n.name: n for n in tree.body if isinstance(n, ast.ClassDef)}
    for name, node in funcs.items():
        if name.startswith("_") or name == "get_hashgrid_cls":
            continue
        assert hasattr(ours, name), f"missing function {name}"
        theirs = [a.arg for a in node.args.args]
        mine = list(inspect.signature(getattr(ours, name)).parameters)
        assert mine[:len(theirs)] == theirs, (name, mine, theirs)
    for name in classes:
        assert hasattr(ours, name), f"missing class {name}"
    init = next(n for n in classes["HashGrid"].body if isinstance(n, ast.FunctionDef) and n.name == "__init__")
    theirs = [a.arg for a in init.args.args][1:]
    mine = list(inspect.signature(ours.HashGrid.__init__).parameters)[1:]
    assert mine[:len(theirs)] == theirs
    defaults = {a.arg: ast.literal_eval(d) for a, d in zip(init.args.args[-len(init.args.defaults):], init.args.defaults)}
    sig = inspect.signature(ours.HashGrid.__init__)
    for k, v in defaults.items():
        assert sig.parameters[k].default == v, k
    # the reference's package exports
    init_tree = ast.parse((REFERENCE / "sphops" / "__init__.py").read_text())
    exported = [a.name for n in init_tree.body if isinstance(n, ast.ImportFrom) for a in n.names]
    import npa_b200.sphops as pkg
    for name in exported:
        assert hasattr(pkg, name), name
    # native module: every method the reference binds with .def("name", ...)
    cu = (REFERENCE / "sphops" / "sph_cuda.cu").read_text()
    bound = set(re.findall(r'\.def\("([a-z_]+)"', cu)) | set(re.findall(r'm\.def\("([a-z_]+)"', cu))
    for m in bound - {"safe_inv_sym_mat"}:
        assert hasattr(sph_cuda.HashGrid3DBox, m), m
    assert hasattr(sph_cuda, "safe_inv_sym_mat")
    for cls in re.findall(r'nb::class_<(\w+)>', cu):
        assert hasattr(sph_cuda, cls), cls


@pytest.mark.skipif(not (REFERENCE / "models" / "npa.py").exists(), reason="reference checkout not present")
def test_reference_model_imports_on_top_of_this_package():
    """models/npa.py of the reference imports unchanged once this package answers to `sphops`."""
    import importlib.util
    import sys
    import npa_b200
    saved = {k: sys.modules.get(k) for k in ("sphops", "sphops.sph", "sphops.sph_cuda")}
    try:
        npa_b200.install_as_sphops()
        spec = importlib.util.spec_from_file_location("ref_models_npa", REFERENCE / "models" / "npa.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        model = mod.NPA(spatial_dims=3, state_dims=16, hidden_dims=128)
        assert model.perception_dim == 16 * 2 + 3 + 3 * 16
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def test_step_update_and_splat_reject_bad_arguments_before_any_launch():
    """Validation happens on the host, ahead of the first CUDA call, so it can be checked without a GPU."""
    from npa_b200 import _native as n
    g = n.make_grid(2, "clamped", "grid", (16, 16), 0.1, 1, 128, 32)
    ref = ctypes.byref(g)
    buf = ctypes.c_void_p(256)  # a non-NULL, 16-byte aligned dummy address; never dereferenced
    null = ctypes.c_void_p(0)
    lib = n.lib
    assert lib.npa_step_update_forward(ref, buf, buf, buf, null, 0, 1.0, 1.0, 0, buf, buf, null) == n.NPA_ERR_INVALID_ARGUMENT
    assert "channels" in n.last_error()
    assert lib.npa_step_update_forward(ref, null, buf, buf, null, 8, 1.0, 1.0, 0, buf, buf, null) == n.NPA_ERR_INVALID_ARGUMENT
    assert lib.npa_step_update_backward(ref, buf, null, 8, 1.0, 1.0, buf, buf, null, null) == n.NPA_ERR_INVALID_ARGUMENT
    # splat: radius outside the supported range, non-positive sizes, missing scratch in normalised mode
    args = lambda radius, scratch, N=64: (buf, buf, 1, N, 64, 2.0, radius, -1.0, 1.0, 0, 1, 1.0, scratch, buf, null)
    assert lib.npa_splat_forward(*args(65, buf)) == n.NPA_ERR_UNSUPPORTED
    assert "radius" in n.last_error()
    assert lib.npa_splat_forward(*args(0, buf)) == n.NPA_ERR_UNSUPPORTED
    assert lib.npa_splat_forward(*args(10, buf, N=0)) == n.NPA_ERR_INVALID_ARGUMENT
    assert lib.npa_splat_forward(*args(10, null)) == n.NPA_ERR_INVALID_ARGUMENT
    assert "scale_scratch" in n.last_error()
    assert lib.npa_splat_backward(buf, buf, null, 1, 64, 64, 2.0, 10, -1.0, 1.0, 0, 1, 1.0, buf, buf, null) == n.NPA_ERR_INVALID_ARGUMENT


def test_splat_wrapper_derives_the_reference_constants():
    """sigma in pixels, patch radius and colour scale as utils/splatting.py:43-46,75-77 derives them."""
    from npa_b200.splatting import _derived
    from oracle.splat import derived
    for kw in (dict(img_size=256, sigma=2.0, lo=-1.0, hi=1.0, normalize_color=True, pixel_size=2.0 / 128.0),
               dict(img_size=64, sigma=1.5, lo=-2.0, hi=1.5, normalize_color=True, pixel_size=0.05),
               dict(img_size=32, sigma=0.1, lo=-1.0, hi=1.0, normalize_color=False, pixel_size=1.0)):
        assert _derived(**kw) == derived(**kw)
    assert _derived(256, 2.0, -1.0, 1.0, True, 2.0 / 128.0) == (4.0, 20, 4.0)
    assert _derived(32, 0.1, -1.0, 1.0, False, 1.0) == (0.1, 1, 1.0)


def test_mlp_weight_grad_rejects_unsupported_shapes_before_any_launch():
    from npa_b200 import _native as n
    buf, null = ctypes.c_void_p(256), ctypes.c_void_p(0)
    lib = n.lib
    need = lib.npa_mlp_weight_grad_scratch_floats(262144, 163, 35)
    assert need == 148 * (128 * 163 + 35 * 128 + 128)
    assert lib.npa_mlp_weight_grad_scratch_floats(40, 66, 18) == 2 * (128 * 66 + 18 * 128 + 128)  # two slabs of 32 rows
    call = lambda rows, k, h, o, scratch_floats=1 << 40: lib.npa_mlp_weight_grad(
        buf, buf, buf, buf, rows, k, h, o, buf, scratch_floats, buf, buf, buf, null)
    assert call(1000, 66, 64, 18) == n.NPA_ERR_UNSUPPORTED and "hidden" in n.last_error()
    assert call(1000, 177, 128, 18) == n.NPA_ERR_UNSUPPORTED
    assert call(1000, 66, 128, 49) == n.NPA_ERR_UNSUPPORTED
    assert call(0, 66, 128, 18) == n.NPA_ERR_INVALID_ARGUMENT
    assert call(1000, 66, 128, 18, scratch_floats=10) == n.NPA_ERR_SCRATCH_TOO_SMALL


def test_linear_tf32x3_rejects_unsupported_shapes_before_any_launch():
    from npa_b200 import _native as n
    buf, null = ctypes.c_void_p(256), ctypes.c_void_p(0)
    call = lambda rows, k, o, a=buf: n.lib.npa_linear_tf32x3(a, buf, null, null, buf, rows, k, o, k, 1, 0, null)
    assert call(1000, 177, 128) == n.NPA_ERR_UNSUPPORTED
    assert call(1000, 128, 200) == n.NPA_ERR_UNSUPPORTED
    assert call(1000, 176, 176) == n.NPA_ERR_UNSUPPORTED and "shared memory" in n.last_error()
    assert call(0, 128, 128) == n.NPA_ERR_INVALID_ARGUMENT
    assert call(1000, 128, 128, null) == n.NPA_ERR_INVALID_ARGUMENT


def test_tcgen05_entry_points_reject_bad_arguments_before_any_launch():
    """The tensor-memory kernels validate shapes, pointers, alignment and scratch size on the host: an
    operand or instruction descriptor outside its range would lose the CUDA context, so nothing may launch."""
    from npa_b200 import _native as n
    lib = n.lib
    buf, odd, null = ctypes.c_void_p(256), ctypes.c_void_p(260), ctypes.c_void_p(0)
    big = 1 << 40
    # linear layer
    assert lib.npa_linear_tcgen05_scratch_bytes(163, 128) == 6 * 2 * 128 * 32 * 4
    assert lib.npa_linear_tcgen05_scratch_bytes(128, 163) == 4 * 2 * 176 * 32 * 4
    lin = lambda rows, k, o, a=buf, scratch=buf, nbytes=big: lib.npa_linear_tcgen05(a, buf, null, null, buf, rows, k, o, k, 1, 0, scratch, nbytes, null)
    assert lin(1000, 128, 257) == n.NPA_ERR_UNSUPPORTED and "out_dim" in n.last_error()
    assert lin(1000, 1025, 128) == n.NPA_ERR_UNSUPPORTED
    assert lin(0, 128, 128) == n.NPA_ERR_INVALID_ARGUMENT
    assert lin(1000, 128, 128, a=null) == n.NPA_ERR_INVALID_ARGUMENT
    assert lin(1000, 128, 128, scratch=odd) == n.NPA_ERR_INVALID_ARGUMENT
    assert lin(1000, 128, 128, nbytes=16) == n.NPA_ERR_INVALID_ARGUMENT and "scratch" in n.last_error()
    # both layers of the forward
    assert lib.npa_mlp_forward_tcgen05_scratch_bytes(163, 35) == 6 * 2 * 128 * 32 * 4 + 4 * 2 * 48 * 32 * 4
    fwd = lambda rows, k, o, z=buf, nbytes=big: lib.npa_mlp_forward_tcgen05(z, buf, buf, buf, buf, buf, rows, k, o, k, 1, 128, 1, buf, nbytes, null)
    assert fwd(1000, 163, 65) == n.NPA_ERR_UNSUPPORTED
    assert fwd(1000, 1025, 35) == n.NPA_ERR_UNSUPPORTED
    assert fwd(-1, 163, 35) == n.NPA_ERR_INVALID_ARGUMENT
    assert fwd(1000, 163, 35, z=null) == n.NPA_ERR_INVALID_ARGUMENT
    assert fwd(1000, 163, 35, nbytes=1024) == n.NPA_ERR_INVALID_ARGUMENT
    # weight gradients
    assert lib.npa_mlp_weight_grad_tcgen05_scratch_floats(262144, 163, 35) == 148 * 128 * (176 + 48)
    wg = lambda rows, k, h, o, z=buf, floats=big: lib.npa_mlp_weight_grad_tcgen05(z, buf, buf, buf, rows, k, h, o, buf, floats, buf, buf, buf, null)
    assert wg(1000, 66, 64, 18) == n.NPA_ERR_UNSUPPORTED and "hidden" in n.last_error()
    assert wg(1000, 176, 128, 18) == n.NPA_ERR_UNSUPPORTED      # in + 1 columns must fit six atoms of 32
    assert wg(1000, 66, 128, 49) == n.NPA_ERR_UNSUPPORTED
    assert wg(0, 66, 128, 18) == n.NPA_ERR_INVALID_ARGUMENT
    assert wg(1000, 66, 128, 18, z=odd) == n.NPA_ERR_INVALID_ARGUMENT and "aligned" in n.last_error()
    assert wg(1000, 66, 128, 18, floats=10) == n.NPA_ERR_SCRATCH_TOO_SMALL
    # hidden-layer gradient
    hg = lambda rows, h, o, dh=buf: lib.npa_mlp_hidden_grad(buf, buf, buf, dh, rows, h, o, 128, 1, null)
    assert hg(1000, 64, 18) == n.NPA_ERR_UNSUPPORTED
    assert hg(1000, 128, 49) == n.NPA_ERR_UNSUPPORTED
    assert hg(0, 128, 18) == n.NPA_ERR_INVALID_ARGUMENT
    assert hg(1000, 128, 18, dh=odd) == n.NPA_ERR_INVALID_ARGUMENT
    # status and self-test arguments
    assert lib.npa_linear_tcgen05_status(null, 0) == n.NPA_ERR_INVALID_ARGUMENT
    assert lib.npa_linear_tcgen05_wait_selftest(0, buf, null) == n.NPA_ERR_INVALID_ARGUMENT
    assert lib.npa_linear_tcgen05_wait_selftest(2000, null, null) == n.NPA_ERR_INVALID_ARGUMENT
