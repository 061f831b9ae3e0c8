"""npa_b200: B200-native (sm_100a) SPH neighbour perception behind the ``sphops`` API.

``npa_b200.sphops`` mirrors the operator package of Neural Particle Automata;
``npa_b200.sharding`` splits a batch of independent particle systems over the
GPUs of one node.  Importing either loads ``libnpa_b200.so`` and fails loudly if
it has not been built (``python -m npa_b200.build``): there is no CPU fallback.
"""
import sys

__version__ = "0.1.0"


def install_as_sphops(fuse=False):
    """Register ``npa_b200.sphops`` under the top-level name ``sphops``.

    After this call ``from sphops import HashGrid`` (what the reference's models
    and trainers do) resolves to the B200 implementation.  ``fuse=True`` also turns
    on sibling-output fusion of the per-operator API (``sphops.enable_fusion``), which
    makes ``NPA.perceive`` run two neighbour sweeps instead of five.
    """
    from . import sphops as _sphops
    from .sphops import sph as _sph, sph_cuda as _sph_cuda

    sys.modules["sphops"] = _sphops
    sys.modules["sphops.sph"] = _sph
    sys.modules["sphops.sph_cuda"] = _sph_cuda
    if fuse:
        _sphops.enable_fusion(True)
    return _sphops
