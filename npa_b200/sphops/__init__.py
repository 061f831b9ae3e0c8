"""Drop-in ``sphops`` package backed by the B200 kernels.

Exports what the reference's ``sphops/__init__.py`` exports (HashGrid and the
operator functions) plus :func:`perceive`, the fused perception step.  Put the
directory that contains this package (``npa_b200/``) on ``sys.path`` ahead of the
reference checkout, or call :func:`npa_b200.install_as_sphops`, and
``from sphops import HashGrid, blur, ...`` resolves here.
"""
from .sph import (HashGrid, HashGridSnapshot, bin_particles, unbin_particles, count, density, blur,
                  gradient, density_gradient, moment_matrix, gradient_hybrid, safe_inv_sym_mat, perceive,
                  enable_fusion, fusion_enabled, set_pair_cache, DensityPair, BlurGradient, perceive_features, PerceiveFeatures,
                  step_update, StepUpdate,
                  Permute, Count, Density, Blur, Gradient, DensityGradient, MomentMatrix, Perception)

__all__ = [
    "HashGrid", "HashGridSnapshot", "bin_particles", "unbin_particles", "count", "density", "blur",
    "gradient", "density_gradient", "moment_matrix", "gradient_hybrid", "safe_inv_sym_mat", "perceive",
    "enable_fusion", "fusion_enabled", "set_pair_cache", "perceive_features", "step_update",
]
