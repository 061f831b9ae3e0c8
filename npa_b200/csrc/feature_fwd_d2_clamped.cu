// Instantiates the blur / feature-gradient forward kernels for dim 2, clamped
// boundary (one translation unit per geometry keeps the build parallel).
#include "feature_kernels.cuh"

namespace npa {
template int launch_feature_forward_geom<2, false>(const Geom &, int, const FeatureFwdArgs &, cudaStream_t);
}  // namespace npa
