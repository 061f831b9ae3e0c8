// Instantiates the blur / feature-gradient forward kernels for dim 3, periodic
// boundary (one translation unit per geometry keeps the build parallel).
#include "feature_kernels.cuh"

namespace npa {
template int launch_feature_forward_geom<3, true>(const Geom &, int, const FeatureFwdArgs &, cudaStream_t);
}  // namespace npa
