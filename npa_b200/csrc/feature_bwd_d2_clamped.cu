// Instantiates the blur / feature-gradient backward kernels for dim 2, clamped
// boundary (one translation unit per geometry keeps the build parallel).
#include "feature_kernels.cuh"

namespace npa {
template int launch_feature_backward_geom<2, false, true>(const Geom &, int, const FeatureBwdArgs &, cudaStream_t);
template int launch_feature_backward_geom<2, false, false>(const Geom &, int, const FeatureBwdArgs &, cudaStream_t);
}  // namespace npa
