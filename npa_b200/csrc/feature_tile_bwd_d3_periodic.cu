// Instantiates the cell-tile backward sweeps (blur + feature gradient) for dim 3, periodic
// boundary (one translation unit per geometry keeps the build parallel).
#include "feature_tile.cuh"

namespace npa {
template int launch_feature_tile_backward<3, true, true>(const Geom &, int, const FeatureBwdArgs &, cudaStream_t, bool *);
template int launch_feature_tile_backward<3, true, false>(const Geom &, int, const FeatureBwdArgs &, cudaStream_t, bool *);
}  // namespace npa
