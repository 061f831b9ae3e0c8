// Instantiates the cell-tile forward sweeps (blur + feature gradient) for dim 2, clamped
// boundary (one translation unit per geometry keeps the build parallel).
#include "feature_tile.cuh"

namespace npa {
template int launch_feature_tile_forward<2, false>(const Geom &, int, const FeatureFwdArgs &, cudaStream_t, bool *);
}  // namespace npa
