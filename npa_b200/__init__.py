"""npa_b200: B200-native SPH neighbour perception (see npa_b200.sphops)."""
