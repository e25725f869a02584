// Host-side validation and geometry: descriptor -> kernel geometry structs.
#pragma once
#include "simnets_b200.h"
#include "geometry.cuh"

namespace simnets {
int sim_geometry(const simnets_sim_desc* d, SimGeo* g);
int mex_geometry(const simnets_mex_desc* d, simnets_mex_geometry* out, MexGeo* g);
}
