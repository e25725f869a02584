// Placeholder until the Similarity tile kernels land: Similarity is not routed to a tiled kernel.
#include "kernels.cuh"
namespace simnets {
bool sim_use_tiled(const SimGeo&, bool, uint32_t) { return false; }
size_t sim_workspace_bytes(const SimGeo&, bool, uint32_t) { return 256; }
cudaError_t launch_sim_fwd_tiled(const SimGeo&, const float*, const float*, const float*, float*, void*, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_sim_dx_tiled(const SimGeo&, const float*, const float*, const float*, const float*, float*, void*, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_sim_dparams_tiled(const SimGeo&, const float*, const float*, const float*, const float*, float*, float*, bool, void*, cudaStream_t) { return cudaErrorNotSupported; }
}
