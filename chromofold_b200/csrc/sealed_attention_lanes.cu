// placeholder until the lane-per-block kernel lands
#include "attention_params.cuh"
namespace cfb {
bool lanes_kernel_supports(const AttentionParams &) { return false; }
cudaError_t launch_lanes_attention(const AttentionParams &, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace cfb
