// placeholder until the uncompressed comparison kernel lands
#include "attention_params.cuh"
namespace cfb {
cudaError_t launch_dense_attention(const AttentionParams &, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace cfb
extern "C" cf_status cf_b200_dense_attention_async(const cf_b200_dense_attention_desc *, void *) { return CF_ERR_UNSUPPORTED; }
