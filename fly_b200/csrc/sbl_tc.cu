// bf16 tensor-core path (tcgen05 + TMA).  Placeholder: reports "unsupported"
// so that every call takes the generic kernels.
#include "sbl_common.cuh"

namespace sbl {
bool tc_supported(const SblParams&) { return false; }
cudaError_t tc_prepare_projection(const SblParams&, const Workspace&, char*, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t tc_key_logscale(const SblParams&, const Workspace&, char*, float*, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t tc_key_summary(const SblParams&, const Workspace&, char*, const float*, float*, float*, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t tc_band(const SblParams&, const Workspace&, char*, const float*, const float*, const float*, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace sbl
