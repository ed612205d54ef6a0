// Instantiations of the split-context tensor-core decode kernel for one K/V mode pair.
#include "decode_mma_kernel.cuh"

namespace knlp {
template int launch_mma_pair<KNLP_KV_INT8_G32, KNLP_KV_INT8_G32>(const DecodeArgs&, const MmaParams&, bool,
                                       const TmaMaps*, cudaStream_t);
}  // namespace knlp
