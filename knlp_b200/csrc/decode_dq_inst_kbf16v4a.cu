// Instantiations of the balanced one-launch decode kernel: unquantized bf16 K, INT4 asymmetric V.
#include "decode_dq_kernel.cuh"

namespace knlp {
template int launch_dq_pair<KNLP_KV_BF16, KNLP_KV_INT4_ASYM>(const DecodeArgs&, const DqParams&, bool, cudaStream_t);
template int dq_chunk_of_pair<KNLP_KV_BF16, KNLP_KV_INT4_ASYM>(int, int);
}  // namespace knlp
