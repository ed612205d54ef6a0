// Instantiations of the balanced one-launch decode kernel: unquantized fp16 K, INT4 symmetric V.
#include "decode_dq_kernel.cuh"

namespace knlp {
template int launch_dq_pair<KNLP_KV_F16, KNLP_KV_INT4_SYM>(const DecodeArgs&, const DqParams&, bool, cudaStream_t);
template int dq_chunk_of_pair<KNLP_KV_F16, KNLP_KV_INT4_SYM>(int, int);
}  // namespace knlp
