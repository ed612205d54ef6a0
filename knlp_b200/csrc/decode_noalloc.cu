// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot provide the split-context workspace that
// knlp_b200_decode_splitk needs: a serving engine that hands all free device
// memory to its own pool at start-up and forbids cudaMalloc afterwards, or a
// plain C / Go / Java host that has no device allocator of its own and does not
// want to manage one just for a few megabytes of softmax partials.  For them
// this file offers one entry point that takes only inputs and the output tensor:
// the (m, l, o) partials live in a fixed array inside the library image.
//
// The array below is reserved on every GPU that loads the library, for as long as
// the process lives.  In host code its name is only a handle of the symbol, not a
// device address, so the address is looked up once per device with
// cudaGetSymbolAddress and that pointer is what the kernels receive.

#include <mutex>

#include "common.cuh"

namespace {

// 8 Mi floats = 32 MiB: room for n_seqs * n_q_heads * n_splits * (head_dim + 2)
// partial values; e.g. 32 sequences x 32 q heads x 37 splits at head_dim 128 needs 4.9 Mi.
constexpr long long kScratchFloats = KNLP_NOALLOC_MAX_FLOATS;
static __device__ __align__(256) float g_partials_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device; looked up on first use.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return KNLP_ERR_NO_DEVICE;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(&p, g_partials_scratch);
    if (rc != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return KNLP_ERR_NO_DEVICE;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return KNLP_OK;
}

}  // namespace

extern "C" {

int knlp_b200_decode_noalloc(const void* query, int q_dtype, const int64_t q_stride[2],
                             const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                             const int32_t* block_table, int64_t bt_stride,
                             const int32_t* seq_lens, int64_t num_blocks, int n_seqs,
                             int n_q_heads, int n_kv_heads, int head_dim, int block_size,
                             int n_splits, int max_seq_len, void* out, int out_dtype,
                             int64_t out_row_stride, void* stream) {
  if (!out) return KNLP_ERR_NULL;
  // everything the merge would reject is rejected here, before the decode kernel is enqueued
  if (out_dtype != KNLP_F32 && out_dtype != KNLP_F16 && out_dtype != KNLP_BF16)
    return KNLP_ERR_DTYPE;
  if (n_seqs < 0 || n_q_heads <= 0 || head_dim <= 0) return KNLP_ERR_SHAPE;
  if (n_seqs == 0) return KNLP_OK;
  const long long rows = static_cast<long long>(n_seqs) * n_q_heads;
  const long long per_split = rows * (static_cast<long long>(head_dim) + 2);
  if (per_split > kScratchFloats) return KNLP_ERR_TOO_LARGE;
  if (n_splits <= 0) {
    // let the library choose, then shrink to what the fixed array can hold
    int planned = 1;
    int64_t unused = 0;
    const int rc = knlp_b200_decode_plan(n_seqs, n_q_heads, n_kv_heads, head_dim, block_size,
                                         max_seq_len, k_plane ? k_plane->mode : 0,
                                         v_plane ? v_plane->mode : 0, &planned, &unused);
    if (rc != KNLP_OK) return rc;
    const long long fit = kScratchFloats / per_split;
    n_splits = planned > fit ? static_cast<int>(fit) : planned;
  } else if (per_split * n_splits > kScratchFloats) {
    return KNLP_ERR_TOO_LARGE;
  }

  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != KNLP_OK) return rc;
  // carve the array: m [rows, n], l [rows, n], o [rows, n, d].  Every slot that the
  // merge reads is written by the decode kernel of this call (empty splits write a
  // neutral partial), so nothing has to be cleared between calls.
  float* part_m = scratch;
  float* part_l = part_m + rows * n_splits;
  float* part_o = part_l + rows * n_splits;

  rc = knlp_b200_decode_splitk(query, q_dtype, q_stride, k_plane, v_plane, block_table, bt_stride,
                               seq_lens, num_blocks, n_seqs, n_q_heads, n_kv_heads, head_dim,
                               block_size, n_splits, max_seq_len, part_m, part_l, part_o, 0u,
                               stream);
  if (rc != KNLP_OK) return rc;
  return knlp_b200_combine(part_m, part_l, part_o, n_splits, n_splits, 1,
                           static_cast<int64_t>(n_splits) * head_dim, head_dim, out, out_dtype,
                           out_row_stride, nullptr, nullptr, 0, static_cast<int>(rows), head_dim,
                           stream);
}

}  // extern "C"
