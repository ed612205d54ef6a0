// Shared device/host definitions for the packed-KV kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/knlp_b200.h"

namespace knlp {

constexpr int kGroup = KNLP_GROUP_SIZE;  // elements per scale/zero group

// Device-side view of one cache plane; mirrors knlp_kv_plane.
struct Plane {
  uint8_t* codes;
  __half* scales;
  __half* zeros;
  int64_t cs[3];  // codes strides: block, token, head (bytes)
  int64_t ss[3];  // scales strides (fp16 elements)
  int64_t zs[3];  // zeros strides
  int mode;
};

inline Plane make_plane(const knlp_kv_plane* p) {
  Plane d{};
  if (!p) {
    d.mode = KNLP_KV_NONE;
    return d;
  }
  d.codes = static_cast<uint8_t*>(p->codes);
  d.scales = static_cast<__half*>(p->scales);
  d.zeros = static_cast<__half*>(p->zeros);
  for (int i = 0; i < 3; ++i) {
    d.cs[i] = p->codes_stride[i];
    d.ss[i] = p->scales_stride[i];
    d.zs[i] = p->zeros ? p->zeros_stride[i] : 0;
  }
  d.mode = p->mode;
  if (p->mode == KNLP_KV_F16 || p->mode == KNLP_KV_BF16) {
    // an unquantized plane: its strides arrive in 2-byte elements, the kernels index bytes
    for (int i = 0; i < 3; ++i) d.cs[i] *= 2;
  }
  return d;
}

// Exact widening load of one source element.
template <int DT>
__device__ __forceinline__ float load_elem(const void* base, int64_t idx) {
  if constexpr (DT == KNLP_F32) {
    return static_cast<const float*>(base)[idx];
  } else if constexpr (DT == KNLP_F16) {
    return __half2float(static_cast<const __half*>(base)[idx]);
  } else {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
  }
}

__device__ __forceinline__ float load_elem_rt(const void* base, int64_t idx, int dt) {
  if (dt == KNLP_F32) return load_elem<KNLP_F32>(base, idx);
  if (dt == KNLP_F16) return load_elem<KNLP_F16>(base, idx);
  return load_elem<KNLP_BF16>(base, idx);
}

__device__ __forceinline__ void store_elem_rt(void* base, int64_t idx, float v, int dt) {
  if (dt == KNLP_F32) {
    static_cast<float*>(base)[idx] = v;
  } else if (dt == KNLP_F16) {
    static_cast<__half*>(base)[idx] = __float2half_rn(v);
  } else {
    static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  }
}

// Split length used by decode_splitk: ceil(max_len / n_splits) rounded up to 64.
__host__ __device__ inline int split_chunk(int max_len, int n_splits) {
  int c = (max_len + n_splits - 1) / n_splits;
  c = (c + 63) / 64 * 64;
  return c < 64 ? 64 : c;
}

// Host-side launch functions implemented in the individual .cu files.
int launch_quant_append(const void* key, const int64_t* kstride, const void* value,
                        const int64_t* vstride, int src_dtype, const Plane& kp, const Plane& vp,
                        const int64_t* slot_mapping, int n_tokens, int n_kv_heads, int head_dim,
                        int block_size, float clip_ratio, cudaStream_t st);

struct DecodeArgs {
  const void* q;
  int q_dtype;
  int64_t q_stride[2];
  Plane k, v;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  int64_t num_blocks;
  int n_seqs, n_q_heads, n_kv_heads, head_dim, block_size;
  int n_splits, chunk;
  float* part_m;
  float* part_l;
  float* part_o;
  // Output of the balanced one-launch kernel (the split-context kernels write partials)
  void* out;
  int out_dtype;
  int64_t out_row_stride;
};

int launch_decode_generic(const DecodeArgs& a, cudaStream_t st);
// Returns KNLP_OK if it launched, 1 if the shape/strides are not eligible for the
// tensor-core kernel (caller falls back to the generic one), <0 on error.
// allow_tma = false keeps the tensor-core kernel on its cp.async loader.
// debug_stall: test aid of the TMA staging, see KNLP_DECODE_DEBUG_STALL.
int launch_decode_mma(const DecodeArgs& a, bool allow_tma, bool debug_stall, cudaStream_t st);
// Shape / layout test of the tensor-core kernels: 0 = eligible (heads per CTA and page
// size filled in as log2), 1 = generic kernel only.
int decode_mma_layout(const DecodeArgs& a, int* hpb_log2, int* page_log2);

// CTA shape of the tensor-core decode kernels, shared with the split planner: one warp
// per (kv head, 16-token tile), so a CTA covers at most kDecodeWarps kv heads; sixteen
// warps of ~128 registers fit on an SM, as four CTAs of four warps (the CTAs of an SM
// wait at their stage barriers independently).
constexpr int kDecodeWarps = 4;
constexpr int kDecodeCtasPerSm = 16 / kDecodeWarps;

// Balanced one-launch decode (decode_dq_kernel.cuh): a.out receives the attention output
// (emit_partial: fp32 rows [o un-normalised, m, l]).  ws / ints: the workspace sized by
// dq_workspace_size; the ints are counters that must be zero on entry and are left zero.  Returns KNLP_OK, 1 if the call is not eligible (nothing launched),
// <0 on error.  per_head_tables: routed decode - block_table and seq_lens have one row /
// entry per (sequence, kv head), the lengths count whole blocks.
int launch_decode_dq(const DecodeArgs& a, float* ws, int64_t ws_floats, int* ints, int64_t n_ints,
                     int max_seq_len, bool emit_partial, int n_sms,
                     const knlp_new_tokens* new_tokens, bool per_head_tables, cudaStream_t st);
void dq_workspace_size(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int n_sms,
                       int64_t* floats, int64_t* ints);
// Low-rank-V decode (lowrank_decode.cu): split-context kernel + finish kernel.
int launch_lowrank_decode(const void* q, const void* k, int qk_dtype, const float* proj,
                          const float* basis, int n_kv_heads, int nq, int T, int head_dim,
                          int n_sms, float* ws, int64_t ws_floats, float* za_out, float* out,
                          cudaStream_t st);
int64_t lowrank_workspace_floats(int n_kv_heads, int nq, int T, int n_sms);
// Device-side status word of the decode kernels (0 = clean); synchronises.
int read_and_clear_decode_status();

int launch_combine(const float* pm, const float* pl, const float* po, int n_parts,
                   int64_t ml_row, int64_t ml_part, int64_t o_row, int64_t o_part, void* out,
                   int out_dtype, int64_t out_row, float* out_m, float* out_l, int64_t out_ml,
                   int n_rows, int head_dim, cudaStream_t st);
// Merge of the balanced kernel's partial slots: row r of pair p = slots
// pair_info[2p] .. + pair_info[2p+1] - 1 (heads rows each).  Launched as a programmatic
// dependent of the kernel before it on the stream.
int launch_combine_pairs(const float* ws_m, const float* ws_l, const float* ws_o,
                         const int* pair_info, int heads, int n_rows, int head_dim, void* out,
                         int out_dtype, int64_t out_row, bool emit_partial, cudaStream_t st);

}  // namespace knlp
