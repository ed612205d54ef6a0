// C ABI of the library: argument validation and dispatch.  No exceptions, no
// C++ types and no allocation cross this boundary.

#include <atomic>

#include "common.cuh"

using namespace knlp;

namespace {

bool dtype_ok(int dt) { return dt == KNLP_F32 || dt == KNLP_F16 || dt == KNLP_BF16; }

bool head_dim_ok(int d) { return d == 32 || d == 64 || d == 128 || d == 256; }

// unquantized_k: the plane may also be an fp16 / bf16 K plane (decode only).
int check_plane(const knlp_kv_plane* p, bool unquantized_k) {
  if (!p) return KNLP_ERR_NULL;
  switch (p->mode) {
    case KNLP_KV_F16:
    case KNLP_KV_BF16:
      if (!unquantized_k) return KNLP_ERR_MODE;
      return p->codes ? KNLP_OK : KNLP_ERR_NULL;
    case KNLP_KV_INT4_SYM:
      break;
    case KNLP_KV_INT4_ASYM:
      if (!p->zeros) return KNLP_ERR_NULL;
      break;
    case KNLP_KV_INT8_G32:
      break;
    default:
      return KNLP_ERR_MODE;
  }
  if (!p->codes || !p->scales) return KNLP_ERR_NULL;
  return KNLP_OK;
}

// SM count of the CURRENT device, looked up once per device index.
int sm_count() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return 148;  // B200
  }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 148;
  }
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace

extern "C" {

int knlp_b200_abi_version(void) { return KNLP_B200_ABI_VERSION; }

int knlp_b200_debug_status(void) { return read_and_clear_decode_status(); }

const char* knlp_b200_strerror(int status) {
  switch (status) {
    case KNLP_OK: return "ok";
    case KNLP_ERR_NULL: return "a required pointer is NULL";
    case KNLP_ERR_SHAPE: return "unsupported shape (head_dim must be 32/64/128/256, heads must divide)";
    case KNLP_ERR_DTYPE: return "unknown dtype code";
    case KNLP_ERR_MODE: return "unknown or unsupported K/V quantization mode";
    case KNLP_ERR_STRIDE: return "stride or alignment not addressable";
    case KNLP_ERR_WORKSPACE: return "split count / workspace arguments out of range";
    case KNLP_ERR_LAUNCH: return "CUDA launch failed";
    case KNLP_ERR_NO_DEVICE: return "no usable sm_100 device or kernel image";
    case KNLP_ERR_TOO_LARGE: return "request exceeds a fixed capacity of this entry point";
    default: return "unknown status";
  }
}

int knlp_b200_quant_append(const void* key, const int64_t key_stride[2], const void* value,
                           const int64_t value_stride[2], int src_dtype,
                           const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                           const int64_t* slot_mapping, int n_tokens, int n_kv_heads,
                           int head_dim, int block_size, float clip_ratio, void* stream) {
  if (!dtype_ok(src_dtype)) return KNLP_ERR_DTYPE;
  if (n_tokens < 0 || n_kv_heads <= 0 || block_size <= 0) return KNLP_ERR_SHAPE;
  if (head_dim <= 0 || head_dim % KNLP_GROUP_SIZE) return KNLP_ERR_SHAPE;
  const bool do_k = key && k_plane && k_plane->mode != KNLP_KV_NONE;
  const bool do_v = value && v_plane && v_plane->mode != KNLP_KV_NONE;
  if (do_k) {
    if (!key_stride) return KNLP_ERR_NULL;
    int rc = check_plane(k_plane, false);
    if (rc) return rc;
  }
  if (do_v) {
    if (!value_stride) return KNLP_ERR_NULL;
    int rc = check_plane(v_plane, false);
    if (rc) return rc;
  }
  if (!do_k && !do_v) return KNLP_OK;
  if (n_tokens == 0) return KNLP_OK;
  if (!slot_mapping) return KNLP_ERR_NULL;
  Plane kp = make_plane(do_k ? k_plane : nullptr);
  Plane vp = make_plane(do_v ? v_plane : nullptr);
  return launch_quant_append(do_k ? key : nullptr, key_stride, do_v ? value : nullptr,
                             value_stride, src_dtype, kp, vp, slot_mapping, n_tokens, n_kv_heads,
                             head_dim, block_size, clip_ratio, static_cast<cudaStream_t>(stream));
}

int knlp_b200_decode_plan(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                          int block_size, int max_seq_len, int k_mode, int v_mode,
                          int* n_splits_out, int64_t* workspace_floats_out) {
  (void)block_size; (void)k_mode; (void)v_mode;
  if (!n_splits_out || !workspace_floats_out) return KNLP_ERR_NULL;
  if (n_seqs <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    return KNLP_ERR_SHAPE;
  if (!head_dim_ok(head_dim) || max_seq_len < 0) return KNLP_ERR_SHAPE;
  // CTAs per split: one per (sequence, block of up to kDecodeWarps kv heads);
  // kDecodeCtasPerSm of them fit on an SM.  Pick the split count that fills whole waves
  // best; prefer at least two waves so the tail is amortised, and never go below 256
  // tokens per split.
  int hpb = kDecodeWarps;
  while (hpb > 1 && n_kv_heads % hpb) hpb >>= 1;
  const int64_t base = static_cast<int64_t>(n_seqs) * (n_kv_heads / hpb);
  const int64_t slots = static_cast<int64_t>(kDecodeCtasPerSm) * sm_count();
  const int max_splits = max_seq_len >= 512 ? (max_seq_len / 256 > 1024 ? 1024 : max_seq_len / 256) : 1;
  // Cost model (microseconds, coarse): a wave of CTAs costs a fixed
  // set-up plus 1.2 us per stage (16 tokens x the CTA's heads) of its split; merging costs a
  // little per split.  Fewer, longer splits amortise the set-up; more splits fill the
  // machine and even out ragged batches.
  const int tokens_per_stage = 16 * (kDecodeWarps / hpb);
  int best = 1;
  double best_cost = 1e30;
  for (int n = 1; n <= max_splits; ++n) {
    const int64_t ctas = base * n;
    const int64_t waves = (ctas + slots - 1) / slots;
    if (waves > 8 && n > 1) break;
    const int chunk = split_chunk(max_seq_len, n);
    const double stages = static_cast<double>((chunk + tokens_per_stage - 1) / tokens_per_stage);
    const double cost = static_cast<double>(waves) * (6.0 + 1.2 * stages) + 0.03 * n + 3.0;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = n;
    }
  }
  *n_splits_out = best;
  *workspace_floats_out =
      static_cast<int64_t>(n_seqs) * n_q_heads * best * (static_cast<int64_t>(head_dim) + 2);
  return KNLP_OK;
}

}  // extern "C"

namespace {

// Argument checks and DecodeArgs shared by the decode entry points.  Returns 1 when
// there is nothing to do (no sequences).
int decode_args(const void* query, int q_dtype, const int64_t q_stride[2],
                const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
                int64_t num_blocks, int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                int block_size, int max_seq_len, DecodeArgs* out) {
  if (!query || !q_stride || !block_table || !seq_lens) return KNLP_ERR_NULL;
  if (!dtype_ok(q_dtype)) return KNLP_ERR_DTYPE;
  if (n_seqs < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    return KNLP_ERR_SHAPE;
  if (!head_dim_ok(head_dim) || block_size <= 0 || num_blocks <= 0) return KNLP_ERR_SHAPE;
  if (n_seqs > 65535 || n_kv_heads * ((n_q_heads / n_kv_heads + 7) / 8) > 65535)
    return KNLP_ERR_SHAPE;
  if (max_seq_len < 0) return KNLP_ERR_WORKSPACE;
  int rc = check_plane(k_plane, true);
  if (rc) return rc;
  rc = check_plane(v_plane, false);
  if (rc) return rc;
  if (n_seqs == 0) return 1;
  DecodeArgs a{};
  a.q = query;
  a.q_dtype = q_dtype;
  a.q_stride[0] = q_stride[0];
  a.q_stride[1] = q_stride[1];
  a.k = make_plane(k_plane);
  a.v = make_plane(v_plane);
  a.block_table = block_table;
  a.bt_stride = bt_stride;
  a.seq_lens = seq_lens;
  a.num_blocks = num_blocks;
  a.n_seqs = n_seqs;
  a.n_q_heads = n_q_heads;
  a.n_kv_heads = n_kv_heads;
  a.head_dim = head_dim;
  a.block_size = block_size;
  *out = a;
  return KNLP_OK;
}

// Split-context launch: tensor-core kernel where the layout allows, else the generic one.
int launch_splitk(const DecodeArgs& a, unsigned flags, cudaStream_t st) {
  int rc = 1;
  if (!(flags & KNLP_DECODE_FORCE_GENERIC)) {
    rc = launch_decode_mma(a, (flags & KNLP_DECODE_USE_TMA) != 0,
                           (flags & KNLP_DECODE_DEBUG_STALL) != 0, st);
    if (rc <= 0) return rc;  // launched, or failed for good
  }
  return launch_decode_generic(a, st);
}

}  // namespace

extern "C" {

int knlp_b200_decode_splitk(const void* query, int q_dtype, const int64_t q_stride[2],
                            const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                            const int32_t* block_table, int64_t bt_stride,
                            const int32_t* seq_lens, int64_t num_blocks, int n_seqs,
                            int n_q_heads, int n_kv_heads, int head_dim, int block_size,
                            int n_splits, int max_seq_len, float* part_m, float* part_l,
                            float* part_o, unsigned flags, void* stream) {
  if (!part_m || !part_l || !part_o) return KNLP_ERR_NULL;
  if (n_splits < 1) return KNLP_ERR_WORKSPACE;
  DecodeArgs a;
  const int rc = decode_args(query, q_dtype, q_stride, k_plane, v_plane, block_table, bt_stride,
                             seq_lens, num_blocks, n_seqs, n_q_heads, n_kv_heads, head_dim,
                             block_size, max_seq_len, &a);
  if (rc) return rc < 0 ? rc : KNLP_OK;
  a.n_splits = n_splits;
  a.chunk = split_chunk(max_seq_len, n_splits);
  a.part_m = part_m;
  a.part_l = part_l;
  a.part_o = part_o;
  return launch_splitk(a, flags, static_cast<cudaStream_t>(stream));
}

int knlp_b200_decode_workspace(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                               int block_size, int max_seq_len, int64_t* workspace_floats_out,
                               int64_t* counter_ints_out) {
  if (!workspace_floats_out || !counter_ints_out) return KNLP_ERR_NULL;
  int n_splits = 1;
  int64_t split_floats = 0;
  const int rc = knlp_b200_decode_plan(n_seqs > 0 ? n_seqs : 1, n_q_heads, n_kv_heads, head_dim,
                                       block_size, max_seq_len, 0, 0, &n_splits, &split_floats);
  if (rc) return rc;
  int64_t dq_floats = 0, dq_ints = 0;
  dq_workspace_size(n_seqs > 0 ? n_seqs : 1, n_q_heads, n_kv_heads, head_dim, sm_count(),
                    &dq_floats, &dq_ints);
  *workspace_floats_out = (dq_floats > split_floats ? dq_floats : split_floats) + 4;
  *counter_ints_out = dq_ints;
  return KNLP_OK;
}

int knlp_b200_decode_append_attention(const void* query, int q_dtype, const int64_t q_stride[2],
                               const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                               const int32_t* block_table, int64_t bt_stride,
                               const int32_t* seq_lens, int64_t num_blocks, int n_seqs,
                               int n_q_heads, int n_kv_heads, int head_dim, int block_size,
                               int max_seq_len, float* workspace, int64_t workspace_floats,
                               int32_t* counters, int64_t counter_ints, void* out, int out_dtype,
                               int64_t out_row_stride, unsigned flags,
                               const knlp_new_tokens* new_tokens, void* stream) {
  if (!out || !workspace || !counters) return KNLP_ERR_NULL;
  if (new_tokens) {
    if (!new_tokens->key || !new_tokens->value) return KNLP_ERR_NULL;
    if (!dtype_ok(new_tokens->dtype)) return KNLP_ERR_DTYPE;
    if (flags & (KNLP_DECODE_FORCE_GENERIC | KNLP_DECODE_USE_TMA | KNLP_DECODE_FIXED_SPLITS))
      return KNLP_ERR_MODE;  // only the balanced kernel appends
  }
  if (!dtype_ok(out_dtype)) return KNLP_ERR_DTYPE;
  const bool emit = (flags & KNLP_DECODE_EMIT_PARTIAL) != 0;
  if (emit && out_dtype != KNLP_F32) return KNLP_ERR_DTYPE;
  DecodeArgs a;
  int rc = decode_args(query, q_dtype, q_stride, k_plane, v_plane, block_table, bt_stride,
                       seq_lens, num_blocks, n_seqs, n_q_heads, n_kv_heads, head_dim, block_size,
                       max_seq_len, &a);
  if (rc) return rc < 0 ? rc : KNLP_OK;
  a.out = out;
  a.out_dtype = out_dtype;
  a.out_row_stride = out_row_stride;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the merge reads the partial outputs as float4
  const uintptr_t mis = reinterpret_cast<uintptr_t>(workspace) % 16;
  if (mis % 4) return KNLP_ERR_STRIDE;
  if (mis) {
    workspace += (16 - mis) / 4;
    workspace_floats -= (16 - mis) / 4;
  }
  if (!(flags & (KNLP_DECODE_FORCE_GENERIC | KNLP_DECODE_USE_TMA | KNLP_DECODE_FIXED_SPLITS))) {
    rc = launch_decode_dq(a, workspace, workspace_floats, counters, counter_ints, max_seq_len, emit,
                          sm_count(), new_tokens, false, st);
    if (rc <= 0) return rc;  // launched, or failed for good
  }
  // a layout only the other kernels can address: they do not append
  if (new_tokens) return KNLP_ERR_STRIDE;
  // fixed splits: split-context kernel into the workspace, then the combine kernel
  int n_splits = 1;
  int64_t need = 0;
  rc = knlp_b200_decode_plan(n_seqs, n_q_heads, n_kv_heads, head_dim, block_size, max_seq_len,
                             k_plane->mode, v_plane->mode, &n_splits, &need);
  if (rc) return rc;
  if (need > workspace_floats) return KNLP_ERR_WORKSPACE;
  const int64_t rows = static_cast<int64_t>(n_seqs) * n_q_heads;
  a.n_splits = n_splits;
  a.chunk = split_chunk(max_seq_len, n_splits);
  a.part_o = workspace;
  a.part_m = workspace + rows * n_splits * head_dim;
  a.part_l = a.part_m + rows * n_splits;
  a.out = nullptr;
  rc = launch_splitk(a, flags, st);
  if (rc != KNLP_OK) return rc;
  float* fo = static_cast<float*>(out);
  return launch_combine(a.part_m, a.part_l, a.part_o, n_splits, n_splits, 1,
                        static_cast<int64_t>(n_splits) * head_dim, head_dim, out, out_dtype,
                        out_row_stride, emit ? fo + head_dim : nullptr,
                        emit ? fo + head_dim + 1 : nullptr, out_row_stride,
                        static_cast<int>(rows), head_dim, st);
}

int knlp_b200_decode_attention(const void* query, int q_dtype, const int64_t q_stride[2],
                               const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                               const int32_t* block_table, int64_t bt_stride,
                               const int32_t* seq_lens, int64_t num_blocks, int n_seqs,
                               int n_q_heads, int n_kv_heads, int head_dim, int block_size,
                               int max_seq_len, float* workspace, int64_t workspace_floats,
                               int32_t* counters, int64_t counter_ints, void* out, int out_dtype,
                               int64_t out_row_stride, unsigned flags, void* stream) {
  return knlp_b200_decode_append_attention(
      query, q_dtype, q_stride, k_plane, v_plane, block_table, bt_stride, seq_lens, num_blocks,
      n_seqs, n_q_heads, n_kv_heads, head_dim, block_size, max_seq_len, workspace,
      workspace_floats, counters, counter_ints, out, out_dtype, out_row_stride, flags, nullptr,
      stream);
}

int knlp_b200_routed_decode_attention(const void* query, int q_dtype, const int64_t q_stride[2],
                                      const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                                      const int32_t* block_tables, int64_t bt_stride,
                                      const int32_t* block_counts, int64_t num_blocks, int n_seqs,
                                      int n_q_heads, int n_kv_heads, int head_dim, int block_size,
                                      int max_selected_blocks, float* workspace,
                                      int64_t workspace_floats, int32_t* counters,
                                      int64_t counter_ints, void* out, int out_dtype,
                                      int64_t out_row_stride, unsigned flags, void* stream) {
  if (!out || !workspace || !counters) return KNLP_ERR_NULL;
  if (!dtype_ok(out_dtype)) return KNLP_ERR_DTYPE;
  if (flags & ~KNLP_DECODE_EMIT_PARTIAL) return KNLP_ERR_MODE;
  const bool emit = (flags & KNLP_DECODE_EMIT_PARTIAL) != 0;
  if (emit && out_dtype != KNLP_F32) return KNLP_ERR_DTYPE;
  if (max_selected_blocks < 0 || block_size <= 0 ||
      static_cast<int64_t>(max_selected_blocks) * block_size > 0x7fffffff)
    return KNLP_ERR_SHAPE;
  const int max_len = max_selected_blocks * block_size;
  DecodeArgs a;
  int rc = decode_args(query, q_dtype, q_stride, k_plane, v_plane, block_tables, bt_stride,
                       block_counts, num_blocks, n_seqs, n_q_heads, n_kv_heads, head_dim,
                       block_size, max_len, &a);
  if (rc) return rc < 0 ? rc : KNLP_OK;
  a.out = out;
  a.out_dtype = out_dtype;
  a.out_row_stride = out_row_stride;
  const uintptr_t mis = reinterpret_cast<uintptr_t>(workspace) % 16;
  if (mis % 4) return KNLP_ERR_STRIDE;
  if (mis) {
    workspace += (16 - mis) / 4;
    workspace_floats -= (16 - mis) / 4;
  }
  rc = launch_decode_dq(a, workspace, workspace_floats, counters, counter_ints, max_len, emit,
                        sm_count(), nullptr, true, static_cast<cudaStream_t>(stream));
  // only layouts of the balanced tensor-core kernel are served
  return rc > 0 ? KNLP_ERR_STRIDE : rc;
}

int knlp_b200_lowrank_decode_workspace(int n_kv_heads, int n_q_per_kv, int n_tokens,
                                       int64_t* workspace_floats_out) {
  if (!workspace_floats_out) return KNLP_ERR_NULL;
  if (n_kv_heads <= 0 || n_q_per_kv <= 0 || n_q_per_kv > 8 || n_tokens < 0) return KNLP_ERR_SHAPE;
  *workspace_floats_out = lowrank_workspace_floats(n_kv_heads, n_q_per_kv, n_tokens, sm_count());
  return KNLP_OK;
}

int knlp_b200_lowrank_decode(const void* query, const void* key, int qk_dtype, const float* proj,
                             const float* basis, int n_kv_heads, int n_q_per_kv, int n_tokens,
                             int head_dim, int rank, float* workspace, int64_t workspace_floats,
                             float* za_out, float* out, void* stream) {
  if (!query || !key || !proj || !basis || !workspace || !out) return KNLP_ERR_NULL;
  if (qk_dtype != KNLP_F16 && qk_dtype != KNLP_BF16) return KNLP_ERR_DTYPE;
  if (n_kv_heads <= 0 || n_kv_heads > 65535 || n_q_per_kv <= 0 || n_q_per_kv > 8 || n_tokens < 1)
    return KNLP_ERR_SHAPE;
  if ((head_dim != 64 && head_dim != 128) || rank != 32) return KNLP_ERR_SHAPE;
  const uintptr_t al = reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(key) |
                       reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(basis);
  if (al % 16) return KNLP_ERR_STRIDE;  // rows are copied and read in 16-byte pieces
  return launch_lowrank_decode(query, key, qk_dtype, proj, basis, n_kv_heads, n_q_per_kv, n_tokens,
                               head_dim, sm_count(), workspace, workspace_floats, za_out, out,
                               static_cast<cudaStream_t>(stream));
}

int knlp_b200_combine(const float* part_m, const float* part_l, const float* part_o,
                      int n_parts, int64_t ml_row_stride, int64_t ml_part_stride,
                      int64_t o_row_stride, int64_t o_part_stride, void* out, int out_dtype,
                      int64_t out_row_stride, float* out_m, float* out_l,
                      int64_t out_ml_stride, int n_rows, int head_dim, void* stream) {
  if (!part_m || !part_l || !part_o || !out) return KNLP_ERR_NULL;
  if ((out_m == nullptr) != (out_l == nullptr)) return KNLP_ERR_NULL;
  if (!dtype_ok(out_dtype)) return KNLP_ERR_DTYPE;
  if (out_m && out_dtype != KNLP_F32) return KNLP_ERR_DTYPE;
  if (n_parts < 1 || n_rows < 0 || head_dim <= 0) return KNLP_ERR_SHAPE;
  return launch_combine(part_m, part_l, part_o, n_parts, ml_row_stride, ml_part_stride,
                        o_row_stride, o_part_stride, out, out_dtype, out_row_stride, out_m,
                        out_l, out_ml_stride, n_rows, head_dim,
                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
