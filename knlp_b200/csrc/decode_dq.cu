// Host side of the balanced one-launch decode (kernel: decode_dq_kernel.cuh): eligibility,
// grid and workspace arithmetic, dispatch to the instantiation of the K/V mode pair.

#include "decode_dq_kernel.cuh"

namespace knlp {

// Defined in decode_dq_inst_*.cu (one translation unit per mode pair).
#define KNLP_DECL_PAIR(K, V)                                                                     \
  extern template int launch_dq_pair<K, V>(const DecodeArgs&, const DqParams&, bool, cudaStream_t); \
  extern template int dq_chunk_of_pair<K, V>(int, int)
KNLP_DECL_PAIR(KNLP_KV_INT4_ASYM, KNLP_KV_INT4_ASYM);
KNLP_DECL_PAIR(KNLP_KV_INT4_SYM, KNLP_KV_INT4_SYM);
KNLP_DECL_PAIR(KNLP_KV_INT8_G32, KNLP_KV_INT4_ASYM);
KNLP_DECL_PAIR(KNLP_KV_INT8_G32, KNLP_KV_INT4_SYM);
KNLP_DECL_PAIR(KNLP_KV_INT8_G32, KNLP_KV_INT8_G32);
KNLP_DECL_PAIR(KNLP_KV_F16, KNLP_KV_INT4_ASYM);
KNLP_DECL_PAIR(KNLP_KV_F16, KNLP_KV_INT4_SYM);
KNLP_DECL_PAIR(KNLP_KV_F16, KNLP_KV_INT8_G32);
KNLP_DECL_PAIR(KNLP_KV_BF16, KNLP_KV_INT4_ASYM);
KNLP_DECL_PAIR(KNLP_KV_BF16, KNLP_KV_INT4_SYM);
KNLP_DECL_PAIR(KNLP_KV_BF16, KNLP_KV_INT8_G32);
#undef KNLP_DECL_PAIR

namespace {

constexpr int kRanks = kDecodeCtasPerSm;  // CTAs per SM = launch ranks that get interleaved

template <class F>
int with_pair(int km, int vm, F&& f) {
  if (km == KNLP_KV_INT4_ASYM && vm == KNLP_KV_INT4_ASYM)
    return f(std::integral_constant<int, KNLP_KV_INT4_ASYM>{},
             std::integral_constant<int, KNLP_KV_INT4_ASYM>{});
  if (km == KNLP_KV_INT4_SYM && vm == KNLP_KV_INT4_SYM)
    return f(std::integral_constant<int, KNLP_KV_INT4_SYM>{},
             std::integral_constant<int, KNLP_KV_INT4_SYM>{});
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT4_ASYM)
    return f(std::integral_constant<int, KNLP_KV_INT8_G32>{},
             std::integral_constant<int, KNLP_KV_INT4_ASYM>{});
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT4_SYM)
    return f(std::integral_constant<int, KNLP_KV_INT8_G32>{},
             std::integral_constant<int, KNLP_KV_INT4_SYM>{});
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT8_G32)
    return f(std::integral_constant<int, KNLP_KV_INT8_G32>{},
             std::integral_constant<int, KNLP_KV_INT8_G32>{});
  // an unquantized K plane (fp16 or bf16) against each V mode
  if (km == KNLP_KV_F16 || km == KNLP_KV_BF16) {
    auto with_v = [&](auto k) -> int {
      if (vm == KNLP_KV_INT4_ASYM) return f(k, std::integral_constant<int, KNLP_KV_INT4_ASYM>{});
      if (vm == KNLP_KV_INT4_SYM) return f(k, std::integral_constant<int, KNLP_KV_INT4_SYM>{});
      if (vm == KNLP_KV_INT8_G32) return f(k, std::integral_constant<int, KNLP_KV_INT8_G32>{});
      return -1000;
    };
    return km == KNLP_KV_F16 ? with_v(std::integral_constant<int, KNLP_KV_F16>{})
                             : with_v(std::integral_constant<int, KNLP_KV_BF16>{});
  }
  return -1000;  // no tensor-core instantiation for this pair
}

int heads_per_cta_log2(int n_kv_heads) {
  int l = kWarpsLog;
  while (l > 0 && (n_kv_heads % (1 << l))) --l;
  return l;
}

}  // namespace

void dq_workspace_size(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int n_sms,
                       int64_t* floats, int64_t* ints) {
  const int hpb = 1 << heads_per_cta_log2(n_kv_heads);
  const int64_t heads = static_cast<int64_t>(hpb) * (n_q_heads / n_kv_heads);
  const int64_t n_pairs = static_cast<int64_t>(n_seqs) * (n_kv_heads / hpb);
  const int64_t slots = static_cast<int64_t>(kRanks) * n_sms + n_pairs;
  // partial slots, then (first slot, parts) per pair for the merge kernel
  *floats = slots * heads * (head_dim + 2) + 2 * n_pairs;
  *ints = 2 * n_pairs;  // ticket and arrival counters
}

int launch_decode_dq(const DecodeArgs& a_in, float* ws, int64_t ws_floats, int* ints,
                     int64_t n_ints, int max_seq_len, bool emit_partial, int n_sms,
                     const knlp_new_tokens* nt, bool per_head_tables, cudaStream_t st) {
  DqParams dp{};
  dp.len_cap = 0x7fffffff;
  if (decode_mma_layout(a_in, &dp.hpb_log2, &dp.page_log2)) return 1;
  DecodeArgs a = a_in;
  if (per_head_tables) {
    // Every (sequence, kv head) becomes a sequence of its own with one kv head: row
    // s * n_kv_heads + h of the tables, of the lengths (given in blocks), of q and of out.
    if (nt) return KNLP_ERR_MODE;
    const int n_rep = a.n_q_heads / a.n_kv_heads;
    if (a.q_stride[0] != static_cast<int64_t>(a.n_q_heads) * a.q_stride[1]) return 1;
    if (static_cast<int64_t>(a.n_seqs) * a.n_kv_heads > 0x7fffffff) return 1;
    dp.vheads = a.n_kv_heads;
    dp.len_cap = max_seq_len;  // = the blocks a table row holds: larger counts are cut there
    dp.hpb_log2 = 0;
    a.n_seqs *= a.n_kv_heads;
    a.n_q_heads = n_rep;
    a.n_kv_heads = 1;
    a.q_stride[0] = n_rep * a.q_stride[1];
  }
  // q rows are fetched with 16-byte loads
  const int q_align = a.q_dtype == KNLP_F32 ? 4 : 8;
  if (reinterpret_cast<uintptr_t>(a.q) % 16 || a.q_stride[0] % q_align || a.q_stride[1] % q_align)
    return 1;
  const int ct = with_pair(a.k.mode, a.v.mode, [&](auto k, auto v) {
    return dq_chunk_of_pair<decltype(k)::value, decltype(v)::value>(a.head_dim, dp.hpb_log2);
  });
  if (ct <= 0) return 1;
  // the page-id ring holds 32 ids per chunk (a chunk that starts inside a page touches one more)
  if ((ct >> dp.page_log2) + 1 > 32) return 1;
  const int hpb = 1 << dp.hpb_log2;
  const int n_rep = a.n_q_heads / a.n_kv_heads;
  const int64_t heads = static_cast<int64_t>(hpb) * n_rep;
  const int64_t n_pairs = static_cast<int64_t>(a.n_seqs) * (a.n_kv_heads / hpb);
  // positions in the chunk sequence are 32-bit in the kernel
  const int64_t bound_chunks = n_pairs * ((static_cast<int64_t>(max_seq_len) + ct - 1) / ct);
  if (bound_chunks >= (1ll << 30) || n_pairs >= (1ll << 28)) return 1;
  int64_t g = static_cast<int64_t>(kRanks) * n_sms;
  if (bound_chunks < g) g = (bound_chunks + kRanks - 1) / kRanks * kRanks;
  if (g < kRanks) g = kRanks;
  dp.n_ranks = kRanks;
  dp.n_cols = static_cast<int>(g / kRanks);
  const int64_t slots = g + n_pairs;
  if (!ws || !ints || ws_floats < slots * heads * (a.head_dim + 2) + 2 * n_pairs ||
      n_ints < 2 * n_pairs)
    return KNLP_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(ws) % 16) return KNLP_ERR_STRIDE;  // merged as float4
  dp.ws_o = ws;
  dp.ws_m = ws + slots * heads * a.head_dim;
  dp.ws_l = dp.ws_m + slots * heads;
  dp.counters = ints;
  // scratch like the partials: nothing of it has to survive the call
  dp.pair_info = reinterpret_cast<int*>(dp.ws_l + slots * heads);
  // With few members per pair the member that arrives last merges them; a pair with many
  // members (one long sequence on the whole machine) is merged by a second, parallel launch.
  dp.fuse = g <= 32 * n_pairs ? 1 : 0;
  dp.emit_partial = emit_partial ? 1 : 0;
  if (nt) {
    dp.new_key = nt->key;
    dp.new_value = nt->value;
    for (int i = 0; i < 2; ++i) {
      dp.nk_stride[i] = nt->key_stride[i];
      dp.nv_stride[i] = nt->value_stride[i];
    }
    dp.new_dtype = nt->dtype;
    dp.clip_ratio = nt->clip_ratio;
  }
  const bool split = n_rep <= 4;
  // bf16 K with one column per head: q enters the product as a single bf16, which is exact
  // only for bf16 queries
  if (a.k.mode == KNLP_KV_BF16 && !split && a.q_dtype != KNLP_BF16) return 1;
  const int rc = with_pair(a.k.mode, a.v.mode, [&](auto k, auto v) {
    return launch_dq_pair<decltype(k)::value, decltype(v)::value>(a, dp, split, st);
  });
  if (rc != KNLP_OK || dp.fuse) return rc;
  return launch_combine_pairs(dp.ws_m, dp.ws_l, dp.ws_o, dp.pair_info, static_cast<int>(heads),
                              a.n_seqs * a.n_q_heads, a.head_dim, a.out, a.out_dtype,
                              a.out_row_stride, emit_partial, st);
}

}  // namespace knlp
