/*
 * knlp_b200 — C ABI of the B200 (sm_100a) packed-KV-cache hot path.
 *
 * Device operations and their helpers:
 *   quant_append      quantize new K/V tokens and scatter them into the paged cache
 *   decode_attention  GQA decode attention over the packed cache, balanced inside one launch
 *   decode_splitk     the same with a fixed split count, emitting (m, l, o) softmax
 *                     partials per (sequence, q head, split)
 *   combine           merge partials into the attention output (or into one partial)
 *
 * Every entry point is plain C: raw device pointers, sizes, strides and a
 * cudaStream_t passed as void*.  Nothing here allocates or synchronises except
 * where a comment says so; all launches go to the given stream, so the calls are
 * stream-ordered and (knlp_b200_decode_noalloc aside, which carries its own notes)
 * capturable.  Return value: 0 on success, a negative
 * knlp_status on an argument error detected on the host before any launch.
 *
 * Threads and devices: every entry point works on the CURRENT device of the calling
 * thread and may be called from several host threads at once (the library's own
 * per-device state is atomic or mutex-protected).  Calls that share a workspace,
 * counters or a cache region they write must be ordered by the caller, as any two
 * kernels on different streams.
 *
 * Reference interfaces replaced (mcgrof/knlp, fused-quant/fused_int4.v0.1.0.py):
 *   reshape_and_cache_int4          :418-472   -> knlp_b200_quant_append
 *   reshape_and_cache_v_only_int4   :603-647   -> knlp_b200_quant_append (K plane NULL)
 *   reshape_and_cache_k_int8        :1287-1312 -> knlp_b200_quant_append (K mode INT8_G32)
 *   fused_int4_decode               :901-979   -> knlp_b200_decode_attention
 *                                                 (or knlp_b200_decode_splitk + knlp_b200_combine)
 *   kint8_vint4_decode              :1496-1554 -> same, K mode INT8_G32
 *   reshape_and_cache_v_int8        :1619-1645 -> knlp_b200_quant_append (V mode INT8_G32)
 *   kint8_vint8_decode              :1796-1843 -> decode entry points, both modes INT8_G32
 *   kfp16_vint4_decode              :1159-1224 -> decode entry points, K mode F16 / BF16
 *   kfp16_vint8_decode              :1975-2028 -> same, V mode INT8_G32
 * Cache layouts are the reference's (:213-223): codes [num_blocks, block_size,
 * num_kv_heads, head_size/2] uint8 (INT4; element 2j in the low nibble of byte j)
 * or [.., head_size] int8 (INT8); scales and zeros [.., head_size/32] fp16.
 */
#ifndef KNLP_B200_H_
#define KNLP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KNLP_B200_ABI_VERSION 2
#define KNLP_GROUP_SIZE 32

typedef enum {
  KNLP_OK = 0,
  KNLP_ERR_NULL = -1,       /* a required pointer is NULL */
  KNLP_ERR_SHAPE = -2,      /* unsupported head_dim / head counts / sizes */
  KNLP_ERR_DTYPE = -3,      /* unknown dtype code */
  KNLP_ERR_MODE = -4,       /* unknown or unsupported K/V mode combination */
  KNLP_ERR_STRIDE = -5,     /* stride or alignment the kernels cannot address */
  KNLP_ERR_WORKSPACE = -6,  /* n_splits / workspace arguments out of range */
  KNLP_ERR_LAUNCH = -7,     /* the CUDA runtime refused the launch */
  KNLP_ERR_NO_DEVICE = -8,  /* no usable sm_100 device / kernel image */
  KNLP_ERR_TOO_LARGE = -9   /* request exceeds a fixed capacity (see the entry point) */
} knlp_status;

typedef enum { KNLP_F32 = 0, KNLP_F16 = 1, KNLP_BF16 = 2 } knlp_dtype;

typedef enum {
  KNLP_KV_NONE = 0,      /* plane absent (skip) */
  KNLP_KV_INT4_SYM = 1,  /* offset-binary nibbles, scale only (reference :328-357) */
  KNLP_KV_INT4_ASYM = 2, /* unsigned nibbles, scale + zero (reference :308-327) */
  KNLP_KV_INT8_G32 = 3,  /* int8 codes, per-group-32 scale (reference :1270-1284) */
  /* Unquantized K plane of the hybrid decodes (reference kfp16_vint4_decode :1159-1224,
   * kfp16_vint8_decode :1975-2028): codes points to [.., head_size] fp16 or bf16 values,
   * codes_stride counts those 2-byte elements, scales / zeros are unused (may be NULL).
   * Decode only, K side only.  knlp_b200_decode_attention runs it on the tensor cores (head_dim
   * 64 / 128, heads of a token adjacent in memory, 16-byte aligned rows); the split-context
   * entry points and other layouts run the stride-generic kernel. */
  KNLP_KV_F16 = 4,
  KNLP_KV_BF16 = 5
} knlp_kv_mode;

/* One cache plane (K or V).  Strides are in ELEMENTS of the array they index
 * (bytes for codes, fp16 elements for scales/zeros), for the three outer
 * dimensions: [0] physical block, [1] token within the block, [2] kv head.
 * The innermost dimension must be contiguous. */
typedef struct {
  void* codes;
  void* scales;
  void* zeros; /* NULL unless mode == KNLP_KV_INT4_ASYM */
  int64_t codes_stride[3];
  int64_t scales_stride[3];
  int64_t zeros_stride[3];
  int32_t mode; /* knlp_kv_mode */
  int32_t reserved;
} knlp_kv_plane;

/* Flags for knlp_b200_decode_splitk. */
#define KNLP_DECODE_FORCE_GENERIC 1u /* use the stride-generic CUDA-core kernel */
#define KNLP_DECODE_USE_TMA 2u       /* stage with TMA tensor copies + mbarriers instead of cp.async */
/* Test aid, with KNLP_DECODE_USE_TMA only: the first stage of every CTA announces 16 bytes
 * more than it copies, so the bounded wait on it runs out (about 2 ms); the kernel then
 * writes empty partials, sets the status word read by knlp_b200_debug_status and returns.
 * It exercises the give-up path without any fault: every copy that is issued lands. */
#define KNLP_DECODE_DEBUG_STALL 16u

/* ABI version of the loaded library (KNLP_B200_ABI_VERSION at build time). */
int knlp_b200_abi_version(void);

/*
 * Debug aid, no counterpart in the reference.  The decode kernel bounds every
 * barrier wait (2 ms); if one ever runs out it sets a device-side status word, reports
 * the split as empty and ends (the attention output is then wrong, not garbage).  This
 * call SYNCHRONISES the current device, returns the word (0 = clean, 1 = a wait ran out,
 * -1 = could not be read) and clears it.  Not for use on a hot path or during capture.
 */
int knlp_b200_debug_status(void);

/* Static description of a knlp_status. */
const char* knlp_b200_strerror(int status);

/*
 * Quantize n_tokens new tokens and write them into the paged cache.
 * Replaces reshape_and_cache_int4 / _v_only_int4 / _k_int8 (see file header).
 *   key, value        [n_tokens, n_kv_heads, head_dim] of src_dtype; stride arrays give
 *                     the token and head strides in elements.  A NULL tensor or a NULL /
 *                     KNLP_KV_NONE plane skips that side.
 *   slot_mapping      int64 [n_tokens]; slot < 0 skips the token (reference :266-268);
 *                     block = slot / block_size, offset = slot % block_size.
 *   clip_ratio        outlier clip of the symmetric INT4 mode (reference :336-347);
 *                     <= 0 disables it.  Ignored by the other modes.
 * Arithmetic is IEEE fp32 with true division and round-half-away-from-zero, so
 * packed bytes, scales and zeros are bit-identical to the reference's.
 */
int knlp_b200_quant_append(const void* key, const int64_t key_stride[2],
                           const void* value, const int64_t value_stride[2],
                           int src_dtype,
                           const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                           const int64_t* slot_mapping,
                           int n_tokens, int n_kv_heads, int head_dim, int block_size,
                           float clip_ratio, void* stream);

/*
 * Recommend a split count for decode_splitk and report the workspace it needs.
 * Pure host arithmetic (queries the SM count of the current device once).
 *   n_splits_out          splits per sequence to pass to decode_splitk
 *   workspace_floats_out  floats needed for part_m + part_l + part_o together:
 *                         n_seqs * n_q_heads * n_splits * (head_dim + 2)
 */
int knlp_b200_decode_plan(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                          int block_size, int max_seq_len, int k_mode, int v_mode,
                          int* n_splits_out, int64_t* workspace_floats_out);

/*
 * Split-context decode attention over the packed cache.  Replaces the kernel
 * launch of fused_int4_decode / kint8_vint4_decode (see file header).
 *   query        [n_seqs, n_q_heads, head_dim] of q_dtype; q_stride = {seq, head} in elements
 *   block_table  int32 [n_seqs, *]; row stride bt_stride; entry i of a row is the
 *                physical block of tokens [i*block_size, (i+1)*block_size)
 *   seq_lens     int32 [n_seqs]; number of cached tokens to attend to (0 allowed)
 *   num_blocks   physical blocks in the cache; table entries are clamped to
 *                [0, num_blocks) before use, so a corrupt table cannot fault
 *   n_splits     >= 1.  Split i of a sequence covers tokens
 *                [i*chunk, min((i+1)*chunk, seq_len)), chunk = ceil(max_seq_len/n_splits)
 *                rounded up to a multiple of 64; the LAST split runs on to seq_len
 *   max_seq_len  bound of seq_lens known on the host.  It only sizes the splits: a
 *                sequence longer than it is still attended to in full (its last split
 *                is then longer than the others), so a bound given too small costs
 *                balance, never tokens
 *   part_m/l     float [n_seqs, n_q_heads, n_splits]   running max (natural-log domain,
 *                of the scaled scores) and sum of exp(s - m); empty split: -inf, 0
 *   part_o       float [n_seqs, n_q_heads, n_splits, head_dim]  UN-normalised sum p*v
 * The softmax scale is head_dim^-1/2, applied after the dot product (reference :805).
 */
int knlp_b200_decode_splitk(const void* query, int q_dtype, const int64_t q_stride[2],
                            const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                            const int32_t* block_table, int64_t bt_stride,
                            const int32_t* seq_lens, int64_t num_blocks,
                            int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                            int block_size, int n_splits, int max_seq_len,
                            float* part_m, float* part_l, float* part_o,
                            unsigned flags, void* stream);

/*
 * Workspace of knlp_b200_decode_attention for a decode shape: the number of floats and of
 * int32 counters it needs (host arithmetic; queries the SM count of the current device).
 * Both depend only on the arguments given here, so a caller sizes them once for its
 * largest batch.
 */
int knlp_b200_decode_workspace(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                               int block_size, int max_seq_len, int64_t* workspace_floats_out,
                               int64_t* counter_ints_out);

/*
 * Decode attention, the whole of fused_int4_decode / kint8_vint4_decode / kint8_vint8_decode
 * (reference :901-979, :1496-1554, :1796-1843): query and packed cache in, attention
 * output out.  Arguments as knlp_b200_decode_splitk, without a split count: the work is
 * balanced inside the launch (a persistent grid; the CTAs that serve one sequence and
 * block of kv heads share its tokens through a ticket counter and the one that finishes
 * last merges their partial softmax states).  One kernel launch for ordinary batches; a
 * second, dependent launch merges when one sequence is spread over most of the machine.
 *   workspace    floats, >= what knlp_b200_decode_workspace reports; contents are scratch
 *   counters     int32, >= what knlp_b200_decode_workspace reports, all ZERO on entry; the
 *                kernel leaves them zero, so one buffer zeroed once serves every later
 *                call on the same stream, whatever its shape (calls that may overlap on
 *                the GPU need separate workspace and counters)
 *   out          [n_seqs * n_q_heads, head_dim] of out_dtype, row stride out_row_stride
 *                elements: normalised attention output, 0 for sequences without tokens.
 *                With KNLP_DECODE_EMIT_PARTIAL: float rows of head_dim + 2 values
 *                [o un-normalised, m, l] (row stride out_row_stride >= head_dim + 2),
 *                the buffer a rank of a context shard sends in its one all-gather
 *   max_seq_len  host-known bound of seq_lens; sizes the grid only
 * Layouts that the tensor-core kernels cannot address (and the flags FORCE_GENERIC,
 * USE_TMA, FIXED_SPLITS) run knlp_b200_decode_splitk + knlp_b200_combine inside the same
 * workspace instead; the result is the same.
 */
#define KNLP_DECODE_EMIT_PARTIAL 4u /* out receives the merged partial, not the output */
#define KNLP_DECODE_FIXED_SPLITS 8u /* use the split-context kernel + combine */
int knlp_b200_decode_attention(const void* query, int q_dtype, const int64_t q_stride[2],
                               const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                               const int32_t* block_table, int64_t bt_stride,
                               const int32_t* seq_lens, int64_t num_blocks,
                               int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                               int block_size, int max_seq_len,
                               float* workspace, int64_t workspace_floats,
                               int32_t* counters, int64_t counter_ints,
                               void* out, int out_dtype, int64_t out_row_stride,
                               unsigned flags, void* stream);

/*
 * One decode step in ONE launch: append the step's new token of every sequence to the
 * packed cache AND attend over the cache including it.  Replaces the two launches of a
 * decode step of the reference, the cache write and the decode kernel
 * (FusedInt4AttentionImpl: do_kv_cache_update :2483-2546 / forward :2600-2689, then
 * _fused_decode :2851-2928); the idea is the reference's own, docs/fused-quant/latency.md:41.
 * Arguments as knlp_b200_decode_attention, plus
 *   new_tokens   key, value [n_seqs, n_kv_heads, head_dim] of dtype; strides {sequence,
 *                head} in elements, innermost dimension contiguous; clip_ratio as in
 *                knlp_b200_quant_append
 *   seq_lens     the lengths BEFORE the append.  Sequence s gets its token at position
 *                seq_lens[s] (block_table must already hold that position's block) and is
 *                attended to over seq_lens[s] + 1 tokens; the caller adds 1 to its lengths
 *                afterwards.  A sequence of length 0 attends to its new token alone.
 * The token is quantized with the arithmetic of knlp_b200_quant_append (the same device
 * function), so the stored bytes, scales and zeros are bit-identical to it; it takes part
 * in the attention as the dequantized values a later step reads back.  Only layouts the
 * balanced tensor-core kernel takes are supported: others return KNLP_ERR_STRIDE and
 * nothing is launched (use knlp_b200_quant_append + knlp_b200_decode_attention there).
 */
typedef struct {
  const void* key;
  const void* value;
  int64_t key_stride[2];
  int64_t value_stride[2];
  int32_t dtype; /* knlp_dtype */
  float clip_ratio;
} knlp_new_tokens;
int knlp_b200_decode_append_attention(const void* query, int q_dtype, const int64_t q_stride[2],
                                      const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                                      const int32_t* block_table, int64_t bt_stride,
                                      const int32_t* seq_lens, int64_t num_blocks,
                                      int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                                      int block_size, int max_seq_len,
                                      float* workspace, int64_t workspace_floats,
                                      int32_t* counters, int64_t counter_ints,
                                      void* out, int out_dtype, int64_t out_row_stride,
                                      unsigned flags, const knlp_new_tokens* new_tokens,
                                      void* stream);

/*
 * Routed (block-sparse) decode over the packed cache: every kv head of every sequence
 * attends to its OWN list of selected cache blocks, all tokens of a selected block count.
 * Same contract as fused_routed_decode of the reference (routing/fused_routed_attention.py
 * :425-492, kernel :45-190), which reads an unquantized cache; this one reads the packed
 * planes of this library through the loader of knlp_b200_decode_attention.
 *   block_tables  int32, row s * n_kv_heads + h (row stride bt_stride elements) lists the
 *                 selected physical blocks of kv head h of sequence s
 *   block_counts  int32 [n_seqs * n_kv_heads]: valid entries of each row (0: the q heads
 *                 of that kv head get zeros, as in the reference; counts above
 *                 max_selected_blocks are cut there, as the reference's loop bound does)
 *   query         [n_seqs, n_q_heads, head_dim], q_stride[0] == n_q_heads * q_stride[1]
 *   workspace / counters: as knlp_b200_decode_attention, sized by
 *                 knlp_b200_decode_workspace(n_seqs * n_kv_heads, n_q_heads / n_kv_heads, 1,
 *                 head_dim, block_size, max_selected_blocks * block_size, ...)
 *   flags         0 or KNLP_DECODE_EMIT_PARTIAL
 * One launch.  Only layouts the balanced tensor-core kernel addresses (head_dim 64 / 128,
 * block_size a power of two >= 16, both planes quantized): others return KNLP_ERR_STRIDE.
 */
int knlp_b200_routed_decode_attention(const void* query, int q_dtype, const int64_t q_stride[2],
                                      const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                                      const int32_t* block_tables, int64_t bt_stride,
                                      const int32_t* block_counts, int64_t num_blocks,
                                      int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                                      int block_size, int max_selected_blocks,
                                      float* workspace, int64_t workspace_floats,
                                      int32_t* counters, int64_t counter_ints,
                                      void* out, int out_dtype, int64_t out_row_stride,
                                      unsigned flags, void* stream);

/*
 * Low-rank-V decode attention: the value side is stored as rank-r coefficients
 * proj_i = B^T v_i with a per-head basis B, the weighted sum is taken in r dimensions and
 * lifted once: out = B (sum_i softmax(q.k_i / sqrt(d))_i proj_i).  Same contract as
 * lowrank_decode of the reference (pos_quant_v/kernel/vlowrank_kernel.py:139-156, kernel
 * _lowrank_decode :25-75, which leaves the lift to a torch.bmm): all tensors contiguous,
 *   query  [n_kv_heads, n_q_per_kv, head_dim]  fp16 or bf16 (qk_dtype), n_q_per_kv <= 8
 *   key    [n_kv_heads, n_tokens, head_dim]    the same dtype, unquantized
 *   proj   [n_kv_heads, n_tokens, rank]        fp32, rank = 32
 *   basis  [n_kv_heads, head_dim, rank]        fp32
 *   out    [n_kv_heads, n_q_per_kv, head_dim]  fp32; za_out (may be NULL): the coefficients
 *          before the lift, [n_kv_heads, n_q_per_kv, rank] fp32
 *   workspace: floats, >= what knlp_b200_lowrank_decode_workspace reports; scratch
 * head_dim 64 or 128; 16-byte aligned bases; n_tokens >= 1.  Two launches (split-context
 * kernel, finish).
 */
int knlp_b200_lowrank_decode_workspace(int n_kv_heads, int n_q_per_kv, int n_tokens,
                                       int64_t* workspace_floats_out);
int knlp_b200_lowrank_decode(const void* query, const void* key, int qk_dtype, const float* proj,
                             const float* basis, int n_kv_heads, int n_q_per_kv, int n_tokens,
                             int head_dim, int rank, float* workspace, int64_t workspace_floats,
                             float* za_out, float* out, void* stream);

/*
 * Merge n_parts partials per (sequence, q head) row.  No counterpart function
 * in the reference: the algebra is its in-loop online-softmax recurrence
 * (:808-815, :883-887) applied across splits.
 *   part_m/l     element (row, p) at row*ml_row_stride + p*ml_part_stride
 *   part_o       element (row, p, :) at row*o_row_stride + p*o_part_stride
 *   out          [n_rows, head_dim] with row stride out_row_stride (elements) of
 *                out_dtype: normalised attention output; rows with no tokens give 0
 *   out_m/out_l  if both non-NULL, the merged partial is emitted instead: out
 *                (must be KNLP_F32) receives the UN-normalised o, and row r's m and l
 *                go to out_m[r*out_ml_stride], out_l[r*out_ml_stride] — so one buffer
 *                of rows [o(head_dim), m, l] can be filled for a single all-gather
 */
int knlp_b200_combine(const float* part_m, const float* part_l, const float* part_o,
                      int n_parts, int64_t ml_row_stride, int64_t ml_part_stride,
                      int64_t o_row_stride, int64_t o_part_stride,
                      void* out, int out_dtype, int64_t out_row_stride,
                      float* out_m, float* out_l, int64_t out_ml_stride,
                      int n_rows, int head_dim, void* stream);

/*
 * Plugin-level simulated quantizers.  Replace the tensor expressions of
 * backends/quant.py: quantize_int8_symmetric (:23-35; group = dim, bits = 8),
 * quantize_int4_block (:43-72; group = block size, bits = 4, one code per int8, the
 * last block of a row may be partial), dequantize_int8_symmetric (:38-40) and
 * dequantize_int4_block (:75-86).
 *   x       [n_rows, dim] of dtype, rows contiguous
 *   q       int8 [n_rows, dim]
 *   scale   [n_rows, ceil(dim / group)] of the SAME dtype as x (as the reference returns)
 *   out     float [n_rows, dim] = q * scale
 * Arithmetic is carried out in x's dtype as the reference does (amax floor 1e-8, scale
 * and quotient each rounded to that dtype), integer rounding is half-to-even, so codes
 * and scales are bit-identical to the reference's.  A row that is all zero in fp16
 * (where the floor rounds to 0) is 0 / 0 in the reference, whose NaN converts to code 0;
 * here too its codes are 0 and its scale 0.
 */
int knlp_b200_plugin_quantize(const void* x, int dtype, int64_t n_rows, int dim, int group,
                              int bits, int8_t* q, void* scale, void* stream);
int knlp_b200_plugin_dequantize(const int8_t* q, const void* scale, int scale_dtype,
                                int64_t n_rows, int dim, int group, float* out, void* stream);

/*
 * Decode attention straight to the output, with NO device allocation by anyone.
 * It has no counterpart in the reference.  It exists for hosts that cannot hand
 * knlp_b200_decode_splitk a workspace: an engine that gave all device memory to its
 * own pool at start-up and may not call cudaMalloc any more, or a C / Go / Java
 * host without a device allocator.  The split partials live in a fixed array of
 * KNLP_NOALLOC_MAX_FLOATS floats (32 MiB) inside the library, present on every GPU
 * that loads it until the process exits.
 *   arguments   as knlp_b200_decode_splitk, plus the output of knlp_b200_combine:
 *               out [n_seqs * n_q_heads, head_dim] of out_dtype, row stride
 *               out_row_stride elements
 *   n_splits    > 0: used as given; <= 0: chosen by the library and reduced to what
 *               the fixed array holds
 *   limit       n_seqs * n_q_heads * n_splits * (head_dim + 2) must not exceed
 *               KNLP_NOALLOC_MAX_FLOATS, else KNLP_ERR_TOO_LARGE is returned and
 *               nothing is launched
 * The first call on a device looks up the array's device address (no allocation);
 * make that first call outside any stream capture.  All calls on a device share the
 * array: two calls whose kernels may overlap on the GPU (different streams) race on
 * it, so keep them on one stream or order them with events.  The array keeps the
 * last call's partials; every value a call reads it has written itself, so nothing
 * needs clearing in between.
 */
#define KNLP_NOALLOC_MAX_FLOATS (8ll << 20)
int knlp_b200_decode_noalloc(const void* query, int q_dtype, const int64_t q_stride[2],
                             const knlp_kv_plane* k_plane, const knlp_kv_plane* v_plane,
                             const int32_t* block_table, int64_t bt_stride,
                             const int32_t* seq_lens, int64_t num_blocks,
                             int n_seqs, int n_q_heads, int n_kv_heads, int head_dim,
                             int block_size, int n_splits, int max_seq_len,
                             void* out, int out_dtype, int64_t out_row_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KNLP_B200_H_ */
