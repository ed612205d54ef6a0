// Balanced GQA decode attention over the packed KV cache in one launch (sm_100a).
//
// Same math and staging as the split-context kernel of decode_mma_kernel.cuh (tokens on
// the M side of m16n8k16 MMAs, codes entering as fp16 subnormals, cp.async stages, scale
// and zero-point folded per group outside the MMA); what differs is who does which
// tokens.  The split-context kernel cuts every sequence into the same number of fixed
// splits, one CTA each.  That leaves the machine idle where it hurts in short launches:
// the last split is short, the grid rarely fills the last wave, ragged batches leave most
// CTAs of short sequences empty, and the CTAs that share an SM do not progress at the same
// rate (the hardware favours the CTAs launched first), so a one-wave launch ends in a
// long tail.  Here the grid is persistent (four CTAs per SM) and the work is handed out
// in two levels:
//   1. static, proportional: the chunks (kStages stages = 48..256 tokens) of all
//      (sequence, head block) pairs form one sequence; CTA i is given the i-th equal
//      share of it, which makes it a member of the group of every pair its share touches;
//   2. dynamic, inside a pair: the members of a pair's group take its chunks from a
//      ticket counter, so a CTA that runs faster simply takes more of them and all
//      members finish within a chunk or two of each other.
// The accumulators of the online softmax do not care which chunks they saw, so a CTA
// writes ONE partial (m, l, o) per pair whatever it processed.  Logical CTA ids are
// interleaved so that the members of a group sit in different launch ranks of their SMs.
// Tickets are taken two chunks ahead of use, the page ids of a chunk one chunk ahead;
// nothing in the loop waits on a global load or an atomic, and no CTA waits on another.
//
// The merge of a pair's partials is done by the member that arrives last (counted with
// an atomic after a fence), straight into the output; with many members per pair the
// host asks for the partials only and runs the combine kernel on them.
//
// Variants of the same kernel: K modes INT4 (sym / asym), INT8 and unquantized fp16 / bf16
// (the K tile is then the MMA's A operand as it lies in memory, bf16 through the bf16 MMA
// with q split into two bf16 parts); V modes INT4 and INT8; the step's new token appended
// by the pair's last member (append_token); per-kv-head page tables for routed decode
// (instantiation ROUTED: one kv head per CTA, scale rows fetched per (token, head)).

#pragma once

#include <atomic>

#include "decode_mma_common.cuh"
#include "quant_row.cuh"

namespace knlp {

// Launch parameters of the balanced kernel computed on the host.
struct DqParams {
  int hpb_log2;    // kv heads per CTA = 1 << hpb_log2
  int page_log2;   // block_size = 1 << page_log2
  int n_cols;      // gridDim.x = n_ranks * n_cols; CTA b is column b % n_cols, rank b / n_cols
  int n_ranks;
  float* ws_o;     // partial slots [n_slots][heads of a pair][head_dim], un-normalised
  float* ws_m;     // [n_slots][heads of a pair], natural-log domain
  float* ws_l;
  int* counters;   // [2 * n_pairs]: chunk tickets, arrivals; zero on entry, left zero
  int* pair_info;  // [2 * n_pairs]: first slot and number of parts (for the combine kernel)
  int fuse;        // 1: the last member of a pair merges its parts into a.out
  int emit_partial;  // fused merge writes fp32 rows [o (un-normalised), m, l] instead
  // The step's new token, appended inside the launch (new_key == nullptr: none):
  // [n_seqs, n_kv_heads, head_dim] of new_dtype, strides {sequence, head} in elements.
  // It is quantized into the cache at position seq_lens[s] and attended to as well.
  const void* new_key;
  const void* new_value;
  int64_t nk_stride[2], nv_stride[2];
  int new_dtype;
  float clip_ratio;
  // Per-kv-head page tables (routed decode).  vheads > 0: the launch sees every (sequence,
  // kv head) as a sequence of its own with ONE kv head - row v of block_table / seq_lens /
  // query / out belongs to kv head v % vheads of a cache that holds vheads heads per token
  // (heads per CTA is 1 then), seq_lens count whole blocks, and lengths are cut at len_cap
  // tokens (a table row holds no more blocks).
  int vheads;
  int len_cap;
};

namespace {

// The 8 q elements of every group that one thread's B fragments need, as fp32: element
// slot e of group g is 32g + 8*quad + e (runs of 8; RUNS4 = false) or 32g + 16(e>>2) +
// 4*quad + (e&3) (two runs of 4; RUNS4 = true).  All vector loads are issued before the
// first conversion so that they are in flight together.
template <int NG, bool RUNS4>
__device__ __forceinline__ void load_q_groups(const void* base, int64_t row, int quad, int dt,
                                              float out[NG][8]) {
  if (dt == KNLP_F32) {
    const float* p = static_cast<const float*>(base) + row;
    float4 v[NG][2];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const float* q0 = p + 32 * g + (RUNS4 ? 4 * quad : 8 * quad);
      v[g][0] = __ldg(reinterpret_cast<const float4*>(q0));
      v[g][1] = __ldg(reinterpret_cast<const float4*>(q0 + (RUNS4 ? 16 : 4)));
    }
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      out[g][0] = v[g][0].x; out[g][1] = v[g][0].y; out[g][2] = v[g][0].z; out[g][3] = v[g][0].w;
      out[g][4] = v[g][1].x; out[g][5] = v[g][1].y; out[g][6] = v[g][1].z; out[g][7] = v[g][1].w;
    }
    return;
  }
  const uint16_t* p = static_cast<const uint16_t*>(base) + row;
  uint32_t w[NG][4];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    if constexpr (RUNS4) {
      const uint2 a0 = __ldg(reinterpret_cast<const uint2*>(p + 32 * g + 4 * quad));
      const uint2 a1 = __ldg(reinterpret_cast<const uint2*>(p + 32 * g + 16 + 4 * quad));
      w[g][0] = a0.x; w[g][1] = a0.y; w[g][2] = a1.x; w[g][3] = a1.y;
    } else {
      const uint4 a0 = __ldg(reinterpret_cast<const uint4*>(p + 32 * g + 8 * quad));
      w[g][0] = a0.x; w[g][1] = a0.y; w[g][2] = a0.z; w[g][3] = a0.w;
    }
  }
  const bool f16 = dt == KNLP_F16;
#pragma unroll
  for (int g = 0; g < NG; ++g) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[g][i]));
      // bf16 is the upper half of an fp32
      out[g][2 * i] = f16 ? f.x : __uint_as_float(w[g][i] << 16);
      out[g][2 * i + 1] = f16 ? f.y : __uint_as_float(w[g][i] & 0xFFFF0000u);
    }
  }
}

// The same for an unquantized K plane, whose tile is the A operand as it lies in memory:
// slot (2i, 2i + 1) of group g is the element pair 32g + 8i + 2*quad (+1), i = 0..3 - the
// B fragment rows of the two 16-wide steps of the group.
template <int NG>
__device__ __forceinline__ void load_q_pairs(const void* base, int64_t row, int quad, int dt,
                                             float out[NG][8]) {
  if (dt == KNLP_F32) {
    const float* p = static_cast<const float*>(base) + row + 2 * quad;
    float2 v[NG][4];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) v[g][i] = __ldg(reinterpret_cast<const float2*>(p + 32 * g + 8 * i));
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[g][2 * i] = v[g][i].x;
        out[g][2 * i + 1] = v[g][i].y;
      }
    return;
  }
  const uint16_t* p = static_cast<const uint16_t*>(base) + row + 2 * quad;
  uint32_t w[NG][4];
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i) w[g][i] = __ldg(reinterpret_cast<const uint32_t*>(p + 32 * g + 8 * i));
  const bool f16 = dt == KNLP_F16;
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[g][i]));
      out[g][2 * i] = f16 ? f.x : __uint_as_float(w[g][i] << 16);
      out[g][2 * i + 1] = f16 ? f.y : __uint_as_float(w[g][i] & 0xFFFF0000u);
    }
}

// The weights of a pair's parts, w_p = l_p e^(m_p - m) / sum_q l_q e^(m_q - m), into
// sw[row * tile + p] (parts <= 32; emit_partial: not normalised, and m and the sum go out
// with the row).  Ends before the barrier that makes them visible.
template <int HD>
__device__ __forceinline__ void merge_weights(const float* pm, const float* pl, const int parts,
                                              const int heads, float* sw, const int tile,
                                              void* out, const int64_t out_row_stride,
                                              const int64_t row0, const int emit_partial) {
  const int tid = threadIdx.x;
  // Four warps run here and nothing hides a round trip to L2 but more
  // loads in flight, so the (row, part) pairs are spread over all 128 threads - thread =
  // (part group j, row), rows fastest, so that the m / l loads of a part coalesce over
  // its heads - every thread's loads are issued together, and the two reductions over
  // the parts go through shared memory instead of dependent loads or shuffles.
  int hp_log = 2;  // rows padded to a power of two, at least 4: at most 32 part groups
  while ((1 << hp_log) < heads) ++hp_log;
  const int hp = 1 << hp_log, n_grp = kThreads >> hp_log;
  const int row = tid & (hp - 1), j = tid >> hp_log;
  const bool row_ok = row < heads;
  float* const red = sw + ((heads * tile + 3) & ~3);  // behind the weights
  constexpr int kPer = 8;  // parts per thread: 32 parts over at least 4 groups
  float lv[kPer], mv[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int p = j + i * n_grp;
    const bool ok = row_ok && p < parts;
    lv[i] = ok ? __ldcg(pl + p * heads + row) : 0.0f;
    mv[i] = ok ? __ldcg(pm + p * heads + row) : -INFINITY;
  }
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPer; ++i) mx = fmaxf(mx, lv[i] > 0.0f ? mv[i] : -INFINITY);
  red[tid] = mx;
  __syncthreads();
  for (int g = 0; g < n_grp; ++g) mx = fmaxf(mx, red[(g << hp_log) + row]);
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    mv[i] = lv[i] > 0.0f ? __expf(mv[i] - mx) : 0.0f;
    sum = fmaf(lv[i], mv[i], sum);
  }
  red[kThreads + tid] = sum;
  __syncthreads();
  sum = 0.0f;
  for (int g = 0; g < n_grp; ++g) sum += red[kThreads + (g << hp_log) + row];
  const float inv = emit_partial ? 1.0f : (sum > 0.0f ? 1.0f / sum : 0.0f);
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int p = j + i * n_grp;
    if (row_ok && p < parts) sw[row * tile + p] = mv[i] * inv;
  }
  if (emit_partial && j == 0 && row_ok) {
    float* orow = static_cast<float*>(out) + (row0 + row) * out_row_stride;
    orow[HD] = mx;
    orow[HD + 1] = sum;
  }
}

// Second half of merge_pair: a thread owns ITEMS (row, four elements) items and keeps
// their sums; the partial outputs are fetched kBatch parts of every item at a time, all
// those loads independent of each other (about 20 vector loads in flight per thread: the
// partials sit in L2, and a dependent round of loads costs over a microsecond while the
// rest of the machine streams).
template <int HD, int ITEMS>
__device__ __forceinline__ void merge_rows(const float* pm, const float* pl, const float* po,
                                           const int parts, const int heads, float* sw,
                                           const int tile, const bool one_pass,
                                           const float* s_mrow, const float* s_irow, void* out,
                                           const int out_dtype, const int64_t out_row_stride,
                                           const int64_t row0, const int emit_partial) {
  const int tid = threadIdx.x;
  constexpr int kVec = HD / 4;
  constexpr int kBatch = ITEMS >= 10 ? 2 : 20 / ITEMS;
  const float4* po4 = reinterpret_cast<const float4*>(po);
  float4 acc[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) acc[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int p0 = 0; p0 < parts; p0 += tile) {
    const int np = min(tile, parts - p0);
    if (!one_pass) {
      __syncthreads();  // the previous tile's weights are no longer read
      for (int i = tid; i < heads * np; i += kThreads) {
        const int r = i / np, p = p0 + i % np;
        const float l1 = __ldcg(pl + p * heads + r);
        sw[r * tile + (p - p0)] =
            l1 > 0.0f ? __expf(__ldcg(pm + p * heads + r) - s_mrow[r]) * s_irow[r] : 0.0f;
      }
      __syncthreads();
    }
    for (int pb = 0; pb < np; pb += kBatch) {
      float4 v[ITEMS][kBatch];
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const int i = tid + k * kThreads;
        const int r = i / kVec, e4 = i % kVec;
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
          // a member that saw no token wrote zeros, so no value needs skipping
          const bool valid = i < heads * kVec && pb + q < np;
          v[k][q] = valid ? __ldcg(po4 + (static_cast<int64_t>(p0 + pb + q) * heads + r) * kVec + e4)
                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
      }
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const int i = tid + k * kThreads;
        const int r = min(i / kVec, heads - 1);
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
          const float wgt = pb + q < np ? sw[r * tile + pb + q] : 0.0f;
          acc[k].x = fmaf(v[k][q].x, wgt, acc[k].x);
          acc[k].y = fmaf(v[k][q].y, wgt, acc[k].y);
          acc[k].z = fmaf(v[k][q].z, wgt, acc[k].z);
          acc[k].w = fmaf(v[k][q].w, wgt, acc[k].w);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = tid + k * kThreads;
    if (i < heads * kVec) {
      const int r = i / kVec, e4 = i % kVec;
      const int64_t o = (row0 + r) * out_row_stride + 4 * e4;
      if (emit_partial) {
        float* orow = static_cast<float*>(out) + o;
        orow[0] = acc[k].x; orow[1] = acc[k].y; orow[2] = acc[k].z; orow[3] = acc[k].w;
      } else {
        store_elem_rt(out, o, acc[k].x, out_dtype);
        store_elem_rt(out, o + 1, acc[k].y, out_dtype);
        store_elem_rt(out, o + 2, acc[k].z, out_dtype);
        store_elem_rt(out, o + 3, acc[k].w, out_dtype);
      }
    }
  }
}

// The whole merge of a pair with at most 32 parts.  The first batch of partial outputs is
// fetched BEFORE the weights are worked out (the loads do not depend on them), so its round
// trip to L2 runs under the weights' own.
template <int HD, int ITEMS>
__device__ __forceinline__ void merge_one_pass(const float* pm, const float* pl, const float* po,
                                               const int parts, const int heads, float* sw,
                                               const int tile, void* out, const int out_dtype,
                                               const int64_t out_row_stride, const int64_t row0,
                                               const int emit_partial) {
  const int tid = threadIdx.x;
  constexpr int kVec = HD / 4;
  constexpr int kBatch = ITEMS >= 10 ? 2 : 20 / ITEMS;
  const int part4 = heads * kVec;  // float4 items of one part
  const float4* po4 = reinterpret_cast<const float4*>(po) + tid;
  float4 acc[ITEMS], v[ITEMS][kBatch];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) acc[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  auto fetch = [&](const int pb) {
#pragma unroll
    for (int q = 0; q < kBatch; ++q) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        // a member that saw no token wrote zeros, so no value needs skipping
        const bool valid = tid + k * kThreads < part4 && pb + q < parts;
        v[k][q] = valid ? __ldcg(po4 + (static_cast<int64_t>(pb + q) * part4 + k * kThreads))
                        : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
  };
  auto add = [&](const int pb) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const float* wr = sw + min((tid + k * kThreads) / kVec, heads - 1) * tile + pb;
#pragma unroll
      for (int q = 0; q < kBatch; ++q) {
        const float wgt = pb + q < parts ? wr[q] : 0.0f;
        acc[k].x = fmaf(v[k][q].x, wgt, acc[k].x);
        acc[k].y = fmaf(v[k][q].y, wgt, acc[k].y);
        acc[k].z = fmaf(v[k][q].z, wgt, acc[k].z);
        acc[k].w = fmaf(v[k][q].w, wgt, acc[k].w);
      }
    }
  };
  fetch(0);
  merge_weights<HD>(pm, pl, parts, heads, sw, tile, out, out_row_stride, row0, emit_partial);
  __syncthreads();
  add(0);
  for (int pb = kBatch; pb < parts; pb += kBatch) {
    fetch(pb);
    add(pb);
  }
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = tid + k * kThreads;
    if (i < part4) {
      const int r = i / kVec, e4 = i % kVec;
      const int64_t o = (row0 + r) * out_row_stride + 4 * e4;
      if (emit_partial) {
        float* orow = static_cast<float*>(out) + o;
        orow[0] = acc[k].x; orow[1] = acc[k].y; orow[2] = acc[k].z; orow[3] = acc[k].w;
      } else {
        store_elem_rt(out, o, acc[k].x, out_dtype);
        store_elem_rt(out, o + 1, acc[k].y, out_dtype);
        store_elem_rt(out, o + 2, acc[k].z, out_dtype);
        store_elem_rt(out, o + 3, acc[k].w, out_dtype);
      }
    }
  }
}

// Merge of the partials of one pair by the CTA that arrived last: out[row] = sum_p w_p o_p
// with w_p = l_p e^(m_p - m) / sum_q l_q e^(m_q - m).  pm, pl: [parts][heads]; po: [parts]
// [heads][HD]; sw: shared-memory scratch of sw_floats floats; s_mrow, s_irow: MAXH floats
// of shared memory.  Kept out of line so that its registers are not the main loop's.
template <int HD, int MAXH>
__device__ __noinline__ void merge_pair(const float* pm, const float* pl, const float* po,
                                        const int parts, const int heads, float* sw,
                                        const int sw_floats, float* s_mrow, float* s_irow,
                                        void* out, const int out_dtype,
                                        const int64_t out_row_stride, const int64_t row0,
                                        const int emit_partial) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = min(parts, sw_floats / heads);
  const bool one_pass = parts <= 32 && parts <= tile;
  if (one_pass) {
    const int n_items = (heads * (HD / 4) + kThreads - 1) / kThreads;
    constexpr int kMaxItems = (MAXH * (HD / 4) + kThreads - 1) / kThreads;
    if (n_items <= 1) {
      merge_one_pass<HD, 1>(pm, pl, po, parts, heads, sw, tile, out, out_dtype, out_row_stride,
                            row0, emit_partial);
    } else if (n_items <= 2) {
      merge_one_pass<HD, 2>(pm, pl, po, parts, heads, sw, tile, out, out_dtype, out_row_stride,
                            row0, emit_partial);
    } else if (n_items <= 4 || kMaxItems <= 4) {
      merge_one_pass<HD, 4>(pm, pl, po, parts, heads, sw, tile, out, out_dtype, out_row_stride,
                            row0, emit_partial);
    } else {
      merge_one_pass<HD, kMaxItems>(pm, pl, po, parts, heads, sw, tile, out, out_dtype,
                                    out_row_stride, row0, emit_partial);
    }
    return;
  }
  {
    constexpr int kRowsW = MAXH / kWarpsCta;
    float rm[kRowsW], rl[kRowsW], lp[kRowsW], mp[kRowsW];
#pragma unroll
    for (int k = 0; k < kRowsW; ++k) {
      rm[k] = -INFINITY;
      rl[k] = 0.0f;
    }
    for (int p0 = 0; p0 < parts; p0 += 32) {
#pragma unroll
      for (int k = 0; k < kRowsW; ++k) {
        const int r = warp + k * kWarpsCta;
        const bool valid = r < heads && p0 + lane < parts;
        lp[k] = valid ? __ldcg(pl + (p0 + lane) * heads + r) : 0.0f;
        mp[k] = valid ? __ldcg(pm + (p0 + lane) * heads + r) : -INFINITY;
      }
#pragma unroll
      for (int k = 0; k < kRowsW; ++k) {
        float mx = lp[k] > 0.0f ? mp[k] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(rm[k], mx);
        float sum = lp[k] > 0.0f ? lp[k] * __expf(mp[k] - m_new) : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        rl[k] = (rl[k] > 0.0f ? rl[k] * __expf(rm[k] - m_new) : 0.0f) + sum;
        rm[k] = m_new;
      }
    }
#pragma unroll
    for (int k = 0; k < kRowsW; ++k) {
      const int r = warp + k * kWarpsCta;
      const float inv = emit_partial ? 1.0f : (rl[k] > 0.0f ? 1.0f / rl[k] : 0.0f);
      if (one_pass && r < heads && lane < parts)
        sw[r * tile + lane] = lp[k] > 0.0f ? __expf(mp[k] - rm[k]) * inv : 0.0f;
      if (lane == 0 && r < heads) {
        s_mrow[r] = rm[k];
        s_irow[r] = inv;
        if (emit_partial) {
          float* orow = static_cast<float*>(out) + (row0 + r) * out_row_stride;
          orow[HD] = rm[k];
          orow[HD + 1] = rl[k];
        }
      }
    }
  }
  __syncthreads();
  // (2) out[row] = sum_p w_p o_p, with as many (row, four elements) items per thread as
  // the pair really has heads: the fewer items, the more parts are fetched at once.
  const int items = (heads * (HD / 4) + kThreads - 1) / kThreads;
  if (items <= 1) {
    merge_rows<HD, 1>(pm, pl, po, parts, heads, sw, tile, one_pass, s_mrow, s_irow, out,
                      out_dtype, out_row_stride, row0, emit_partial);
  } else if (items <= 2) {
    merge_rows<HD, 2>(pm, pl, po, parts, heads, sw, tile, one_pass, s_mrow, s_irow, out,
                      out_dtype, out_row_stride, row0, emit_partial);
  } else if (items <= 4 || MAXH * (HD / 4) <= 4 * kThreads) {
    merge_rows<HD, 4>(pm, pl, po, parts, heads, sw, tile, one_pass, s_mrow, s_irow, out,
                      out_dtype, out_row_stride, row0, emit_partial);
  } else {
    merge_rows<HD, (MAXH * (HD / 4) + kThreads - 1) / kThreads>(
        pm, pl, po, parts, heads, sw, tile, one_pass, s_mrow, s_irow, out, out_dtype,
        out_row_stride, row0, emit_partial);
  }
}

// Four consecutive elements (index a multiple of 4) of a row of runtime dtype, with one
// vector load where the address allows it.
__device__ __forceinline__ void load4_rt(const void* base, int64_t idx, int dt, float out[4]) {
  if (dt == KNLP_F32) {
    const float* p = static_cast<const float*>(base) + idx;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p));
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) out[i] = __ldg(p + i);
    }
    return;
  }
  const uint16_t* p = static_cast<const uint16_t*>(base) + idx;
  uint32_t w0, w1;
  if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
    w0 = v.x;
    w1 = v.y;
  } else {
    w0 = __ldg(p) | (static_cast<uint32_t>(__ldg(p + 1)) << 16);
    w1 = __ldg(p + 2) | (static_cast<uint32_t>(__ldg(p + 3)) << 16);
  }
  if (dt == KNLP_F16) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w0));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w1));
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
  } else {  // bf16: the upper half of an fp32
    out[0] = __uint_as_float(w0 << 16);
    out[1] = __uint_as_float(w0 & 0xFFFF0000u);
    out[2] = __uint_as_float(w1 << 16);
    out[3] = __uint_as_float(w1 & 0xFFFF0000u);
  }
}

// The step's new token of one (sequence, kv head), done by ONE warp of the pair's last
// member: quantize K and V with the write path's own arithmetic (quant_row.cuh), store
// them at the token's slot, and leave what the attention needs of it in shared memory -
// the scaled scores of the head's q rows against the DEQUANTIZED key (as later steps will
// read it) and the dequantized value row - so that the token joins this CTA's partial as
// one more tile, without a round trip through global memory.
template <int HD, int KMODE, int VMODE>
__device__ __noinline__ void append_token(const void* ksrc, const void* vsrc, const int src_dt,
                                          uint8_t* k_crow, __half* k_srow, __half* k_zrow,
                                          uint8_t* v_crow, __half* v_srow, __half* v_zrow,
                                          const void* q, const int q_dt, const int64_t q_row0,
                                          const int64_t q_head_stride, const int n_rep,
                                          const float clip_ratio, float* s_new, float* v_new) {
  const int lane = threadIdx.x & 31;
  const int e0 = lane * 4;
  const bool active = e0 < HD;
  const bool leader = active && ((lane & 7) == 0);
  float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  int c[4];
  float sc, mn;
  // ---- key (the value row and the q rows are fetched up front as well)
  float xv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float qv[8][4];
  if (active) {
    load4_rt(ksrc, e0, src_dt, x);
    load4_rt(vsrc, e0, src_dt, xv);
#pragma unroll
    for (int hs = 0; hs < 8; ++hs)
      if (hs < n_rep) load4_rt(q, q_row0 + hs * q_head_stride + e0, q_dt, qv[hs]);
  }
  quantize4(KMODE, x, lane, clip_ratio, c, sc, mn);
  if (active) store_quantized4(KMODE, c, sc, mn, k_crow, k_srow, k_zrow, e0, leader, true);
  {
    const float s16 = __half2float(__float2half_rn(sc));
    const float z16 = KMODE == KNLP_KV_INT4_ASYM ? __half2float(__float2half_rn(mn)) : 0.0f;
    float kh[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float code = static_cast<float>(KMODE == KNLP_KV_INT4_SYM ? c[i] - 8 : c[i]);
      kh[i] = active ? code * s16 + z16 : 0.0f;
    }
    const float mul = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f;  // log2 domain
#pragma unroll
    for (int hs = 0; hs < 8; ++hs) {
      if (hs < n_rep) {
        float dot = 0.0f;
        if (active) {
#pragma unroll
          for (int i = 0; i < 4; ++i) dot = fmaf(qv[hs][i], kh[i], dot);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) s_new[hs] = dot * mul;
      }
    }
  }
  // ---- value
  quantize4(VMODE, xv, lane, clip_ratio, c, sc, mn);
  if (active) {
    store_quantized4(VMODE, c, sc, mn, v_crow, v_srow, v_zrow, e0, leader, true);
    const float s16 = __half2float(__float2half_rn(sc));
    const float z16 = VMODE == KNLP_KV_INT4_ASYM ? __half2float(__float2half_rn(mn)) : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float code = static_cast<float>(VMODE == KNLP_KV_INT4_SYM ? c[i] - 8 : c[i]);
      v_new[e0 + i] = code * s16 + z16;
    }
  }
}

// CTAs per SM the register budget is set for: as many as the stages leave room for in
// shared memory (an unquantized K plane: three; the packed planes: kCtasPerSm).
template <int HD, int KMODE, int VMODE>
constexpr int dq_ctas_per_sm() {
  using G = Geo<HD, KMODE, VMODE, kTilePad>;
  constexpr int fit = 232448 / (G::kSmemBytes + 2048);
  return fit < 1 ? 1 : fit < kCtasPerSm ? fit : kCtasPerSm;
}

template <int HD, int KMODE, int VMODE, bool SPLIT, int HPBL, bool ROUTED = false>
__global__ void __launch_bounds__(kThreads, dq_ctas_per_sm<HD, KMODE, VMODE>())
decode_dq_kernel(const DecodeArgs a, const DqParams dp) {
  static_assert(!ROUTED || HPBL == 0, "per-kv-head page tables: one kv head per CTA");
  using G = Geo<HD, KMODE, VMODE, kTilePad>;
  constexpr int kStages = G::kStages;
  constexpr bool kInt8V = G::kInt8V;
  constexpr int NG = G::NG;
  constexpr bool kInt8K = G::kInt8K;
  constexpr bool kFpK = G::kFpK;  // unquantized K: no scale rows, the tile IS the A operand
  constexpr bool kBf16K = (KMODE == KNLP_KV_BF16);
  constexpr bool kAsymK = (KMODE == KNLP_KV_INT4_ASYM);
  constexpr bool kAsymV = (VMODE == KNLP_KV_INT4_ASYM);
  constexpr int hpb_log2 = HPBL;
  constexpr int HPB = 1 << hpb_log2;
  constexpr int TT = (kWarpsCta >> hpb_log2) * 16;  // tokens per stage
  constexpr int CT = kStages * TT;                  // tokens per chunk
  constexpr int tiles = kWarpsCta >> hpb_log2;      // 16-token tiles per stage
  static_assert(kStages >= 3, "tickets and page ids are handed over at stages 0, k-2, k-1");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  __shared__ int pg_tab[4][32];  // page ids of the chunk of round r at [r & 3]
  __shared__ int ch_tok[4];      // first token of the chunk of round r, -1 = none
  __shared__ int s_scan[kWarpsCta];
  __shared__ int s_find[2];
  __shared__ int s_last, s_flag;
  // Values that are needed again only after the long loop over the chunks are parked
  // here meanwhile (they would otherwise hold registers the loop needs)
  __shared__ int s_park[12];
  __shared__ float s_mrow[HPB * 8], s_irow[HPB * 8];  // merge: row maximum and weight scale
  // the step's new token of the pair (its last member only): scaled scores of the q rows
  // (log2 domain) and the dequantized value rows, from the prologue to the epilogue
  __shared__ float sm_snew[HPB * 8];
  __shared__ __align__(16) float sm_vnew[HPB * HD];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int fr = lane >> 2;
  const int ft = lane & 3;
  const int n_rep = a.n_q_heads / a.n_kv_heads;
  const int heads = HPB * n_rep;  // q heads (output rows) of a pair
  const int HBn = a.n_kv_heads >> hpb_log2;
  const int S = a.n_seqs;
  const int n_pairs = S * HBn;
  const int Gn = static_cast<int>(gridDim.x);
  // interleave the launch ranks: consecutive logical ids sit in different ranks
  const int Lid = static_cast<int>(blockIdx.x % dp.n_cols) * dp.n_ranks +
                  static_cast<int>(blockIdx.x / dp.n_cols);

  // a sequence without cached tokens still has work when the step appends one to it
  const bool appending = dp.new_key != nullptr;
  auto seq_chunks = [&](int s) -> int {
    const int L = ROUTED ? min(__ldg(a.seq_lens + s) << dp.page_log2, dp.len_cap)
                         : __ldg(a.seq_lens + s);
    if (L < 0 || (L == 0 && !appending)) return 0;
    return L > CT ? (L + CT - 1) / CT : 1;
  };

  // ---------------- sequences without tokens: their output rows are zero ----------------
  if (dp.fuse) {
    for (int s = Lid; s < S; s += Gn) {
      if (seq_chunks(s) > 0) continue;
      const int row_elems = dp.emit_partial ? HD + 2 : HD;
      for (int i = tid; i < a.n_q_heads * row_elems; i += kThreads) {
        const int r = i / row_elems, e = i % row_elems;
        const int64_t o = (static_cast<int64_t>(s) * a.n_q_heads + r) * a.out_row_stride + e;
        if (dp.emit_partial) {
          static_cast<float*>(a.out)[o] = e == HD ? -INFINITY : 0.0f;
        } else {
          store_elem_rt(a.out, o, 0.0f, a.out_dtype);
        }
      }
    }
  } else {
    for (int p = Lid * kThreads + tid; p < n_pairs; p += Gn * kThreads) {
      if (seq_chunks(p / HBn) == 0) {
        dp.pair_info[2 * p] = 0;
        dp.pair_info[2 * p + 1] = 0;
      }
    }
  }

  // ---------------- this CTA's share of the chunk sequence ----------------
  // chunks before sequence s (per head block): an exclusive scan over the sequences,
  // each thread summing a contiguous run of them
  const int per_thread = (S + kThreads - 1) / kThreads;
  const int s0 = min(S, tid * per_thread), s1 = min(S, s0 + per_thread);
  int mine = 0;
  for (int s = s0; s < s1; ++s) mine += seq_chunks(s);
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) s_scan[warp] = incl;
  __syncthreads();
  int before = 0, total_seq = 0;
#pragma unroll
  for (int w = 0; w < kWarpsCta; ++w) {
    if (w < warp) before += s_scan[w];
    total_seq += s_scan[w];
  }
  const int excl = before + incl - mine;
  const int total = total_seq * HBn;  // chunks of all pairs (the host bounds this below 2^31)
  const int per = max(1, (total + Gn - 1) / Gn);
  const int lo = Lid * per;
  const int hi = min(lo + per, total);
  if (lo >= total) return;  // CTA-uniform
  if (mine > 0 && HBn * excl <= lo && lo < HBn * (excl + mine)) {
    int pre = excl;
    for (int s = s0; s < s1; ++s) {
      const int n = seq_chunks(s);
      if (lo < HBn * (pre + n)) {
        s_find[0] = s;
        s_find[1] = pre;
        break;
      }
      pre += n;
    }
  }
  __syncthreads();
  int seq = s_find[0];
  int pre = s_find[1];

  // ---------------- per-thread roles that do not depend on the pair ----------------
  const int w_head = warp & (HPB - 1);
  const int w_tile = warp >> hpb_log2;
  const int page_mask = (1 << dp.page_log2) - 1;
  const int max_blk = static_cast<int>(a.num_blocks) - 1;
  const uint32_t smem_base = smem_u32(smem);
  const float score_mul = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f * kTwo24;
  // per-kv-head page tables: the heads of a token lie in different blocks, so the scale
  // rows are fetched per (token, head), G::SB bytes a piece
  constexpr bool routed = ROUTED;
  const bool page16 = dp.page_log2 == 4;

  // copy role: the 16-byte pieces of a stage are dealt to the threads in memory order
  // (token, head, piece); a thread owns pieces tid, tid + 128, ... of each plane
  constexpr int kKPer = G::KCH / 2, kVPer = G::VCH / 2;
  constexpr int kKChLog = G::KCH == 16 ? 4 : G::KCH == 8 ? 3 : G::KCH == 4 ? 2 : 1;
  constexpr int kVChLog = G::VCH == 8 ? 3 : G::VCH == 4 ? 2 : 1;
  constexpr int k_lg = hpb_log2 + kKChLog, v_lg = hpb_log2 + kVChLog;
  const int k_tt0 = tid >> k_lg, v_tt0 = tid >> v_lg;
  constexpr int k_dtt = kThreads >> k_lg, v_dtt = kThreads >> v_lg;
  const int k_j = tid & ((1 << k_lg) - 1), v_j = tid & ((1 << v_lg) - 1);
  const uint32_t kcs0 = static_cast<uint32_t>(a.k.cs[0]), kcs1 = static_cast<uint32_t>(a.k.cs[1]);
  const uint32_t vcs0 = static_cast<uint32_t>(a.v.cs[0]), vcs1 = static_cast<uint32_t>(a.v.cs[1]);
  uint32_t k_dst[kKPer], v_dst[kVPer];
#pragma unroll
  for (int n = 0; n < kKPer; ++n) {
    const int tt = k_tt0 + n * k_dtt, r = tt & 15;
    const int ws = (k_j >> kKChLog) + ((tt >> 4) << hpb_log2);
    k_dst[n] = smem_base + G::kOffK + ws * G::kTileK + r * G::KB +
               (((k_j & (G::KCH - 1)) ^ swz<G::KCH>(r)) << 4);
  }
#pragma unroll
  for (int n = 0; n < kVPer; ++n) {
    const int tt = v_tt0 + n * v_dtt, r = tt & 15;
    const int ws = (v_j >> kVChLog) + ((tt >> 4) << hpb_log2);
    v_dst[n] = smem_base + G::kOffV + ws * G::kTileV + r * G::VB +
               (((v_j & (G::VCH - 1)) ^ swz<G::VCH>(r)) << 4);
  }
  constexpr int kSPieces = kRows * G::SB / 16;
  const int s_arr = tid / kSPieces;
  const int s_byte = (tid % kSPieces) * 16;
  constexpr int s_tb = G::SB << hpb_log2;
  const int s_tt = s_byte / s_tb;
  const bool s_on = s_arr < 4 && !((s_arr == 0 && kFpK) || (s_arr == 1 && !kAsymK) ||
                                   (s_arr == 3 && !kAsymV));
  const Plane& s_pl = (s_arr >= 2) ? a.v : a.k;
  const bool s_zero = (s_arr & 1) != 0;
  const __half* s_base = s_zero ? s_pl.zeros : s_pl.scales;
  const int64_t* s_st = s_zero ? s_pl.zs : s_pl.ss;
  const uint32_t s_st0 = s_on ? static_cast<uint32_t>(s_st[0]) * 2 : 0;
  const uint32_t s_st1 = s_on ? static_cast<uint32_t>(s_st[1]) * 2 : 0;
  constexpr int s_tb_log = hpb_log2 + (G::SB == 8 ? 3 : 2);
  auto sc_swz = [&](int t, int byte_in_row) -> int {
    if (s_tb_log < 5) return byte_in_row;
    constexpr int kPieceLog = s_tb_log >= 5 ? s_tb_log - 4 : 0;
    constexpr int kPeriodLog = s_tb_log >= 5 ? 7 - s_tb_log : 0;
    return byte_in_row ^ (((t >> kPeriodLog) & ((1 << kPieceLog) - 1)) << 4);
  };
  const uint32_t s_dst =
      smem_base + (s_arr == 0 ? G::kOffKs : s_arr == 1 ? G::kOffKz : s_arr == 2 ? G::kOffVs
                                                                               : G::kOffVz) +
      (s_tb_log >= 5 ? s_tt * s_tb + sc_swz(s_tt, s_byte % s_tb) : s_byte);

  // ldmatrix addresses and scale rows of this lane
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_q = lane >> 4;
  const uint32_t k_lm0 = smem_base + G::kOffK + warp * G::kTileK + lm_row * G::KB;
  const uint32_t v_lm0 = smem_base + G::kOffV + warp * G::kTileV + lm_row * G::VB;
  constexpr int kKLoads = kFpK ? 2 * NG : kInt8K ? NG : NG / 2;
  constexpr int kVLoads = kInt8V ? NG : NG / 2;
  uint32_t k_lm[kKLoads], v_lm[kVLoads];
#pragma unroll
  for (int i = 0; i < kKLoads; ++i) k_lm[i] = k_lm0 + (((2 * i + lm_q) ^ swz<G::KCH>(lm_row)) << 4);
#pragma unroll
  for (int i = 0; i < kVLoads; ++i) v_lm[i] = v_lm0 + (((2 * i + lm_q) ^ swz<G::VCH>(lm_row)) << 4);
  const int sc_row0 =
      (((w_tile << 4) + fr) << s_tb_log) + sc_swz((w_tile << 4) + fr, w_head * G::SB);
  constexpr int sc_row8 = (8 * G::SB) << hpb_log2;

  constexpr int NH = SPLIT ? 1 : 2;
  constexpr int kHeadSlots = SPLIT ? 4 : 8;

  // =====================================================================================
  // one (sequence, head block) pair: take chunks until its ticket counter runs out
  // =====================================================================================
  // Chunks of a pair are handed out in two ways.  A member for which the pair is the first
  // of its share ("home": all members but possibly the first, whose share may begin in an
  // earlier pair) owns two chunks outright - js and js + n_static - so that it can start
  // without an atomic round trip; every further chunk, 2 * n_static + t, goes to whoever
  // draws ticket t.  A member that comes to the pair late from an earlier one only draws
  // tickets, and if none is left it files an empty partial at once.  A member whose share
  // goes on into further pairs takes no more chunks here than its share holds (quota), or
  // the pairs behind, which may have no other member, would wait for it.
  auto process_pair = [&](const int seq_in, const int hb_in, const int n_chunks,
                          const int parts_in, const int slot_in, const int first_slot_in,
                          const bool last_pair, const bool home, const int js,
                          const int n_static, const int quota) {
    {
    const int seq = seq_in, hb = hb_in, slot = slot_in, first_slot = first_slot_in;
    const int parts = parts_in;
    int* const ticket = dp.counters + (seq * HBn + hb);
    const int kvh = hb * HPB + w_head;
    const int len = ROUTED ? min(__ldg(a.seq_lens + seq) << dp.page_log2, dp.len_cap)
                           : __ldg(a.seq_lens + seq);
    const int32_t* bt_row = a.block_table + static_cast<int64_t>(seq) * a.bt_stride;
    const int hmem = hb + (routed ? seq % dp.vheads : 0);  // head block within the cache
    const int dyn0 = 2 * n_static;  // chunk of ticket 0
    if (tid == 0) {
      s_park[0] = slot;
      s_park[1] = first_slot;
      s_park[2] = parts;
      s_park[3] = seq;
      s_park[4] = hb;
      s_park[5] = last_pair ? 1 : 0;
    }

    // the pair's last member also appends the step's new token
    const bool has_new = !kFpK && appending && slot - first_slot == parts - 1;
    bool have_work = true;
    if (!home && !has_new) {  // one thread looks, so that the whole CTA goes the same way
      if (tid == 0) s_flag = dyn0 + *reinterpret_cast<volatile int*>(ticket) < n_chunks ? 1 : 0;
      __syncthreads();
      have_work = s_flag != 0;
    }
    if (!have_work) {
      // nothing left to take: an empty partial (the merge reads every member's slot)
      float4* po = reinterpret_cast<float4*>(dp.ws_o + static_cast<int64_t>(slot) * heads * HD);
      for (int i = tid; i < heads * (HD / 4); i += kThreads)
        po[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int i = tid; i < heads; i += kThreads) {
        dp.ws_m[static_cast<int64_t>(slot) * heads + i] = -INFINITY;
        dp.ws_l[static_cast<int64_t>(slot) * heads + i] = 0.0f;
      }
      if (last_pair) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    } else {
    // tickets of the first two chunks of a late member (in flight while q is fetched)
    int t0 = 0, t1 = 0x3fffffff;
    if (!home && tid == 0) {
      t0 = atomicAdd(ticket, 1);
      if (quota >= 2) t1 = atomicAdd(ticket, 1);
    }
    int taken = (home || quota >= 2) ? 2 : 1;  // thread 0: chunks drawn or owned so far

    // source pointers of this thread's pieces in block 0 (at token tt % 16 of the block)
    const uint8_t* k_pp[kKPer];
    const uint8_t* v_pp[kVPer];
#pragma unroll
    for (int n = 0; n < kKPer; ++n)
      k_pp[n] = a.k.codes + (hmem * (G::KB << hpb_log2) + k_j * 16) +
                static_cast<uint32_t>((k_tt0 + n * k_dtt) & 15) * kcs1;
#pragma unroll
    for (int n = 0; n < kVPer; ++n)
      v_pp[n] = a.v.codes + (hmem * (G::VB << hpb_log2) + v_j * 16) +
                static_cast<uint32_t>((v_tt0 + n * v_dtt) & 15) * vcs1;
    const uint8_t* s_pp = reinterpret_cast<const uint8_t*>(s_base) +
                          (hmem * s_tb + (s_tb >= 16 ? s_byte % s_tb : 0)) +
                          static_cast<uint32_t>(s_tt & 15) * s_st1;

    // routed: this thread's two scale pieces per stage - token tid % 64 of array tid / 64
    // (K scales or K zeros) and of array 2 + tid / 64 (V scales or V zeros); the address
    // within a block and the destination within a stage
    const __half* r_base[2] = {nullptr, nullptr};
    uint32_t r_st0[2] = {0u, 0u}, r_st1[2] = {0u, 0u}, r_dst[2] = {0u, 0u};
    if constexpr (ROUTED) {
      {
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const int arr = (tid >> 6) + 2 * n;
          if ((arr == 0 && kFpK) || (arr == 1 && !kAsymK) || (arr == 3 && !kAsymV)) continue;
          const Plane& pl = n ? a.v : a.k;
          const __half* base = (arr & 1) ? pl.zeros : pl.scales;
          const int64_t* st = (arr & 1) ? pl.zs : pl.ss;
          r_base[n] = base + hmem * NG;
          r_st0[n] = static_cast<uint32_t>(st[0]);
          r_st1[n] = static_cast<uint32_t>(st[1]);
          r_dst[n] = smem_base + (tid & 63) * G::SB +
                     (arr == 0 ? G::kOffKs : arr == 1 ? G::kOffKz : arr == 2 ? G::kOffVs
                                                                             : G::kOffVz);
        }
      }
    }

    // page ids of a chunk: lane i of warp 0 fetches the i-th page the chunk touches
    auto load_pages = [&](int T) -> int {
      const int p = (T >> dp.page_log2) + lane;
      int b = 0;
      if (T >= 0 && (p << dp.page_log2) < len) b = __ldg(bt_row + p);
      return b;
    };
    auto clamp_blk = [&](int raw) -> uint32_t {
      return static_cast<uint32_t>(raw < 0 ? 0 : (raw > max_blk ? max_blk : raw));
    };

    // copies of one stage, any page size, any position: predicated, zero-filling
    auto issue_general = [&](const int T, const int ring, const int st, const uint32_t stage_off) {
      if (T < 0) return;
      const int stage_tok0 = T + st * TT;
      const int page0 = T >> dp.page_log2;
#pragma unroll
      for (int n = 0; n < kKPer; ++n) {
        const int tt = k_tt0 + n * k_dtt;
        const int tok = stage_tok0 + tt;
        const bool live = tok < len;
        const uint32_t blk = live ? clamp_blk(pg_tab[ring][(tok >> dp.page_log2) - page0]) : 0u;
        const int dt = (tok & page_mask) - (tt & 15);
        const uint8_t* src = k_pp[n] + (static_cast<int64_t>(blk) * kcs0 +
                                        static_cast<int64_t>(dt) * kcs1);
        cp_async16(k_dst[n] + stage_off, live ? src : a.k.codes, live ? 16 : 0);
      }
#pragma unroll
      for (int n = 0; n < kVPer; ++n) {
        const int tt = v_tt0 + n * v_dtt;
        const int tok = stage_tok0 + tt;
        const bool live = tok < len;
        const uint32_t blk = live ? clamp_blk(pg_tab[ring][(tok >> dp.page_log2) - page0]) : 0u;
        const int dt = (tok & page_mask) - (tt & 15);
        const uint8_t* src = v_pp[n] + (static_cast<int64_t>(blk) * vcs0 +
                                        static_cast<int64_t>(dt) * vcs1);
        cp_async16(v_dst[n] + stage_off, live ? src : a.v.codes, live ? 16 : 0);
      }
      if constexpr (ROUTED) {
        {
          // one piece per (array, token): the scale row of this head alone
          const int tok = stage_tok0 + (tid & 63);
          const bool live = tok < len;
          const uint32_t blk = live ? clamp_blk(pg_tab[ring][(tok >> dp.page_log2) - page0]) : 0u;
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            if (!r_base[n]) continue;
            const __half* src = r_base[n] + (static_cast<int64_t>(blk) * r_st0[n] +
                                             static_cast<int64_t>(tok & page_mask) * r_st1[n]);
            cp_async_small<G::SB>(r_dst[n] + stage_off, live ? src : r_base[n], live ? G::SB : 0);
          }
          return;
        }
      }
      if (s_on) {
        const int tok = stage_tok0 + s_tt;
        const bool live = tok < len;
        const uint32_t blk = live ? clamp_blk(pg_tab[ring][(tok >> dp.page_log2) - page0]) : 0u;
        const int dt = (tok & page_mask) - (s_tt & 15);
        const uint8_t* src = s_pp + (static_cast<int64_t>(blk) * s_st0 +
                                     static_cast<int64_t>(dt) * s_st1);
        cp_async16(s_dst + stage_off, live ? src : reinterpret_cast<const uint8_t*>(s_base),
                   live ? 16 : 0);
      }
    };
    // copies of one stage of a FULL chunk with 16-token blocks: a 16-token tile is one
    // block, a piece costs one table read, one multiply-add and the copy
    auto issue_steady = [&](const int ring, auto st_tag) {
      constexpr int st = decltype(st_tag)::value;
      constexpr int stage_off = st * G::kStageBytes;
      constexpr int pg0 = st * TT / 16;  // first page of the stage within the chunk
      uint64_t kb[kKPer], vb[kVPer];
#pragma unroll
      for (int n = 0; n < kKPer; ++n)
        kb[n] = (TT > 16 || n == 0) ? clamp_blk(pg_tab[ring][pg0 + ((k_tt0 + n * k_dtt) >> 4)])
                                    : kb[0];
#pragma unroll
      for (int n = 0; n < kVPer; ++n)
        vb[n] = TT > 16 ? clamp_blk(pg_tab[ring][pg0 + ((v_tt0 + n * v_dtt) >> 4)]) : kb[0];
      const uint64_t sb = TT > 16 ? clamp_blk(pg_tab[ring][pg0 + (s_tt >> 4)]) : kb[0];
#pragma unroll
      for (int n = 0; n < kKPer; ++n) cp_async16_full_at<stage_off>(k_dst[n], k_pp[n] + kb[n] * kcs0);
#pragma unroll
      for (int n = 0; n < kVPer; ++n) cp_async16_full_at<stage_off>(v_dst[n], v_pp[n] + vb[n] * vcs0);
      if constexpr (ROUTED) {
        {
          const uint64_t rb = clamp_blk(pg_tab[ring][pg0 + ((tid & 63) >> 4)]);
#pragma unroll
          for (int n = 0; n < 2; ++n)
            if (r_base[n])
              cp_async_small<G::SB>(r_dst[n] + stage_off,
                                    r_base[n] + (rb * r_st0[n] + (tid & 15) * r_st1[n]), G::SB);
          return;
        }
      }
      if (s_on) cp_async16_full_at<stage_off>(s_dst, s_pp + sb * s_st0);
    };

    // ---------------- accumulators ----------------
    float oacc[NG][2][4];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) oacc[g][j][i] = 0.0f;
    float zacc[NG][NH];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int h = 0; h < NH; ++h) zacc[g][h] = 0.0f;
    float m_run[NH], l_run[NH];
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      m_run[h] = -INFINITY;
      l_run[h] = 0.0f;
    }

    // ---------------- prologue: first two chunks, their page ids, first stages ----------------
    int pg_reg = 0;     // warp 0: page ids of the chunk after next, parked for one iteration
    int grab_reg = 0;   // thread 0: ticket taken for the round after next
    bool more = false;  // thread 0: the last ticket was inside the pair
    if (warp == 0) {
      int c0 = js, c1 = js + n_static;
      if (!home) {
        c0 = dyn0 + __shfl_sync(0xffffffffu, t0, 0);
        c1 = dyn0 + __shfl_sync(0xffffffffu, t1, 0);
      }
      const int T0 = c0 < n_chunks ? c0 * CT : -1;
      const int T1 = c1 < n_chunks ? c1 * CT : -1;
      if (lane == 0) {
        ch_tok[0] = T0;
        ch_tok[1] = T1;
        ch_tok[2] = -1;
        ch_tok[3] = -1;
      }
      more = T1 >= 0;
      pg_tab[0][lane] = load_pages(T0);
      pg_reg = load_pages(T1);
    }
    __syncthreads();
    {
      const int T0 = ch_tok[0];
      auto first_fill = [&](int, auto st_tag) -> bool {
        constexpr int st = decltype(st_tag)::value;
        if (page16 && T0 >= 0 && T0 + CT <= len) {
          issue_steady(0, st_tag);
        } else {
          issue_general(T0, 0, st, st * G::kStageBytes);
        }
        cp_async_commit();
        return true;
      };
      run_stages<0, kStages - 1, false>(first_fill, 0, kStages);
    }

    // ---------------- the step's new token (the pair's last member): while the first
    // copies are in flight, one warp per kv head quantizes it, stores it and leaves its
    // scores and value row in shared memory for the epilogue ----------------
    if constexpr (!kFpK)  // (an unquantized K plane takes no fused append)
    if (has_new && w_tile == 0) {
      const int kvh_e = hb * HPB + w_head;
      int blk = __ldg(bt_row + (len >> dp.page_log2));
      blk = blk < 0 ? 0 : (blk > max_blk ? max_blk : blk);
      const int off = len & page_mask;
      auto row = [&](auto* base, const int64_t* st) {
        return base + (static_cast<int64_t>(blk) * st[0] + static_cast<int64_t>(off) * st[1] +
                       static_cast<int64_t>(kvh_e) * st[2]);
      };
      const int esz = dp.new_dtype == KNLP_F32 ? 4 : 2;
      append_token<HD, KMODE, VMODE>(
          static_cast<const uint8_t*>(dp.new_key) +
              (seq * dp.nk_stride[0] + kvh_e * dp.nk_stride[1]) * esz,
          static_cast<const uint8_t*>(dp.new_value) +
              (seq * dp.nv_stride[0] + kvh_e * dp.nv_stride[1]) * esz,
          dp.new_dtype, row(a.k.codes, a.k.cs), row(a.k.scales, a.k.ss),
          kAsymK ? row(a.k.zeros, a.k.zs) : nullptr, row(a.v.codes, a.v.cs),
          row(a.v.scales, a.v.ss), kAsymV ? row(a.v.zeros, a.v.zs) : nullptr, a.q, a.q_dtype,
          static_cast<int64_t>(seq) * a.q_stride[0] + kvh_e * n_rep * a.q_stride[1],
          a.q_stride[1], n_rep, dp.clip_ratio, sm_snew + w_head * 8, sm_vnew + w_head * HD);
    }

    // ---------------- q fragments (B operand), kept in registers ----------------
    // (built while the first copies are in flight)
    // B column n = fr.  SPLIT: head n/2, part n%2 (hi, lo); else head n.
    uint32_t bq[NG][2][2];
    float qsum[NG][2];
    {
      const int col = fr;
      const int head = SPLIT ? (col >> 1) : col;
      const bool lo_part = SPLIT && (col & 1);
      const bool live = head < n_rep;
      const int qh = kvh * n_rep + (live ? head : 0);
      const int64_t qbase = static_cast<int64_t>(seq) * a.q_stride[0] + qh * a.q_stride[1];
      float xq[NG][8];
      // slot e of group g is element 32g + 8ft + e (INT4 K) or 32g + 16(e>>2) + 4ft + (e&3)
      if (live) {
        if constexpr (kFpK) {
          load_q_pairs<NG>(a.q, qbase, ft, a.q_dtype, xq);
        } else {
          load_q_groups<NG, kInt8K>(a.q, qbase, ft, a.q_dtype, xq);
        }
      } else {
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
          for (int e = 0; e < 8; ++e) xq[g][e] = 0.0f;
      }
      float colsum[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        if constexpr (kBf16K) {
          // bf16 parts of q: hi = bf16(q), lo = bf16(q - hi)
          uint32_t u[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float x = xq[g][e];
            __nv_bfloat16 b = __float2bfloat16_rn(x);
            if (lo_part) b = __float2bfloat16_rn(x - __bfloat162float(b));
            u[e] = *reinterpret_cast<const uint16_t*>(&b);
          }
          colsum[g] = 0.0f;
          bq[g][0][0] = u[0] | (u[1] << 16);
          bq[g][0][1] = u[2] | (u[3] << 16);
          bq[g][1][0] = u[4] | (u[5] << 16);
          bq[g][1][1] = u[6] | (u[7] << 16);
          continue;
        }
        __half v[8];
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float x = xq[g][e];
          float wgt = 1.0f;
          if constexpr (!kInt8K && !kFpK) {
            // the A operand holds, per byte, the even nibble alone and the whole byte (even
            // + 16 * odd): the even slot takes q_e - q_o / 16, the odd slot q_o / 16 (with q
            // as a single fp16 the nibbles are isolated and only the odd slot is scaled)
            if (e & 1) {
              x *= 0.0625f;
              if constexpr (SPLIT) wgt = 17.0f; else wgt = 16.0f;
            } else if constexpr (SPLIT) {
              x -= xq[g][e + 1] * 0.0625f;
            }
          }
          __half h = __float2half_rn(x);
          if (lo_part) h = __float2half_rn(x - __half2float(h));
          s += wgt * __half2float(h);
          v[e] = h;
        }
        colsum[g] = s;
        if constexpr (kInt8K || kFpK) {
          bq[g][0][0] = pack_h2(v[0], v[1]);
          bq[g][0][1] = pack_h2(v[2], v[3]);
          bq[g][1][0] = pack_h2(v[4], v[5]);
          bq[g][1][1] = pack_h2(v[6], v[7]);
        } else {
          bq[g][0][0] = pack_h2(v[0], v[4]);
          bq[g][0][1] = pack_h2(v[1], v[5]);
          bq[g][1][0] = pack_h2(v[2], v[6]);
          bq[g][1][1] = pack_h2(v[3], v[7]);
        }
      }
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float s = colsum[g];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        qsum[g][0] = __shfl_sync(0xffffffffu, s, (2 * ft) * 4) * kTwoM24;
        qsum[g][1] = __shfl_sync(0xffffffffu, s, (2 * ft + 1) * 4) * kTwoM24;
        if constexpr (SPLIT) qsum[g][0] += qsum[g][1];
      }
    }

    // One iteration consumes stage kS of the chunk of round R and refills the slot freed
    // by the previous iteration.  MATH_STEADY: the chunk of this round is full (no
    // end-of-sequence tests in the body).  ISSUE_STEADY: so is the chunk the refill
    // belongs to, and blocks are 16 tokens.
    auto iteration = [&](const int R, const int T_cur, const int T_next, auto stage_tag,
                         auto math_tag, auto issue_tag) {
      constexpr int kS = decltype(stage_tag)::value;
      constexpr bool kMathSteady = decltype(math_tag)::value;
      constexpr bool kIssueSteady = decltype(issue_tag)::value;
      constexpr int kNextS = (kS + kStages - 1) % kStages;  // slot refilled now
      cp_async_wait<kStages - 2>();
      __syncthreads();
      // hand-over of tickets and page ids (warp 0; CTA-uniform conditions)
      if constexpr (kS == 0) {
        if (warp == 0) pg_tab[(R + 1) & 3][lane] = pg_reg;  // pages of the next round's chunk
        if (tid == 0) {  // a ticket for the round after next
          if (more && taken < quota) {
            grab_reg = atomicAdd(ticket, 1);
            ++taken;
          } else {
            more = false;
          }
        }
      }
      if constexpr (kS == kStages - 2) {
        if (tid == 0) {
          const int T2 = (more && dyn0 + grab_reg < n_chunks) ? (dyn0 + grab_reg) * CT : -1;
          more = T2 >= 0;
          ch_tok[(R + 2) & 3] = T2;
        }
      }
      if constexpr (kS == kStages - 1) {
        if (warp == 0) pg_reg = load_pages(ch_tok[(R + 2) & 3]);
      }
      // refill: stage kNextS of this round's chunk (kS == 0) or of the next round's
      {
        const int Tt = kS == 0 ? T_cur : T_next;
        const int ring = (kS == 0 ? R : R + 1) & 3;
        if constexpr (kIssueSteady) {
          issue_steady(ring, std::integral_constant<int, kNextS>{});
        } else if constexpr (kMathSteady) {
          // this round's chunk is full; the next one is partial or absent
          if (kS == 0 && page16) {
            issue_steady(ring, std::integral_constant<int, kNextS>{});
          } else {
            issue_general(Tt, ring, kNextS, kNextS * G::kStageBytes);
          }
        } else {
          issue_general(Tt, ring, kNextS, kNextS * G::kStageBytes);
        }
        cp_async_commit();
      }

      constexpr int stage_off = kS * G::kStageBytes;
      const uint8_t* st = smem + stage_off;
      const int tok0 = T_cur + kS * TT + w_tile * 16;  // first token of this warp's tile
      if constexpr (!kMathSteady) {
        if (tok0 >= len) return;  // whole tile past the end (warp-uniform)
      }
      const bool partial = !kMathSteady && tok0 + 16 > len;

      // ---------------- scores ----------------
      float sacc[NG][4];
#pragma unroll
      for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i) sacc[g][i] = 0.0f;
      if constexpr (kFpK) {
        // the tile as it lies in memory is the A operand: one ldmatrix and one MMA per 16
        // elements of the head dimension, all into one accumulator (no per-group scale)
#pragma unroll
        for (int i = 0; i < 2 * NG; ++i) {
          uint32_t w[4];
          ldmatrix_x4_at<stage_off>(k_lm[i], w);
          if constexpr (kBf16K) {
            mma16816_bf16(sacc[0], w[0], w[1], w[2], w[3], bq[i >> 1][i & 1][0], bq[i >> 1][i & 1][1]);
          } else {
            mma16816(sacc[0], w[0], w[1], w[2], w[3], bq[i >> 1][i & 1][0], bq[i >> 1][i & 1][1]);
          }
        }
      } else if constexpr (kInt8K) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          uint32_t w[4];
          ldmatrix_x4_at<stage_off>(k_lm[g], w);
          uint32_t lo0[2], hi0[2], lo1[2], hi1[2];
          unpack_int8x4(w[0], lo0);
          unpack_int8x4(w[1], hi0);
          unpack_int8x4(w[2], lo1);
          unpack_int8x4(w[3], hi1);
          mma16816(sacc[g], lo0[0], hi0[0], lo0[1], hi0[1], bq[g][0][0], bq[g][0][1]);
          mma16816(sacc[g], lo1[0], hi1[0], lo1[1], hi1[1], bq[g][1][0], bq[g][1][1]);
        }
      } else {
#pragma unroll
        for (int gp = 0; gp < NG / 2; ++gp) {
          uint32_t w[4];
          ldmatrix_x4_at<stage_off>(k_lm[gp], w);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const int g = 2 * gp + s;
            uint32_t top[4], bot[4];
            if constexpr (SPLIT) {
              unpack_nibbles8(w[2 * s], top);
              unpack_nibbles8(w[2 * s + 1], bot);
            } else {
              unpack_nibbles8_pure(w[2 * s], top);
              unpack_nibbles8_pure(w[2 * s + 1], bot);
            }
            mma16816(sacc[g], top[0], bot[0], top[1], bot[1], bq[g][0][0], bq[g][0][1]);
            mma16816(sacc[g], top[2], bot[2], top[3], bot[3], bq[g][1][0], bq[g][1][1]);
          }
        }
      }

      // ---------------- fold scales / zeros, mask, online softmax ----------------
      float sc[2][NH];
      {
        if constexpr (kFpK) {
          constexpr float kMulFp = 1.4426950408889634f;  // scores in the log2 domain
          const float mul = rsqrtf(static_cast<float>(HD)) * kMulFp;
#pragma unroll
          for (int rh = 0; rh < 2; ++rh) {
            if constexpr (SPLIT) {
              sc[rh][0] = (sacc[0][2 * rh] + sacc[0][2 * rh + 1]) * mul;
            } else {
              sc[rh][0] = sacc[0][2 * rh] * mul;
              sc[rh][NH - 1] = sacc[0][2 * rh + 1] * mul;
            }
          }
        }
#pragma unroll
        for (int rh = 0; rh < (kFpK ? 0 : 2); ++rh) {
          float ks[NG], kz[NG];
          const __half2* sp2 =
              reinterpret_cast<const __half2*>(st + G::kOffKs + sc_row0 + rh * sc_row8);
#pragma unroll
          for (int g2 = 0; g2 < NG / 2; ++g2) {
            const float2 f = __half22float2(sp2[g2]);
            ks[2 * g2] = f.x;
            ks[2 * g2 + 1] = f.y;
          }
          if constexpr (kAsymK) {
            const __half2* zp2 =
                reinterpret_cast<const __half2*>(st + G::kOffKz + sc_row0 + rh * sc_row8);
#pragma unroll
            for (int g2 = 0; g2 < NG / 2; ++g2) {
              const float2 f = __half22float2(zp2[g2]);
              kz[2 * g2] = f.x;
              kz[2 * g2 + 1] = f.y;
            }
          } else {
#pragma unroll
            for (int g = 0; g < NG; ++g) kz[g] = (kInt8K ? -128.0f : -8.0f) * ks[g];
          }
          float c0 = 0.0f, c1 = 0.0f;
          if constexpr (SPLIT) {
#pragma unroll
            for (int g = 0; g < NG; ++g) {
              c0 = fmaf(ks[g], sacc[g][2 * rh] + sacc[g][2 * rh + 1], c0);
              c1 = fmaf(kz[g], qsum[g][0], c1);
            }
            sc[rh][0] = (c0 + c1) * score_mul;
          } else {
#pragma unroll
            for (int g = 0; g < NG; ++g) {
              c0 = fmaf(ks[g], sacc[g][2 * rh], c0);
              c1 = fmaf(ks[g], sacc[g][2 * rh + 1], c1);
              c0 = fmaf(kz[g], qsum[g][0], c0);
              c1 = fmaf(kz[g], qsum[g][1], c1);
            }
            sc[rh][0] = c0 * score_mul;
            sc[rh][1] = c1 * score_mul;
          }
        }
        if (partial) {
#pragma unroll
          for (int rh = 0; rh < 2; ++rh) {
            if (tok0 + fr + rh * 8 >= len) {
#pragma unroll
              for (int h = 0; h < NH; ++h) sc[rh][h] = -INFINITY;
            }
          }
        }
      }
      float alpha[NH], pr[2][NH];
      bool moved = false;
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        float tmax = fmaxf(sc[0][h], sc[1][h]);
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
        const float m_new = fmaxf(m_run[h], tmax);  // finite: the tile has >= 1 valid token
        alpha[h] = fast_exp2(m_run[h] - m_new);
        moved |= (m_new != m_run[h]);
        m_run[h] = m_new;
        pr[0][h] = fast_exp2(sc[0][h] - m_new);
        pr[1][h] = fast_exp2(sc[1][h] - m_new);
        l_run[h] = l_run[h] * alpha[h] + pr[0][h] + pr[1][h];
      }
      if (__any_sync(0xffffffffu, moved)) {
        const float a0 = alpha[0];
        const float a1 = alpha[NH - 1];
#pragma unroll
        for (int g = 0; g < NG; ++g) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            oacc[g][j][0] *= a0;
            oacc[g][j][1] *= a1;
            oacc[g][j][2] *= a0;
            oacc[g][j][3] *= a1;
          }
#pragma unroll
          for (int h = 0; h < NH; ++h) zacc[g][h] *= alpha[h];
        }
      }

      // ---------------- P' = p * vscale per group, transposed into the B operand ----
      float vs[2][NG];
#pragma unroll
      for (int rh = 0; rh < 2; ++rh) {
        const __half2* sp2 =
            reinterpret_cast<const __half2*>(st + G::kOffVs + sc_row0 + rh * sc_row8);
        float vz[NG];
#pragma unroll
        for (int g2 = 0; g2 < NG / 2; ++g2) {
          const float2 f = __half22float2(sp2[g2]);
          vs[rh][2 * g2] = f.x;
          vs[rh][2 * g2 + 1] = f.y;
        }
        if constexpr (kAsymV) {
          const __half2* zp2 =
              reinterpret_cast<const __half2*>(st + G::kOffVz + sc_row0 + rh * sc_row8);
#pragma unroll
          for (int g2 = 0; g2 < NG / 2; ++g2) {
            const float2 f = __half22float2(zp2[g2]);
            vz[2 * g2] = f.x;
            vz[2 * g2 + 1] = f.y;
          }
        } else {
#pragma unroll
          for (int g = 0; g < NG; ++g) vz[g] = (kInt8V ? -128.0f : -8.0f) * vs[rh][g];
        }
        if (partial && (tok0 + fr + rh * 8) >= len) {
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            vs[rh][g] = 0.0f;
            vz[g] = 0.0f;
          }
        }
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
          for (int g = 0; g < NG; ++g) zacc[g][h] = fmaf(pr[rh][h], vz[g], zacc[g][h]);
      }
      auto p_operand = [&](int g, uint32_t pb[2]) {
#pragma unroll
        for (int rh = 0; rh < 2; ++rh) {
          uint32_t packed;
          if constexpr (SPLIT) {
            const float x = pr[rh][0] * vs[rh][g];
            const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
            packed = pack_f2h2(hi, x - hi);
          } else {
            packed = pack_f2h2(pr[rh][0] * vs[rh][g], pr[rh][1] * vs[rh][g]);
          }
          pb[rh] = movmatrix_trans(packed);
        }
      };
      if constexpr (kInt8V) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          uint32_t w[4];
          ldmatrix_x4_trans_at<stage_off>(v_lm[g], w);
          uint32_t pb[2];
          p_operand(g, pb);
          uint32_t a0[2], a1[2], b0[2], b1[2];
          unpack_int8_pairs(w[0], a0);
          unpack_int8_pairs(w[1], a1);
          unpack_int8_pairs(w[2], b0);
          unpack_int8_pairs(w[3], b1);
          mma16816(oacc[g][0], a0[0], a0[1], a1[0], a1[1], pb[0], pb[1]);
          mma16816(oacc[g][1], b0[0], b0[1], b1[0], b1[1], pb[0], pb[1]);
        }
      } else {
#pragma unroll
        for (int gp = 0; gp < NG / 2; ++gp) {
          uint32_t w[4];
          ldmatrix_x4_trans_at<stage_off>(v_lm[gp], w);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const int g = 2 * gp + s;
            uint32_t pb[2];
            p_operand(g, pb);
            uint32_t e0[4], e1[4];
            unpack_nibbles8(w[2 * s], e0);
            unpack_nibbles8(w[2 * s + 1], e1);
            mma16816(oacc[g][0], e0[0], e0[1], e1[0], e1[1], pb[0], pb[1]);
            mma16816(oacc[g][1], e0[2], e0[3], e1[2], e1[3], pb[0], pb[1]);
          }
        }
      }
    };

    // ---------------- rounds ----------------
    for (int R = 0;; ++R) {
      const int T_cur = ch_tok[R & 3];
      if (T_cur < 0) break;  // CTA-uniform: published at least one barrier ago
      const int T_next = ch_tok[(R + 1) & 3];
      const bool cur_full = page16 && T_cur + CT <= len;
      const bool next_full = T_next >= 0 && T_next + CT <= len;
      if (cur_full && next_full) {
        auto body = [&](int, auto stage_tag) -> bool {
          iteration(R, T_cur, T_next, stage_tag, std::true_type{}, std::true_type{});
          return true;
        };
        run_stages<0, kStages, false>(body, 0, kStages);
      } else if (cur_full) {
        auto body = [&](int, auto stage_tag) -> bool {
          iteration(R, T_cur, T_next, stage_tag, std::true_type{}, std::false_type{});
          return true;
        };
        run_stages<0, kStages, false>(body, 0, kStages);
      } else {
        auto body = [&](int, auto stage_tag) -> bool {
          iteration(R, T_cur, T_next, stage_tag, std::false_type{}, std::false_type{});
          return true;
        };
        run_stages<0, kStages, false>(body, 0, kStages);
      }
    }

    // ---------------- epilogue: reduce lanes, merge the warps of a head, write ----
    cp_async_wait<0>();
    __syncthreads();  // all stages consumed; shared memory is reused below
    // a dependent launch (the merge kernel, when the host uses one) may be set up from here
    if (s_park[5]) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      float l = l_run[h];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      l_run[h] = l;
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float z = zacc[g][h];
        z += __shfl_xor_sync(0xffffffffu, z, 4);
        z += __shfl_xor_sync(0xffffffffu, z, 8);
        z += __shfl_xor_sync(0xffffffffu, z, 16);
        zacc[g][h] = z;
      }
    }
    float* sm_o = reinterpret_cast<float*>(smem);
    float* sm_m = sm_o + kWarpsCta * kHeadSlots * HD;
    float* sm_l = sm_m + kWarpsCta * kHeadSlots;
    {
      float* wo = sm_o + warp * kHeadSlots * HD;
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        if constexpr (kInt8V) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int dj = 32 * g + 16 * j + 2 * fr;
            if constexpr (SPLIT) {
              float2 v;
              v.x = fmaf(oacc[g][j][0] + oacc[g][j][1], kTwo24, zacc[g][0]);
              v.y = fmaf(oacc[g][j][2] + oacc[g][j][3], kTwo24, zacc[g][0]);
              *reinterpret_cast<float2*>(wo + ft * HD + dj) = v;
            } else {
              float2 v0, v1;
              v0.x = fmaf(oacc[g][j][0], kTwo24, zacc[g][0]);
              v0.y = fmaf(oacc[g][j][2], kTwo24, zacc[g][0]);
              v1.x = fmaf(oacc[g][j][1], kTwo24, zacc[g][NH - 1]);
              v1.y = fmaf(oacc[g][j][3], kTwo24, zacc[g][NH - 1]);
              *reinterpret_cast<float2*>(wo + (2 * ft) * HD + dj) = v0;
              *reinterpret_cast<float2*>(wo + (2 * ft + 1) * HD + dj) = v1;
            }
          }
          continue;
        }
        const int d0 = 32 * g + 4 * fr;
        if constexpr (SPLIT) {
          float4 v;
          const float e0 = oacc[g][0][0] + oacc[g][0][1], m0 = oacc[g][0][2] + oacc[g][0][3];
          const float e1 = oacc[g][1][0] + oacc[g][1][1], m1 = oacc[g][1][2] + oacc[g][1][3];
          v.x = fmaf(e0, kTwo24, zacc[g][0]);
          v.y = fmaf(m0 - e0, kTwo20, zacc[g][0]);
          v.z = fmaf(e1, kTwo24, zacc[g][0]);
          v.w = fmaf(m1 - e1, kTwo20, zacc[g][0]);
          *reinterpret_cast<float4*>(wo + ft * HD + d0) = v;
        } else {
          float4 v0, v1;
          v0.x = fmaf(oacc[g][0][0], kTwo24, zacc[g][0]);
          v0.y = fmaf(oacc[g][0][2] - oacc[g][0][0], kTwo20, zacc[g][0]);
          v0.z = fmaf(oacc[g][1][0], kTwo24, zacc[g][0]);
          v0.w = fmaf(oacc[g][1][2] - oacc[g][1][0], kTwo20, zacc[g][0]);
          v1.x = fmaf(oacc[g][0][1], kTwo24, zacc[g][NH - 1]);
          v1.y = fmaf(oacc[g][0][3] - oacc[g][0][1], kTwo20, zacc[g][NH - 1]);
          v1.z = fmaf(oacc[g][1][1], kTwo24, zacc[g][NH - 1]);
          v1.w = fmaf(oacc[g][1][3] - oacc[g][1][1], kTwo20, zacc[g][NH - 1]);
          *reinterpret_cast<float4*>(wo + (2 * ft) * HD + d0) = v0;
          *reinterpret_cast<float4*>(wo + (2 * ft + 1) * HD + d0) = v1;
        }
      }
      if (fr == 0) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          const int hslot = SPLIT ? ft : 2 * ft + h;
          sm_m[warp * kHeadSlots + hslot] = m_run[h];
          sm_l[warp * kHeadSlots + hslot] = l_run[h];
        }
      }
    }
    // the step's new token was quantized, stored and scored in the prologue (sm_snew, sm_vnew)
    const bool new_here = appending && s_park[0] - s_park[1] == s_park[2] - 1;
    __syncthreads();
    // this CTA's partial of the pair: rows (kv head hl, q head hs), merged over the tiles
    {
      constexpr int kVec = HD / 4;
      const int slot = s_park[0];
      float4* po = reinterpret_cast<float4*>(dp.ws_o + static_cast<int64_t>(slot) * heads * HD);
      for (int i = tid; i < heads * kVec; i += kThreads) {
        const int e4 = i % kVec;
        const int row = i / kVec;
        const int hs = row % n_rep;
        const int hl = row / n_rep;
        float mm = -INFINITY;
#pragma unroll
        for (int t = 0; t < tiles; ++t) {
          const int w = hl + (t << hpb_log2);
          if (sm_l[w * kHeadSlots + hs] > 0.0f) mm = fmaxf(mm, sm_m[w * kHeadSlots + hs]);
        }
        if (new_here) mm = fmaxf(mm, sm_snew[hl * 8 + hs]);
        float ll = 0.0f;
        float4 oo = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (new_here) {  // the appended token: one more tile of one token, p = 2^(s - m)
          const float wgt = fast_exp2(sm_snew[hl * 8 + hs] - mm);
          const float4 v = *reinterpret_cast<const float4*>(sm_vnew + hl * HD + 4 * e4);
          ll = wgt;
          oo = make_float4(v.x * wgt, v.y * wgt, v.z * wgt, v.w * wgt);
        }
#pragma unroll
        for (int t = 0; t < tiles; ++t) {
          const int w = hl + (t << hpb_log2);
          const float lw = sm_l[w * kHeadSlots + hs];
          if (lw > 0.0f) {
            const float wgt = fast_exp2(sm_m[w * kHeadSlots + hs] - mm);
            const float4 v = *reinterpret_cast<const float4*>(sm_o + (w * kHeadSlots + hs) * HD + 4 * e4);
            ll += lw * wgt;
            oo.x += v.x * wgt;
            oo.y += v.y * wgt;
            oo.z += v.z * wgt;
            oo.w += v.w * wgt;
          }
        }
        po[i] = oo;
        if (e4 == 0) {
          dp.ws_m[static_cast<int64_t>(slot) * heads + row] = mm * 0.6931471805599453f;
          dp.ws_l[static_cast<int64_t>(slot) * heads + row] = ll;
        }
      }
    }
    }  // have_work
    }

    // ---------------- arrival; the last member merges the pair ----------------
    if (dp.fuse) __threadfence();  // this thread's partial is visible device-wide ...
    __syncthreads();               // ... and every other thread's, before the CTA is counted
    const int first_slot = s_park[1], parts = s_park[2], seq = s_park[3], hb = s_park[4];
    const int pair = seq * HBn + hb;
    int* const ticket = dp.counters + pair;
    int* const arrive = dp.counters + n_pairs + pair;
    if (tid == 0) {
      const int old = atomicAdd(arrive, 1);
      const int last = (old == parts - 1) ? 1 : 0;
      if (last) {
        // the other members' partials are read after this point (the CTA's loads come
        // after the barrier below); nothing of this thread is in flight, so the fence is
        // cheap here - after the counter resets it would wait for their round trip
        __threadfence();
        if (!dp.fuse) {  // every member has taken its last ticket: ready for the next launch
          *arrive = 0;
          *ticket = 0;
          dp.pair_info[2 * pair] = first_slot;
          dp.pair_info[2 * pair + 1] = parts;
        }
      }
      s_last = last;
    }
    __syncthreads();
    if (!dp.fuse || !s_last) return;
    if (tid == 0) {  // ready for the next launch; off the merge's critical path
      *arrive = 0;
      *ticket = 0;
    }
    merge_pair<HD, HPB * 8>(dp.ws_m + static_cast<int64_t>(first_slot) * heads,
                            dp.ws_l + static_cast<int64_t>(first_slot) * heads,
                            dp.ws_o + static_cast<int64_t>(first_slot) * heads * HD, parts, heads,
                            reinterpret_cast<float*>(smem), static_cast<int>(G::kSmemBytes / 4),
                            s_mrow, s_irow, a.out, a.out_dtype, a.out_row_stride,
                            static_cast<int64_t>(seq) * a.n_q_heads + hb * heads,
                            dp.emit_partial);
  };

  // ---------------- the pairs this CTA's share touches ----------------
  int g = lo;
  while (g < hi && seq < S) {
    const int n = seq_chunks(seq);
    const int base = HBn * pre;
    const int hb = n > 0 ? (g - base) / n : HBn;
    if (hb >= HBn) {
      pre += n;
      ++seq;
      continue;
    }
    const int off = base + hb * n;
    const int first = off / per;
    const int last = (off + n - 1) / per;
    const int pair = seq * HBn + hb;
    const int boundary = (off % per) != 0 ? 1 : 0;  // the first member's share begins earlier
    const int j = Lid - first;
    if (tid == 0) {
      s_park[6] = seq;
      s_park[7] = pre;
      s_park[8] = off + n;
    }
    const bool last_pair = off + n >= hi;
    process_pair(seq, hb, n, last - first + 1, Lid + pair, first + pair, last_pair,
                 j >= boundary, j - boundary, last - first + 1 - boundary,
                 last_pair ? 0x3fffffff : off + n - max(g, off));
    __syncthreads();  // the shared-memory rings and buffers are reused by the next pair
    seq = s_park[6];
    pre = s_park[7];
    g = s_park[8];
  }
}

template <int HD, int KMODE, int VMODE, bool SPLIT, int HPBL, bool ROUTED = false>
int launch_dq_hpb(const DecodeArgs& a, const DqParams& dp, cudaStream_t st) {
  using G = Geo<HD, KMODE, VMODE, kTilePad>;
  constexpr int kSmem = G::kSmemBytes + 128;
  auto kern = decode_dq_kernel<HD, KMODE, VMODE, SPLIT, HPBL, ROUTED>;
  static std::atomic<uint64_t> configured{0};  // bit d: attribute set on device d
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
        cudaSuccess) {
      cudaGetLastError();
      return KNLP_ERR_NO_DEVICE;
    }
    configured.fetch_or(bit, std::memory_order_release);
  }
  // the grid must be resident as a whole (shares are static): as many CTAs per SM as fit
  static std::atomic<int> occupancy{0};
  int occ = occupancy.load(std::memory_order_relaxed);
  if (occ == 0) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, kSmem) !=
            cudaSuccess || occ < 1) {
      cudaGetLastError();
      occ = 1;
    }
    occupancy.store(occ, std::memory_order_relaxed);
  }
  DqParams p = dp;
  if (p.n_ranks > occ) p.n_ranks = occ;
  kern<<<p.n_cols * p.n_ranks, kThreads, kSmem, st>>>(a, p);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

template <int HD, int KMODE, int VMODE, bool SPLIT>
int launch_dq_inst(const DecodeArgs& a, const DqParams& dp, cudaStream_t st) {
  switch (dp.hpb_log2) {
    case 0:
      return dp.vheads > 0 ? launch_dq_hpb<HD, KMODE, VMODE, SPLIT, 0, true>(a, dp, st)
                           : launch_dq_hpb<HD, KMODE, VMODE, SPLIT, 0>(a, dp, st);
    case 1: return launch_dq_hpb<HD, KMODE, VMODE, SPLIT, 1>(a, dp, st);
    default: return launch_dq_hpb<HD, KMODE, VMODE, SPLIT, 2>(a, dp, st);
  }
}

}  // namespace

// Tokens per chunk of the balanced kernel for a mode pair and heads-per-CTA count.
template <int HD, int KMODE, int VMODE>
constexpr int dq_chunk_tokens(int hpb_log2) {
  return Geo<HD, KMODE, VMODE, kTilePad>::kStages * ((kWarpsCta >> hpb_log2) * 16);
}

// One pair of K/V modes, both head sizes; instantiated in decode_dq_inst_*.cu.
template <int KMODE, int VMODE>
int launch_dq_pair(const DecodeArgs& a, const DqParams& dp, bool split, cudaStream_t st) {
  if (a.head_dim == 128)
    return split ? launch_dq_inst<128, KMODE, VMODE, true>(a, dp, st)
                 : launch_dq_inst<128, KMODE, VMODE, false>(a, dp, st);
  return split ? launch_dq_inst<64, KMODE, VMODE, true>(a, dp, st)
               : launch_dq_inst<64, KMODE, VMODE, false>(a, dp, st);
}
template <int KMODE, int VMODE>
int dq_chunk_of_pair(int head_dim, int hpb_log2) {
  return head_dim == 128 ? dq_chunk_tokens<128, KMODE, VMODE>(hpb_log2)
                         : dq_chunk_tokens<64, KMODE, VMODE>(hpb_log2);
}

}  // namespace knlp
