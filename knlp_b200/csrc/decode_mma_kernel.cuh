// Split-context GQA decode attention over the packed KV cache (sm_100a).
//
// The hot kernel of the library.  It replaces the reference's
// _fused_int4_decode_kernel (fused-quant/fused_int4.v0.1.0.py:656-894) and
// _kint8_vint4_decode_kernel (:1318-1493), which run one program per
// (sequence, q head), stream the whole context through it and re-read K/V once
// per q head of a group.  Here a CTA owns (sequence, block of kv heads,
// context split); every K/V byte is read from HBM once and serves all q heads
// of its group.
//
// Data movement: each stage of the pipeline is TT tokens x HPB kv heads of
// codes, scales and zeros (HPB <= 4 heads, one warp per head and 16-token tile),
// copied global -> shared with cp.async in 16-byte pieces dealt in memory order,
// three or four stages deep.  Code rows are stored warp-major in shared memory
// (the 16 rows a warp consumes are contiguous) with an xor swizzle of the 16-byte
// column, scale rows xor-permuted by their place in the bank period, so that the
// cp.async writes, the ldmatrix reads and the scale loads are bank-conflict free.
// While whole stages lie ahead the loop body carries no end-of-sequence test.
//
// Math: the per-token work is far too much for CUDA-core FMAs at HBM speed
// (2 * n_rep * head_dim FMAs per 160 bytes), so both products run on the tensor
// cores as m16n8k16 f16 MMAs with the 16 TOKENS of a tile on the M side and the
// q heads of the kv group on the N side, which keeps the tile dense for GQA:
//   scores  S_g[token, col] = sum_{d in group g} code[token, d] * q[col, d]
//   output  O[d, col]      += sum_token code_v[token, d] * (p[token, col] * vscale[token, g(d)])
// The codes enter the MMA as exact integers at no conversion cost: a nibble (or a
// whole byte, even nibble + 16 x odd nibble) masked in place inside an fp16 lane IS
// the fp16 subnormal value * 2^-24.  The mix of two nibbles in a byte is resolved by
// the other operand (scores: the q slots are q_even - q_odd/16 and q_odd/16) or in the
// epilogue (output: odd row = (mixed row - even row) / 16), the power of two likewise.
// int8 codes are biased to unsigned and byte-permuted into the low mantissa bits the
// same way.  Scale and zero-point
// are applied per group outside the MMA:
//   s = sum_g kscale_g * S_g + kzero_g * sum_{d in g} q[d]
//   o += sum_token p * vzero_g   (accumulated on CUDA cores)
// With at most 4 q heads per kv head the 8 MMA columns carry a hi/lo fp16 split
// of q (and of p * vscale), so the products are accurate to ~2^-22; with 5..8
// q heads the columns are the heads themselves and q, p are rounded to fp16.
// Accumulation is fp32 throughout.
//
// Softmax is the usual online recurrence in the log2 domain, one 16-token tile
// per warp per stage; accumulators are rescaled only when a running maximum
// moves.  The partial written per (sequence, q head, split) is (m, l, o) with m
// in the natural-log domain and o un-normalised.
//
// Synchronisation on the default path is cp.async group completion and
// __syncthreads only; no CTA ever waits for another.  The TMA staging option waits on
// "stage landed" mbarriers of its own CTA, every wait bounded (a wait that runs out sets
// the device status word and ends the CTA).
//
// This kernel cuts every sequence into a FIXED number of splits (the caller's n_splits),
// one CTA each, and writes one partial per split in a public layout; it serves
// knlp_b200_decode_splitk.  The default decode path of the library is the balanced kernel
// of decode_dq_kernel.cuh, which shares this math and hands the work out inside the launch.
//
// Included by the host file (which only declares the instantiations) and by one small
// translation unit per pair of K/V modes, so the instantiations compile in parallel.
#pragma once

#include <atomic>

#include "decode_mma_common.cuh"

namespace knlp {
namespace {

// TMA = true: stages are filled by cp.async.bulk.tensor copies (one box per plane and
// tile) and announced by a "stage landed" mbarrier; the warp that is last to finish
// with a slot refills it; the warps never meet at a CTA barrier inside the main loop.
// TMA = false: stages are filled by cp.async from all threads (any 16-byte
// aligned strides), one __syncthreads per stage.
template <int HD, int KMODE, int VMODE, bool SPLIT, bool TMA, int HPBL>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
decode_mma_kernel(const DecodeArgs a, const MmaParams mp, const __grid_constant__ TmaMaps tm) {
  using G = Geo<HD, KMODE, VMODE, TMA ? 0 : kTilePad>;
  constexpr int kStages = G::kStages;
  constexpr bool kInt8V = G::kInt8V;
  constexpr int NG = G::NG;
  constexpr bool kInt8K = G::kInt8K;
  constexpr bool kAsymK = (KMODE == KNLP_KV_INT4_ASYM);
  constexpr bool kAsymV = (VMODE == KNLP_KV_INT4_ASYM);

  extern __shared__ uint8_t smem_raw[];
  // swizzled TMA tiles need their natural alignment: round the base up to 1 KB
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t bars[kMaxStages];  // TMA path: "stage has landed" barriers
  __shared__ unsigned slot_done[kMaxStages];          // TMA path: warps finished with the slot
  static_assert(kMaxStages < 8, "the page table ring has 8 slots");
  __shared__ int pg_tab[8][16];  // page ids of the stages in flight (ring, slot = stage & 7)

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int fr = lane >> 2;  // fragment row / column-of-B index
  const int ft = lane & 3;   // fragment quad index

  constexpr int hpb_log2 = HPBL;  // kv heads per CTA = 1 << HPBL, a compile-time constant
  constexpr int HPB = 1 << hpb_log2;
  constexpr int TT = (kWarpsCta >> hpb_log2) * 16;  // tokens per stage
  const int split = blockIdx.x;
  const int hb = blockIdx.y;
  const int seq = blockIdx.z;
  const int n_rep = a.n_q_heads / a.n_kv_heads;

  const int seq_len = a.seq_lens[seq];
  const int start = split * a.chunk;
  // the last split takes whatever lies beyond n_splits * chunk (a max_seq_len given too
  // small must not drop tokens)
  const int end = split == a.n_splits - 1 ? seq_len : min(start + a.chunk, seq_len);

  // this warp's role in every stage: one kv head, one 16-token tile
  const int w_head = warp & (HPB - 1);
  const int w_tile = warp >> hpb_log2;
  const int kvh = hb * HPB + w_head;

  if (end <= start) {
    // empty split: neutral partials for every q head of this head block
    const int heads = HPB * n_rep;
    for (int i = tid; i < heads * HD; i += kThreads) {
      const int hh = i / HD, e = i % HD;
      const int64_t row = static_cast<int64_t>(seq) * a.n_q_heads + hb * HPB * n_rep + hh;
      const int64_t pidx = row * a.n_splits + split;
      a.part_o[pidx * HD + e] = 0.0f;
      if (e == 0) {
        a.part_m[pidx] = -INFINITY;
        a.part_l[pidx] = 0.0f;
      }
    }
    return;
  }

  // ---------------- Q fragments (B operand), kept in registers ----------------
  // B column n = fr.  SPLIT: head n/2, part n%2 (hi, lo); else head n.
  // Accumulator columns of this thread are 2ft, 2ft+1: with SPLIT both belong to q
  // head ft (hi, lo), else they are heads 2ft and 2ft+1.
  uint32_t bq[NG][2][2];
  float qsum[NG][2];  // per-group column sums * 2^-24 for accumulator columns 2ft, 2ft+1
  {
    const int col = fr;
    const int head = SPLIT ? (col >> 1) : col;
    const bool lo_part = SPLIT && (col & 1);
    const bool live = head < n_rep;
    const int qh = kvh * n_rep + (live ? head : 0);
    const int64_t qbase = static_cast<int64_t>(seq) * a.q_stride[0] + qh * a.q_stride[1];
    float colsum[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      __half v[8];
      float s = 0.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        // element index of slot e of this thread in group g (see the A-side unpack)
        int d;
        if constexpr (kInt8K) {
          d = 32 * g + 16 * (e >> 2) + 4 * ft + (e & 3);
        } else {
          d = 32 * g + 8 * ft + e;
        }
        float x = live ? load_elem_rt(a.q, qbase + d, a.q_dtype) : 0.0f;
        float wgt = 1.0f;
        if constexpr (!kInt8K) {
          // The A operand holds, per byte, the even nibble alone and the whole byte
          // (even + 16 * odd), see unpack_nibbles8: the even slot takes q_e - q_o / 16,
          // the odd slot q_o / 16.  What multiplies the zero-point is then
          // sum_e x_e + 17 sum_o x_o over the rounded slots.
          // (With q as a single fp16 the nibbles are isolated instead and only the
          // odd slot is scaled.)
          if (e & 1) {
            x *= 0.0625f;
            if constexpr (SPLIT) wgt = 17.0f; else wgt = 16.0f;
          } else if constexpr (SPLIT) {
            const float xo = live ? load_elem_rt(a.q, qbase + d + 1, a.q_dtype) : 0.0f;
            x -= xo * 0.0625f;
          }
        }
        __half h = __float2half_rn(x);
        if (lo_part) h = __float2half_rn(x - __half2float(h));
        s += wgt * __half2float(h);
        v[e] = h;
      }
      colsum[g] = s;
      if constexpr (kInt8K) {
        // k-step = 16-byte piece: reg0 = (e0, e1), reg1 = (e2, e3) of that piece
        bq[g][0][0] = pack_h2(v[0], v[1]);
        bq[g][0][1] = pack_h2(v[2], v[3]);
        bq[g][1][0] = pack_h2(v[4], v[5]);
        bq[g][1][1] = pack_h2(v[6], v[7]);
      } else {
        // k-step 0: reg0 = (n0, n4), reg1 = (n1, n5); k-step 1: (n2, n6), (n3, n7)
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
      // every lane of column fr now holds the full group sum; fetch columns 2ft, 2ft+1
      qsum[g][0] = __shfl_sync(0xffffffffu, s, (2 * ft) * 4) * kTwoM24;
      qsum[g][1] = __shfl_sync(0xffffffffu, s, (2 * ft + 1) * 4) * kTwoM24;
      if constexpr (SPLIT) qsum[g][0] += qsum[g][1];  // hi + lo of head ft
    }
  }
  // scores leave the MMA scaled by 2^-24; softmax runs in the log2 domain
  const float score_mul = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f * kTwo24;

  // ---------------- cp.async path: copy role of this thread ----------------
  // The 16-byte pieces of a stage are dealt to the threads in MEMORY order (token,
  // then head, then piece), so a warp-wide cp.async reads 512 contiguous bytes (the
  // natural layout keeps the heads of a token adjacent) and, thanks to the pad
  // between the warps' tiles, writes them to distinct banks.  Piece i of a plane:
  // token i / (HPB * CH), head (i / CH) % HPB, piece i % CH; a thread owns pieces
  // tid, tid + 256, ...  (same head and piece, tokens 256 / (HPB * CH) apart).
  const int page_mask = (1 << mp.page_log2) - 1;
  const int32_t* bt_row = a.block_table + static_cast<int64_t>(seq) * a.bt_stride;
  const int max_blk = static_cast<int>(a.num_blocks) - 1;
  const uint32_t smem_base = smem_u32(smem);
  constexpr int kKPer = G::KCH / 2, kVPer = G::VCH / 2;  // pieces per thread and stage
  constexpr int kKChLog = G::KCH == 8 ? 3 : G::KCH == 4 ? 2 : 1;
  constexpr int kVChLog = G::VCH == 8 ? 3 : G::VCH == 4 ? 2 : 1;
  const int k_lg = hpb_log2 + kKChLog, v_lg = hpb_log2 + kVChLog;
  const int k_tt0 = tid >> k_lg, v_tt0 = tid >> v_lg;       // token of piece 0 in the stage
  const int k_dtt = kThreads >> k_lg, v_dtt = kThreads >> v_lg;  // token step between pieces
  const int k_j = tid & ((1 << k_lg) - 1), v_j = tid & ((1 << v_lg) - 1);
  const uint32_t kcs0 = static_cast<uint32_t>(a.k.cs[0]), kcs1 = static_cast<uint32_t>(a.k.cs[1]);
  const uint32_t vcs0 = static_cast<uint32_t>(a.v.cs[0]), vcs1 = static_cast<uint32_t>(a.v.cs[1]);
  // k_pp[n] / v_pp[n]: this thread's n-th piece (token tt of the stage) in block 0 of
  // a cache with 16-token blocks, i.e. at token tt % 16 of the block; every other
  // address is an offset from these
  const uint8_t* k_pp[kKPer];
  const uint8_t* v_pp[kVPer];
#pragma unroll
  for (int n = 0; n < kKPer; ++n)
    k_pp[n] = a.k.codes + (hb * (G::KB << hpb_log2) + k_j * 16) +
              static_cast<uint32_t>((k_tt0 + n * k_dtt) & 15) * kcs1;
#pragma unroll
  for (int n = 0; n < kVPer; ++n)
    v_pp[n] = a.v.codes + (hb * (G::VB << hpb_log2) + v_j * 16) +
              static_cast<uint32_t>((v_tt0 + n * v_dtt) & 15) * vcs1;
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
  // Scales and zeros: each array of a stage is 128 rows of SB bytes laid out
  // [token][head], also copied in 16-byte pieces in memory order; thread tid serves
  // array tid / (8 * SB) (ks, kz, vs, vz), piece tid % (8 * SB).
  constexpr int kSPieces = kRows * G::SB / 16;  // per array and stage
  const int s_arr = tid / kSPieces;
  const int s_byte = (tid % kSPieces) * 16;        // byte offset inside the stage's array
  const int s_tb = G::SB << hpb_log2;              // bytes of one token's row (CTA's heads)
  const int s_tt = s_byte / s_tb;                  // (first) token of the piece
  const bool s_on = s_arr < 4 && !((s_arr == 1 && !kAsymK) || (s_arr == 3 && !kAsymV));
  const Plane& s_pl = (s_arr >= 2) ? a.v : a.k;
  const bool s_zero = (s_arr & 1) != 0;
  const __half* s_base = s_zero ? s_pl.zeros : s_pl.scales;
  const int64_t* s_st = s_zero ? s_pl.zs : s_pl.ss;
  const uint32_t s_st0 = s_on ? static_cast<uint32_t>(s_st[0]) * 2 : 0;  // bytes
  const uint32_t s_st1 = s_on ? static_cast<uint32_t>(s_st[1]) * 2 : 0;
  // the same for this thread's scale / zero piece (token s_tt of the stage)
  const uint8_t* s_pp = reinterpret_cast<const uint8_t*>(s_base) +
                        (hb * s_tb + (s_tb >= 16 ? s_byte % s_tb : 0)) +
                        static_cast<uint32_t>(s_tt & 15) * s_st1;
  // A warp later reads the 8 rows fr = 0..7 of ONE head in a single instruction; with
  // token rows of 32 or 64 bytes these would fall on the same banks (2- or 4-way
  // conflict).  So the 16-byte pieces of token row t are stored xor-permuted by the
  // row's index within the 128-byte bank period (see sc_swz below).
  constexpr int s_tb_log = hpb_log2 + (G::SB == 8 ? 3 : 2);
  auto sc_swz = [&](int t, int byte_in_row) -> int {
    if (TMA || s_tb_log < 5) return byte_in_row;  // TMA boxes land unpermuted
    constexpr int kPieceLog = s_tb_log >= 5 ? s_tb_log - 4 : 0;  // 16-byte pieces per row
    constexpr int kPeriodLog = s_tb_log >= 5 ? 7 - s_tb_log : 0;  // rows per 128 bytes
    return byte_in_row ^ (((t >> kPeriodLog) & ((1 << kPieceLog) - 1)) << 4);
  };
  const uint32_t s_dst =
      smem_base + (s_arr == 0 ? G::kOffKs : s_arr == 1 ? G::kOffKz : s_arr == 2 ? G::kOffVs
                                                                               : G::kOffVz) +
      (s_tb_log >= 5 ? s_tt * s_tb + sc_swz(s_tt, s_byte % s_tb) : s_byte);

  // Page ids reach the copiers through a small table in shared memory: 16 threads
  // load the ids of a stage two iterations before it is issued and park them in a
  // register for one iteration, so no instruction ever waits on the page-table load.
  auto load_pages = [&](int st_it) -> int {  // raw id of page `tid` of stage st_it
    const int p = ((start + st_it * TT) >> mp.page_log2) + tid;
    int b = 0;
    if (tid < 16 && (p << mp.page_log2) < end) b = __ldg(bt_row + p);
    return b;
  };
  auto page_id = [&](int slot, int tok, int page0) -> uint32_t {
    const int raw = pg_tab[slot][(tok >> mp.page_log2) - page0];
    return static_cast<uint32_t>(raw < 0 ? 0 : (raw > max_blk ? max_blk : raw));
  };

  // The copies of a stage: part 0 = K codes, 1 = V codes, 2 = scales and zeros.  They
  // are all issued at the top of an iteration (spreading them over the iteration
  // measured slower).
  auto issue_part = [&](int it, int part, uint32_t stage_off) {
    const int stage_tok0 = start + it * TT;
    const int page0 = stage_tok0 >> mp.page_log2;
    const int slot = it & 7;
    if (part == 0) {
#pragma unroll
      for (int n = 0; n < kKPer; ++n) {
        const int tok = stage_tok0 + k_tt0 + n * k_dtt;
        const bool live = tok < end;
        const uint32_t blk = live ? page_id(slot, tok, page0) : 0u;
        const int dt = (tok & page_mask) - ((k_tt0 + n * k_dtt) & 15);  // tokens from k_pp[n]
        const uint8_t* src = k_pp[n] + (static_cast<int64_t>(blk) * kcs0 +
                                        static_cast<int64_t>(dt) * kcs1);
        cp_async16(k_dst[n] + stage_off, src, live ? 16 : 0);  // 0 -> zero fill
      }
    } else if (part == 1) {
#pragma unroll
      for (int n = 0; n < kVPer; ++n) {
        const int tok = stage_tok0 + v_tt0 + n * v_dtt;
        const bool live = tok < end;
        const uint32_t blk = live ? page_id(slot, tok, page0) : 0u;
        const int dt = (tok & page_mask) - ((v_tt0 + n * v_dtt) & 15);
        const uint8_t* src = v_pp[n] + (static_cast<int64_t>(blk) * vcs0 +
                                        static_cast<int64_t>(dt) * vcs1);
        cp_async16(v_dst[n] + stage_off, src, live ? 16 : 0);
      }
    } else if (s_on) {
      const int tok = stage_tok0 + s_tt;
      const bool live = tok < end;
      const uint32_t blk = live ? page_id(slot, tok, page0) : 0u;
      const int dt = (tok & page_mask) - (s_tt & 15);
      const uint8_t* src = s_pp + (static_cast<int64_t>(blk) * s_st0 +
                                   static_cast<int64_t>(dt) * s_st1);
      cp_async16(s_dst + stage_off, src, live ? 16 : 0);
    }
  };
  // Fast path for the common stage: it lies inside one page (TT <= block size) and
  // entirely before the end of the sequence.  One page lookup, one base address per
  // array, constant steps between a thread's pieces, no predicates.
  const bool one_page = TT <= (1 << mp.page_log2);
  auto issue_stage = [&](int it, auto stage_tag) {  // stage_tag: it % kStages as a constant
    constexpr int stage_off = decltype(stage_tag)::value * G::kStageBytes;
    const int stage_tok0 = start + it * TT;
    if (one_page && stage_tok0 + TT <= end) {
      const int raw = pg_tab[it & 7][0];
      const uint32_t blk = static_cast<uint32_t>(raw < 0 ? 0 : (raw > max_blk ? max_blk : raw));
      const uint32_t off_s = static_cast<uint32_t>(stage_tok0 & page_mask);
      const uint64_t ko = static_cast<uint64_t>(blk) * kcs0 + off_s * kcs1;
#pragma unroll
      for (int n = 0; n < kKPer; ++n)
        cp_async16_full_at<stage_off>(
            k_dst[n], k_pp[n] + (ko + (TT > 16 ? ((k_tt0 + n * k_dtt) & ~15u) * kcs1 : 0u)));
      const uint64_t vo = static_cast<uint64_t>(blk) * vcs0 + off_s * vcs1;
#pragma unroll
      for (int n = 0; n < kVPer; ++n)
        cp_async16_full_at<stage_off>(
            v_dst[n], v_pp[n] + (vo + (TT > 16 ? ((v_tt0 + n * v_dtt) & ~15u) * vcs1 : 0u)));
      if (s_on)
        cp_async16_full_at<stage_off>(
            s_dst, s_pp + (static_cast<uint64_t>(blk) * s_st0 +
                           (off_s + (TT > 16 ? (s_tt & ~15u) : 0u)) * s_st1));
      return;
    }
    issue_part(it, 0, stage_off);
    issue_part(it, 1, stage_off);
    issue_part(it, 2, stage_off);
  };

  // Steady state: 16-token blocks, and the stage lies before the end of the sequence.
  // Each of its 16-token tiles is then exactly one block, and a piece's address is the
  // thread's pointer into block 0 plus block id x block stride: one page-table read, one
  // multiply-add and one copy per piece, no predicates.
  auto steady_blk = [&](int it, int tt) -> uint64_t {
    const int raw = pg_tab[it & 7][TT > 16 ? (tt >> 4) : 0];
    return static_cast<uint64_t>(raw < 0 ? 0 : (raw > max_blk ? max_blk : raw));
  };
  auto issue_steady = [&](int it, auto stage_tag) {
    constexpr int stage_off = decltype(stage_tag)::value * G::kStageBytes;
    // all page ids first: the copies below are memory barriers to the compiler, a
    // lookup placed between them would be repeated
    uint64_t kb[kKPer], vb[kVPer];
#pragma unroll
    for (int n = 0; n < kKPer; ++n)
      kb[n] = (TT > 16 || n == 0) ? steady_blk(it, k_tt0 + n * k_dtt) : kb[0];
#pragma unroll
    for (int n = 0; n < kVPer; ++n)
      vb[n] = TT > 16 ? steady_blk(it, v_tt0 + n * v_dtt) : kb[0];
    const uint64_t sb = TT > 16 ? steady_blk(it, s_tt) : kb[0];
#pragma unroll
    for (int n = 0; n < kKPer; ++n) cp_async16_full_at<stage_off>(k_dst[n], k_pp[n] + kb[n] * kcs0);
#pragma unroll
    for (int n = 0; n < kVPer; ++n) cp_async16_full_at<stage_off>(v_dst[n], v_pp[n] + vb[n] * vcs0);
    if (s_on) cp_async16_full_at<stage_off>(s_dst, s_pp + sb * s_st0);
  };

  const int n_iters = (end - start + TT - 1) / TT;

  // ---------------- TMA path: one warp fills a whole stage ----------------
  const uint32_t bar0 = smem_u32(bars);
  constexpr int tiles = kWarpsCta >> hpb_log2;  // 16-token tiles per stage
  constexpr int kScaleArrays = 2 + (kAsymK ? 1 : 0) + (kAsymV ? 1 : 0);
  // bytes one live tile (16 tokens x HPB heads) brings into a stage
  const uint32_t tile_bytes =
      static_cast<uint32_t>((16 * (G::KB + G::VB) + kScaleArrays * 16 * G::SB) << hpb_log2);
  // Shared-memory placement of the code tiles under TMA.  seg = bytes the CTA's heads
  // take in one token row.  Wide (seg >= 128): one box per 128-byte column, rows =
  // tokens.  Narrow: one box per tile, a row holds 128 / seg tokens.
  const int k_seg = G::KB << hpb_log2, v_seg = G::VB << hpb_log2;
  const int k_box = k_seg >= 128 ? k_seg >> 7 : 1, v_box = v_seg >= 128 ? v_seg >> 7 : 1;
  // byte offset, inside the K or V region of a stage, of 16-byte piece q of token t of
  // (head hl, tile tl), after the 128-byte swizzle
  auto code_off = [&](int row_bytes, int seg, int nbox, int tl, int hl, int t, int q) -> int {
    if (seg >= 128) {
      const int hoff = hl * row_bytes;
      const int c = ((hoff & 127) >> 4) + q;
      return ((tl * nbox + (hoff >> 7)) << 11) + t * 128 + ((c ^ (t & 7)) << 4);
    }
    const int off = t * seg + hl * row_bytes + q * 16;
    const int rho = off >> 7;
    return tl * 16 * seg + rho * 128 + ((((off >> 4) & 7) ^ (rho & 7)) << 4);
  };

  // A stage is K, V, ks, kz, vs, vz boxes for each of its 16-token tiles; lane c of the
  // issuing warp owns copies c and c + 32.  Every warp keeps, for its own copies, the
  // page ids of the stage that will next land in the slot it is working on (loaded at
  // the top of the iteration, used at its end), so a refill never waits on the table.
  constexpr int n_copies = 6 * tiles;
  constexpr int kCopySlots = (n_copies + 31) / 32;
  int pg_next[kCopySlots];
  auto copy_tok = [&](int it, int c) -> int { return start + it * TT + (c & (tiles - 1)) * 16; };
  auto prefetch_pages = [&](int it) {
#pragma unroll
    for (int j = 0; j < kCopySlots; ++j) {
      // The address is clamped, not the result: nothing may depend on the loaded value
      // here, or the warp (which issues in order) would sit out the load's latency.
      const int tok = min(copy_tok(it, lane + 32 * j), end - 1);
      pg_next[j] = __ldg(bt_row + (tok >> mp.page_log2));
    }
  };
  auto issue_tma = [&](int it, auto stage_tag, bool prefetched) {
    constexpr int sn = decltype(stage_tag)::value;  // == it % kStages
    const int stage_tok0 = start + it * TT;
    const int live_tiles = min(tiles, (end - stage_tok0 + 15) >> 4);
    const uint32_t full = bar0 + sn * 8;
    // (debug_stall: 16 bytes that never come, so that the bounded wait on this stage runs
    // out; every copy that IS issued still lands)
    if (lane == 0)
      mbar_arrive_expect_tx(full, static_cast<uint32_t>(live_tiles) * tile_bytes +
                                      ((mp.debug_stall && it == 0) ? 16u : 0u));
    __syncwarp();
    const uint32_t stage_base = smem_base + static_cast<uint32_t>(sn) * G::kStageBytes;
#pragma unroll
    for (int j = 0; j < kCopySlots; ++j) {
      const int c = lane + 32 * j;
      if (c >= n_copies) continue;
      const int tl = c & (tiles - 1);
      if (tl >= live_tiles) continue;
      const int tok = stage_tok0 + tl * 16;
      int blk = prefetched ? pg_next[j] : __ldg(bt_row + (tok >> mp.page_log2));
      blk = blk < 0 ? 0 : (blk > max_blk ? max_blk : blk);
      const int off = tok & page_mask;
      const int arr = c / tiles;  // 0 K codes, 1 V codes, 2 ks, 3 kz, 4 vs, 5 vz
      if (arr < 2) {
        const bool is_v = arr == 1;
        const int nbox = is_v ? v_box : k_box;
        const int seg = is_v ? v_seg : k_seg;
        const void* map = is_v ? static_cast<const void*>(&tm.v) : static_cast<const void*>(&tm.k);
        const uint32_t region = stage_base + (is_v ? G::kOffV : G::kOffK);
        if (seg >= 128) {
          tma_load_4d(region + ((tl * nbox) << 11), map, full, 0, off, (hb * seg) >> 7, blk);
        } else {
          tma_load_3d(region + tl * 16 * seg, map, full, 0, (off * seg) >> 7, blk);
        }
      } else {
        if ((arr == 3 && !kAsymK) || (arr == 5 && !kAsymV)) continue;
        const void* map = arr == 2 ? &tm.ks : arr == 3 ? &tm.kz : arr == 4 ? &tm.vs : &tm.vz;
        const int aoff =
            arr == 2 ? G::kOffKs : arr == 3 ? G::kOffKz : arr == 4 ? G::kOffVs : G::kOffVz;
        const uint32_t dst = stage_base + aoff + ((tl * 16 * G::SB) << hpb_log2);
        if (tm.scale_merged) {
          tma_load_3d(dst, map, full, ((off * G::SB) << hpb_log2) >> 2, 0, blk);
        } else {
          tma_load_3d(dst, map, full, hb * HPB * G::SB, off, blk);
        }
      }
    }
  };
  // A warp that has finished reading a slot counts itself off; the LAST one to do so
  // refills the slot at once with the stage kStages ahead.  The acq_rel counter orders
  // every warp's reads of the slot before the refill that overwrites it.
  auto release_slot = [&](int it, auto stage_tag) {
    constexpr int sn = decltype(stage_tag)::value;
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      unsigned old;
      asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;\n"
                   : "=r"(old)
                   : "r"(smem_u32(&slot_done[sn]))
                   : "memory");
      last = (old == kWarpsCta - 1) ? 1 : 0;
      if (last) *reinterpret_cast<volatile unsigned*>(&slot_done[sn]) = 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last && it + kStages < n_iters) issue_tma(it + kStages, stage_tag, true);
  };

  // ---------------- accumulators ----------------
  // oacc[g][j]: c0, c1 = output row d = 32g + 4fr + 2j; c2, c3 = that row + 16 x row
  // d + 1 (the byte-wide operand); all scaled 2^-24; columns 2ft, 2ft+1
  float oacc[NG][2][4];
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) oacc[g][j][i] = 0.0f;
  constexpr int NH = SPLIT ? 1 : 2;  // q heads this thread tracks
  float zacc[NG][NH];                // sum_token p * vzero_g, this thread's rows only
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

  // ---------------- prologue: fill kStages-1 stages ----------------
  int pg_reg = 0;  // cp.async path: page id parked by threads 0..15 (see load_pages)
  bool lost = false;  // a bounded barrier wait ran out
  if constexpr (TMA) {
    if (tid == 0) {
#pragma unroll
      for (int s = 0; s < kStages; ++s) {
        mbar_init(bar0 + s * 8, 1);  // the issuing lane's arrival + the bytes of the stage
        slot_done[s] = 0;
      }
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
      auto first_fill = [&](int it, auto stage_tag) -> bool {
        issue_tma(it, stage_tag, false);
        return true;
      };
      run_stages<0, kStages>(first_fill, 0, n_iters);
    }
  } else {
    if (tid < 16) {
#pragma unroll
      for (int s = 0; s < kStages; ++s) pg_tab[s][tid] = load_pages(s);
      pg_reg = load_pages(kStages);
    }
    __syncthreads();
    auto first_fill = [&](int it, auto stage_tag) -> bool {
      issue_stage(it, stage_tag);
      cp_async_commit();
      return true;
    };
    run_stages<0, kStages - 1>(first_fill, 0, n_iters);
    for (int s = n_iters; s < kStages - 1; ++s) cp_async_commit();  // keep the group count
  }

  // ldmatrix source row of this lane: row (lane & 7) + 8 * ((lane >> 3) & 1), piece + (lane >> 4)
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_q = lane >> 4;
  const uint32_t k_lm0 = smem_base + G::kOffK + warp * G::kTileK + lm_row * G::KB;
  const uint32_t v_lm0 = smem_base + G::kOffV + warp * G::kTileV + lm_row * G::VB;
  // piece offsets of the ldmatrix calls (piece index xor row swizzle), fixed per thread
  constexpr int kKLoads = kInt8K ? NG : NG / 2;
  constexpr int kVLoads = kInt8V ? NG : NG / 2;
  uint32_t k_lm[kKLoads], v_lm[kVLoads];
#pragma unroll
  for (int i = 0; i < kKLoads; ++i) {
    if constexpr (TMA) {
      k_lm[i] = smem_base + G::kOffK +
                code_off(G::KB, k_seg, k_box, w_tile, w_head, lm_row, 2 * i + lm_q);
    } else {
      k_lm[i] = k_lm0 + (((2 * i + lm_q) ^ swz<G::KCH>(lm_row)) << 4);
    }
  }
#pragma unroll
  for (int i = 0; i < kVLoads; ++i) {
    if constexpr (TMA) {
      v_lm[i] = smem_base + G::kOffV +
                code_off(G::VB, v_seg, v_box, w_tile, w_head, lm_row, 2 * i + lm_q);
    } else {
      v_lm[i] = v_lm0 + (((2 * i + lm_q) ^ swz<G::VCH>(lm_row)) << 4);
    }
  }
  // scale / zero rows of this thread's two accumulator rows (fr and fr + 8)
  // scale / zero arrays of a stage are [token][head of the CTA] rows of SB bytes
  // (the piece permutation of row t depends on t only through bits that rows t and
  // t + 8 share, so one offset serves both)
  const int sc_row0 =
      (((w_tile << 4) + fr) << s_tb_log) + sc_swz((w_tile << 4) + fr, w_head * G::SB);
  const int sc_row8 = (8 * G::SB) << hpb_log2;

  // One iteration consumes one stage.  The stage index kS (== it % kStages) is a
  // compile-time constant, so every shared-memory offset of the body is an immediate;
  // the driver loop below steps through the stages kStages at a time.  Returns false
  // if a bounded barrier wait ran out.
  // steady_tag = true_type: the caller guarantees that this stage and the one refilled
  // now are whole (and, for cp.async, that a stage is one page), which removes every
  // end-of-sequence test from the body.
  auto iteration = [&](const int it, auto stage_tag, auto steady_tag) -> bool {
    constexpr int kS = decltype(stage_tag)::value;
    constexpr bool kSteady = decltype(steady_tag)::value;
    [[maybe_unused]] constexpr int kNextS = (kS + kStages - 1) % kStages;  // slot refilled now
    if constexpr (TMA) {
      prefetch_pages(it + kStages);  // for the refill this warp may issue at the end
      if (!mbar_wait(bar0 + kS * 8, static_cast<uint32_t>(it / kStages) & 1u)) lost = true;
      if (__any_sync(0xffffffffu, lost)) {
        if (lane == 0) atomicExch(mp.status, 1);
        return false;
      }
    } else {
      cp_async_wait<kStages - 2>();
      __syncthreads();
      if (tid < 16) {
        pg_tab[(it + kStages) & 7][tid] = pg_reg;  // loaded one iteration ago
        pg_reg = load_pages(it + kStages + 1);
      }
    }
    if constexpr (!TMA) {
      const int nx = it + kStages - 1;
      if constexpr (kSteady) {
        issue_steady(nx, std::integral_constant<int, kNextS>{});
      } else {
        if (nx < n_iters) issue_stage(nx, std::integral_constant<int, kNextS>{});
      }
      cp_async_commit();
    }

    constexpr int stage_off = kS * G::kStageBytes;
    const uint8_t* st = smem + stage_off;
    const int tok0 = start + it * TT + w_tile * 16;  // first token of this warp's tile
    if constexpr (!kSteady) {
      if (tok0 >= end) {  // whole tile past the end (warp-uniform): nothing was loaded for it
        if constexpr (TMA) release_slot(it, stage_tag);
        return true;
      }
    }
    // Rows past the end of a partial tile may hold whatever the page holds there (a TMA
    // box is always whole; a 16-byte scale piece can span two tokens), so their scales
    // are masked before use.
    const bool partial = !kSteady && tok0 + 16 > end;

    // ---------------- scores ----------------
    float sacc[NG][4];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i) sacc[g][i] = 0.0f;
    {
      if constexpr (kInt8K) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          uint32_t w[4];
          ldmatrix_x4_at<stage_off>(k_lm[g], w);
          // w0: rows 0-7 piece 2g; w1: rows 8-15 piece 2g; w2/w3: piece 2g+1
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
          // w0: rows 0-7 group 2gp; w1: rows 8-15 group 2gp; w2/w3: group 2gp+1
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
    }

    // ---------------- fold scales / zeros, mask, online softmax ----------------
    // this thread's rows: fr (token tok0 + fr) and fr + 8
    float sc[2][NH];  // [row half][head]
    {
#pragma unroll
      for (int rh = 0; rh < 2; ++rh) {
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
          // symmetric int4 stores code + 8, int8 enters the MMA as code + 128
#pragma unroll
          for (int g = 0; g < NG; ++g) kz[g] = (kInt8K ? -128.0f : -8.0f) * ks[g];
        }
        float c0 = 0.0f, c1 = 0.0f;  // columns 2ft, 2ft+1 (still scaled by 2^-24)
        if constexpr (SPLIT) {
          // hi and lo columns of one head share scale and zero: add them first
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
      if (partial) {  // warp-uniform: only the last tile of a split masks rows
#pragma unroll
        for (int rh = 0; rh < 2; ++rh) {
          if (tok0 + fr + rh * 8 >= end) {
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
      if (partial && (tok0 + fr + rh * 8) >= end) {
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

    // P' of group g as the B operand: rows = the 16 tokens (two registers), columns as
    // in the score accumulators
    auto p_operand = [&](int g, uint32_t pb[2]) {
#pragma unroll
      for (int rh = 0; rh < 2; ++rh) {
        uint32_t packed;
        if constexpr (SPLIT) {
          // hi = x with the low 13 mantissa bits cleared (exact in fp16), lo = x - hi
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
        // w0: tokens 0-7, 16-byte piece 2g; w1: tokens 8-15, piece 2g; w2 / w3: piece 2g+1.
        // A register holds elements 2fr, 2fr+1 of its piece for tokens 2ft and 2ft+1.
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
        // w0: tokens 0-7 group 2gp; w1: tokens 8-15 group 2gp; w2/w3: group 2gp+1
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int g = 2 * gp + s;
          uint32_t pb[2];
          p_operand(g, pb);
          // a ldmatrix.trans register is (token 2ft | token 2ft+1) x nibbles 4fr..4fr+3 of
          // the group, so the same unpack yields (token, token+1) pairs per element
          uint32_t e0[4], e1[4];
          unpack_nibbles8(w[2 * s], e0);
          unpack_nibbles8(w[2 * s + 1], e1);
          mma16816(oacc[g][0], e0[0], e0[1], e1[0], e1[1], pb[0], pb[1]);
          mma16816(oacc[g][1], e0[2], e0[3], e1[2], e1[3], pb[0], pb[1]);
        }
      }
    }
    if constexpr (TMA) release_slot(it, stage_tag);  // done reading the stage
    return true;
  };
  {
    const int n_full = (end - start) / TT;  // whole stages
    int n_steady = n_full - (kStages - 1);  // iterations whose own and refilled stage are whole
    if (!TMA && mp.page_log2 != 4) n_steady = 0;  // the steady copies assume 16-token blocks
    n_steady = n_steady > 0 ? n_steady - n_steady % kStages : 0;
    auto steady = [&](int it, auto stage_tag) -> bool {
      return iteration(it, stage_tag, std::true_type{});
    };
    auto general = [&](int it, auto stage_tag) -> bool {
      return iteration(it, stage_tag, std::false_type{});
    };
    bool ok = true;
    int it0 = 0;
    for (; ok && it0 < n_steady; it0 += kStages)
      ok = run_stages<0, kStages, false>(steady, it0, n_steady);
    for (; ok && it0 < n_iters; it0 += kStages) ok = run_stages<0, kStages>(general, it0, n_iters);
  }

  // ---------------- epilogue: reduce lanes, merge the warps of a head, write ----
  cp_async_wait<0>();
  if constexpr (TMA) {
    // A wait ran out in some warp (never expected; the status word is set): the stage
    // buffers may still be the target of copies, so they are not reused; this split
    // reports no tokens and the CTA ends.
    if (__syncthreads_or(lost ? 1 : 0)) {
      const int heads = HPB * n_rep;
      for (int i = tid; i < heads * HD; i += kThreads) {
        const int hh = i / HD, e = i % HD;
        const int64_t row = static_cast<int64_t>(seq) * a.n_q_heads + hb * HPB * n_rep + hh;
        const int64_t pidx = row * a.n_splits + split;
        a.part_o[pidx * HD + e] = 0.0f;
        if (e == 0) {
          a.part_m[pidx] = -INFINITY;
          a.part_l[pidx] = 0.0f;
        }
      }
      return;
    }
  }
  __syncthreads();  // all stages consumed; shared memory is reused below

  // per-warp totals over the 8 fragment rows
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

  // shared layout: per warp [head slots][HD] floats of o, then m and l per head slot
  constexpr int kHeadSlots = SPLIT ? 4 : 8;
  float* sm_o = reinterpret_cast<float*>(smem);
  float* sm_m = sm_o + kWarpsCta * kHeadSlots * HD;
  float* sm_l = sm_m + kWarpsCta * kHeadSlots;
  {
    float* wo = sm_o + warp * kHeadSlots * HD;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      if constexpr (kInt8V) {
        // accumulator j of the group = its 16-byte piece j; rows fr | fr + 8 = elements
        // 2fr | 2fr + 1 of the piece, all scaled 2^-24
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
      // undo the 2^-24 of the subnormals; odd rows = (mixed - even) / 16
      if constexpr (SPLIT) {
        // head ft: hi column + lo column + zero term
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
        const int slot = SPLIT ? ft : 2 * ft + h;
        sm_m[warp * kHeadSlots + slot] = m_run[h];
        sm_l[warp * kHeadSlots + slot] = l_run[h];
      }
    }
  }
  __syncthreads();

  // merge: thread i handles (kv head hl, q head slot, element e)
  const int total = HPB * n_rep * HD;
  for (int i = tid; i < total; i += kThreads) {
    const int e = i % HD;
    const int hs = (i / HD) % n_rep;
    const int hl = i / (HD * n_rep);
    float mm = -INFINITY;
    for (int t = 0; t < tiles; ++t) {
      const int w = hl + (t << hpb_log2);
      if (sm_l[w * kHeadSlots + hs] > 0.0f) mm = fmaxf(mm, sm_m[w * kHeadSlots + hs]);
    }
    float ll = 0.0f, oo = 0.0f;
    for (int t = 0; t < tiles; ++t) {
      const int w = hl + (t << hpb_log2);
      const float lw = sm_l[w * kHeadSlots + hs];
      if (lw > 0.0f) {
        const float wgt = fast_exp2(sm_m[w * kHeadSlots + hs] - mm);
        ll += lw * wgt;
        oo += sm_o[(w * kHeadSlots + hs) * HD + e] * wgt;
      }
    }
    const int64_t row =
        static_cast<int64_t>(seq) * a.n_q_heads + (hb * HPB + hl) * n_rep + hs;
    const int64_t pidx = row * a.n_splits + split;
    a.part_o[pidx * HD + e] = oo;
    if (e == 0) {
      a.part_m[pidx] = mm * 0.6931471805599453f;  // log2 domain -> natural log
      a.part_l[pidx] = ll;
    }
  }
}

template <int HD, int KMODE, int VMODE, bool SPLIT, bool TMA, int HPBL>
int launch_hpb(const DecodeArgs& a, const MmaParams& mp, const TmaMaps& tm, cudaStream_t st) {
  using G = Geo<HD, KMODE, VMODE, TMA ? 0 : kTilePad>;
  constexpr int kSmem = G::kSmemBytes + 1024;  // slack for the 1 KB alignment of the stages
  auto kern = decode_mma_kernel<HD, KMODE, VMODE, SPLIT, TMA, HPBL>;
  // per instantiation: bit d set = the attribute has been set on device d (it is a
  // per-device property of the function); any host thread may get here
  static std::atomic<uint64_t> configured{0};
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
  const int hpb = 1 << mp.hpb_log2;
  dim3 grid(a.n_splits, a.n_kv_heads / hpb, a.n_seqs);
  kern<<<grid, kThreads, kSmem, st>>>(a, mp, tm);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

template <int HD, int KMODE, int VMODE, bool SPLIT, bool TMA>
int launch_inst(const DecodeArgs& a, const MmaParams& mp, const TmaMaps& tm, cudaStream_t st) {
  switch (mp.hpb_log2) {
    case 0: return launch_hpb<HD, KMODE, VMODE, SPLIT, TMA, 0>(a, mp, tm, st);
    case 1: return launch_hpb<HD, KMODE, VMODE, SPLIT, TMA, 1>(a, mp, tm, st);
    case 2:
      return launch_hpb<HD, KMODE, VMODE, SPLIT, TMA, (kWarpsLog < 2 ? kWarpsLog : 2)>(a, mp, tm, st);
    default:
      return launch_hpb<HD, KMODE, VMODE, SPLIT, TMA, (kWarpsLog < 3 ? kWarpsLog : 3)>(a, mp, tm, st);
  }
}

template <int HD, int KMODE, int VMODE>
int launch_split(const DecodeArgs& a, const MmaParams& mp, bool split, const TmaMaps* tm,
                 cudaStream_t st) {
  static const TmaMaps none{};
  // TMA staging is compiled for the INT4 caches and for INT8 K with asymmetric INT4 V; the
  // other mode pairs are always staged with cp.async
  constexpr bool kTmaBuilt = VMODE != KNLP_KV_INT8_G32 &&
                             !(KMODE == KNLP_KV_INT8_G32 && VMODE == KNLP_KV_INT4_SYM);
  if constexpr (kTmaBuilt) {
    if (tm) {
      return split ? launch_inst<HD, KMODE, VMODE, true, true>(a, mp, *tm, st)
                   : launch_inst<HD, KMODE, VMODE, false, true>(a, mp, *tm, st);
    }
  }
  return split ? launch_inst<HD, KMODE, VMODE, true, false>(a, mp, none, st)
               : launch_inst<HD, KMODE, VMODE, false, false>(a, mp, none, st);
}

}  // namespace

// One pair of K/V modes, both head sizes, every heads-per-CTA count; instantiated
// explicitly in decode_mma_inst_*.cu.
template <int KMODE, int VMODE>
int launch_mma_pair(const DecodeArgs& a, const MmaParams& mp, bool split, const TmaMaps* tm,
                    cudaStream_t st) {
  return a.head_dim == 128 ? launch_split<128, KMODE, VMODE>(a, mp, split, tm, st)
                           : launch_split<64, KMODE, VMODE>(a, mp, split, tm, st);
}

}  // namespace knlp
