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
// codes, scales and zeros, copied global -> shared with cp.async (16-byte
// pieces for codes, whole scale/zero rows of 4 or 8 bytes), kStages deep.
// Rows are stored warp-major in shared memory (the 16 rows a warp consumes are
// contiguous) with an xor swizzle of the 16-byte column, so that both the
// cp.async writes and the ldmatrix reads are bank-conflict free.
//
// Math: the per-token work is far too much for CUDA-core FMAs at HBM speed
// (2 * n_rep * head_dim FMAs per 160 bytes), so both products run on the tensor
// cores as m16n8k16 f16 MMAs with the 16 TOKENS of a tile on the M side and the
// q heads of the kv group on the N side, which keeps the tile dense for GQA:
//   scores  S_g[token, col] = sum_{d in group g} code[token, d] * q[col, d]
//   output  O[d, col]      += sum_token code_v[token, d] * (p[token, col] * vscale[token, g(d)])
// The codes enter the MMA as exact integers at no conversion cost: a nibble
// masked in place inside an fp16 lane IS the fp16 subnormal code * 2^-24 (bits
// 0-3) or code * 2^-20 (bits 4-7); the power of two is undone on the q side
// (scores) or in the epilogue (output).  int8 codes are biased to unsigned and
// byte-permuted into the low mantissa bits the same way.  Scale and zero-point
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
// Nothing in this kernel waits on another CTA or on an mbarrier: the only
// synchronisation is cp.async group completion and __syncthreads.

#include "common.cuh"

namespace knlp {
namespace {

constexpr int kWarpsCta = 8;
constexpr int kThreads = kWarpsCta * 32;
#ifndef KNLP_STAGES
#define KNLP_STAGES 4
#endif
constexpr int kStages = KNLP_STAGES;
constexpr int kRows = kWarpsCta * 16;  // (token, head) rows per stage

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t r[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t r[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
// D += A(16x16, row) * B(16x8, col), f16 inputs, f32 accumulate
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
  __half2 h = __halves2half2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f2h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

constexpr float kTwo24 = 16777216.0f;
constexpr float kTwo20 = 1048576.0f;
constexpr float kTwoM24 = 1.0f / 16777216.0f;

// Eight nibbles of a 32-bit word -> four fp16x2 registers of fp16 SUBNORMALS:
//   out[0] = (n0, n4) * 2^-24   out[1] = (n1, n5) * 2^-20
//   out[2] = (n2, n6) * 2^-24   out[3] = (n3, n7) * 2^-20     n_i = bits [4i, 4i+4)
// A half whose exponent field is zero has the value mantissa * 2^-24, so masking
// a nibble in place is the whole conversion.
__device__ __forceinline__ void unpack_nibbles8(uint32_t w, uint32_t out[4]) {
  const uint32_t w8 = w >> 8;
  out[0] = w & 0x000F000Fu;
  out[1] = w & 0x00F000F0u;
  out[2] = w8 & 0x000F000Fu;
  out[3] = w8 & 0x00F000F0u;
}

// Four int8 of a word -> two fp16x2 registers of subnormals (b + 128) * 2^-24:
// out[0] = (b0, b1), out[1] = (b2, b3).  The +128 bias is removed with the
// per-group sum of q, like a zero-point.
__device__ __forceinline__ void unpack_int8x4(uint32_t w, uint32_t out[2]) {
  const uint32_t u = w ^ 0x80808080u;
  out[0] = __byte_perm(u, 0u, 0x4140);
  out[1] = __byte_perm(u, 0u, 0x4342);
}

template <int HD, int KMODE>
struct Geo {
  static constexpr bool kInt8K = (KMODE == KNLP_KV_INT8_G32);
  static constexpr int NG = HD / 32;
  static constexpr int KB = kInt8K ? HD : HD / 2;  // K row bytes
  static constexpr int VB = HD / 2;                // V row bytes
  static constexpr int KCH = KB / 16;              // 16-byte pieces per K row
  static constexpr int VCH = VB / 16;
  static constexpr int SB = NG * 2;                // scale row bytes
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kOffK + kRows * KB;
  static constexpr int kOffKs = kOffV + kRows * VB;
  static constexpr int kOffKz = kOffKs + kRows * SB;
  static constexpr int kOffVs = kOffKz + kRows * SB;
  static constexpr int kOffVz = kOffVs + kRows * SB;
  static constexpr int kStageBytes = kOffVz + kRows * SB;
  static constexpr int kSmemBytes = kStages * kStageBytes;
};

// xor swizzle of the 16-byte column index of row r (0..15) for rows of CH pieces
template <int CH>
__device__ __forceinline__ int swz(int r) {
  return (r / (8 / CH)) & (CH - 1);
}

// Extra launch parameters computed on the host.
struct MmaParams {
  int hpb_log2;   // kv heads per CTA = 1 << hpb_log2
  int page_log2;  // block_size = 1 << page_log2
};

template <int HD, int KMODE, int VMODE, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 2)
decode_mma_kernel(const DecodeArgs a, const MmaParams mp) {
  using G = Geo<HD, KMODE>;
  constexpr int NG = G::NG;
  constexpr bool kInt8K = G::kInt8K;
  constexpr bool kAsymK = (KMODE == KNLP_KV_INT4_ASYM);
  constexpr bool kAsymV = (VMODE == KNLP_KV_INT4_ASYM);

  extern __shared__ __align__(128) uint8_t smem[];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int fr = lane >> 2;  // fragment row / column-of-B index
  const int ft = lane & 3;   // fragment quad index

  const int hpb_log2 = mp.hpb_log2;
  const int HPB = 1 << hpb_log2;
  const int TT = (kWarpsCta >> hpb_log2) * 16;  // tokens per stage
  const int split = blockIdx.x;
  const int hb = blockIdx.y;
  const int seq = blockIdx.z;
  const int n_rep = a.n_q_heads / a.n_kv_heads;

  const int seq_len = a.seq_lens[seq];
  const int start = split * a.chunk;
  const int end = min(start + a.chunk, seq_len);

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
        __half h = __float2half_rn(x);
        if (lo_part) h = __float2half_rn(x - __half2float(h));
        s += __half2float(h);
        if constexpr (!kInt8K) {
          // odd elements sit in bits 4-7 of their byte: their code arrives * 2^-20
          // instead of * 2^-24, so the matching q is pre-divided by 16 (exact)
          if (e & 1) h = __hmul(h, __float2half_rn(0.0625f));
        }
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

  // ---------------- copy role of this thread: half of one shared-memory row ----
  // Row R of a stage belongs to consumer warp R / 16 (kv head (R/16) % HPB, token
  // tile (R/16) / HPB) and is token R % 16 of that tile.  A warp of copiers fills
  // the 16 rows of one consumer warp: contiguous in shared memory (conflict-free
  // writes), 16 rows of one head in global memory (whole 32-byte sectors).
  const int c_R = tid >> 1;
  const int c_sub = tid & 1;
  const int c_r16 = c_R & 15;
  const int c_ws = c_R >> 4;
  const int c_tt = ((c_ws >> hpb_log2) << 4) + c_r16;  // token within the stage
  const int c_kvh = hb * HPB + (c_ws & (HPB - 1));
  const int page_mask = (1 << mp.page_log2) - 1;
  const int32_t* bt_row = a.block_table + static_cast<int64_t>(seq) * a.bt_stride;
  const int max_blk = static_cast<int>(a.num_blocks) - 1;

  const uint8_t* k_src0 = a.k.codes + c_kvh * a.k.cs[2] + c_sub * (G::KCH / 2) * 16;
  const uint8_t* v_src0 = a.v.codes + c_kvh * a.v.cs[2] + c_sub * (G::VCH / 2) * 16;
  const Plane& sp = c_sub ? a.v : a.k;
  const __half* s_src0 = sp.scales + c_kvh * sp.ss[2];
  const __half* z_src0 = sp.zeros ? sp.zeros + c_kvh * sp.zs[2] : nullptr;
  const uint32_t kcs0 = static_cast<uint32_t>(a.k.cs[0]), kcs1 = static_cast<uint32_t>(a.k.cs[1]);
  const uint32_t vcs0 = static_cast<uint32_t>(a.v.cs[0]), vcs1 = static_cast<uint32_t>(a.v.cs[1]);
  const uint32_t sss0 = static_cast<uint32_t>(sp.ss[0]), sss1 = static_cast<uint32_t>(sp.ss[1]);
  const uint32_t szs0 = static_cast<uint32_t>(sp.zs[0]), szs1 = static_cast<uint32_t>(sp.zs[1]);
  const bool c_has_zero = c_sub ? kAsymV : kAsymK;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t k_dst0 = smem_base + G::kOffK + c_R * G::KB;
  const uint32_t v_dst0 = smem_base + G::kOffV + c_R * G::VB;
  const uint32_t s_dst0 = smem_base + (c_sub ? G::kOffVs : G::kOffKs) + c_R * G::SB;
  const uint32_t z_dst0 = smem_base + (c_sub ? G::kOffVz : G::kOffKz) + c_R * G::SB;
  const int k_swz = swz<G::KCH>(c_r16);
  const int v_swz = swz<G::VCH>(c_r16);

  auto page_of = [&](int tok) -> uint32_t {
    int b = (tok < end) ? __ldg(bt_row + (tok >> mp.page_log2)) : 0;
    b = b < 0 ? 0 : (b > max_blk ? max_blk : b);
    return static_cast<uint32_t>(b);
  };

  auto issue_stage = [&](int it, uint32_t blk) {
    const int tok = start + it * TT + c_tt;
    const bool live = tok < end;
    const int nbytes = live ? 16 : 0;  // 0 -> zero fill, source not read
    const uint32_t off = static_cast<uint32_t>(tok & page_mask);
    const uint32_t stage_off = static_cast<uint32_t>(it % kStages) * G::kStageBytes;
    {
      const uint8_t* src = k_src0 + (static_cast<uint64_t>(blk) * kcs0 + off * kcs1);
      const uint32_t dst = k_dst0 + stage_off;
      constexpr int per = G::KCH / 2;
#pragma unroll
      for (int j = 0; j < per; ++j) {
        const int q = c_sub * per + j;
        cp_async16(dst + ((q ^ k_swz) << 4), src + (j << 4), nbytes);
      }
    }
    {
      const uint8_t* src = v_src0 + (static_cast<uint64_t>(blk) * vcs0 + off * vcs1);
      const uint32_t dst = v_dst0 + stage_off;
      constexpr int per = G::VCH / 2;
#pragma unroll
      for (int j = 0; j < per; ++j) {
        const int q = c_sub * per + j;
        cp_async16(dst + ((q ^ v_swz) << 4), src + (j << 4), nbytes);
      }
    }
    // scale / zero rows: sub 0 copies the K side, sub 1 the V side
#ifndef KNLP_EXP_NOSCALECOPY
    {
      const int sb = live ? G::SB : 0;
      const __half* ssrc = s_src0 + (static_cast<uint64_t>(blk) * sss0 + off * sss1);
      if constexpr (G::SB == 8) {
        cp_async8(s_dst0 + stage_off, ssrc, sb);
      } else {
        cp_async4(s_dst0 + stage_off, ssrc, sb);
      }
      if (c_has_zero) {
        const __half* zsrc = z_src0 + (static_cast<uint64_t>(blk) * szs0 + off * szs1);
        if constexpr (G::SB == 8) {
          cp_async8(z_dst0 + stage_off, zsrc, sb);
        } else {
          cp_async4(z_dst0 + stage_off, zsrc, sb);
        }
      }
    }
#endif
  };

  const int n_iters = (end - start + TT - 1) / TT;

  // ---------------- accumulators ----------------
  // oacc[g][j]: output rows d = 32g + 4fr + 2j (c0, c1; scaled 2^-24) and
  // d = 32g + 4fr + 2j + 1 (c2, c3; scaled 2^-20), columns 2ft, 2ft+1
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
  uint32_t blk_next = page_of(start + c_tt);
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_iters) {
      issue_stage(s, blk_next);
      blk_next = page_of(start + (s + 1) * TT + c_tt);
    }
    cp_async_commit();
  }

  // ldmatrix source row of this lane: row (lane & 7) + 8 * ((lane >> 3) & 1), piece + (lane >> 4)
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_q = lane >> 4;
  const int Rbase = warp * 16;
  const uint32_t k_lm0 = smem_base + G::kOffK + (Rbase + lm_row) * G::KB;
  const uint32_t v_lm0 = smem_base + G::kOffV + (Rbase + lm_row) * G::VB;
  // piece offsets of the ldmatrix calls (piece index xor row swizzle), fixed per thread
  constexpr int kKLoads = kInt8K ? NG : NG / 2;
  uint32_t k_lm[kKLoads], v_lm[NG / 2];
#pragma unroll
  for (int i = 0; i < kKLoads; ++i)
    k_lm[i] = k_lm0 + (((2 * i + lm_q) ^ swz<G::KCH>(lm_row)) << 4);
#pragma unroll
  for (int i = 0; i < NG / 2; ++i)
    v_lm[i] = v_lm0 + (((2 * i + lm_q) ^ swz<G::VCH>(lm_row)) << 4);
  // scale / zero rows of this thread's two accumulator rows (fr and fr + 8)
  const int sc_row0 = (Rbase + fr) * G::SB;

  for (int it = 0; it < n_iters; ++it) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    {
      const int nx = it + kStages - 1;
#ifdef KNLP_EXP_NOCOPY
      if (false) {
#else
      if (nx < n_iters) {
#endif
        issue_stage(nx, blk_next);
        blk_next = page_of(start + (nx + 1) * TT + c_tt);
      }
      cp_async_commit();
    }

    const uint32_t stage_off = static_cast<uint32_t>(it % kStages) * G::kStageBytes;
    const uint8_t* st = smem + stage_off;
    const int tok0 = start + it * TT + w_tile * 16;  // first token of this warp's tile
    if (tok0 >= end) continue;                        // whole tile past the end (warp-uniform)
#ifdef KNLP_EXP_NOCOMPUTE
    if (st[tid] == 255 && st[tid + 999] == 254) oacc[0][0][0] += 1.0f;
    continue;
#endif

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
          ldmatrix_x4(k_lm[g] + stage_off, w);
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
          ldmatrix_x4(k_lm[gp] + stage_off, w);
          // w0: rows 0-7 group 2gp; w1: rows 8-15 group 2gp; w2/w3: group 2gp+1
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const int g = 2 * gp + s;
            uint32_t top[4], bot[4];
            unpack_nibbles8(w[2 * s], top);
            unpack_nibbles8(w[2 * s + 1], bot);
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
            reinterpret_cast<const __half2*>(st + G::kOffKs + sc_row0 + rh * 8 * G::SB);
#pragma unroll
        for (int g2 = 0; g2 < NG / 2; ++g2) {
          const float2 f = __half22float2(sp2[g2]);
          ks[2 * g2] = f.x;
          ks[2 * g2 + 1] = f.y;
        }
        if constexpr (kAsymK) {
          const __half2* zp2 =
              reinterpret_cast<const __half2*>(st + G::kOffKz + sc_row0 + rh * 8 * G::SB);
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
        const bool valid = (tok0 + fr + rh * 8) < end;
        if constexpr (SPLIT) {
          // hi and lo columns of one head share scale and zero: add them first
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            c0 = fmaf(ks[g], sacc[g][2 * rh] + sacc[g][2 * rh + 1], c0);
            c1 = fmaf(kz[g], qsum[g][0], c1);
          }
          sc[rh][0] = valid ? (c0 + c1) * score_mul : -INFINITY;
        } else {
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            c0 = fmaf(ks[g], sacc[g][2 * rh], c0);
            c1 = fmaf(ks[g], sacc[g][2 * rh + 1], c1);
            c0 = fmaf(kz[g], qsum[g][0], c0);
            c1 = fmaf(kz[g], qsum[g][1], c1);
          }
          sc[rh][0] = valid ? c0 * score_mul : -INFINITY;
          sc[rh][1] = valid ? c1 * score_mul : -INFINITY;
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
          reinterpret_cast<const __half2*>(st + G::kOffVs + sc_row0 + rh * 8 * G::SB);
      float vz[NG];
#pragma unroll
      for (int g2 = 0; g2 < NG / 2; ++g2) {
        const float2 f = __half22float2(sp2[g2]);
        vs[rh][2 * g2] = f.x;
        vs[rh][2 * g2 + 1] = f.y;
      }
      if constexpr (kAsymV) {
        const __half2* zp2 =
            reinterpret_cast<const __half2*>(st + G::kOffVz + sc_row0 + rh * 8 * G::SB);
#pragma unroll
        for (int g2 = 0; g2 < NG / 2; ++g2) {
          const float2 f = __half22float2(zp2[g2]);
          vz[2 * g2] = f.x;
          vz[2 * g2 + 1] = f.y;
        }
      } else {
#pragma unroll
        for (int g = 0; g < NG; ++g) vz[g] = -8.0f * vs[rh][g];
      }
#pragma unroll
      for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int g = 0; g < NG; ++g) zacc[g][h] = fmaf(pr[rh][h], vz[g], zacc[g][h]);
    }

#pragma unroll
    for (int gp = 0; gp < NG / 2; ++gp) {
      uint32_t w[4];
      ldmatrix_x4_trans(v_lm[gp] + stage_off, w);
      // w0: tokens 0-7 group 2gp; w1: tokens 8-15 group 2gp; w2/w3: group 2gp+1
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int g = 2 * gp + s;
        uint32_t pb[2];
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

  // ---------------- epilogue: reduce lanes, merge the warps of a head, write ----
  cp_async_wait<0>();
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
      const int d0 = 32 * g + 4 * fr;
      // undo the subnormal scaling: even elements 2^-24, odd elements 2^-20
      if constexpr (SPLIT) {
        // head ft: hi column + lo column + zero term
        float4 v;
        v.x = fmaf(oacc[g][0][0] + oacc[g][0][1], kTwo24, zacc[g][0]);
        v.y = fmaf(oacc[g][0][2] + oacc[g][0][3], kTwo20, zacc[g][0]);
        v.z = fmaf(oacc[g][1][0] + oacc[g][1][1], kTwo24, zacc[g][0]);
        v.w = fmaf(oacc[g][1][2] + oacc[g][1][3], kTwo20, zacc[g][0]);
        *reinterpret_cast<float4*>(wo + ft * HD + d0) = v;
      } else {
        float4 v0, v1;
        v0.x = fmaf(oacc[g][0][0], kTwo24, zacc[g][0]);
        v0.y = fmaf(oacc[g][0][2], kTwo20, zacc[g][0]);
        v0.z = fmaf(oacc[g][1][0], kTwo24, zacc[g][0]);
        v0.w = fmaf(oacc[g][1][2], kTwo20, zacc[g][0]);
        v1.x = fmaf(oacc[g][0][1], kTwo24, zacc[g][NH - 1]);
        v1.y = fmaf(oacc[g][0][3], kTwo20, zacc[g][NH - 1]);
        v1.z = fmaf(oacc[g][1][1], kTwo24, zacc[g][NH - 1]);
        v1.w = fmaf(oacc[g][1][3], kTwo20, zacc[g][NH - 1]);
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
  const int tiles = kWarpsCta >> hpb_log2;
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

template <int HD, int KMODE, int VMODE, bool SPLIT>
int launch_inst(const DecodeArgs& a, const MmaParams& mp, cudaStream_t st) {
  using G = Geo<HD, KMODE>;
  auto kern = decode_mma_kernel<HD, KMODE, VMODE, SPLIT>;
  static int configured_dev = -1;  // per instantiation; the attribute is per device function
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             G::kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return KNLP_ERR_NO_DEVICE;
    }
    configured_dev = dev;
  }
  const int hpb = 1 << mp.hpb_log2;
  dim3 grid(a.n_splits, a.n_kv_heads / hpb, a.n_seqs);
  kern<<<grid, kThreads, G::kSmemBytes, st>>>(a, mp);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

template <int HD, int KMODE, int VMODE>
int launch_split(const DecodeArgs& a, const MmaParams& mp, bool split, cudaStream_t st) {
  return split ? launch_inst<HD, KMODE, VMODE, true>(a, mp, st)
               : launch_inst<HD, KMODE, VMODE, false>(a, mp, st);
}

template <int HD>
int launch_modes(const DecodeArgs& a, const MmaParams& mp, bool split, cudaStream_t st) {
  const int km = a.k.mode, vm = a.v.mode;
  if (km == KNLP_KV_INT4_ASYM && vm == KNLP_KV_INT4_ASYM)
    return launch_split<HD, KNLP_KV_INT4_ASYM, KNLP_KV_INT4_ASYM>(a, mp, split, st);
  if (km == KNLP_KV_INT4_SYM && vm == KNLP_KV_INT4_SYM)
    return launch_split<HD, KNLP_KV_INT4_SYM, KNLP_KV_INT4_SYM>(a, mp, split, st);
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT4_ASYM)
    return launch_split<HD, KNLP_KV_INT8_G32, KNLP_KV_INT4_ASYM>(a, mp, split, st);
  if (km == KNLP_KV_INT8_G32 && vm == KNLP_KV_INT4_SYM)
    return launch_split<HD, KNLP_KV_INT8_G32, KNLP_KV_INT4_SYM>(a, mp, split, st);
  return 1;  // other combinations go to the generic kernel
}

bool aligned(const void* p, uintptr_t n) { return reinterpret_cast<uintptr_t>(p) % n == 0; }

// The copy loop addresses with 32-bit strides and 16-byte pieces.
bool plane_ok(const Plane& p, int head_dim) {
  const int sb = head_dim / 32;  // fp16 elements per scale row
  constexpr int64_t kMax = 0x7fffffff;
  if (!aligned(p.codes, 16)) return false;
  for (int i = 0; i < 3; ++i) {
    if (p.cs[i] % 16 || p.cs[i] < 0 || p.cs[i] > kMax) return false;
    if (p.ss[i] % sb || p.ss[i] < 0 || p.ss[i] > kMax) return false;
    if (p.zeros && (p.zs[i] % sb || p.zs[i] < 0 || p.zs[i] > kMax)) return false;
  }
  if (!aligned(p.scales, sb * 2)) return false;
  if (p.zeros && !aligned(p.zeros, sb * 2)) return false;
  return true;
}

}  // namespace

int launch_decode_mma(const DecodeArgs& a, cudaStream_t st) {
  if (a.head_dim != 64 && a.head_dim != 128) return 1;
  if (a.n_q_heads % a.n_kv_heads) return 1;
  const int n_rep = a.n_q_heads / a.n_kv_heads;
  if (n_rep > 8) return 1;
  if (a.block_size & (a.block_size - 1)) return 1;  // pages must be a power of two
  if (a.num_blocks > 0x7fffffff) return 1;
  if (!plane_ok(a.k, a.head_dim) || !plane_ok(a.v, a.head_dim)) return 1;
  MmaParams mp{};
  mp.hpb_log2 = 3;
  while (mp.hpb_log2 > 0 && (a.n_kv_heads % (1 << mp.hpb_log2))) --mp.hpb_log2;
  mp.page_log2 = 0;
  while ((1 << mp.page_log2) < a.block_size) ++mp.page_log2;
  const bool split = n_rep <= 4;
  return a.head_dim == 128 ? launch_modes<128>(a, mp, split, st)
                           : launch_modes<64>(a, mp, split, st);
}

}  // namespace knlp
