// Device helpers shared by the tensor-core decode kernels (sm_100a): cp.async, ldmatrix,
// mma.sync and mbarrier / TMA wrappers, the conversion-free unpack of packed codes into
// fp16 MMA operands, and the shared-memory geometry of a pipeline stage.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "common.cuh"

namespace knlp {

constexpr int kWarpsCta = kDecodeWarps;
constexpr int kWarpsLog = kWarpsCta == 8 ? 3 : kWarpsCta == 4 ? 2 : 1;
constexpr int kCtasPerSm = kDecodeCtasPerSm;
constexpr int kThreads = kWarpsCta * 32;
constexpr int kMaxStages = 4;  // pipeline depth; one less where shared memory is short
constexpr int kRows = kWarpsCta * 16;  // (token, head) rows per stage

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// .ca (allocate in L1) rather than .cg: the fills reach shared memory in fewer, wider
// writes.  The data is streamed once either way.
#define KNLP_CP_MODE "ca"
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async." KNLP_CP_MODE ".shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
template <int BYTES>  // 4- or 8-byte piece, zero-filled beyond src_bytes
__device__ __forceinline__ void cp_async_small(uint32_t dst, const void* src, int src_bytes) {
  static_assert(BYTES == 4 || BYTES == 8, "cp.async piece sizes below 16 are 4 and 8");
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;\n" ::"r"(dst), "l"(src), "n"(BYTES),
               "r"(src_bytes)
               : "memory");
}
template <int OFF>  // destination = dst + OFF, the offset folded into the address operand
__device__ __forceinline__ void cp_async16_full_at(uint32_t dst, const void* src) {
  asm volatile("cp.async." KNLP_CP_MODE ".shared.global [%0+%2], [%1], 16;\n" ::"r"(dst), "l"(src),
               "n"(OFF)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ldmatrix x4 (and its transposing form) with a compile-time byte offset folded into the
// address operand
template <int OFF>
__device__ __forceinline__ void ldmatrix_x4_at(uint32_t addr, uint32_t r[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ void ldmatrix_x4_trans_at(uint32_t addr, uint32_t r[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr), "n"(OFF));
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
// the same with bf16 inputs (an unquantized bf16 K plane against q split into bf16 parts)
__device__ __forceinline__ void mma16816_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// ---- mbarrier + TMA (cp.async.bulk.tensor) primitives, CTA scope, no multicast ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kWaitLimitNs of wall time (the %globaltimer), so a lost
// completion ends the kernel within milliseconds instead of hanging it.
constexpr unsigned long long kWaitLimitNs = 2000000ull;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  do {
    if (mbar_try_wait(bar, parity)) return true;
  } while (global_ns() - t0 < kWaitLimitNs);
  return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Tensor maps of one launch, passed by value as a __grid_constant__ parameter.
// Every code box has 128-byte rows under the 128-byte swizzle, because shared-memory
// fills are only efficient in whole 128-byte lines:
//   k, v   wide (the CTA's heads of one token span >= 128 bytes): 4-D (128 bytes,
//          128-byte columns of a token row, tokens of a page, blocks), box = one
//          column x 16 tokens, i.e. 128/row_bytes adjacent heads per shared-memory row;
//          narrow (they span < 128 bytes and the tokens of the CTA's heads are
//          contiguous): 3-D (128 bytes, 128-byte rows of a page, blocks), box = the rows
//          of 16 tokens, i.e. several tokens per shared-memory row
//   ks..vz 3-D byte tensors of the scale / zero arrays; box = 16 tokens x the kv heads
//          of the CTA, as [token][head] rows (scale_merged: the box is one contiguous run)
struct alignas(64) TmaMaps {
  CUtensorMap k, v, ks, kz, vs, vz;
  int scale_merged;
  int k_narrow, v_narrow;
};

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

// Eight nibbles of a 32-bit word -> four fp16x2 registers of fp16 SUBNORMALS
// (n_i = bits [4i, 4i+4) of the word):
//   out[0] = (n0,          n4         ) * 2^-24
//   out[1] = (n0 + 16 n1,  n4 + 16 n5 ) * 2^-24      a whole byte left in place
//   out[2] = (n2,          n6         ) * 2^-24
//   out[3] = (n2 + 16 n3,  n6 + 16 n7 ) * 2^-24
// A half whose exponent field is zero has the value mantissa * 2^-24, so masking in
// place is the whole conversion (a byte still fits the 10-bit mantissa).  The odd
// nibbles are never isolated - that would need a shift per word; instead the other
// operand of the product absorbs the mix:
//   n0 q0 + n1 q1 = n0 (q0 - q1/16) + (n0 + 16 n1) (q1/16)          (scores)
// or the pure row is subtracted from the mixed one afterwards          (output rows).
__device__ __forceinline__ void unpack_nibbles8(uint32_t w, uint32_t out[4]) {
  out[0] = w & 0x000F000Fu;
  out[1] = w & 0x00FF00FFu;
  out[3] = __byte_perm(w, 0u, 0x4341);  // bytes 1 and 3 moved down, upper bytes cleared
  out[2] = out[3] & 0x000F000Fu;
}
// The same with every nibble isolated (one more instruction per word):
//   out[0] = (n0, n4) * 2^-24   out[1] = (n1, n5) * 2^-20
//   out[2] = (n2, n6) * 2^-24   out[3] = (n3, n7) * 2^-20
// Used for the scores when q is held as a single fp16 (5..8 q heads per kv head): there
// the q slot of an odd nibble is just q_odd / 16 (exact), while the mixed form above
// would round q_even - q_odd / 16 a second time.
__device__ __forceinline__ void unpack_nibbles8_pure(uint32_t w, uint32_t out[4]) {
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

// A transposed int8 V register: bytes 0, 1 = elements d, d+1 of one token, bytes 2, 3 the
// same elements of the next token.  Biased to unsigned and split by element:
// out[0] = (d of both tokens), out[1] = (d+1 of both tokens), fp16 subnormals * 2^-24.
__device__ __forceinline__ void unpack_int8_pairs(uint32_t w, uint32_t out[2]) {
  const uint32_t u = w ^ 0x80808080u;
  out[0] = u & 0x00FF00FFu;
  out[1] = __byte_perm(u, 0u, 0x4341);
}

// Shared-memory geometry of a stage.  PAD (cp.async path: kTilePad = 64 bytes) separates
// the 16-row code tiles of the warps.  A warp-wide copy of a token row scatters one 64-byte
// run per head, i.e. per tile; with tiles half a 128-byte line apart the runs of two heads
// complete one line between them.
constexpr int kTilePad = 64;
template <int HD, int KMODE, int VMODE, int PAD>
struct Geo {
  static constexpr bool kInt8K = (KMODE == KNLP_KV_INT8_G32);
  static constexpr bool kInt8V = (VMODE == KNLP_KV_INT8_G32);
  // an unquantized fp16 / bf16 K plane: rows of 2 * HD bytes, no scale or zero rows
  static constexpr bool kFpK = (KMODE == KNLP_KV_F16 || KMODE == KNLP_KV_BF16);
  static constexpr int NG = HD / 32;
  static constexpr int KB = kFpK ? 2 * HD : kInt8K ? HD : HD / 2;  // K row bytes
  static constexpr int VB = kInt8V ? HD : HD / 2;  // V row bytes
  static constexpr int KCH = KB / 16;              // 16-byte pieces per K row
  static constexpr int VCH = VB / 16;
  static constexpr int SB = NG * 2;                // scale row bytes
  static constexpr int kTileK = 16 * KB + PAD;     // one warp's 16 K rows
  static constexpr int kTileV = 16 * VB + PAD;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kOffK + kWarpsCta * kTileK;
  static constexpr int kOffKs = kOffV + kWarpsCta * kTileV;
  static constexpr int kOffKz = kOffKs + (kFpK ? 0 : kRows * SB);
  static constexpr int kOffVs = kOffKz + (kFpK ? 0 : kRows * SB);
  static constexpr int kOffVz = kOffVs + kRows * SB;
  static constexpr int kStageBytes = kOffVz + kRows * SB;
  // Four stages, or three where four would no longer let kCtasPerSm CTAs share the
  // 227 KB of an SM (the INT8 planes); depth 3 and 4 measured the same.
  static constexpr int kStages =
      kCtasPerSm * (kMaxStages * kStageBytes + 2048) <= 232448 ? kMaxStages : kMaxStages - 1;
  static constexpr int kSmemBytes = kStages * kStageBytes;
};

// xor swizzle of the 16-byte column index of row r (0..15) for rows of CH pieces
template <int CH>
__device__ __forceinline__ int swz(int r) {
  if constexpr (CH >= 8) {
    return r & 7;  // rows of 128 bytes or more: the eight rows of an 8x8 matrix differ
  } else {
    return (r / (8 / CH)) & (CH - 1);
  }
}

// Extra launch parameters computed on the host.
struct MmaParams {
  int hpb_log2;   // kv heads per CTA = 1 << hpb_log2
  int page_log2;  // block_size = 1 << page_log2
  int* status;    // device status word: set to 1 by a kernel whose bounded wait ran out
  int debug_stall;  // test aid (TMA staging): the first stage announces more bytes than it copies
};

// Calls f(it0 + S, integral_constant<S>) for S = FIRST .. N-1 while it0 + S < n; stops
// and returns false as soon as a call does.
// (CHECK = false: the caller guarantees it0 + N <= n.)
template <int S, int N, bool CHECK = true, class F>
__device__ __forceinline__ bool run_stages(F& f, int it0, int n) {
  if constexpr (S < N) {
    if (CHECK && it0 + S >= n) return true;
    if (!f(it0 + S, std::integral_constant<int, S>{})) return false;
    return run_stages<S + 1, N, CHECK>(f, it0, n);
  } else {
    return true;
  }
}

}  // namespace knlp
