// The quantizers of one 32-element group, four elements per lane (eight lanes a group),
// shared by the quantize-append kernel for general layouts and by the decode kernel that
// appends the step's new token itself.  Arithmetic of the reference's cache-write kernels
// (fused-quant/fused_int4.v0.1.0.py:308-327 asymmetric, :328-357 symmetric with outlier
// clip, :1270-1284 INT8), bit for bit: every step that decides a code or a stored fp16 is
// an explicit round-to-nearest intrinsic (never contracted into an FMA, never a
// reciprocal), rounding is round-half-away-from-zero written as floor(y + 0.5) /
// ceil(y - 0.5) with an fp32 add (:199-202).  All 32 lanes of the warp must call.
#pragma once

#include "common.cuh"

namespace knlp {

__device__ __forceinline__ float rha(float y) {
  return y >= 0.0f ? floorf(__fadd_rn(y, 0.5f)) : ceilf(__fsub_rn(y, 0.5f));
}

__device__ __forceinline__ float group_min(float v) {
  v = fminf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fminf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fminf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}
__device__ __forceinline__ float group_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}

// Sum of the 32 values of a group (a[s] = this lane's element s; lane L of the
// group holds elements 4L..4L+3) in the order numpy's pairwise reduction uses for
// 32 contiguous floats: r[j] = ((e[j] + e[8+j]) + e[16+j]) + e[24+j], then
// ((r0+r1)+(r2+r3)) + ((r4+r5)+(r6+r7)).  The reference's trimmed mean
// (:339-343) is reduced in that order when its kernel runs under the Triton
// interpreter, which is where the golden vectors come from.
__device__ __forceinline__ float group_sum_numpy_order(const float a[4], int lane) {
  const int gbase = lane & ~7;
  const int par = lane & 1;
  float r[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    float v0 = __shfl_sync(0xffffffffu, a[s], gbase + par + 0);
    float v1 = __shfl_sync(0xffffffffu, a[s], gbase + par + 2);
    float v2 = __shfl_sync(0xffffffffu, a[s], gbase + par + 4);
    float v3 = __shfl_sync(0xffffffffu, a[s], gbase + par + 6);
    r[s] = __fadd_rn(__fadd_rn(__fadd_rn(v0, v1), v2), v3);
  }
  // even lanes hold r[0..3], odd lanes r[4..7]
  float half = __fadd_rn(__fadd_rn(r[0], r[1]), __fadd_rn(r[2], r[3]));
  float other = __shfl_xor_sync(0xffffffffu, half, 1);
  return __fadd_rn(half, other);
}

// Quantizes this lane's four elements x of its group.  c: the stored codes (INT4: 0..15,
// offset binary in the symmetric mode; INT8: -128..127); sc: the group's scale and mn its
// zero-point (asymmetric mode only) BEFORE their rounding to fp16.
__device__ __forceinline__ void quantize4(int mode, const float x[4], int lane, float clip_ratio,
                                          int c[4], float& sc, float& mn) {
  mn = 0.0f;
  if (mode == KNLP_KV_INT4_ASYM) {
    mn = group_min(fminf(fminf(x[0], x[1]), fminf(x[2], x[3])));
    const float mx = group_max(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])));
    const float range = fmaxf(__fsub_rn(mx, mn), 1e-8f);
    sc = __fdiv_rn(range, 15.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float q = rha(__fdiv_rn(__fsub_rn(x[i], mn), sc));
      q = fmaxf(fminf(q, 15.0f), 0.0f);
      c[i] = static_cast<int>(static_cast<unsigned>(q));
    }
  } else if (mode == KNLP_KV_INT4_SYM) {
    const float a[4] = {fabsf(x[0]), fabsf(x[1]), fabsf(x[2]), fabsf(x[3])};
    float amax = group_max(fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3])));
    amax = fmaxf(amax, 1e-8f);
    if (clip_ratio > 0.0f) {
      float below[4], ind[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool lt = a[i] < amax;
        below[i] = lt ? a[i] : 0.0f;
        ind[i] = lt ? 1.0f : 0.0f;
      }
      const float cnt = fmaxf(group_sum_numpy_order(ind, lane), 1.0f);
      const float tmean = __fdiv_rn(group_sum_numpy_order(below, lane), cnt);
      const float clip = __fmul_rn(tmean, clip_ratio);
      amax = fminf(amax, fmaxf(clip, 1e-8f));
    }
    sc = __fdiv_rn(amax, 7.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float q = rha(__fdiv_rn(x[i], sc));
      q = fmaxf(fminf(q, 7.0f), -8.0f);
      c[i] = static_cast<int>(static_cast<unsigned>(__fadd_rn(q, 8.0f)));
    }
  } else {  // KNLP_KV_INT8_G32
    float amax = group_max(
        fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
    amax = fmaxf(amax, 1e-8f);
    sc = __fdiv_rn(amax, 127.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float q = rha(__fdiv_rn(x[i], sc));
      q = fmaxf(fminf(q, 127.0f), -128.0f);
      c[i] = static_cast<int>(q);
    }
  }
}

// Stores the four codes of a lane (elements e0..e0+3 of the row) and, by the group's
// leading lane, the fp16 scale and zero-point.  wide: the code row allows 2-byte (INT4) /
// 4-byte (INT8) stores.
__device__ __forceinline__ void store_quantized4(int mode, const int c[4], float sc, float mn,
                                                 uint8_t* crow, __half* srow, __half* zrow,
                                                 int e0, bool leader, bool wide) {
  if (mode == KNLP_KV_INT8_G32) {
    if (wide) {
      const unsigned w32 = (c[0] & 0xff) | ((c[1] & 0xff) << 8) | ((c[2] & 0xff) << 16) |
                           (static_cast<unsigned>(c[3] & 0xff) << 24);
      *reinterpret_cast<unsigned*>(crow + e0) = w32;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) crow[e0 + i] = static_cast<uint8_t>(c[i] & 0xff);
    }
  } else {
    const unsigned b0 = c[0] | (c[1] << 4), b1 = c[2] | (c[3] << 4);
    if (wide) {
      *reinterpret_cast<uint16_t*>(crow + (e0 >> 1)) = static_cast<uint16_t>(b0 | (b1 << 8));
    } else {
      crow[(e0 >> 1)] = static_cast<uint8_t>(b0);
      crow[(e0 >> 1) + 1] = static_cast<uint8_t>(b1);
    }
  }
  if (leader) {
    srow[e0 >> 5] = __float2half_rn(sc);
    if (mode == KNLP_KV_INT4_ASYM) zrow[e0 >> 5] = __float2half_rn(mn);
  }
}

}  // namespace knlp
