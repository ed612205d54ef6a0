// Low-rank-V decode attention: o = B (sum_i softmax(q.k_i)_i proj_i), the value side kept as
// rank-r coefficients proj_i = B^T v_i with a per-head basis B.  Counterpart of
// pos_quant_v/kernel/vlowrank_kernel.py of the reference (kernel _lowrank_decode :25-75,
// host lowrank_decode :139-156): unquantized K [Hkv, T, dh] (fp16 / bf16, as the queries),
// proj [Hkv, T, r] fp32, basis [Hkv, dh, r] fp32, out [Hkv, nq, dh] fp32.
//
// Two launches.  (1) lowrank_splitk_kernel: grid (split, kv head); a CTA streams its token
// range through shared memory in 64-token stages (cp.async, two stages, four CTAs per SM), the scores of
// a 16-token tile are one ldmatrix + one m16n8k16 MMA per 16 elements of the head
// dimension with the head's queries as the B columns (the K tile is the A operand as it
// lies in memory, as in the unquantized-K mode of the paged decode kernel), the softmax is
// online in the log2 domain, and the r-wide accumulation sum_t p_t proj_t runs on the CUDA
// cores with lane = coefficient index (r = 32: 128 FMAs per token against 512 for the
// scores).  (2) lowrank_finish_kernel: merges the splits' partial states per (head, query)
// and lifts the r coefficients through the basis.
//
// HBM-bound like the paged decode: 2 dh + 4 r bytes per (token, kv head) are read once.

#include <atomic>

#include "decode_mma_common.cuh"

namespace knlp {
namespace {

constexpr int kLrRank = 32;             // coefficients per token: one per lane
constexpr int kLrStageTok = 64;         // tokens per stage: one 16-token tile per warp
constexpr int kLrStages = 2;

template <int DH>
struct LrGeo {
  static constexpr int kKRow = 2 * DH;                       // bytes of a K row
  static constexpr int kKCh = kKRow / 16;                    // 16-byte pieces per K row
  static constexpr int kOffP = kLrStageTok * kKRow;          // proj rows after the K rows
  static constexpr int kStageBytes = kOffP + kLrStageTok * kLrRank * 4;
  static constexpr int kSmemBytes = kLrStages * kStageBytes;
};

// part_m / part_l: [rows][n_splits]; part_o: [rows][n_splits][r]; rows = kv head * nq + query
template <int DH, bool BF16>
__global__ void __launch_bounds__(kThreads)
lowrank_splitk_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k,
                      const float* __restrict__ proj, const int nq, const int T, const int chunk,
                      float* __restrict__ part_m, float* __restrict__ part_l,
                      float* __restrict__ part_o) {
  using G = LrGeo<DH>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(16) float s_p[kWarpsCta][16][8];  // probabilities of a warp's tile: [token][query]
  __shared__ __align__(16) float s_alpha[kWarpsCta][8];  // rescale of the running sums, per query
  __shared__ float s_m[kWarpsCta][8], s_l[kWarpsCta][8];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fr = lane >> 2, ft = lane & 3;
  const int split = blockIdx.x, head = blockIdx.y, n_splits = gridDim.x;
  const int t0 = split * chunk;
  const int t1 = min(T, t0 + chunk);
  const uint32_t smem_base = smem_u32(smem);
  const uint8_t* kh = reinterpret_cast<const uint8_t*>(k) + static_cast<int64_t>(head) * T * G::kKRow;
  const float* ph = proj + static_cast<int64_t>(head) * T * kLrRank;

  // ---- q as B fragments: column n = query n (zero beyond nq), 16 elements per step
  uint32_t bq[DH / 16][2];
  {
    const int col = fr;
    const uint16_t* qrow = q + (static_cast<int64_t>(head) * nq + min(col, nq - 1)) * DH;
#pragma unroll
    for (int j = 0; j < DH / 16; ++j) {
      const uint32_t b0 = __ldg(reinterpret_cast<const uint32_t*>(qrow + 16 * j + 2 * ft));
      const uint32_t b1 = __ldg(reinterpret_cast<const uint32_t*>(qrow + 16 * j + 8 + 2 * ft));
      bq[j][0] = col < nq ? b0 : 0u;
      bq[j][1] = col < nq ? b1 : 0u;
    }
  }

  // ---- copies of one stage: K rows swizzled for ldmatrix, proj rows as they are.  A
  // thread's pieces of a stage lie a fixed distance apart (8 K rows, 16 coefficient rows),
  // so a full stage costs one address per plane and immediate offsets.
  constexpr int kKPer = kLrStageTok * G::kKCh / kThreads;  // K pieces per thread and stage
  constexpr int kKRowStep = kThreads / G::kKCh;            // rows between them
  constexpr int kPPer = kLrStageTok * 8 / kThreads;        // coefficient pieces (8 per row)
  const int k_row = tid / G::kKCh, k_col = tid % G::kKCh;
  const int p_row = tid >> 3, p_col = tid & 7;
  const uint32_t k_dst = k_row * G::kKRow + ((k_col ^ (k_row & 7)) << 4);  // row & 7 survives + 8i
  const uint32_t p_dst = G::kOffP + p_row * 128 + p_col * 16;
  const uint8_t* const k_src = kh + (static_cast<int64_t>(k_row) * G::kKRow + k_col * 16);
  const float* const p_src = ph + (p_row * kLrRank + p_col * 4);
  static_assert(kKRowStep % 8 == 0, "the swizzle of a thread's pieces must not change");
  auto fill = [&](const int c, const int slot) {
    const int tok0 = t0 + c * kLrStageTok;
    const uint32_t base = smem_base + slot * G::kStageBytes;
    if (tok0 + kLrStageTok <= t1) {  // a full stage: no predicates
      const uint8_t* ks = k_src + static_cast<int64_t>(tok0) * G::kKRow;
      const float* ps = p_src + static_cast<int64_t>(tok0) * kLrRank;
#pragma unroll
      for (int i = 0; i < kKPer; ++i)
        cp_async16(base + k_dst + i * kKRowStep * G::kKRow, ks + i * kKRowStep * G::kKRow, 16);
#pragma unroll
      for (int i = 0; i < kPPer; ++i)
        cp_async16(base + p_dst + i * 16 * 128, ps + i * 16 * kLrRank, 16);
    } else if (tok0 < t1) {
#pragma unroll
      for (int i = 0; i < kKPer; ++i) {
        const int row = k_row + i * kKRowStep;
        const bool live = tok0 + row < t1;
        const uint8_t* src = k_src + static_cast<int64_t>(tok0 + i * kKRowStep) * G::kKRow;
        cp_async16(base + k_dst + i * kKRowStep * G::kKRow, live ? src : kh, live ? 16 : 0);
      }
#pragma unroll
      for (int i = 0; i < kPPer; ++i) {
        const int row = p_row + i * 16;
        const bool live = tok0 + row < t1;
        const float* src = p_src + static_cast<int64_t>(tok0 + i * 16) * kLrRank;
        cp_async16(base + p_dst + i * 16 * 128, live ? src : ph, live ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  const int n_chunks = t1 > t0 ? (t1 - t0 + kLrStageTok - 1) / kLrStageTok : 0;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};  // queries 2ft, 2ft + 1
  float acc[8];                                                        // coefficient `lane`
#pragma unroll
  for (int h = 0; h < 8; ++h) acc[h] = 0.0f;
  const float mul = rsqrtf(static_cast<float>(DH)) * 1.4426950408889634f;
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_q = lane >> 4;

  for (int c = 0; c < kLrStages - 1; ++c) fill(c, c);
  for (int c = 0; c < n_chunks; ++c) {
    cp_async_wait<kLrStages - 2>();
    __syncthreads();
    fill(c + kLrStages - 1, (c + kLrStages - 1) % kLrStages);
    const int slot = c % kLrStages;
    const int tok0 = t0 + c * kLrStageTok + warp * 16;
    if (tok0 < t1) {  // warp-uniform
      const uint32_t kt = smem_base + slot * G::kStageBytes + (warp * 16 + lm_row) * G::kKRow;
      float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sacc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < DH / 16; ++j) {  // two chains of dependent MMAs instead of one
        uint32_t w[4];
        ldmatrix_x4_at<0>(kt + (((2 * j + lm_q) ^ (lm_row & 7)) << 4), w);
        float* const dst = (j & 1) ? sacc2 : sacc;
        if constexpr (BF16) {
          mma16816_bf16(dst, w[0], w[1], w[2], w[3], bq[j][0], bq[j][1]);
        } else {
          mma16816(dst, w[0], w[1], w[2], w[3], bq[j][0], bq[j][1]);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) sacc[i] += sacc2[i];
      // sacc: (token fr, queries 2ft, 2ft+1), (token fr + 8, the same queries)
      float sc[2][2];
#pragma unroll
      for (int rh = 0; rh < 2; ++rh)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          sc[rh][h] = tok0 + fr + 8 * rh < t1 ? sacc[2 * rh + h] * mul : -INFINITY;
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float tmax = fmaxf(sc[0][h], sc[1][h]);
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
        const float m_new = fmaxf(m_run[h], tmax);  // finite: the tile has a valid token
        alpha[h] = fast_exp2(m_run[h] - m_new);
        m_run[h] = m_new;
        const float p0 = fast_exp2(sc[0][h] - m_new), p1 = fast_exp2(sc[1][h] - m_new);
        float ps = p0 + p1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 4);
        ps += __shfl_xor_sync(0xffffffffu, ps, 8);
        ps += __shfl_xor_sync(0xffffffffu, ps, 16);
        l_run[h] = l_run[h] * alpha[h] + ps;
        s_p[warp][fr][2 * ft + h] = p0;
        s_p[warp][fr + 8][2 * ft + h] = p1;
      }
      if (fr == 0) {
        s_alpha[warp][2 * ft] = alpha[0];
        s_alpha[warp][2 * ft + 1] = alpha[1];
      }
      __syncwarp();
      // coefficient `lane` of every query: acc = acc * alpha + sum_t p[t] proj[t][lane]
      {
        const float4 a0 = *reinterpret_cast<const float4*>(&s_alpha[warp][0]);
        const float4 a1 = *reinterpret_cast<const float4*>(&s_alpha[warp][4]);
        acc[0] *= a0.x; acc[1] *= a0.y; acc[2] *= a0.z; acc[3] *= a0.w;
        acc[4] *= a1.x; acc[5] *= a1.y; acc[6] *= a1.z; acc[7] *= a1.w;
        const float* pt = reinterpret_cast<const float*>(smem + slot * G::kStageBytes + G::kOffP) +
                          warp * 16 * kLrRank + lane;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const float x = pt[t * kLrRank];
          const float4 p0 = *reinterpret_cast<const float4*>(&s_p[warp][t][0]);
          const float4 p1 = *reinterpret_cast<const float4*>(&s_p[warp][t][4]);
          acc[0] = fmaf(p0.x, x, acc[0]); acc[1] = fmaf(p0.y, x, acc[1]);
          acc[2] = fmaf(p0.z, x, acc[2]); acc[3] = fmaf(p0.w, x, acc[3]);
          acc[4] = fmaf(p1.x, x, acc[4]); acc[5] = fmaf(p1.y, x, acc[5]);
          acc[6] = fmaf(p1.z, x, acc[6]); acc[7] = fmaf(p1.w, x, acc[7]);
        }
      }
      __syncwarp();  // s_p and s_alpha are rewritten by the next tile
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // the stages are dead: their memory takes the warps' sums

  // ---- merge the four warps, write the split's partial (m in the natural-log domain)
  float (*s_o)[8][kLrRank] = reinterpret_cast<float (*)[8][kLrRank]>(smem);
  if (fr == 0) {
    s_m[warp][2 * ft] = m_run[0];
    s_m[warp][2 * ft + 1] = m_run[1];
    s_l[warp][2 * ft] = l_run[0];
    s_l[warp][2 * ft + 1] = l_run[1];
  }
#pragma unroll
  for (int h = 0; h < 8; ++h) s_o[warp][h][lane] = acc[h];
  __syncthreads();
  for (int i = tid; i < nq * kLrRank; i += kThreads) {
    const int h = i / kLrRank, e = i % kLrRank;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarpsCta; ++w) m = fmaxf(m, s_m[w][h]);
    float l = 0.0f, o = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarpsCta; ++w) {
      const float f = s_m[w][h] == -INFINITY ? 0.0f : fast_exp2(s_m[w][h] - m);
      l = fmaf(s_l[w][h], f, l);
      o = fmaf(s_o[w][h][e], f, o);
    }
    const int64_t row = static_cast<int64_t>(head) * nq + h;
    part_o[(row * n_splits + split) * kLrRank + e] = o;
    if (e == 0) {
      part_m[row * n_splits + split] = m * 0.6931471805599453f;
      part_l[row * n_splits + split] = l;
    }
  }
}

// One CTA per (kv head, query) row: merge the splits into the r coefficients za (warp 0,
// lane = coefficient), then out[d] = sum_r za[r] basis[head][d][r].
__global__ void __launch_bounds__(kThreads)
lowrank_finish_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                      const float* __restrict__ part_o, const int n_splits, const int nq,
                      const float* __restrict__ basis, const int dh, float* __restrict__ za_out,
                      float* __restrict__ out) {
  __shared__ float s_za[kLrRank];
  __shared__ float s_wl[kWarpsCta], s_wz[kWarpsCta][kLrRank];
  const int row = blockIdx.x, head = row / nq;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* pm = part_m + static_cast<int64_t>(row) * n_splits;
  const float* pl = part_l + static_cast<int64_t>(row) * n_splits;
  const float* po = part_o + static_cast<int64_t>(row) * n_splits * kLrRank;
  // the row's maximum (every warp computes it), then each warp sums a quarter of the splits
  float m = -INFINITY;
  for (int p = lane; p < n_splits; p += 32) {
    const float lp = pl[p], mp = pm[p];
    m = fmaxf(m, lp > 0.0f ? mp : -INFINITY);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float l = 0.0f, z = 0.0f;
#pragma unroll 4
  for (int p = warp; p < n_splits; p += kWarpsCta) {
    const float lp = pl[p], mp = pm[p], zp = po[p * kLrRank + lane];  // issued together
    const float f = lp > 0.0f ? __expf(mp - m) : 0.0f;
    l = fmaf(lp, f, l);
    z = fmaf(lp > 0.0f ? zp : 0.0f, f, z);
  }
  s_wz[warp][lane] = z;
  if (lane == 0) s_wl[warp] = l;
  __syncthreads();
  if (tid < 32) {
    float lt = 0.0f, zt = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarpsCta; ++w) {
      lt += s_wl[w];
      zt += s_wz[w][lane];
    }
    const float za = lt > 0.0f ? zt / lt : 0.0f;
    s_za[lane] = za;
    if (za_out) za_out[static_cast<int64_t>(row) * kLrRank + lane] = za;
  }
  __syncthreads();
  for (int d = tid; d < dh; d += kThreads) {
    const float4* b = reinterpret_cast<const float4*>(
        basis + (static_cast<int64_t>(head) * dh + d) * kLrRank);
    float o = 0.0f;
#pragma unroll
    for (int i = 0; i < kLrRank / 4; ++i) {
      const float4 v = __ldg(b + i);
      o = fmaf(s_za[4 * i], v.x, o);
      o = fmaf(s_za[4 * i + 1], v.y, o);
      o = fmaf(s_za[4 * i + 2], v.z, o);
      o = fmaf(s_za[4 * i + 3], v.w, o);
    }
    out[static_cast<int64_t>(row) * dh + d] = o;
  }
}

template <int DH, bool BF16>
int launch_lr(const void* q, const void* k, const float* proj, int n_kv_heads, int nq, int T,
              int n_splits, int chunk, float* pm, float* pl, float* po, cudaStream_t st) {
  using G = LrGeo<DH>;
  auto kern = lowrank_splitk_kernel<DH, BF16>;
  static std::atomic<uint64_t> configured{0};
  int dev = 0;
  cudaGetDevice(&dev);
  const uint64_t bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes) !=
        cudaSuccess) {
      cudaGetLastError();
      return KNLP_ERR_NO_DEVICE;
    }
    configured.fetch_or(bit, std::memory_order_release);
  }
  kern<<<dim3(n_splits, n_kv_heads), kThreads, G::kSmemBytes, st>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(k), proj, nq, T, chunk, pm, pl,
      po);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

}  // namespace

// Split count: as many CTAs as the machine holds at once (four fit an SM; twice and four
// times as many, smaller splits measured slower), no split below 256 tokens.
int lowrank_plan(int n_kv_heads, int T, int n_sms, int* chunk_out) {
  int n = 4 * n_sms / n_kv_heads;
  const int cap = (T + 255) / 256;
  if (n > cap) n = cap;
  if (n < 1) n = 1;
  int chunk = (T + n - 1) / n;
  chunk = (chunk + kLrStageTok - 1) / kLrStageTok * kLrStageTok;
  if (chunk < kLrStageTok) chunk = kLrStageTok;
  n = T > 0 ? (T + chunk - 1) / chunk : 1;
  *chunk_out = chunk;
  return n;
}

int launch_lowrank_decode(const void* q, const void* k, int qk_dtype, const float* proj,
                          const float* basis, int n_kv_heads, int nq, int T, int head_dim,
                          int n_sms, float* ws, int64_t ws_floats, float* za_out, float* out,
                          cudaStream_t st) {
  int chunk = 0;
  const int n_splits = lowrank_plan(n_kv_heads, T, n_sms, &chunk);
  const int64_t rows = static_cast<int64_t>(n_kv_heads) * nq;
  if (ws_floats < rows * n_splits * (kLrRank + 2)) return KNLP_ERR_WORKSPACE;
  float* po = ws;
  float* pm = ws + rows * n_splits * kLrRank;
  float* pl = pm + rows * n_splits;
  const bool bf16 = qk_dtype == KNLP_BF16;
  int rc;
  if (head_dim == 128) {
    rc = bf16 ? launch_lr<128, true>(q, k, proj, n_kv_heads, nq, T, n_splits, chunk, pm, pl, po, st)
              : launch_lr<128, false>(q, k, proj, n_kv_heads, nq, T, n_splits, chunk, pm, pl, po, st);
  } else {
    rc = bf16 ? launch_lr<64, true>(q, k, proj, n_kv_heads, nq, T, n_splits, chunk, pm, pl, po, st)
              : launch_lr<64, false>(q, k, proj, n_kv_heads, nq, T, n_splits, chunk, pm, pl, po, st);
  }
  if (rc != KNLP_OK) return rc;
  lowrank_finish_kernel<<<static_cast<unsigned>(rows), kThreads, 0, st>>>(
      pm, pl, po, n_splits, nq, basis, head_dim, za_out, out);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

int64_t lowrank_workspace_floats(int n_kv_heads, int nq, int T, int n_sms) {
  int chunk = 0;
  const int n_splits = lowrank_plan(n_kv_heads, T, n_sms, &chunk);
  return static_cast<int64_t>(n_kv_heads) * nq * n_splits * (kLrRank + 2);
}

}  // namespace knlp
