// Merge (m, l, o) softmax partials of split-context decode attention (sm_100a).
//
// The reference has no split path, hence no such kernel; the algebra is the
// online-softmax recurrence of its decode loop
// (fused-quant/fused_int4.v0.1.0.py:808-815, 883-887) applied across parts:
//   m = max_i m_i,  l = sum_i l_i e^(m_i - m),  o = sum_i o_i e^(m_i - m) [/ l]
// One CTA of 8 warps per (sequence, q head) row.  The parts are dealt to the warps
// round-robin and every lane owns head_dim/32 consecutive elements, so a warp reads
// one part's o row as one contiguous run and the loads of different parts are
// independent (several in flight per warp).  The warps' sums meet in shared memory.
// Parts with l == 0 (empty splits) are skipped; a row with no tokens gives 0.

#include "common.cuh"

namespace knlp {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxEpl = 8;  // head_dim <= 256

__global__ void __launch_bounds__(kThreads)
combine_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
               const float* __restrict__ po, int n_parts, int64_t ml_row, int64_t ml_part,
               int64_t o_row, int64_t o_part, void* out, int out_dtype, int64_t out_row,
               float* out_m, float* out_l, int64_t out_ml, int head_dim) {
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* rm = pm + row * ml_row;
  const float* rl = pl + row * ml_row;
  const float* ro = po + row * o_row;
  const int epl = head_dim >> 5;  // elements per lane (head_dim is a multiple of 32)

  __shared__ float s_red[kWarps];
  __shared__ float s_l[kWarps];
  __shared__ float s_o[kWarps][32 * kMaxEpl];

  // global maximum over the non-empty parts
  float m = -INFINITY;
  for (int p = threadIdx.x; p < n_parts; p += kThreads) {
    const float lp = rl[p * ml_part], mp = rm[p * ml_part];  // both loads issued at once
    m = fmaxf(m, lp > 0.0f ? mp : -INFINITY);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) m = fmaxf(m, s_red[w]);

  // this warp's share of the parts
  float l = 0.0f;
  float acc[kMaxEpl];
#pragma unroll
  for (int i = 0; i < kMaxEpl; ++i) acc[i] = 0.0f;
  // every load of a part is issued whatever its weight turns out to be (a value of an
  // empty part is dropped by the select, not by skipping its load): no load waits for
  // another, and four parts are in flight per warp
#pragma unroll 4
  for (int p = warp; p < n_parts; p += kWarps) {
    const float lp = rl[p * ml_part];
    const float mp = rm[p * ml_part];
    const float* src = ro + p * o_part + lane * epl;
    float v[kMaxEpl];
#pragma unroll
    for (int i = 0; i < kMaxEpl; ++i) v[i] = i < epl ? src[i] : 0.0f;
    const float w = lp > 0.0f ? __expf(mp - m) : 0.0f;
    l += lp * w;
#pragma unroll
    for (int i = 0; i < kMaxEpl; ++i)
      if (i < epl) acc[i] = fmaf(w > 0.0f ? v[i] : 0.0f, w, acc[i]);
  }
  if (lane == 0) s_l[warp] = l;
#pragma unroll
  for (int i = 0; i < kMaxEpl; ++i)
    if (i < epl) s_o[warp][lane * epl + i] = acc[i];
  __syncthreads();

  for (int e = threadIdx.x; e < head_dim; e += kThreads) {
    float lt = 0.0f, ot = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      lt += s_l[w];
      ot += s_o[w][e];
    }
    if (out_m != nullptr) {
      static_cast<float*>(out)[row * out_row + e] = ot;
      if (e == 0) {
        out_m[row * out_ml] = m;
        out_l[row * out_ml] = lt;
      }
    } else {
      store_elem_rt(out, row * out_row + e, lt > 0.0f ? ot / lt : 0.0f, out_dtype);
    }
  }
}

// Merge of the balanced decode kernel's partial slots.  The parts of a pair are
// consecutive slots of `heads` rows each; pair_info holds (first slot, parts) per pair.
// Grid (row, 32-element slice of the head): with one long sequence spread over the whole
// machine a row has hundreds of parts, and the slices give the merge enough CTAs.  The
// kernel is launched as a programmatic dependent of the decode kernel: it may become
// resident while that one drains and waits here for its memory to be complete.
__global__ void __launch_bounds__(kThreads)
combine_pairs_kernel(const float* __restrict__ ws_m, const float* __restrict__ ws_l,
                     const float* __restrict__ ws_o, const int* __restrict__ pair_info,
                     int heads, int head_dim, void* out, int out_dtype, int64_t out_row,
                     int emit_partial) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const int row = blockIdx.x;
  const int pair = row / heads, r = row % heads;
  const int e = blockIdx.y * 32 + (threadIdx.x & 31);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot0 = pair_info[2 * pair];
  const int parts = pair_info[2 * pair + 1];
  const float* rm = ws_m + static_cast<int64_t>(slot0) * heads + r;
  const float* rl = ws_l + static_cast<int64_t>(slot0) * heads + r;
  const float* ro = ws_o + (static_cast<int64_t>(slot0) * heads + r) * head_dim + e;
  const int64_t o_part = static_cast<int64_t>(heads) * head_dim;

  __shared__ float s_red[kWarps];
  __shared__ float s_l[kWarps];
  __shared__ float s_o[kWarps][32];

  float m = -INFINITY;
  for (int p = threadIdx.x; p < parts; p += kThreads) {
    const float lp = __ldcg(rl + p * heads), mp = __ldcg(rm + p * heads);
    m = fmaxf(m, lp > 0.0f ? mp : -INFINITY);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) m = fmaxf(m, s_red[w]);

  // all three loads of a part are issued unconditionally and eight parts at a time: with
  // four warps on the SM only loads in flight hide the round trips to L2
  float l = 0.0f, acc = 0.0f;
#pragma unroll 8
  for (int p = warp; p < parts; p += kWarps) {
    const float lp = __ldcg(rl + p * heads);
    const float mp = __ldcg(rm + p * heads);
    const float op = __ldcg(ro + p * o_part);
    const float w = lp > 0.0f ? __expf(mp - m) : 0.0f;
    l = fmaf(lp, w, l);
    acc = fmaf(lp > 0.0f ? op : 0.0f, w, acc);
  }
  if (lane == 0) s_l[warp] = l;
  s_o[warp][lane] = acc;
  __syncthreads();
  if (warp == 0) {
    float lt = 0.0f, ot = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      lt += s_l[w];
      ot += s_o[w][lane];
    }
    if (emit_partial) {
      float* orow = static_cast<float*>(out) + row * out_row;
      orow[e] = ot;
      if (e == 0) {
        orow[head_dim] = m;
        orow[head_dim + 1] = lt;
      }
    } else {
      store_elem_rt(out, row * out_row + e, lt > 0.0f ? ot / lt : 0.0f, out_dtype);
    }
  }
}

}  // namespace

int launch_combine_pairs(const float* ws_m, const float* ws_l, const float* ws_o,
                         const int* pair_info, int heads, int n_rows, int head_dim, void* out,
                         int out_dtype, int64_t out_row, bool emit_partial, cudaStream_t st) {
  if (n_rows == 0) return KNLP_OK;
  if (head_dim % 32) return KNLP_ERR_SHAPE;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(n_rows, head_dim / 32);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int emit = emit_partial ? 1 : 0;
  const cudaError_t rc =
      cudaLaunchKernelEx(&cfg, combine_pairs_kernel, ws_m, ws_l, ws_o, pair_info, heads, head_dim,
                         out, out_dtype, out_row, emit);
  if (rc != cudaSuccess) {
    cudaGetLastError();
    return KNLP_ERR_LAUNCH;
  }
  return KNLP_OK;
}

int launch_combine(const float* pm, const float* pl, const float* po, int n_parts,
                   int64_t ml_row, int64_t ml_part, int64_t o_row, int64_t o_part, void* out,
                   int out_dtype, int64_t out_row, float* out_m, float* out_l, int64_t out_ml,
                   int n_rows, int head_dim, cudaStream_t st) {
  if (n_rows == 0) return KNLP_OK;
  if (head_dim % 32 || head_dim > 32 * kMaxEpl) return KNLP_ERR_SHAPE;
  combine_kernel<<<n_rows, kThreads, 0, st>>>(pm, pl, po, n_parts, ml_row, ml_part, o_row, o_part,
                                              out, out_dtype, out_row, out_m, out_l, out_ml,
                                              head_dim);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

}  // namespace knlp
