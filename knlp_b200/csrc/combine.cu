// Merge (m, l, o) softmax partials of split-context decode attention (sm_100a).
//
// The reference has no split path, hence no such kernel; the algebra is the
// online-softmax recurrence of its decode loop
// (fused-quant/fused_int4.v0.1.0.py:808-815, 883-887) applied across parts:
//   m = max_i m_i,  l = sum_i l_i e^(m_i - m),  o = sum_i o_i e^(m_i - m) [/ l]
// One CTA per (sequence, q head) row; a thread owns head_dim/blockDim elements.
// Parts with l == 0 (empty splits) are skipped; a row with no tokens gives 0.

#include "common.cuh"

namespace knlp {
namespace {

constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads)
combine_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
               const float* __restrict__ po, int n_parts, int64_t ml_row, int64_t ml_part,
               int64_t o_row, int64_t o_part, void* out, int out_dtype, int64_t out_row,
               float* out_m, float* out_l, int64_t out_ml, int head_dim) {
  const int64_t row = blockIdx.x;
  const float* rm = pm + row * ml_row;
  const float* rl = pl + row * ml_row;
  const float* ro = po + row * o_row;

  float m = -INFINITY;
  for (int p = 0; p < n_parts; ++p) {
    if (rl[p * ml_part] > 0.0f) m = fmaxf(m, rm[p * ml_part]);
  }
  for (int e = threadIdx.x; e < head_dim; e += kThreads) {
    float l = 0.0f, o = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
      const float lp = rl[p * ml_part];
      if (lp > 0.0f) {
        const float w = __expf(rm[p * ml_part] - m);
        l += lp * w;
        o += ro[p * o_part + e] * w;
      }
    }
    if (out_m != nullptr) {
      static_cast<float*>(out)[row * out_row + e] = o;
      if (e == 0) {
        out_m[row * out_ml] = m;
        out_l[row * out_ml] = l;
      }
    } else {
      store_elem_rt(out, row * out_row + e, l > 0.0f ? o / l : 0.0f, out_dtype);
    }
  }
}

}  // namespace

int launch_combine(const float* pm, const float* pl, const float* po, int n_parts,
                   int64_t ml_row, int64_t ml_part, int64_t o_row, int64_t o_part, void* out,
                   int out_dtype, int64_t out_row, float* out_m, float* out_l, int64_t out_ml,
                   int n_rows, int head_dim, cudaStream_t st) {
  if (n_rows == 0) return KNLP_OK;
  combine_kernel<<<n_rows, kThreads, 0, st>>>(pm, pl, po, n_parts, ml_row, ml_part, o_row, o_part,
                                              out, out_dtype, out_row, out_m, out_l, out_ml, head_dim);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

}  // namespace knlp
