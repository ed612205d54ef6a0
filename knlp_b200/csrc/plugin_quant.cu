// Plugin-level simulated quantizers on the GPU (sm_100a).
//
// Replaces the tensor expressions of the reference's backends/quant.py:
//   quantize_int8_symmetric   (:23-35)  one scale per row (last dimension), range [-128, 127]
//   quantize_int4_block       (:43-72)  one scale per block of 32, range [-8, 7], one code
//                                        per int8, last block of a row zero-padded
//   dequantize_int8_symmetric (:38-40), dequantize_int4_block (:75-86)   code * scale in fp32
// The reference evaluates them in the tensor's own dtype, so that is what happens here:
// the 1e-8 floor of amax, the scale amax / qmax and the quotient x / scale are each
// rounded to the input dtype (fp16 / bf16 / fp32, nearest even) before the next step; the
// quotient is then rounded half-to-even to an integer (torch.round) and clamped.  Codes
// and scales are therefore bit-identical to the reference's.
//
// One warp owns one (row, group): a strided read, a shuffle max, then each lane
// quantizes the elements it read.  The work is a single pass over the data (HBM bound).

#include "common.cuh"

namespace knlp {
namespace {

template <int DT>
__device__ __forceinline__ float round_to_dtype(float v) {
  if constexpr (DT == KNLP_F16) {
    return __half2float(__float2half_rn(v));
  } else if constexpr (DT == KNLP_BF16) {
    return __bfloat162float(__float2bfloat16_rn(v));
  } else {
    return v;
  }
}

constexpr int kWarpsPerCta = 8;

template <int DT>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
plugin_quantize_kernel(const void* __restrict__ x, int8_t* __restrict__ q,
                       void* __restrict__ scale, int64_t n_rows, int dim, int group,
                       int n_groups, float qmax, float qmin) {
  const int lane = threadIdx.x & 31;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (unit >= n_rows * n_groups) return;
  const int64_t row = unit / n_groups;
  const int g = static_cast<int>(unit % n_groups);
  const int lo = g * group;
  const int hi = min(lo + group, dim);  // elements past the row end count as zeros
  const int64_t base = row * dim;

  float amax = 0.0f;
  for (int i = lo + lane; i < hi; i += 32) amax = fmaxf(amax, fabsf(load_elem<DT>(x, base + i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, round_to_dtype<DT>(1e-8f));  // in fp16 the floor itself rounds to 0
  const float sc = round_to_dtype<DT>(__fdiv_rn(amax, qmax));
  if (lane == 0) {
    if constexpr (DT == KNLP_F32) {
      static_cast<float*>(scale)[unit] = sc;
    } else if constexpr (DT == KNLP_F16) {
      static_cast<__half*>(scale)[unit] = __float2half_rn(sc);
    } else {
      static_cast<__nv_bfloat16*>(scale)[unit] = __float2bfloat16_rn(sc);
    }
  }
  for (int i = lo + lane; i < hi; i += 32) {
    const float y = round_to_dtype<DT>(__fdiv_rn(load_elem<DT>(x, base + i), sc));
    // 0 / 0 (an all-zero row in fp16, where the 1e-8 floor rounds to 0) is NaN: code 0, which
    // is what the reference's NaN -> int8 conversion yields
    const float r = y != y ? 0.0f : fminf(fmaxf(rintf(y), qmin), qmax);
    q[base + i] = static_cast<int8_t>(static_cast<int>(r));
  }
}

__global__ void __launch_bounds__(256)
plugin_dequantize_kernel(const int8_t* __restrict__ q, const void* __restrict__ scale,
                         int scale_dtype, float* __restrict__ out, int64_t n_elems, int dim,
                         int group, int n_groups) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_elems) return;
  const int64_t row = i / dim;
  const int g = static_cast<int>(i % dim) / group;
  out[i] = static_cast<float>(q[i]) * load_elem_rt(scale, row * n_groups + g, scale_dtype);
}

}  // namespace
}  // namespace knlp

extern "C" {

int knlp_b200_plugin_quantize(const void* x, int dtype, int64_t n_rows, int dim, int group,
                              int bits, int8_t* q, void* scale, void* stream) {
  using namespace knlp;
  if (n_rows == 0) return KNLP_OK;
  if (!x || !q || !scale) return KNLP_ERR_NULL;
  if (n_rows < 0 || dim <= 0 || group <= 0) return KNLP_ERR_SHAPE;
  if (bits != 8 && bits != 4) return KNLP_ERR_MODE;
  const int n_groups = (dim + group - 1) / group;
  const int64_t units = n_rows * n_groups;
  const int64_t ctas = (units + kWarpsPerCta - 1) / kWarpsPerCta;
  if (ctas > 0x7fffffffLL) return KNLP_ERR_SHAPE;
  const float qmax = bits == 8 ? 127.0f : 7.0f;
  const float qmin = bits == 8 ? -128.0f : -8.0f;
  auto st = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(ctas)), block(kWarpsPerCta * 32);
  switch (dtype) {
    case KNLP_F32:
      plugin_quantize_kernel<KNLP_F32><<<grid, block, 0, st>>>(x, q, scale, n_rows, dim, group,
                                                               n_groups, qmax, qmin);
      break;
    case KNLP_F16:
      plugin_quantize_kernel<KNLP_F16><<<grid, block, 0, st>>>(x, q, scale, n_rows, dim, group,
                                                               n_groups, qmax, qmin);
      break;
    case KNLP_BF16:
      plugin_quantize_kernel<KNLP_BF16><<<grid, block, 0, st>>>(x, q, scale, n_rows, dim, group,
                                                                n_groups, qmax, qmin);
      break;
    default:
      return KNLP_ERR_DTYPE;
  }
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

int knlp_b200_plugin_dequantize(const int8_t* q, const void* scale, int scale_dtype,
                                int64_t n_rows, int dim, int group, float* out, void* stream) {
  using namespace knlp;
  if (n_rows == 0) return KNLP_OK;
  if (!q || !scale || !out) return KNLP_ERR_NULL;
  if (n_rows < 0 || dim <= 0 || group <= 0) return KNLP_ERR_SHAPE;
  if (scale_dtype != KNLP_F32 && scale_dtype != KNLP_F16 && scale_dtype != KNLP_BF16)
    return KNLP_ERR_DTYPE;
  const int n_groups = (dim + group - 1) / group;
  const int64_t n = n_rows * dim;
  const int64_t ctas = (n + 255) / 256;
  if (ctas > 0x7fffffffLL) return KNLP_ERR_SHAPE;
  plugin_dequantize_kernel<<<static_cast<unsigned>(ctas), 256, 0,
                             static_cast<cudaStream_t>(stream)>>>(q, scale, scale_dtype, out, n,
                                                                  dim, group, n_groups);
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

}  // extern "C"
