// Stride-generic split-context decode attention on CUDA cores (sm_100a).
//
// This is the kernel for cache views the tensor-core kernel does not take
// (unaligned or exotic strides, head sizes 32/256, more than 8 q heads per kv
// head) and the in-library cross-check of that kernel.  It follows the math of
// the reference's _fused_int4_decode_kernel (fused-quant/fused_int4.v0.1.0.py:
// 656-894) and _kint8_vint4_decode_kernel (:1318-1493): dequantize in registers
// (c*s+z, (c-8)*s or q8*s), score = (q.k) * d^-1/2, online softmax, acc += p*v.
//
// Mapping: grid (split, kv head x q-head group, sequence); 4 warps per CTA take
// the split's tokens round-robin; a lane owns head_dim/32 consecutive elements
// of every row; all q heads of the group share each K/V row read.  The warps'
// partials are merged through shared memory and written as one (m, l, o)
// partial per (sequence, q head, split).

#include "common.cuh"

namespace knlp {
namespace {

constexpr int kWarps = 4;

template <int EPL>
__device__ __forceinline__ void load_row(const Plane& p, const uint8_t* crow, const __half* srow,
                                         const __half* zrow, int lane, float out[EPL]) {
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane * EPL + i;
    const int g = e >> 5;
    if (p.mode == KNLP_KV_F16) {  // unquantized K (kfp16_* decodes, reference :1076-1083)
      out[i] = __half2float(reinterpret_cast<const __half*>(crow)[e]);
      continue;
    }
    if (p.mode == KNLP_KV_BF16) {
      out[i] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(crow)[e]);
      continue;
    }
    const float s = __half2float(srow[g]);
    if (p.mode == KNLP_KV_INT8_G32) {
      out[i] = static_cast<float>(static_cast<int8_t>(crow[e])) * s;
    } else {
      const unsigned b = crow[e >> 1];
      const float c = static_cast<float>((e & 1) ? (b >> 4) : (b & 0xFu));
      if (p.mode == KNLP_KV_INT4_ASYM) {
        out[i] = c * s + __half2float(zrow[g]);
      } else {
        out[i] = (c - 8.0f) * s;
      }
    }
  }
}

template <int EPL, int QH>
__global__ void __launch_bounds__(kWarps * 32)
decode_generic_kernel(const DecodeArgs a, int n_rep, int q_groups) {
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / q_groups;
  const int qg = blockIdx.y % q_groups;
  const int seq = blockIdx.z;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int d = a.head_dim;
  const int P = a.block_size;

  int seq_len = a.seq_lens[seq];
  if (seq_len < 0) seq_len = 0;
  const int start = split * a.chunk;
  const int end = split == a.n_splits - 1 ? seq_len : min(start + a.chunk, seq_len);

  // q heads handled here: kvh*n_rep + qg*QH + [0, QH), masked to n_rep
  const int h_first = qg * QH;
  float q[QH][EPL];
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    const int hr = h_first + h;
    const int qh = kvh * n_rep + (hr < n_rep ? hr : 0);
    const int64_t base = seq * a.q_stride[0] + qh * a.q_stride[1] + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) q[h][i] = load_elem_rt(a.q, base + i, a.q_dtype);
  }
  const float sm_scale = rsqrtf(static_cast<float>(d));

  float m[QH], l[QH], acc[QH][EPL];
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[h][i] = 0.0f;
  }

  for (int t = start + warp; t < end; t += kWarps) {
    int64_t blk = a.block_table[seq * a.bt_stride + t / P];
    blk = blk < 0 ? 0 : (blk >= a.num_blocks ? a.num_blocks - 1 : blk);
    const int off = t % P;
    float kv[EPL];
    {
      const Plane& p = a.k;
      const uint8_t* crow = p.codes + blk * p.cs[0] + off * p.cs[1] + kvh * p.cs[2];
      const __half* srow = p.scales + blk * p.ss[0] + off * p.ss[1] + kvh * p.ss[2];
      const __half* zrow = p.zeros ? p.zeros + blk * p.zs[0] + off * p.zs[1] + kvh * p.zs[2]
                                   : nullptr;
      load_row<EPL>(p, crow, srow, zrow, lane, kv);
    }
    float s[QH];
#pragma unroll
    for (int h = 0; h < QH; ++h) {
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) dot = fmaf(q[h][i], kv[i], dot);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      s[h] = dot * sm_scale;
    }
    {
      const Plane& p = a.v;
      const uint8_t* crow = p.codes + blk * p.cs[0] + off * p.cs[1] + kvh * p.cs[2];
      const __half* srow = p.scales + blk * p.ss[0] + off * p.ss[1] + kvh * p.ss[2];
      const __half* zrow = p.zeros ? p.zeros + blk * p.zs[0] + off * p.zs[1] + kvh * p.zs[2]
                                   : nullptr;
      load_row<EPL>(p, crow, srow, zrow, lane, kv);
    }
#pragma unroll
    for (int h = 0; h < QH; ++h) {
      const float m_new = fmaxf(m[h], s[h]);
      const float alpha = __expf(m[h] - m_new);  // exp(-inf) = 0 on the first token
      const float pr = __expf(s[h] - m_new);
      l[h] = l[h] * alpha + pr;
#pragma unroll
      for (int i = 0; i < EPL; ++i) acc[h][i] = acc[h][i] * alpha + pr * kv[i];
      m[h] = m_new;
    }
  }

  // merge the warps
  __shared__ float sm_m[kWarps][QH];
  __shared__ float sm_l[kWarps][QH];
  __shared__ float sm_o[kWarps][QH][EPL * 32];
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < QH; ++h) {
      sm_m[warp][h] = m[h];
      sm_l[warp][h] = l[h];
    }
  }
#pragma unroll
  for (int h = 0; h < QH; ++h)
#pragma unroll
    for (int i = 0; i < EPL; ++i) sm_o[warp][h][lane * EPL + i] = acc[h][i];
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    const int hr = h_first + h;
    if (hr >= n_rep) continue;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, sm_m[w][h]);
    float ll = 0.0f;
    float o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[i] = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float lw = sm_l[w][h];
      const float wgt = lw > 0.0f ? __expf(sm_m[w][h] - mm) : 0.0f;
      ll += lw * wgt;
#pragma unroll
      for (int i = 0; i < EPL; ++i) o[i] += sm_o[w][h][lane * EPL + i] * wgt;
    }
    const int64_t row = static_cast<int64_t>(seq) * a.n_q_heads + kvh * n_rep + hr;
    const int64_t pidx = row * a.n_splits + split;
    if (lane == 0) {
      a.part_m[pidx] = mm;
      a.part_l[pidx] = ll;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) a.part_o[pidx * d + lane * EPL + i] = o[i];
  }
}

template <int EPL>
int launch_epl(const DecodeArgs& a, cudaStream_t st) {
  const int n_rep = a.n_q_heads / a.n_kv_heads;
  dim3 block(kWarps * 32);
  if (n_rep == 1) {
    dim3 grid(a.n_splits, a.n_kv_heads, a.n_seqs);
    decode_generic_kernel<EPL, 1><<<grid, block, 0, st>>>(a, n_rep, 1);
  } else if (n_rep <= 4) {
    dim3 grid(a.n_splits, a.n_kv_heads, a.n_seqs);
    decode_generic_kernel<EPL, 4><<<grid, block, 0, st>>>(a, n_rep, 1);
  } else {
    const int qg = (n_rep + 7) / 8;
    dim3 grid(a.n_splits, a.n_kv_heads * qg, a.n_seqs);
    decode_generic_kernel<EPL, 8><<<grid, block, 0, st>>>(a, n_rep, qg);
  }
  return cudaGetLastError() == cudaSuccess ? KNLP_OK : KNLP_ERR_LAUNCH;
}

}  // namespace

int launch_decode_generic(const DecodeArgs& a, cudaStream_t st) {
  switch (a.head_dim) {
    case 32: return launch_epl<1>(a, st);
    case 64: return launch_epl<2>(a, st);
    case 128: return launch_epl<4>(a, st);
    case 256: return launch_epl<8>(a, st);
    default: return KNLP_ERR_SHAPE;
  }
}

}  // namespace knlp
