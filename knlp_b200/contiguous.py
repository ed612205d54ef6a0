"""The contiguous, head-major symmetric INT4 cache of the reference's kernel benches.

mcgrof/knlp's published kernel numbers were taken on this layout
(``scripts/v29_flash_bench.py:40-97``, ``scripts/spev01/tier5_fused_decode.py:116-145``,
``scripts/v35_h100_bench.py:66-93``): K and V quantized with ``quantize_and_pack_int4``
into ``[B, n_kv, T, head_dim/2]`` uint8 (codes + 8, low nibble = even element) with fp16
scales ``[B, n_kv, T, head_dim/32]``, and a decode kernel (or dequantize-then-SDPA,
``pipeline_A``) over them.  The functions here keep those names and signatures.

The quantizer is the block quantizer of the plugin surface (same arithmetic: amax floor
1e-8, scale = amax / 7 in the tensor's dtype, round-half-even, clamp to [-8, 7]) followed by
the nibble packing, so it is bit-identical to the reference's tensor expression.  The decode
reads the layout with the tensor-core kernel through a re-interpretation that moves no
data: every (batch, kv head) is one sequence with ONE kv head, whose pages are the
consecutive 16-token runs of its rows.
"""

from __future__ import annotations

import torch

from . import backends, ops

GROUP_SIZE = 32


def quantize_and_pack_int4(tensor: torch.Tensor, group_size: int = GROUP_SIZE):
    """Quantize to symmetric INT4 and pack two codes per byte.  Returns (packed uint8
    [..., hd/2], scales [..., hd/group_size] in the tensor's dtype).  CUDA tensors only."""
    if tensor.shape[-1] % group_size or tensor.shape[-1] % 2:
        raise ValueError("the last dimension must be a multiple of the group size")
    x4 = tensor.reshape(1, 1, -1, tensor.shape[-1])
    q, scales = backends.quantize_int4_block(x4, group_size)
    qu = (q + 8).to(torch.uint8).reshape(*tensor.shape)
    packed = qu[..., 0::2] | (qu[..., 1::2] << 4)
    return packed, scales.reshape(*tensor.shape[:-1], tensor.shape[-1] // group_size)


def dequant_int4(packed: torch.Tensor, scales: torch.Tensor, group_size: int = GROUP_SIZE):
    """Packed INT4 back to fp16: (code - 8) * scale, as the reference's control path does."""
    low = (packed & 0x0F).to(torch.int8) - 8
    high = ((packed >> 4) & 0x0F).to(torch.int8) - 8
    hd = packed.shape[-1] * 2
    out = torch.empty(*packed.shape[:-1], hd, device=packed.device, dtype=torch.float16)
    out[..., 0::2] = low.to(torch.float16)
    out[..., 1::2] = high.to(torch.float16)
    out = out.reshape(*packed.shape[:-1], hd // group_size, group_size) * scales.unsqueeze(-1)
    return out.reshape(*packed.shape[:-1], hd)


def fused_int4_decode_contiguous(Q: torch.Tensor, K_packed: torch.Tensor, V_packed: torch.Tensor,
                                 scale_k: torch.Tensor, scale_v: torch.Tensor,
                                 seq_len=None, out_dtype=None) -> torch.Tensor:
    """Decode attention over the contiguous cache.  Q [B, n_heads, 1, hd] (or [B, n_heads,
    hd]); K_packed, V_packed [B, n_kv, T, hd/2]; scales [B, n_kv, T, hd/32] fp16.  Returns
    the shape of Q.  ``seq_len`` (int) attends to the first tokens only.

    With T a multiple of 16 every (batch, kv head) becomes a sequence of T/16 pages with one
    kv head and the balanced tensor-core kernel runs on it; other T go through a strided
    view of the same memory (stride-generic kernel)."""
    squeeze = Q.dim() == 4
    q3 = Q.reshape(Q.shape[0], Q.shape[1], Q.shape[-1]) if squeeze else Q
    B, Hq, hd = q3.shape
    Bk, Hkv, T, half = K_packed.shape
    if Bk != B or half * 2 != hd or Hq % Hkv:
        raise ValueError("shapes of Q and the cache do not match")
    if scale_k.dtype != torch.float16 or scale_v.dtype != torch.float16:
        raise TypeError("scales must be float16")
    n_rep = Hq // Hkv
    L = T if seq_len is None else int(seq_len)
    dev = Q.device
    ng = hd // GROUP_SIZE
    contiguous = all(t.is_contiguous() for t in (K_packed, V_packed, scale_k, scale_v))
    if T % 16 == 0 and contiguous and q3.is_contiguous():
        n_seq = B * Hkv
        pages = T // 16
        view = lambda t, w: t.view(n_seq * pages, 16, 1, w)
        bt = torch.arange(n_seq * pages, dtype=torch.int32, device=dev).view(n_seq, pages)
        lens = torch.full((n_seq,), L, dtype=torch.int32, device=dev)
        out = ops.fused_int4_decode(q3.view(n_seq, n_rep, hd), view(K_packed, half),
                                    view(V_packed, half), view(scale_k, ng), view(scale_v, ng),
                                    bt, lens, 1, hd, asymmetric=False, out_dtype=out_dtype,
                                    max_seq_len=T)
        out = out.view(B, Hq, hd)
    else:
        # [B, n_kv, T, w] seen as one block per batch entry: [B, T, n_kv, w]
        perm = lambda t: t.permute(0, 2, 1, 3)
        bt = torch.arange(B, dtype=torch.int32, device=dev).view(B, 1)
        lens = torch.full((B,), L, dtype=torch.int32, device=dev)
        out = ops.fused_int4_decode(q3, perm(K_packed), perm(V_packed), perm(scale_k),
                                    perm(scale_v), bt, lens, Hkv, hd, asymmetric=False,
                                    out_dtype=out_dtype, max_seq_len=T, force_generic=True)
    return out.unsqueeze(2) if squeeze else out
