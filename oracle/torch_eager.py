"""PyTorch-eager CPU restatement of the reference's dequantize-then-attend control path.

TEST / BASELINE INFRASTRUCTURE ONLY: nothing in the shipped package imports this.  It is
what ``bench.py`` times as the CPU baseline and as ``--impl reference``, and what a
CPU test compares with the numpy oracle.

It follows the structure of mcgrof/knlp's control pipeline
(``scripts/v29_flash_bench.py:86-97``, ``pipeline_A``): dequantize the whole packed cache of
a sequence, expand the kv heads to the query heads with ``repeat_interleave``, then one
``F.scaled_dot_product_attention(is_causal=False)`` in fp32.  Dequantization is the
definition of ``_cpu_dequant_slot`` (``fused-quant/fused_int4.v0.1.0.py:150-195``): low
nibble = even element, ``code * float(scale_fp16) + float(zero_fp16)`` per group of 32
(symmetric: ``(code - 8) * scale``; INT8: ``q * scale``, ``:1420``).

All tensors are CPU tensors; threads are torch's intra-op pool (set by the caller).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

GROUP = 32


def dequant_int4(packed: torch.Tensor, scales: torch.Tensor, zeros=None) -> torch.Tensor:
    """[T, H, d/2] uint8 + [T, H, d/32] fp16 (+ zeros) -> [T, H, d] fp32."""
    T, H, half = packed.shape
    lo = (packed & 0xF).to(torch.float32)
    hi = (packed >> 4).to(torch.float32)
    full = torch.stack((lo, hi), dim=-1).reshape(T, H, half * 2 // GROUP, GROUP)
    s = scales.to(torch.float32).unsqueeze(-1)
    if zeros is None:  # symmetric codes are stored + 8 (:176-178)
        return ((full - 8.0) * s).reshape(T, H, half * 2)
    return (full * s + zeros.to(torch.float32).unsqueeze(-1)).reshape(T, H, half * 2)


def dequant_int8(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """[T, H, d] int8 + [T, H, d/32] fp16 -> [T, H, d] fp32 (:1420)."""
    T, H, d = codes.shape
    full = codes.to(torch.float32).reshape(T, H, d // GROUP, GROUP)
    return (full * scales.to(torch.float32).unsqueeze(-1)).reshape(T, H, d)


def _gather(cache: torch.Tensor, table_row: torch.Tensor, seq_len: int) -> torch.Tensor:
    """Rows of one sequence out of the paged cache: [T, H, w]."""
    P = cache.shape[1]
    n = (seq_len + P - 1) // P
    return cache[table_row[:n].long()].reshape(n * P, *cache.shape[2:])[:seq_len]


def decode(query, key_cache, value_cache, k_scales, v_scales, block_table, seq_lens,
           num_kv_heads: int, head_size: int, k_zeros=None, v_zeros=None,
           k_int8: bool = False, v_int8: bool = False) -> torch.Tensor:
    """Dequantize-then-attend for every sequence.  query [S, Hq, d]; returns [S, Hq, d] fp32.
    The kv heads are streamed one at a time, so that the fp32 K/V of a long context never
    exist for all heads at once (each head still sees one whole-context SDPA call)."""
    S, Hq, d = query.shape
    n_rep = Hq // num_kv_heads
    out = torch.zeros(S, Hq, d, dtype=torch.float32)
    scale = float(d) ** -0.5
    for s in range(S):
        L = int(seq_lens[s])
        if L <= 0:
            continue
        row = block_table[s]
        for h in range(num_kv_heads):
            sl = slice(h, h + 1)
            kc = _gather(key_cache[:, :, sl], row, L)
            vc = _gather(value_cache[:, :, sl], row, L)
            ks = _gather(k_scales[:, :, sl], row, L)
            vs = _gather(v_scales[:, :, sl], row, L)
            if k_int8:
                k = dequant_int8(kc, ks)
            else:
                k = dequant_int4(kc, ks, None if k_zeros is None else _gather(k_zeros[:, :, sl], row, L))
            if v_int8:
                v = dequant_int8(vc, vs)
            else:
                v = dequant_int4(vc, vs, None if v_zeros is None else _gather(v_zeros[:, :, sl], row, L))
            # [1, n_rep, 1, d] x [1, n_rep, L, d]: the kv head repeated for its query heads
            q = query[s, h * n_rep:(h + 1) * n_rep].to(torch.float32).reshape(1, n_rep, 1, d)
            kk = k.permute(1, 0, 2).unsqueeze(0).repeat_interleave(n_rep, dim=1)
            vv = v.permute(1, 0, 2).unsqueeze(0).repeat_interleave(n_rep, dim=1)
            o = F.scaled_dot_product_attention(q, kk, vv, is_causal=False, scale=scale)
            out[s, h * n_rep:(h + 1) * n_rep] = o.reshape(n_rep, d)
    return out
