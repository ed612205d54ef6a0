"""Routed (block-sparse) decode attention over the packed KV cache.

Host-side mirror of mcgrof/knlp's ``routing/fused_routed_attention.py``:

    fused_routed_decode       :425-492   every kv head of every sequence attends to its own
                                         list of selected cache blocks (kernel :45-190)
    select_top_k_blocks       :551-571   top-k blocks per kv head from a routing prior

The reference's kernel reads an unquantized ``[max_blocks, block_size, n_kv_heads,
head_dim]`` cache.  Here the cache is the packed one of this library (INT4 or INT8 codes,
fp16 scale / zero per group of 32) and the kernel is the balanced tensor-core decode kernel
with per-kv-head page tables (``knlp_b200_routed_decode_attention``): one launch, the same
staging pipeline as the dense decode.  The semantics are the reference's: all tokens of a
selected block count, a head with no selected block yields zeros, the q heads of a GQA
group share their kv head's selection, the softmax scale is ``head_dim ** -0.5``.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib, ops


def fused_routed_decode(
    q: torch.Tensor,  # [batch, n_heads, head_dim]
    k_plane: _lib.KvPlane,  # packed K plane (ops._plane) of [max_blocks, block_size, n_kv_heads, ...]
    v_plane: _lib.KvPlane,
    num_blocks: int,
    block_size: int,
    n_kv_heads: int,
    block_tables: torch.Tensor,  # [batch, n_kv_heads, max_selected_blocks] int32 (int64 is cast)
    block_counts: torch.Tensor,  # [batch, n_kv_heads] int32
    scale: Optional[float] = None,
    out_dtype=None,
    emit_partial: bool = False,
) -> torch.Tensor:
    """Routed decode attention; returns [batch, n_heads, head_dim] in ``out_dtype``
    (default: q's).  ``emit_partial``: fp32 [batch, n_heads, head_dim + 2] rows
    [o un-normalised, m, l] instead, mergeable with other partials by the combine kernel
    (e.g. a dense near window)."""
    dev = ops._need_cuda(q, block_tables, block_counts)
    batch, n_heads, head_dim = q.shape
    if n_heads % n_kv_heads:
        raise ValueError("n_heads must be a multiple of n_kv_heads")
    if scale is not None and abs(scale - head_dim ** -0.5) > 1e-6 * head_dim ** -0.5:
        raise NotImplementedError("only the default scale head_dim ** -0.5 is built")
    if block_tables.shape[:2] != (batch, n_kv_heads) or block_counts.shape != (batch, n_kv_heads):
        raise ValueError("block_tables must be [batch, n_kv_heads, max_selected], "
                         "block_counts [batch, n_kv_heads]")
    if block_tables.dtype != torch.int32:
        block_tables = block_tables.to(torch.int32)  # torch.topk yields int64
    if block_counts.dtype != torch.int32:
        block_counts = block_counts.to(torch.int32)
    block_tables = block_tables.contiguous()
    block_counts = block_counts.contiguous()
    if not q.is_contiguous():
        q = q.contiguous()
    max_sel = block_tables.shape[2]
    n_rep = n_heads // n_kv_heads
    ws, counters = ops._decode_workspace(dev, batch * n_kv_heads, n_rep, 1, head_dim, block_size,
                                         max_sel * block_size)
    flags = 0
    if emit_partial:
        out = torch.empty((batch, n_heads, head_dim + 2), dtype=torch.float32, device=dev)
        flags |= _lib.DECODE_EMIT_PARTIAL
    else:
        out = torch.empty((batch, n_heads, head_dim),
                          dtype=q.dtype if out_dtype is None else out_dtype, device=dev)
    with ops._on(dev):
        rc = _lib.load().knlp_b200_routed_decode_attention(
            q.data_ptr(), ops._dt(q), ops._stride2(q), C.byref(k_plane), C.byref(v_plane),
            block_tables.data_ptr(), max_sel, block_counts.data_ptr(), num_blocks,
            batch, n_heads, n_kv_heads, head_dim, block_size, max_sel,
            ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
            out.data_ptr(), ops._DT[out.dtype], out.shape[-1], flags, ops._stream(dev))
    _lib.check(rc, "knlp_b200_routed_decode_attention")
    return out


def select_top_k_blocks(routing_prior: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k blocks per kv head from a routing prior [n_layers, n_kv_heads, n_blocks]
    (reference :551-571): block_tables [n_layers, n_kv_heads, k] and block_counts
    [n_layers, n_kv_heads], all equal to min(k, n_blocks)."""
    k = min(int(k), routing_prior.shape[-1])
    tables = routing_prior.topk(k, dim=-1).indices
    counts = torch.full(tuple(routing_prior.shape[:2]), k, dtype=torch.int32)
    return tables, counts
