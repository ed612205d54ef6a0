"""The packed KV cache of one attention layer: buffers, byte accounting and the dispatch
of a decode step over the K/V precisions.

Host-side mirror of the cache plumbing in mcgrof/knlp's fused backend
(``fused-quant/fused_int4.v0.1.0.py``), so that code written against it finds the same
pieces here:

    get_kv_cache_shape            :2123-2158   allocator-compatible shape of the fp16 planes
    _ensure_int4_cache            :2334-2480   the dedicated packed buffers and their
                                               per-block byte formula (:2451-2470)
    FusedInt4AttentionMetadata    :2078-2090   per-step metadata
    FusedInt4AttentionBackend     :2096-2176   name, supported dtypes / head sizes, the
                                               classes that belong together
    FusedInt4AttentionMetadataBuilder :2182-2252  scheduler's common metadata -> per-step metadata
    do_kv_cache_update            :2483-2546   cache write of a step's new tokens
    _fused_decode                 :2851-2928   decode dispatch over k_precision / v_precision

The kernels behind it are this package's (``ops``); nothing here touches vLLM.  One
addition the reference does not have: ``decode_step`` appends the step's token and
attends in ONE launch when both planes are quantized (the reference writes, then decodes).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import ops

GROUP_SIZE = ops.GROUP_SIZE


def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                       cache_dtype_str: str = "int4_fused",
                       replace_cache: bool = False) -> Tuple[int, ...]:
    """Shape of the framework-allocated fp16 cache (reference :2123-2158): two planes (one
    when the V plane is replaced by the packed cache), each [num_blocks, block_size,
    num_kv_heads, head_size] in the model dtype."""
    return (1 if replace_cache else 2, num_blocks, block_size, num_kv_heads, head_size)


def shadow_bytes_per_block(block_size: int, num_kv_heads: int, head_size: int, k_precision: str,
                           v_precision: str, asymmetric: bool) -> int:
    """Bytes of packed cache per block, the planner formula of the reference (:2451-2470):
    INT4 plane = head_size/2 code bytes + 2 bytes of fp16 scale (+ 2 of zero-point when
    asymmetric) per group of 32; INT8 plane = head_size + 2 per group; fp16 K lives in the
    framework's own cache and costs nothing here.  (The reference adds 3 bytes for a
    placeholder tensor it keeps when V is INT8; there is no placeholder here.)"""
    if head_size % GROUP_SIZE:
        raise ValueError("head_size must be a multiple of 32")
    ng = head_size // GROUP_SIZE
    rows = block_size * num_kv_heads

    def plane(precision: str) -> int:
        if precision == "int8":
            return rows * head_size + rows * ng * 2
        if precision == "int4":
            return rows * (head_size // 2) + rows * ng * 2 * (2 if asymmetric else 1)
        if precision == "fp16":
            return 0
        raise ValueError(f"unknown precision {precision!r}")

    if v_precision == "fp16":
        raise ValueError("V is always quantized (int4 or int8)")
    return plane(k_precision) + plane(v_precision)


@dataclass
class AttentionMetadata:
    """Per-step metadata of the decode path (reference FusedInt4AttentionMetadata,
    :2078-2090; the FlashAttention-only fields are left out)."""
    num_actual_tokens: int
    max_query_len: int
    query_start_loc: Optional[torch.Tensor]
    max_seq_len: int
    seq_lens: torch.Tensor
    block_table: torch.Tensor
    slot_mapping: torch.Tensor


class AttentionMetadataBuilder:
    """Builds the per-step metadata from the scheduler's common metadata (reference
    FusedInt4AttentionMetadataBuilder.build, :2210-2252): the fields are taken over as they
    are; the FlashAttention scheduler metadata the reference pre-computes for its fp16-K
    path has no use here.  ``common_attn_metadata`` is any object with the attributes
    num_actual_tokens, max_query_len, query_start_loc, max_seq_len, seq_lens,
    block_table_tensor and slot_mapping (vLLM's CommonAttentionMetadata has them)."""

    # a decode step is one query token per sequence; such batches may be captured in a
    # CUDA graph (reference _cudagraph_support = UNIFORM_SINGLE_TOKEN_DECODE)
    reorder_batch_threshold = 1

    def __init__(self, block_size: int, num_kv_heads: int, head_size: int, device=None):
        self.block_size, self.num_kv_heads, self.head_size = block_size, num_kv_heads, head_size
        self.device = device

    def build(self, common_prefix_len: int, common_attn_metadata,
              fast_build: bool = False) -> AttentionMetadata:
        m = common_attn_metadata
        return AttentionMetadata(
            num_actual_tokens=m.num_actual_tokens, max_query_len=m.max_query_len,
            query_start_loc=m.query_start_loc, max_seq_len=m.max_seq_len, seq_lens=m.seq_lens,
            block_table=m.block_table_tensor, slot_mapping=m.slot_mapping)


class AttentionBackend:
    """What the serving engine asks a backend before it uses it (reference
    FusedInt4AttentionBackend, :2096-2176), answered for this library's kernels."""

    accept_output_buffer = True
    forward_includes_kv_cache_update = False
    supported_dtypes = [torch.float16, torch.bfloat16]
    supported_kv_cache_dtypes = ["int4_fused"]

    @staticmethod
    def get_name() -> str:
        return "FUSED_INT4"

    @staticmethod
    def get_builder_cls():
        return AttentionMetadataBuilder

    @staticmethod
    def get_cache_cls():
        return PackedKVCache

    get_kv_cache_shape = staticmethod(get_kv_cache_shape)

    @classmethod
    def supports_kv_cache_dtype(cls, kv_cache_dtype) -> bool:
        return kv_cache_dtype is None or kv_cache_dtype == "int4_fused"

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        # the groups of 32 must tile the head (the tensor-core kernels take 64 and 128,
        # other multiples of 32 run the stride-generic kernel)
        return head_size > 0 and head_size % GROUP_SIZE == 0


class PackedKVCache:
    """The dedicated packed buffers of one layer (reference ``_ensure_int4_cache``), with
    the cache write and the decode dispatch as methods.

    k_precision: "int4" | "int8" | "fp16" (fp16 / bf16 K stays in the framework's cache and
    is passed to ``decode``); v_precision: "int4" | "int8"."""

    def __init__(self, num_kv_heads: int, head_size: int, k_precision: str = "int4",
                 v_precision: str = "int4", asymmetric: bool = False):
        if k_precision not in ("int4", "int8", "fp16") or v_precision not in ("int4", "int8"):
            raise ValueError("k_precision must be int4/int8/fp16, v_precision int4/int8")
        if head_size % GROUP_SIZE:
            raise ValueError("head_size must be a multiple of 32")
        self.num_kv_heads, self.head_size = num_kv_heads, head_size
        self.k_precision, self.v_precision, self.asymmetric = k_precision, v_precision, asymmetric
        self.num_groups = head_size // GROUP_SIZE
        self.num_blocks = 0
        self.block_size = 0
        self.key_cache = self.value_cache = None
        self.k_scales = self.v_scales = self.k_zeros = self.v_zeros = None

    # ---- allocation and accounting (reference :2334-2480)
    def ensure(self, num_blocks: int, block_size: int, device) -> None:
        """Allocate (or re-allocate larger; contents are not carried over, as in the
        reference) the packed buffers for ``num_blocks`` blocks."""
        if self.value_cache is not None and self.num_blocks >= num_blocks and (
                self.block_size == block_size):
            return
        h, d, ng = self.num_kv_heads, self.head_size, self.num_groups

        def plane(precision):
            if precision == "fp16":
                return None, None, None
            codes = torch.zeros(num_blocks, block_size, h, d if precision == "int8" else d // 2,
                                device=device,
                                dtype=torch.int8 if precision == "int8" else torch.uint8)
            scales = torch.zeros(num_blocks, block_size, h, ng, device=device, dtype=torch.float16)
            zeros = (torch.zeros_like(scales)
                     if precision == "int4" and self.asymmetric else None)
            return codes, scales, zeros

        self.key_cache, self.k_scales, self.k_zeros = plane(self.k_precision)
        self.value_cache, self.v_scales, self.v_zeros = plane(self.v_precision)
        self.num_blocks, self.block_size = num_blocks, block_size

    def tensors(self):
        return [t for t in (self.key_cache, self.value_cache, self.k_scales, self.v_scales,
                            self.k_zeros, self.v_zeros) if t is not None]

    def actual_bytes_per_block(self) -> int:
        total = sum(t.numel() * t.element_size() for t in self.tensors())
        return total // max(self.num_blocks, 1)

    def expected_bytes_per_block(self) -> int:
        return shadow_bytes_per_block(self.block_size, self.num_kv_heads, self.head_size,
                                      self.k_precision, self.v_precision, self.asymmetric)

    # ---- planes as the C ABI takes them
    def _k_plane(self, key_cache_fp16=None):
        L = ops._lib
        if self.k_precision == "fp16":
            if key_cache_fp16 is None:
                raise ValueError("k_precision=fp16: pass the framework's K cache")
            return ops._fp_plane(key_cache_fp16)
        if self.k_precision == "int8":
            return ops._plane(self.key_cache, self.k_scales, None, L.KV_INT8_G32)
        return ops._plane(self.key_cache, self.k_scales, self.k_zeros,
                          L.KV_INT4_ASYM if self.asymmetric else L.KV_INT4_SYM)

    def _v_plane(self):
        L = ops._lib
        if self.v_precision == "int8":
            return ops._plane(self.value_cache, self.v_scales, None, L.KV_INT8_G32)
        return ops._plane(self.value_cache, self.v_scales, self.v_zeros,
                          L.KV_INT4_ASYM if self.asymmetric else L.KV_INT4_SYM)

    # ---- cache write of a step (reference do_kv_cache_update :2483-2546, forward :2661-2689)
    def write(self, key: Optional[torch.Tensor], value: torch.Tensor,
              slot_mapping: torch.Tensor) -> None:
        """Quantize new tokens into the packed planes (one launch for both).  With
        k_precision=fp16 only V is written (K goes to the framework's own cache)."""
        value = value.view(-1, self.num_kv_heads, self.head_size)
        kp = None
        if self.k_precision != "fp16":
            if key is None:
                raise ValueError("key is needed unless k_precision is fp16")
            key = key.view(-1, self.num_kv_heads, self.head_size)
            kp = self._k_plane()
        ops.quant_append(key if kp is not None else None, value, kp, self._v_plane(),
                         slot_mapping, self.block_size)

    # ---- decode dispatch (reference _fused_decode :2851-2928)
    def decode(self, decode_query: torch.Tensor, block_table: torch.Tensor,
               seq_lens: torch.Tensor, key_cache_fp16: Optional[torch.Tensor] = None,
               **kw) -> torch.Tensor:
        """Attention of one query token per sequence over the cache; the same five-way
        dispatch as the reference: K fp16 x V int8/int4, K int8 x V int8/int4, K int4 x V int4."""
        common = dict(num_kv_heads=self.num_kv_heads, head_size=self.head_size, **kw)
        if self.k_precision == "fp16":
            if self.v_precision == "int8":
                return ops.kfp16_vint8_decode(decode_query, key_cache_fp16, self.value_cache,
                                              self.v_scales, block_table, seq_lens, **common)
            return ops.kfp16_vint4_decode(decode_query, key_cache_fp16, self.value_cache,
                                          self.v_scales, block_table, seq_lens,
                                          v_zeros=self.v_zeros, asymmetric=self.asymmetric,
                                          **common)
        if self.k_precision == "int8":
            if self.v_precision == "int8":
                return ops.kint8_vint8_decode(decode_query, self.key_cache, self.value_cache,
                                              self.k_scales, self.v_scales, block_table, seq_lens,
                                              **common)
            return ops.kint8_vint4_decode(decode_query, self.key_cache, self.value_cache,
                                          self.k_scales, self.v_scales, block_table, seq_lens,
                                          v_zeros=self.v_zeros, asymmetric=self.asymmetric,
                                          **common)
        if self.v_precision != "int4":
            raise NotImplementedError("K int4 with V int8 is not a mode of the reference")
        return ops.fused_int4_decode(decode_query, self.key_cache, self.value_cache,
                                     self.k_scales, self.v_scales, block_table, seq_lens,
                                     k_zeros=self.k_zeros, v_zeros=self.v_zeros,
                                     asymmetric=self.asymmetric, **common)

    # ---- a whole decode step
    def decode_step(self, decode_query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    meta: AttentionMetadata, key_cache_fp16: Optional[torch.Tensor] = None,
                    out_dtype=None) -> torch.Tensor:
        """One uniform single-token decode step: the step's token of every sequence goes
        into the cache and the query attends over the cache including it.
        ``meta.seq_lens`` are the lengths INCLUDING the new token (as the reference's
        metadata has them), ``meta.slot_mapping`` the new tokens' slots.

        Both planes quantized: one launch (append fused into the decode kernel).
        Otherwise: the cache write, then the decode, as the reference does."""
        S = decode_query.shape[0]
        if self.k_precision != "fp16" and value.shape[0] == S:
            before = meta.seq_lens - 1
            return ops.decode_attention(
                decode_query, self._k_plane(), self._v_plane(), self.num_blocks,
                meta.block_table, before, self.num_kv_heads, self.head_size, self.block_size,
                out_dtype=out_dtype, max_seq_len=meta.max_seq_len,
                new_key=key.view(S, self.num_kv_heads, self.head_size),
                new_value=value.view(S, self.num_kv_heads, self.head_size))
        self.write(key, value, meta.slot_mapping)
        return self.decode(decode_query, meta.block_table, meta.seq_lens,
                           key_cache_fp16=key_cache_fp16, out_dtype=out_dtype,
                           max_seq_len=meta.max_seq_len)
