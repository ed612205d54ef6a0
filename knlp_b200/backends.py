"""Plugin surface of knlp's KV-compression harness, B200 side.

Mirrors the interface of the reference's ``backends/base.py`` (``V14StepStats``,
``CompressionBackend``, ``DenseBackend``; :23-134) and ``backends/quant.py`` (the four
module-level quantizer functions :23-86 and ``QuantBackend`` :89-319) so that the
evaluation harnesses that import those names (``eval_v14b.py:54-104``) can import these
instead.  Names, arguments, return types, byte accounting and error behaviour are the
reference's; the quantizers run as CUDA kernels of ``libknlp_b200.so`` and produce
bit-identical codes and scales.  CUDA tensors only: there is no CPU path.
"""

from __future__ import annotations

import ctypes as C
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import List, Tuple

import numpy as np
import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


# --------------------------------------------------------------------------- quantizers
def _check_input(x: torch.Tensor, what: str) -> int:
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise RuntimeError(f"{what}: knlp_b200 quantizers take CUDA tensors only (no CPU path)")
    if x.dtype not in _DT:
        raise TypeError(f"{what}: unsupported dtype {x.dtype}; expected float32/float16/bfloat16")
    return _DT[x.dtype]


def _quantize(x: torch.Tensor, group: int, bits: int, what: str):
    dt = _check_input(x, what)
    dim = x.shape[-1]
    xc = x.contiguous()
    n_rows = xc.numel() // dim if dim else 0
    n_groups = (dim + group - 1) // group
    q = torch.empty(xc.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(xc.shape[:-1] + (n_groups,), dtype=x.dtype, device=x.device)
    if n_rows:
        with torch.cuda.device(x.device):
            rc = _lib.load().knlp_b200_plugin_quantize(
                xc.data_ptr(), dt, n_rows, dim, group, bits, q.data_ptr(), scale.data_ptr(),
                torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc, what)
    return q, scale


def _dequantize(x_q: torch.Tensor, scale: torch.Tensor, group: int, what: str) -> torch.Tensor:
    if not x_q.is_cuda or not scale.is_cuda:
        raise RuntimeError(f"{what}: knlp_b200 quantizers take CUDA tensors only (no CPU path)")
    if x_q.dtype != torch.int8:
        raise TypeError(f"{what}: codes must be int8")
    if scale.dtype not in _DT:
        raise TypeError(f"{what}: unsupported scale dtype {scale.dtype}")
    dim = x_q.shape[-1]
    n_groups = (dim + group - 1) // group
    if tuple(scale.shape) != tuple(x_q.shape[:-1]) + (n_groups,):
        raise ValueError(f"{what}: scale shape {tuple(scale.shape)} does not match the codes")
    qc, sc = x_q.contiguous(), scale.contiguous()
    out = torch.empty(qc.shape, dtype=torch.float32, device=x_q.device)
    n_rows = qc.numel() // dim if dim else 0
    if n_rows:
        with torch.cuda.device(x_q.device):
            rc = _lib.load().knlp_b200_plugin_dequantize(
                qc.data_ptr(), sc.data_ptr(), _DT[scale.dtype], n_rows, dim, group,
                out.data_ptr(), torch.cuda.current_stream(x_q.device).cuda_stream)
        _lib.check(rc, what)
    return out


def quantize_int8_symmetric(x):
    """Symmetric INT8 with one scale per row of the last dimension
    (reference ``backends/quant.py:23-35``).

    x: [..., dim] fp16 / bf16 / fp32 CUDA tensor.
    Returns (x_q [..., dim] int8, scale [..., 1] in x's dtype)."""
    return _quantize(x, max(int(x.shape[-1]), 1), 8, "quantize_int8_symmetric")


def dequantize_int8_symmetric(x_q, scale):
    """codes * scale as fp32 (reference ``backends/quant.py:38-40``)."""
    return _dequantize(x_q, scale, max(int(x_q.shape[-1]), 1), "dequantize_int8_symmetric")


def quantize_int4_block(x, block_size=32):
    """Simulated INT4: one symmetric scale per block of ``block_size`` elements, codes in
    [-8, 7] kept one per int8 (reference ``backends/quant.py:43-72``).

    x: [B, H, T, D].  Returns (x_q [B, H, T, D] int8, scales [B, H, T, ceil(D / block_size)])."""
    if x.dim() != 4:
        raise ValueError("quantize_int4_block expects a [B, H, T, D] tensor")
    return _quantize(x, int(block_size), 4, "quantize_int4_block")


def dequantize_int4_block(x_q, scale, block_size=32):
    """Inverse of :func:`quantize_int4_block` (reference ``backends/quant.py:75-86``), fp32."""
    if x_q.dim() != 4:
        raise ValueError("dequantize_int4_block expects [B, H, T, D] codes")
    return _dequantize(x_q, scale, int(block_size), "dequantize_int4_block")


# --------------------------------------------------------------------------- plugin base
@dataclass
class V14StepStats:
    """Per-step statistics a backend reports (reference ``backends/base.py:23-35``)."""

    kv_kept: int = 0
    kv_bytes_full: int = 0
    kv_bytes_compressed: int = 0
    kv_bytes_total: int = 0
    compress_ms: float = 0.0
    decompress_ms: float = 0.0
    gate_ms: float = 0.0
    n_full: int = 0
    n_compressed: int = 0


class CompressionBackend(ABC):
    """KV-cache compression plugin (reference ``backends/base.py:38-81``).  The harness
    fixes the routing: the last ``W_min`` tokens and the first ``W_sink`` stay full
    precision, what lies between is the backend's to compress; nothing is dropped."""

    W_min: int = 1024
    W_sink: int = 4

    @property
    @abstractmethod
    def name(self) -> str:
        ...

    @abstractmethod
    def configure(self, L: int, model_config: dict, **kwargs):
        """Set the backend's parameters for context length L."""

    def calibrate(self, model, token_data, L, device_str, model_config):
        """Optional one-time calibration on sample data."""

    @abstractmethod
    def run_decode(self, model, prefix_ids: torch.Tensor, continuation_ids: torch.Tensor,
                   device_str: str, max_ctx: int) -> Tuple[torch.Tensor, List[V14StepStats]]:
        """Prefill on ``prefix_ids`` then feed ``continuation_ids`` one token at a time.
        Returns (logits [B, decode_steps + 1, V], one V14StepStats per decode step)."""

    def compression_ratio(self) -> float:
        return 1.0

    def description(self) -> str:
        return self.name


def _layer_kv(past, li):
    """(key, value) of layer ``li`` from a DynamicCache of any transformers generation or
    from a legacy tuple."""
    layers = getattr(past, "layers", None)
    if layers is not None:
        return layers[li].keys, layers[li].values
    k, v = past[li][0], past[li][1]
    return k, v


def _n_layers(past) -> int:
    layers = getattr(past, "layers", None)
    return len(layers) if layers is not None else len(past)


def _kv_bytes_per_token(mc: dict, elem: int = 2) -> int:
    return 2 * mc["n_kv_heads"] * mc["head_dim"] * elem


class DenseBackend(CompressionBackend):
    """No compression (reference ``backends/base.py:84-134``)."""

    @property
    def name(self):
        return "dense"

    def configure(self, L, model_config, **kwargs):
        self.L = L
        self.mc = model_config

    @torch.no_grad()
    def run_decode(self, model, prefix_ids, continuation_ids, device_str, max_ctx):
        out = model(prefix_ids, use_cache=True)
        past = out.past_key_values
        logits = [out.logits[:, -1:, :]]
        stats = []
        bpt = _kv_bytes_per_token(self.mc)
        for step in range(continuation_ids.shape[1]):
            out = model(continuation_ids[:, step:step + 1], past_key_values=past, use_cache=True)
            past = out.past_key_values
            logits.append(out.logits)
            cache_len = _layer_kv(past, 0)[0].shape[2]
            total = cache_len * bpt * self.mc["n_layers"]
            stats.append(V14StepStats(kv_kept=cache_len, kv_bytes_full=total,
                                      kv_bytes_compressed=0, kv_bytes_total=total,
                                      n_full=cache_len, n_compressed=0))
        return torch.cat(logits, dim=1), stats

    def compression_ratio(self):
        return 1.0

    def description(self):
        return "dense (no compression)"


# --------------------------------------------------------------------------- quant backend
class QuantBackend(CompressionBackend):
    """Per-layer 4- or 8-bit quantization of the far tokens (reference
    ``backends/quant.py:89-319``).  The far segment of every layer is quantized and put
    back dequantized into a DynamicCache (the memory saving is accounted, the quality
    effect is real), exactly as the reference does; the quantizers are the CUDA ones of
    this module."""

    @property
    def name(self):
        return "quant_int4" if getattr(self, "_force_int4", False) else "quant"

    def configure(self, L, model_config, **kwargs):
        self.L = L
        self.mc = model_config
        self.W_min = kwargs.get("W_min", 1024)
        self.W_sink = kwargs.get("W_sink", 4)
        self.default_bits = kwargs.get("default_bits", 8)
        self.block_size = kwargs.get("block_size", 32)
        if not hasattr(self, "calibrated"):  # a calibration survives re-configuration
            self.calibrated = False
            self.layer_bits = None

    # -- calibration -----------------------------------------------------------------
    @staticmethod
    def _text_window(token_data, seq_len, rng):
        """One random window of ``seq_len`` token ids (the harness' ``get_text_batch`` with
        batch size 1, ``scripts/bpa_v11_bench.py:222-229``)."""
        max_start = len(token_data) - seq_len
        if max_start <= 0:
            raise ValueError(f"Token data too short: {len(token_data)} < {seq_len}")
        start = int(rng.randint(0, max_start, size=1)[0])
        return torch.from_numpy(np.asarray(token_data[start:start + seq_len])[None].astype(np.int64))

    def _roundtrip(self, t, bits):
        if bits == 8:
            q, s = quantize_int8_symmetric(t)
            return dequantize_int8_symmetric(q, s)
        q, s = quantize_int4_block(t, self.block_size)
        return dequantize_int4_block(q, s, self.block_size)

    def calibrate(self, model, token_data, L, device_str, model_config):
        """Choose 4 or 8 bits per layer: INT4 where its round-trip error stays below twice
        the median INT8 error (reference :110-168)."""
        n_layers = model_config["n_layers"]
        rng = np.random.RandomState(42)
        idx = self._text_window(token_data, min(L, 4096), rng).to(device_str)
        with torch.no_grad():
            past = model(idx, use_cache=True).past_key_values
        err8, err4 = [], []
        for li in range(n_layers):
            k, v = _layer_kv(past, li)
            e = {}
            for bits in (8, 4):
                kh = self._roundtrip(k, bits).to(k.dtype)
                vh = self._roundtrip(v, bits).to(v.dtype)
                e[bits] = ((k - kh) ** 2).mean().item() + ((v - vh) ** 2).mean().item()
            err8.append(e[8])
            err4.append(e[4])
        if getattr(self, "_force_int4", False):
            self.layer_bits = [4] * n_layers
        else:
            bar = 2.0 * np.median(err8)
            self.layer_bits = [4 if err4[li] < bar else 8 for li in range(n_layers)]
        n4 = sum(1 for b in self.layer_bits if b == 4)
        print(f"    quant calibrated: {n4} layers@INT4, {n_layers - n4} layers@INT8")
        del past
        torch.cuda.empty_cache()
        self.calibrated = True

    # -- decode ----------------------------------------------------------------------
    def _compressed_bytes(self, n_compressed):
        mc = self.mc
        avg_bits = np.mean(self.layer_bits) if self.layer_bits else 8
        per_tok = 2 * mc["n_kv_heads"] * mc["head_dim"] * (avg_bits / 8)
        if avg_bits == 4:
            overhead = 2 * mc["n_kv_heads"] * (mc["head_dim"] / self.block_size) * 2
        else:
            overhead = 2 * mc["n_kv_heads"] * 2
        return int(n_compressed * (per_tok + overhead) * mc["n_layers"])

    @torch.no_grad()
    def run_decode(self, model, prefix_ids, continuation_ids, device_str, max_ctx):
        n_layers = self.mc["n_layers"]
        bpt = _kv_bytes_per_token(self.mc)
        out = model(prefix_ids, use_cache=True)
        past = out.past_key_values
        dtype = _layer_kv(past, 0)[0].dtype
        logits = [out.logits[:, -1:, :]]
        stats = []
        pos = prefix_ids.shape[1]
        if self.calibrated:
            t0 = time.perf_counter()
            past, n_full, n_compressed = self._quantize_far(past, device_str, dtype)
            compress_ms = (time.perf_counter() - t0) * 1000
        else:
            n_full, n_compressed, compress_ms = _layer_kv(past, 0)[0].shape[2], 0, 0

        for step in range(continuation_ids.shape[1]):
            pos_ids = None
            if self.calibrated:
                pos_ids = torch.tensor([[pos]], device=device_str, dtype=torch.long)
            out = model(continuation_ids[:, step:step + 1], past_key_values=past, use_cache=True,
                        position_ids=pos_ids)
            past = out.past_key_values
            logits.append(out.logits)
            pos += 1
            cache_len = _layer_kv(past, 0)[0].shape[2]
            if self.calibrated:
                bytes_full = n_full * bpt * n_layers
                bytes_comp = self._compressed_bytes(n_compressed)
            else:
                bytes_full, bytes_comp = cache_len * bpt * n_layers, 0
            stats.append(V14StepStats(
                kv_kept=cache_len, kv_bytes_full=bytes_full, kv_bytes_compressed=bytes_comp,
                kv_bytes_total=bytes_full + bytes_comp,
                compress_ms=compress_ms if step == 0 else 0,
                n_full=n_full + step + 1, n_compressed=n_compressed))
        return torch.cat(logits, dim=1), stats

    def _quantize_far(self, past, device_str, dtype):
        """Replace tokens [W_sink, len - W_min) of every layer by their quantize ->
        dequantize image (reference :253-306).  Returns (cache, n_full, n_compressed)."""
        from transformers.cache_utils import DynamicCache

        cache_len = _layer_kv(past, 0)[0].shape[2]
        far_end = cache_len - self.W_min
        n_far = far_end - self.W_sink
        if cache_len <= self.W_min + self.W_sink or n_far <= 0:
            return past, cache_len, 0
        new_cache = DynamicCache()
        for li in range(_n_layers(past)):
            k, v = _layer_kv(past, li)
            bits = self.layer_bits[li] if self.layer_bits else 8
            pieces = []
            for t in (k, v):
                far = self._roundtrip(t[:, :, self.W_sink:far_end, :], bits).to(dtype)
                pieces.append(torch.cat([t[:, :, :self.W_sink, :], far, t[:, :, far_end:, :]], dim=2))
            new_cache.update(pieces[0], pieces[1], li)
        return new_cache, self.W_sink + self.W_min, n_far

    def compression_ratio(self):
        if self.calibrated and self.layer_bits:
            return np.mean(self.layer_bits) / 16.0
        return self.default_bits / 16.0

    def description(self):
        if self.calibrated and self.layer_bits:
            n4 = sum(1 for b in self.layer_bits if b == 4)
            return f"quant ({n4}xINT4 + {len(self.layer_bits) - n4}xINT8)"
        return f"quant (default={self.default_bits}bit)"


# --------------------------------------------------------------------------- packed far cache
_ACTIVE_PACKED = None  # the PackedQuantBackend whose run_decode is in progress
_ATTN_NAME = "knlp_b200_packed"


def _packed_attention(module, query, key, value, attention_mask=None, dropout=0.0, scaling=None,
                      **kwargs):
    """Attention function installed into the model while ``PackedQuantBackend.run_decode``
    steps: ``key`` / ``value`` hold only the tokens kept in full (sink + near + new), the
    far tokens of this layer live in a packed cache and are attended to by the decode
    kernel; the two softmax partials are merged by the combine kernel."""
    from . import ops
    st = _ACTIVE_PACKED
    if st is None or query.shape[2] != 1:
        raise RuntimeError("the packed attention function only serves single-token decode steps "
                           "of PackedQuantBackend.run_decode")
    B, H, _, D = query.shape
    if scaling is not None and abs(scaling - D ** -0.5) > 1e-6 * D ** -0.5:
        raise NotImplementedError("only the standard head_dim^-1/2 softmax scale is supported")
    far = st._far[module.layer_idx]
    q3 = query.reshape(B, H, D).contiguous()
    # dense part (sink + near + the new token): one partial (o un-normalised, m, l) per row
    n_rep = H // key.shape[1]
    k = key if n_rep == 1 else key.repeat_interleave(n_rep, dim=1)
    v = value if n_rep == 1 else value.repeat_interleave(n_rep, dim=1)
    s = torch.einsum("bhd,bhtd->bht", q3.float(), k.float()) * (D ** -0.5)
    m = s.max(dim=-1, keepdim=True).values
    pr = torch.exp(s - m)
    dense = torch.cat([torch.einsum("bht,bhtd->bhd", pr, v.float()), m,
                       pr.sum(dim=-1, keepdim=True)], dim=-1)
    if far is None:
        packed = dense.unsqueeze(0)
    else:
        cache, table, lens = far
        far_part = ops.decode_attention(q3, cache._k_plane(), cache._v_plane(), cache.num_blocks,
                                        table, lens, cache.num_kv_heads, D, cache.block_size,
                                        max_seq_len=st._n_far, emit_partial=True)
        packed = torch.stack([far_part, dense.contiguous()])
    out = ops.combine_packed(packed.contiguous(), out_dtype=query.dtype)
    return out.view(B, 1, H, D), None


class PackedQuantBackend(QuantBackend):
    """``QuantBackend`` with a REAL packed far segment: the far tokens of every layer are
    quantized once into a packed paged cache (4-bit layers: INT4 asymmetric group-32 K and
    V; 8-bit layers: INT8 group-32 K and V) by the quantize-append kernel and are read by
    the decode-attention kernel at every step; sink, near and new tokens stay in full
    precision.  The reference simulates this (``backends/quant.py:253-306`` puts the
    dequantized far tokens back into a float cache), so the evaluation harness never
    reaches its fused kernels; here it does, and the byte accounting is that of the
    buffers that exist.  Interface, calibration and statistics as ``QuantBackend``."""

    PAGE = 16

    @property
    def name(self):
        return "quant_packed"

    def _pack_far(self, past, dtype):
        """Packed caches for tokens [W_sink, len - W_min) and a DynamicCache of the rest."""
        from transformers.cache_utils import DynamicCache
        from .cache import PackedKVCache

        cache_len = _layer_kv(past, 0)[0].shape[2]
        far_end = cache_len - self.W_min
        n_far = far_end - self.W_sink
        if cache_len <= self.W_min + self.W_sink or n_far <= 0:
            self._far = [None] * _n_layers(past)
            self._n_far = 0
            return past, cache_len, 0
        P = self.PAGE
        self._far, self._n_far = [], n_far
        dense = DynamicCache()
        for li in range(_n_layers(past)):
            k, v = _layer_kv(past, li)
            B, Hkv, _, D = k.shape
            bits = self.layer_bits[li] if self.layer_bits else 8
            prec = "int4" if bits == 4 else "int8"
            c = PackedKVCache(Hkv, D, prec, prec, asymmetric=(bits == 4))
            pages = (n_far + P - 1) // P
            c.ensure(B * pages, P, k.device)
            table = torch.arange(B * pages, dtype=torch.int32, device=k.device).view(B, pages)
            pos = torch.arange(n_far, device=k.device)
            slots = (table[:, pos // P].to(torch.int64) * P + pos % P).reshape(-1)
            # [B, H, T, D] -> token-major rows [B * n_far, H, D]
            rows = lambda t: t[:, :, self.W_sink:far_end, :].permute(0, 2, 1, 3).reshape(-1, Hkv, D)
            c.write(rows(k).contiguous(), rows(v).contiguous(), slots)
            lens = torch.full((B,), n_far, dtype=torch.int32, device=k.device)
            self._far.append((c, table, lens))
            dense.update(torch.cat([k[:, :, :self.W_sink], k[:, :, far_end:]], dim=2),
                         torch.cat([v[:, :, :self.W_sink], v[:, :, far_end:]], dim=2), li)
        return dense, self.W_sink + self.W_min, n_far

    def _compressed_bytes(self, n_compressed):
        """Bytes of the packed far segment as allocated (codes, scales, zero-points)."""
        total = 0
        for far in getattr(self, "_far", []):
            if far is not None:
                c = far[0]
                total += n_compressed * c.expected_bytes_per_block() // c.block_size
        return int(total)

    @torch.no_grad()
    def run_decode(self, model, prefix_ids, continuation_ids, device_str, max_ctx):
        global _ACTIVE_PACKED
        from transformers import AttentionInterface

        n_layers = self.mc["n_layers"]
        bpt = _kv_bytes_per_token(self.mc)
        out = model(prefix_ids, use_cache=True)
        past = out.past_key_values
        dtype = _layer_kv(past, 0)[0].dtype
        logits = [out.logits[:, -1:, :]]
        stats = []
        pos = prefix_ids.shape[1]
        t0 = time.perf_counter()
        past, n_full, n_compressed = self._pack_far(past, dtype)
        compress_ms = (time.perf_counter() - t0) * 1000
        AttentionInterface.register(_ATTN_NAME, _packed_attention)
        old_impl = model.config._attn_implementation
        _ACTIVE_PACKED = self
        try:
            model.config._attn_implementation = _ATTN_NAME
            for step in range(continuation_ids.shape[1]):
                pos_ids = torch.tensor([[pos]], device=device_str, dtype=torch.long)
                out = model(continuation_ids[:, step:step + 1], past_key_values=past,
                            use_cache=True, position_ids=pos_ids)
                past = out.past_key_values
                logits.append(out.logits)
                pos += 1
                bytes_full = (n_full + step + 1) * bpt * n_layers
                bytes_comp = self._compressed_bytes(n_compressed)
                stats.append(V14StepStats(
                    kv_kept=n_full + step + 1 + n_compressed, kv_bytes_full=bytes_full,
                    kv_bytes_compressed=bytes_comp, kv_bytes_total=bytes_full + bytes_comp,
                    compress_ms=compress_ms if step == 0 else 0,
                    n_full=n_full + step + 1, n_compressed=n_compressed))
        finally:
            model.config._attn_implementation = old_impl
            _ACTIVE_PACKED = None
        return torch.cat(logits, dim=1), stats

    def description(self):
        return "packed far cache: " + super().description()


def get_backend(name: str) -> CompressionBackend:
    """The two names of the reference's registry (``eval_v14b.py:54-104``) that this
    library serves, plus the dense control."""
    if name == "dense":
        return DenseBackend()
    if name == "quant":
        return QuantBackend()
    if name == "quant_int4":
        b = QuantBackend()
        b._force_int4 = True
        return b
    if name == "quant_packed":  # no counterpart in the reference's registry
        return PackedQuantBackend()
    raise ValueError(f"unknown backend {name!r}; knlp_b200 provides dense, quant, quant_int4, "
                     "quant_packed")
