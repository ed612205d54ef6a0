"""Operator surface of the packed-KV hot path, with the reference's signatures.

Drop-in for the module-level functions of mcgrof/knlp's
``fused-quant/fused_int4.v0.1.0.py``:

    reshape_and_cache_int4          (:418-472)
    reshape_and_cache_v_only_int4   (:603-647)
    reshape_and_cache_k_int8        (:1287-1312)
    fused_int4_decode               (:901-979)
    kint8_vint4_decode              (:1496-1554)
    reshape_and_cache_v_int8        (:1619-1645)
    kint8_vint8_decode              (:1796-1843)
    kfp16_vint4_decode              (:1159-1224)   stride-generic kernel
    kfp16_vint8_decode              (:1975-2028)   stride-generic kernel

Same argument names, order, meaning and in-place behaviour; tensors are CUDA
tensors owned by the caller.  The work is done by hand-written sm_100a kernels in
libknlp_b200.so, reached through its C ABI (include/knlp_b200.h) with raw device
pointers; torch only supplies memory and the current stream.  There is no CPU or
eager fallback: a CPU tensor, or a missing library, raises.

Additions that the reference does not have (keyword-only, all optional):
``out_dtype`` (fp32 output straight from the fp32 accumulator), ``max_seq_len``
(host-known bound on ``seq_lens``; default ``block_table.shape[1] * block_size``,
so that no device value is read back), ``n_splits``, ``force_generic``, and the
split-context entry points ``decode_partials`` / ``combine_partials`` used by the
multi-GPU context shard.
"""

from __future__ import annotations

import contextlib
import ctypes as C
import os
from typing import Optional, Tuple

import torch

from . import _lib

# Environment defaults honoured like the reference (fused_int4.v0.1.0.py:55-78).
GROUP_SIZE: int = int(os.environ.get("VLLM_FUSED_INT4_GROUP_SIZE", "32"))
OUTLIER_CLIP_RATIO: float = float(os.environ.get("VLLM_FUSED_INT4_OUTLIER_CLIP_RATIO", "10.0"))
ASYMMETRIC: bool = os.environ.get("VLLM_FUSED_INT4_ASYMMETRIC", "0") == "1"

if GROUP_SIZE != 32:
    raise RuntimeError("knlp_b200 is built for VLLM_FUSED_INT4_GROUP_SIZE=32 only")

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32/float16/bfloat16") from None


def _need_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("knlp_b200 operators take CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("all tensors must live on the same CUDA device")
    return dev


def _stride3(t: torch.Tensor):
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError("cache tensors must be 4-D with a contiguous last dimension")
    return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def _stride2(t: torch.Tensor):
    if t.dim() != 3 or t.stride(2) != 1:
        raise ValueError("expected [n, heads, head_size] with a contiguous last dimension")
    return (C.c_int64 * 2)(t.stride(0), t.stride(1))


_planes = {}  # (pointers, strides, dtype, mode) -> marshalled knlp_kv_plane


def _plane(codes, scales, zeros, mode) -> _lib.KvPlane:
    """The knlp_kv_plane of a cache.  A decode step passes the same tensors every time, so
    the marshalled struct is kept per (pointers, strides, dtype, mode)."""
    key = (codes.data_ptr(), scales.data_ptr(), 0 if zeros is None else zeros.data_ptr(), mode,
           codes.stride(), scales.stride(), None if zeros is None else zeros.stride(),
           codes.dtype)
    p = _planes.get(key)
    if p is not None:
        return p
    p = _lib.KvPlane()
    if codes.dtype not in (torch.uint8, torch.int8):
        raise TypeError("code cache must be uint8 (INT4) or int8 (INT8)")
    if scales.dtype != torch.float16 or (zeros is not None and zeros.dtype != torch.float16):
        raise TypeError("scales and zeros must be float16")
    p.codes = codes.data_ptr()
    p.scales = scales.data_ptr()
    p.zeros = zeros.data_ptr() if zeros is not None else None
    p.codes_stride = _stride3(codes)
    p.scales_stride = _stride3(scales)
    p.zeros_stride = _stride3(zeros) if zeros is not None else (C.c_int64 * 3)(0, 0, 0)
    p.mode = mode
    if len(_planes) >= 4096:
        _planes.clear()
    _planes[key] = p
    return p


def _int4_mode(asymmetric: bool, zeros) -> int:
    if asymmetric:
        if zeros is None:
            raise ValueError("asymmetric=True needs the zero-point cache")
        return _lib.KV_INT4_ASYM
    return _lib.KV_INT4_SYM


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


_SAME_DEVICE = contextlib.nullcontext()


def _on(dev):
    """Context that makes ``dev`` the current CUDA device (nothing to do when it already is)."""
    return _SAME_DEVICE if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)


def _quant_append(key, value, k_plane, v_plane, slot_mapping, head_size, block_size, clip_ratio):
    src = key if key is not None else value
    dev = _need_cuda(key, value, slot_mapping)
    if slot_mapping.dtype != torch.int64 or slot_mapping.dim() != 1 or (
            slot_mapping.numel() and slot_mapping.stride(0) != 1):
        raise TypeError("slot_mapping must be a contiguous int64 vector")
    if key is not None and value is not None and key.dtype != value.dtype:
        raise TypeError("key and value must have the same dtype")
    n_tokens, n_heads = src.shape[0], src.shape[1]
    if slot_mapping.numel() != n_tokens:
        raise ValueError("slot_mapping length must equal the number of tokens")
    lib = _lib.load()
    with _on(dev):
        rc = lib.knlp_b200_quant_append(
            key.data_ptr() if key is not None else None,
            _stride2(key) if key is not None else None,
            value.data_ptr() if value is not None else None,
            _stride2(value) if value is not None else None,
            _dt(src),
            C.byref(k_plane) if k_plane is not None else None,
            C.byref(v_plane) if v_plane is not None else None,
            slot_mapping.data_ptr(), n_tokens, n_heads, head_size, block_size,
            float(clip_ratio), _stream(dev))
    _lib.check(rc, "knlp_b200_quant_append")


def quant_append(key, value, k_plane, v_plane, slot_mapping, block_size: int,
                 clip_ratio: Optional[float] = None) -> None:
    """Quantize new tokens into both cache planes in ONE launch, whatever their modes (the
    reference needs two calls when K and V differ: reshape_and_cache_k_int8 :1287-1312 and
    reshape_and_cache_v_only_int4 :603-647).  Planes as built by ``_plane``; ``key`` /
    ``value`` [num_tokens, num_kv_heads, head_size]; either side may be None."""
    src = key if key is not None else value
    _quant_append(key, value, k_plane, v_plane, slot_mapping, src.shape[2], block_size,
                  OUTLIER_CLIP_RATIO if clip_ratio is None else clip_ratio)


def reshape_and_cache_int4(
    key: torch.Tensor,  # [num_tokens, num_heads, head_size]
    value: torch.Tensor,
    key_cache: torch.Tensor,  # [num_blocks, block_size, num_heads, head_size//2] uint8
    value_cache: torch.Tensor,
    k_scales: torch.Tensor,  # [num_blocks, block_size, num_heads, head_size//32] fp16
    v_scales: torch.Tensor,
    slot_mapping: torch.Tensor,  # [num_tokens] int64, <0 = skip
    k_zeros: Optional[torch.Tensor] = None,
    v_zeros: Optional[torch.Tensor] = None,
    asymmetric: bool = False,
    *,
    clip_ratio: Optional[float] = None,
) -> None:
    """Quantize K/V to INT4 and write them into the paged cache, in place
    (reference fused_int4.v0.1.0.py:418-472).  Packed bytes, scales and zeros are
    bit-identical to the reference kernel's."""
    _need_cuda(key_cache, value_cache, k_scales, v_scales, k_zeros, v_zeros)
    head_size = key.shape[2]
    kp = _plane(key_cache, k_scales, k_zeros if asymmetric else None,
                _int4_mode(asymmetric, k_zeros))
    vp = _plane(value_cache, v_scales, v_zeros if asymmetric else None,
                _int4_mode(asymmetric, v_zeros))
    _quant_append(key, value, kp, vp, slot_mapping, head_size, key_cache.shape[1],
                  OUTLIER_CLIP_RATIO if clip_ratio is None else clip_ratio)


def reshape_and_cache_v_only_int4(
    value: torch.Tensor,
    value_cache: torch.Tensor,
    v_scales: torch.Tensor,
    slot_mapping: torch.Tensor,
    v_zeros: Optional[torch.Tensor] = None,
    asymmetric: bool = False,
    *,
    clip_ratio: Optional[float] = None,
) -> None:
    """V-only variant (reference fused_int4.v0.1.0.py:603-647)."""
    _need_cuda(value_cache, v_scales, v_zeros)
    vp = _plane(value_cache, v_scales, v_zeros if asymmetric else None,
                _int4_mode(asymmetric, v_zeros))
    _quant_append(None, value, None, vp, slot_mapping, value.shape[2], value_cache.shape[1],
                  OUTLIER_CLIP_RATIO if clip_ratio is None else clip_ratio)


def reshape_and_cache_k_int8(
    key: torch.Tensor,
    key_cache_int8: torch.Tensor,  # [num_blocks, block_size, num_heads, head_size] int8
    k_scales: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """K -> symmetric INT8 with per-group-32 fp16 scales (reference :1287-1312)."""
    _need_cuda(key_cache_int8, k_scales)
    kp = _plane(key_cache_int8, k_scales, None, _lib.KV_INT8_G32)
    _quant_append(key, None, kp, None, slot_mapping, key.shape[2], key_cache_int8.shape[1], 0.0)


def reshape_and_cache_v_int8(
    value: torch.Tensor,
    value_cache_int8: torch.Tensor,  # [num_blocks, block_size, num_heads, head_size] int8
    v_scales: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """V -> symmetric INT8 with per-group-32 fp16 scales (reference :1619-1645)."""
    _need_cuda(value_cache_int8, v_scales)
    vp = _plane(value_cache_int8, v_scales, None, _lib.KV_INT8_G32)
    _quant_append(None, value, None, vp, slot_mapping, value.shape[2],
                  value_cache_int8.shape[1], 0.0)


def plan_splits(num_seqs: int, num_heads: int, num_kv_heads: int, head_size: int,
                block_size: int, max_seq_len: int) -> int:
    """Split count the library recommends for this decode shape (host arithmetic)."""
    n = C.c_int(0)
    ws = C.c_int64(0)
    rc = _lib.load().knlp_b200_decode_plan(num_seqs, num_heads, num_kv_heads, head_size,
                                           block_size, max_seq_len, 0, 0, C.byref(n), C.byref(ws))
    _lib.check(rc, "knlp_b200_decode_plan")
    return n.value


def _decode_flags(force_generic) -> int:
    """``force_generic``: False = best kernel for the layout (tensor-core kernel staged
    with cp.async, else the generic one); "tma" = tensor-core kernel staged with TMA
    tensor copies and mbarriers (measured slower for this access pattern; kept
    selectable); True = stride-generic CUDA-core kernel."""
    if force_generic == "tma":
        return _lib.DECODE_USE_TMA
    if force_generic == "tma_stall":  # test aid: makes the kernel's bounded wait run out
        return _lib.DECODE_USE_TMA | _lib.DECODE_DEBUG_STALL
    return _lib.DECODE_FORCE_GENERIC if force_generic else 0


def device_status() -> int:
    """Synchronise and return (then clear) the decode kernels' device status word:
    0 = clean, 1 = a bounded barrier wait ran out inside a kernel."""
    return _lib.load().knlp_b200_debug_status()


def decode_partials(
    query: torch.Tensor, k_plane: _lib.KvPlane, v_plane: _lib.KvPlane, num_blocks: int,
    block_table: torch.Tensor, seq_lens: torch.Tensor, num_kv_heads: int, head_size: int,
    block_size: int, *, max_seq_len: Optional[int] = None, n_splits: Optional[int] = None,
    force_generic: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Run the split-context decode kernel and return the softmax partials
    (m [S, Hq, n], l [S, Hq, n], o [S, Hq, n, d]) — m in the natural-log domain,
    o un-normalised."""
    dev = _need_cuda(query, block_table, seq_lens)
    if block_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TypeError("block_table and seq_lens must be int32")
    if block_table.dim() != 2 or block_table.stride(1) != 1 or seq_lens.dim() != 1 or (
            seq_lens.numel() and seq_lens.stride(0) != 1):
        raise ValueError("block_table must be [S, max_blocks] (contiguous rows), seq_lens [S]")
    S, Hq, d = query.shape
    if d != head_size or Hq % num_kv_heads:
        raise ValueError("query shape does not match num_kv_heads / head_size")
    if max_seq_len is None:
        max_seq_len = block_table.shape[1] * block_size
    if n_splits is None:
        n_splits = plan_splits(S, Hq, num_kv_heads, head_size, block_size, max_seq_len)
    pm = torch.empty((S, Hq, n_splits), dtype=torch.float32, device=dev)
    pl = torch.empty((S, Hq, n_splits), dtype=torch.float32, device=dev)
    po = torch.empty((S, Hq, n_splits, d), dtype=torch.float32, device=dev)
    lib = _lib.load()
    with _on(dev):
        rc = lib.knlp_b200_decode_splitk(
            query.data_ptr(), _dt(query), _stride2(query), C.byref(k_plane), C.byref(v_plane),
            block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(), num_blocks,
            S, Hq, num_kv_heads, head_size, block_size, n_splits, max_seq_len,
            pm.data_ptr(), pl.data_ptr(), po.data_ptr(),
            _decode_flags(force_generic), _stream(dev))
    _lib.check(rc, "knlp_b200_decode_splitk")
    return pm, pl, po


def combine_partials(pm: torch.Tensor, pl: torch.Tensor, po: torch.Tensor,
                     out: Optional[torch.Tensor] = None, out_dtype=torch.float32,
                     emit_partial: bool = False, parts_dim: int = -1):
    """Merge softmax partials.

    pm, pl: [..., n_parts] and po: [..., n_parts, d] (``parts_dim=-1``), or with the
    parts dimension first, pm, pl: [n_parts, ...], po: [n_parts, ..., d]
    (``parts_dim=0``, the layout an all-gather of per-rank partials produces).
    Returns the normalised output [..., d] in ``out_dtype``; with
    ``emit_partial=True`` returns the merged partial (m [...], l [...], o [..., d])
    in fp32 instead.
    """
    dev = _need_cuda(pm, pl, po)
    if not (pm.is_contiguous() and pl.is_contiguous() and po.is_contiguous()):
        raise ValueError("partials must be contiguous")
    d = po.shape[-1]
    if parts_dim == 0:
        n_parts = pm.shape[0]
        rows_shape = tuple(pm.shape[1:])
        n_rows = pm[0].numel()
        ml_row, ml_part, o_row, o_part = 1, n_rows, d, n_rows * d
    else:
        n_parts = pm.shape[-1]
        rows_shape = tuple(pm.shape[:-1])
        n_rows = pm.numel() // max(n_parts, 1)
        ml_row, ml_part, o_row, o_part = n_parts, 1, n_parts * d, d
    lib = _lib.load()
    if emit_partial:
        om = torch.empty(rows_shape, dtype=torch.float32, device=dev)
        ol = torch.empty(rows_shape, dtype=torch.float32, device=dev)
        oo = torch.empty(rows_shape + (d,), dtype=torch.float32, device=dev)
        with _on(dev):
            rc = lib.knlp_b200_combine(pm.data_ptr(), pl.data_ptr(), po.data_ptr(), n_parts,
                                       ml_row, ml_part, o_row, o_part, oo.data_ptr(), _lib.F32, d,
                                       om.data_ptr(), ol.data_ptr(), 1, n_rows, d, _stream(dev))
        _lib.check(rc, "knlp_b200_combine")
        return om, ol, oo
    if out is None:
        out = torch.empty(rows_shape + (d,), dtype=out_dtype, device=dev)
    elif not out.is_contiguous() or out.numel() != n_rows * d:
        raise ValueError("out must be contiguous [..., d]")
    with _on(dev):
        rc = lib.knlp_b200_combine(pm.data_ptr(), pl.data_ptr(), po.data_ptr(), n_parts,
                                   ml_row, ml_part, o_row, o_part, out.data_ptr(), _DT[out.dtype],
                                   d, None, None, 0, n_rows, d, _stream(dev))
    _lib.check(rc, "knlp_b200_combine")
    return out


def combine_to_packed(pm: torch.Tensor, pl: torch.Tensor, po: torch.Tensor) -> torch.Tensor:
    """Merge the splits of each row into ONE partial and return it packed as
    fp32 rows [o (d, un-normalised), m, l] of shape [..., d + 2]: the buffer a rank
    of a context shard sends in its single all-gather."""
    dev = _need_cuda(pm, pl, po)
    if not (pm.is_contiguous() and pl.is_contiguous() and po.is_contiguous()):
        raise ValueError("partials must be contiguous")
    d = po.shape[-1]
    n_parts = pm.shape[-1]
    rows_shape = tuple(pm.shape[:-1])
    n_rows = pm.numel() // max(n_parts, 1)
    packed = torch.empty(rows_shape + (d + 2,), dtype=torch.float32, device=dev)
    base = packed.data_ptr()
    with _on(dev):
        rc = _lib.load().knlp_b200_combine(
            pm.data_ptr(), pl.data_ptr(), po.data_ptr(), n_parts, n_parts, 1, n_parts * d, d,
            base, _lib.F32, d + 2, base + 4 * d, base + 4 * (d + 1), d + 2, n_rows, d,
            _stream(dev))
    _lib.check(rc, "knlp_b200_combine")
    return packed


def combine_packed(gathered: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """Final merge of packed partials gathered from all ranks: ``gathered`` is
    [n_ranks, ..., d + 2] (rows as written by ``combine_to_packed``); returns the
    normalised attention output [..., d]."""
    dev = _need_cuda(gathered)
    if not gathered.is_contiguous() or gathered.dtype != torch.float32:
        raise ValueError("gathered partials must be a contiguous fp32 tensor")
    n_parts = gathered.shape[0]
    d = gathered.shape[-1] - 2
    rows_shape = tuple(gathered.shape[1:-1])
    n_rows = gathered[0].numel() // (d + 2)
    out = torch.empty(rows_shape + (d,), dtype=out_dtype, device=dev)
    base = gathered.data_ptr()
    part = n_rows * (d + 2)
    with _on(dev):
        rc = _lib.load().knlp_b200_combine(
            base + 4 * d, base + 4 * (d + 1), base, n_parts, d + 2, part, d + 2, part,
            out.data_ptr(), _DT[out.dtype], d, None, None, 0, n_rows, d, _stream(dev))
    _lib.check(rc, "knlp_b200_combine")
    return out


_workspaces = {}  # (device index, stream) -> (float workspace, int32 counters left zero)


_ws_sizes = {}  # shape -> (floats, counters) of knlp_b200_decode_workspace


def _decode_workspace(dev: torch.device, S: int, Hq: int, Hkv: int, d: int, block_size: int,
                      max_seq_len: int):
    """Workspace of ``knlp_b200_decode_attention`` for the current stream: grown on demand,
    reused by every later call on that stream (calls on one stream are ordered)."""
    shape = (dev.index, S, Hq, Hkv, d, block_size, max_seq_len)
    need = _ws_sizes.get(shape)
    if need is None:
        nf, ni = C.c_int64(0), C.c_int64(0)
        with _on(dev):  # the size depends on the device's SM count
            rc = _lib.load().knlp_b200_decode_workspace(S, Hq, Hkv, d, block_size, max_seq_len,
                                                        C.byref(nf), C.byref(ni))
        _lib.check(rc, "knlp_b200_decode_workspace")
        if len(_ws_sizes) >= 4096:
            _ws_sizes.clear()
        need = _ws_sizes[shape] = (nf.value, ni.value)
    key = (dev.index, _stream(dev))
    cur = _workspaces.get(key)
    if cur is None or cur[0].numel() < need[0] or cur[1].numel() < need[1]:
        cur = (torch.empty(max(need[0], 1 << 20), dtype=torch.float32, device=dev),
               torch.zeros(max(need[1], 4096), dtype=torch.int32, device=dev))
        _workspaces[key] = cur
    return cur


def decode_workspace_floats(S: int, Hq: int, Hkv: int, d: int, block_size: int,
                            max_seq_len: int) -> int:
    """Floats of scratch ``knlp_b200_decode_attention`` asks for at this shape."""
    nf, ni = C.c_int64(0), C.c_int64(0)
    rc = _lib.load().knlp_b200_decode_workspace(S, Hq, Hkv, d, block_size, max_seq_len,
                                                C.byref(nf), C.byref(ni))
    _lib.check(rc, "knlp_b200_decode_workspace")
    return nf.value


def decode_attention(
    query: torch.Tensor, k_plane: _lib.KvPlane, v_plane: _lib.KvPlane, num_blocks: int,
    block_table: torch.Tensor, seq_lens: torch.Tensor, num_kv_heads: int, head_size: int,
    block_size: int, *, out_dtype=None, max_seq_len: Optional[int] = None,
    emit_partial: bool = False, out: Optional[torch.Tensor] = None, flags: int = 0,
    new_key: Optional[torch.Tensor] = None, new_value: Optional[torch.Tensor] = None,
    clip_ratio: Optional[float] = None,
) -> torch.Tensor:
    """Decode attention balanced inside one launch (``knlp_b200_decode_attention``).
    Returns [S, Hq, d] in ``out_dtype`` (default: the query's); with ``emit_partial`` the
    merged softmax partial per row instead, fp32 [S, Hq, d + 2] = [o un-normalised, m, l]
    (what a rank of a context shard all-gathers).

    With ``new_key`` / ``new_value`` ([S, Hkv, d]) the same launch first appends the
    step's new token of every sequence to the cache at position ``seq_lens[s]`` (the
    lengths BEFORE the append) and attends over ``seq_lens[s] + 1`` tokens
    (``knlp_b200_decode_append_attention``)."""
    dev = _need_cuda(query, block_table, seq_lens)
    if block_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TypeError("block_table and seq_lens must be int32")
    if block_table.dim() != 2 or block_table.stride(1) != 1 or seq_lens.dim() != 1 or (
            seq_lens.numel() and seq_lens.stride(0) != 1):
        raise ValueError("block_table must be [S, max_blocks] (contiguous rows), seq_lens [S]")
    S, Hq, d = query.shape
    if d != head_size or Hq % num_kv_heads:
        raise ValueError("query shape does not match num_kv_heads / head_size")
    if max_seq_len is None:
        max_seq_len = block_table.shape[1] * block_size
    ws, counters = _decode_workspace(dev, S, Hq, num_kv_heads, d, block_size, max_seq_len)
    if emit_partial:
        if out is None:
            out = torch.empty((S, Hq, d + 2), dtype=torch.float32, device=dev)
        flags |= _lib.DECODE_EMIT_PARTIAL
    elif out is None:
        out = torch.empty((S, Hq, d), dtype=query.dtype if out_dtype is None else out_dtype,
                          device=dev)
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")
    nt = None
    if new_key is not None or new_value is not None:
        if new_key is None or new_value is None:
            raise ValueError("the fused append needs both new_key and new_value")
        _need_cuda(new_key, new_value)
        if new_key.dtype != new_value.dtype or new_key.shape != (S, num_kv_heads, d) or (
                new_value.shape != new_key.shape):
            raise ValueError("new_key / new_value must be [S, num_kv_heads, head_size] of one dtype")
        nt = _lib.NewTokens()
        nt.key, nt.value = new_key.data_ptr(), new_value.data_ptr()
        nt.key_stride, nt.value_stride = _stride2(new_key), _stride2(new_value)
        nt.dtype = _dt(new_key)
        nt.clip_ratio = float(OUTLIER_CLIP_RATIO if clip_ratio is None else clip_ratio)
    with _on(dev):
        rc = _lib.load().knlp_b200_decode_append_attention(
            query.data_ptr(), _dt(query), _stride2(query), C.byref(k_plane), C.byref(v_plane),
            block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(), num_blocks,
            S, Hq, num_kv_heads, head_size, block_size, max_seq_len,
            ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
            out.data_ptr(), _DT[out.dtype], out.shape[-1], flags,
            C.byref(nt) if nt is not None else None, _stream(dev))
    _lib.check(rc, "knlp_b200_decode_append_attention" if nt is not None
               else "knlp_b200_decode_attention")
    return out


def _decode(query, k_plane, v_plane, num_blocks, block_table, seq_lens, num_kv_heads,
            head_size, block_size, out_dtype, max_seq_len, n_splits, force_generic,
            two_launches=False):
    # Default: the balanced one-launch kernel.  A given split count, a forced kernel or
    # two_launches=True run the split-context kernel and the combine kernel instead.
    if two_launches or n_splits is not None or force_generic:
        pm, pl, po = decode_partials(query, k_plane, v_plane, num_blocks, block_table, seq_lens,
                                     num_kv_heads, head_size, block_size,
                                     max_seq_len=max_seq_len, n_splits=n_splits,
                                     force_generic=force_generic)
        return combine_partials(pm, pl, po,
                                out_dtype=query.dtype if out_dtype is None else out_dtype)
    return decode_attention(query, k_plane, v_plane, num_blocks, block_table, seq_lens,
                            num_kv_heads, head_size, block_size, out_dtype=out_dtype,
                            max_seq_len=max_seq_len)


def fused_int4_decode(
    query: torch.Tensor,  # [num_seqs, num_heads, head_size]
    key_cache: torch.Tensor,  # [num_blocks, block_size, num_kv_heads, head_size//2]
    value_cache: torch.Tensor,
    k_scales: torch.Tensor,  # [num_blocks, block_size, num_kv_heads, head_size//32]
    v_scales: torch.Tensor,
    block_table: torch.Tensor,  # [num_seqs, max_num_blocks_per_seq] int32
    seq_lens: torch.Tensor,  # [num_seqs] int32
    num_kv_heads: int,
    head_size: int,
    block_n: int = 64,  # tuning hint of the reference kernel; ignored here
    k_zeros: Optional[torch.Tensor] = None,
    v_zeros: Optional[torch.Tensor] = None,
    asymmetric: bool = False,
    *,
    out_dtype: Optional[torch.dtype] = None,
    max_seq_len: Optional[int] = None,
    n_splits: Optional[int] = None,
    force_generic: bool = False,
    two_launches: bool = False,
) -> torch.Tensor:
    """Decode attention over the packed INT4 cache (reference :901-979).

    Returns [num_seqs, num_heads, head_size] in the query dtype (``out_dtype``
    overrides; fp32 is the un-rounded accumulator).  Sequences of length 0 give 0.
    """
    _need_cuda(key_cache, value_cache, k_scales, v_scales, k_zeros, v_zeros)
    kp = _plane(key_cache, k_scales, k_zeros if asymmetric else None,
                _int4_mode(asymmetric, k_zeros))
    vp = _plane(value_cache, v_scales, v_zeros if asymmetric else None,
                _int4_mode(asymmetric, v_zeros))
    return _decode(query, kp, vp, key_cache.shape[0], block_table, seq_lens, num_kv_heads,
                   head_size, key_cache.shape[1], out_dtype, max_seq_len, n_splits, force_generic,
                   two_launches)


def kint8_vint4_decode(
    query: torch.Tensor,
    key_cache_int8: torch.Tensor,  # [num_blocks, block_size, kv_heads, head_size] int8
    value_cache_int4: torch.Tensor,  # [num_blocks, block_size, kv_heads, head_size//2] uint8
    k_scales: torch.Tensor,
    v_scales: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    num_kv_heads: int,
    head_size: int,
    block_n: int = 64,
    v_zeros: Optional[torch.Tensor] = None,
    asymmetric: bool = False,
    *,
    out_dtype: Optional[torch.dtype] = None,
    max_seq_len: Optional[int] = None,
    n_splits: Optional[int] = None,
    force_generic: bool = False,
    two_launches: bool = False,
) -> torch.Tensor:
    """K INT8 (group-32 scales) / V INT4 decode attention (reference :1496-1554)."""
    _need_cuda(key_cache_int8, value_cache_int4, k_scales, v_scales, v_zeros)
    kp = _plane(key_cache_int8, k_scales, None, _lib.KV_INT8_G32)
    vp = _plane(value_cache_int4, v_scales, v_zeros if asymmetric else None,
                _int4_mode(asymmetric, v_zeros))
    return _decode(query, kp, vp, key_cache_int8.shape[0], block_table, seq_lens, num_kv_heads,
                   head_size, key_cache_int8.shape[1], out_dtype, max_seq_len, n_splits,
                   force_generic, two_launches)


def kint8_vint8_decode(
    query: torch.Tensor,
    key_cache_int8: torch.Tensor,  # [num_blocks, block_size, kv_heads, head_size] int8
    value_cache_int8: torch.Tensor,  # same shape, int8
    k_scales: torch.Tensor,
    v_scales: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    num_kv_heads: int,
    head_size: int,
    block_n: int = 64,
    *,
    out_dtype: Optional[torch.dtype] = None,
    max_seq_len: Optional[int] = None,
    n_splits: Optional[int] = None,
    force_generic: bool = False,
    two_launches: bool = False,
) -> torch.Tensor:
    """K INT8 / V INT8 decode attention, group-32 scales on both (reference :1796-1843)."""
    _need_cuda(key_cache_int8, value_cache_int8, k_scales, v_scales)
    kp = _plane(key_cache_int8, k_scales, None, _lib.KV_INT8_G32)
    vp = _plane(value_cache_int8, v_scales, None, _lib.KV_INT8_G32)
    return _decode(query, kp, vp, key_cache_int8.shape[0], block_table, seq_lens, num_kv_heads,
                   head_size, key_cache_int8.shape[1], out_dtype, max_seq_len, n_splits,
                   force_generic, two_launches)


def _fp_plane(cache: torch.Tensor) -> _lib.KvPlane:
    """An unquantized [num_blocks, block_size, kv_heads, head_size] fp16 / bf16 K cache."""
    if cache.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("the unquantized K cache must be float16 or bfloat16")
    p = _lib.KvPlane()
    p.codes = cache.data_ptr()
    p.scales = None
    p.zeros = None
    p.codes_stride = _stride3(cache)  # in 2-byte elements, as the C ABI expects for this mode
    p.scales_stride = (C.c_int64 * 3)(0, 0, 0)
    p.zeros_stride = (C.c_int64 * 3)(0, 0, 0)
    p.mode = _lib.KV_F16 if cache.dtype == torch.float16 else _lib.KV_BF16
    return p


def kfp16_vint4_decode(
    query: torch.Tensor,
    key_cache_fp16: torch.Tensor,  # [num_blocks, block_size, kv_heads, head_size] fp16 / bf16
    value_cache_int4: torch.Tensor,  # [num_blocks, block_size, kv_heads, head_size//2] uint8
    v_scales: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    num_kv_heads: int,
    head_size: int,
    block_n: int = 64,
    v_zeros: Optional[torch.Tensor] = None,
    asymmetric: bool = False,
    *,
    out_dtype: Optional[torch.dtype] = None,
    max_seq_len: Optional[int] = None,
    n_splits: Optional[int] = None,
) -> torch.Tensor:
    """K unquantized / V INT4 hybrid decode (reference :1159-1224).  The balanced
    tensor-core launch takes it (the fp16 / bf16 K tile is the MMA operand as it lies in
    memory); a given ``n_splits`` or a layout it cannot address runs the stride-generic
    kernel."""
    _need_cuda(key_cache_fp16, value_cache_int4, v_scales, v_zeros)
    kp = _fp_plane(key_cache_fp16)
    vp = _plane(value_cache_int4, v_scales, v_zeros if asymmetric else None,
                _int4_mode(asymmetric, v_zeros))
    return _decode(query, kp, vp, key_cache_fp16.shape[0], block_table, seq_lens, num_kv_heads,
                   head_size, key_cache_fp16.shape[1], out_dtype, max_seq_len, n_splits,
                   False, False)


def kfp16_vint8_decode(
    query: torch.Tensor,
    key_cache_fp16: torch.Tensor,
    value_cache_int8: torch.Tensor,  # [num_blocks, block_size, kv_heads, head_size] int8
    v_scales: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    num_kv_heads: int,
    head_size: int,
    block_n: int = 64,
    *,
    out_dtype: Optional[torch.dtype] = None,
    max_seq_len: Optional[int] = None,
    n_splits: Optional[int] = None,
) -> torch.Tensor:
    """K unquantized / V INT8 hybrid decode (reference :1975-2028).  Kernels as for
    ``kfp16_vint4_decode``."""
    _need_cuda(key_cache_fp16, value_cache_int8, v_scales)
    kp = _fp_plane(key_cache_fp16)
    vp = _plane(value_cache_int8, v_scales, None, _lib.KV_INT8_G32)
    return _decode(query, kp, vp, key_cache_fp16.shape[0], block_table, seq_lens, num_kv_heads,
                   head_size, key_cache_fp16.shape[1], out_dtype, max_seq_len, n_splits,
                   False, False)
