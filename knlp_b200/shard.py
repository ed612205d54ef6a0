"""Multi-GPU partitioning of the decode path: one process per GPU.

The reference never runs this path on more than one GPU
(``tensor_parallel_size=1`` wherever its fused backend is driven,
scripts/fused-quant/profiles/stage1_quick_profile.py:25-32 of mcgrof/knlp), so
both shards below are new.  They need no custom communication: a kv-head shard
exchanges nothing inside attention, a context shard exchanges one small buffer.

kv-head shard
    Rank r owns kv heads [r*Hkv/G, (r+1)*Hkv/G) and their q heads.  Its cache is
    born with Hkv/G heads; attention over it is an ordinary single-GPU call and
    its output slice [S, Hq/G, d] stays on the rank (a tensor-parallel o_proj
    consumes it sharded).  ``gather_heads`` assembles the full output when a
    caller wants it.

context shard
    Rank r owns tokens [r*T/G, (r+1)*T/G) of every sequence (page aligned).  It
    runs the decode kernel over its segment, which leaves ONE partial per
    (sequence, q head), packed as fp32 rows [o(d), m, l], in the send buffer; a
    single all-gather (NCCL over NVLink) moves S*Hq*(d+2)*4 bytes per rank; every
    rank then merges the G partials with the combine kernel.

The plumbing here (ownership arithmetic, the all-gather) is device agnostic so
that it can be tested with gloo ranks on CPU; the kernels are CUDA only.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def head_shard(n_kv_heads: int, world: int, rank: int) -> slice:
    """kv heads owned by ``rank`` (contiguous, equal sized)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    if n_kv_heads % world:
        raise ValueError(f"{world} ranks do not divide {n_kv_heads} kv heads")
    per = n_kv_heads // world
    return slice(rank * per, (rank + 1) * per)


def q_heads_of(kv: slice, n_rep: int) -> slice:
    """q heads that read the kv heads ``kv`` (GQA: q head h reads kv head h // n_rep)."""
    return slice(kv.start * n_rep, kv.stop * n_rep)


def context_shard(seq_len: int, world: int, rank: int, page: int = 16) -> Tuple[int, int]:
    """Token range [start, end) of one sequence owned by ``rank``: contiguous
    segments whose boundaries are multiples of ``page`` (so a page never spans two
    ranks); the last rank takes the remainder.  Ranks past the end own nothing."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    pages = (seq_len + page - 1) // page
    per = (pages + world - 1) // world
    start = min(rank * per * page, seq_len)
    end = min((rank + 1) * per * page, seq_len)
    return start, end


def context_shard_lens(seq_lens: List[int], world: int, rank: int, page: int = 16) -> List[int]:
    """Local lengths of every sequence on ``rank`` (its segment may be empty)."""
    out = []
    for L in seq_lens:
        s, e = context_shard(L, world, rank, page)
        out.append(e - s)
    return out


def all_gather_packed(packed: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather the packed partials of every rank: [..., d+2] -> [G, ..., d+2].
    One collective; NCCL for CUDA tensors, gloo for CPU tensors."""
    if not (dist.is_available() and dist.is_initialized()):
        return packed.unsqueeze(0).contiguous()
    world = dist.get_world_size(group)
    packed = packed.contiguous()
    out = torch.empty((world,) + tuple(packed.shape), dtype=packed.dtype, device=packed.device)
    if packed.is_cuda:
        dist.all_gather_into_tensor(out, packed, group=group)
    else:
        parts = list(out.unbind(0))
        dist.all_gather(parts, packed, group=group)
    return out


def gather_heads(out_slice: torch.Tensor, group=None) -> torch.Tensor:
    """[S, Hq/G, d] per rank -> [S, Hq, d] on every rank (kv-head shard)."""
    if not (dist.is_available() and dist.is_initialized()):
        return out_slice
    world = dist.get_world_size(group)
    out_slice = out_slice.contiguous()
    buf = torch.empty((world,) + tuple(out_slice.shape), dtype=out_slice.dtype,
                      device=out_slice.device)
    if out_slice.is_cuda:
        dist.all_gather_into_tensor(buf, out_slice, group=group)
    else:
        dist.all_gather(list(buf.unbind(0)), out_slice, group=group)
    S, hq, d = out_slice.shape
    return buf.permute(1, 0, 2, 3).reshape(S, world * hq, d)


def context_sharded_attention(query, k_plane, v_plane, num_blocks, block_table, local_seq_lens,
                              num_kv_heads: int, head_size: int, block_size: int, *,
                              max_seq_len=None, group=None, out_dtype=None) -> torch.Tensor:
    """One decode step of a context shard on CUDA: this rank's segment of every sequence is
    attended to by the balanced kernel, which writes the rank's ONE packed softmax partial
    per (sequence, q head) straight into the buffer that the all-gather sends (the only
    exchange of the step); the merge of the ranks' partials follows.  ``block_table`` and
    ``local_seq_lens`` describe the rank's own segment.  Returns [S, Hq, d] on every rank."""
    from . import ops
    packed = ops.decode_attention(query, k_plane, v_plane, num_blocks, block_table,
                                  local_seq_lens, num_kv_heads, head_size, block_size,
                                  max_seq_len=max_seq_len, emit_partial=True)
    gathered = all_gather_packed(packed, group)
    return ops.combine_packed(gathered,
                              out_dtype=query.dtype if out_dtype is None else out_dtype)


def context_sharded_decode(local_partials, group=None, out_dtype=torch.float32) -> torch.Tensor:
    """Finish a context-sharded decode step on CUDA.

    ``local_partials`` = (m, l, o) of this rank's segment as returned by
    ``ops.decode_partials`` ([S, Hq, n], [S, Hq, n], [S, Hq, n, d]).  Merges the local
    splits into one packed partial, all-gathers it (the only exchange of the step)
    and merges the ranks.  Returns the attention output [S, Hq, d] on every rank.
    """
    from . import ops
    pm, pl, po = local_partials
    packed = ops.combine_to_packed(pm, pl, po)        # [S, Hq, d+2]
    gathered = all_gather_packed(packed, group)        # [G, S, Hq, d+2]
    return ops.combine_packed(gathered, out_dtype=out_dtype)
