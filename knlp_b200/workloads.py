"""Seeded synthetic decode workloads with the shapes and value distributions of
the benchmark configurations (stand-ins for the reference's own synthetic-tensor
kernel benches, scripts/spev01/tier5_fused_decode.py:403-451 of mcgrof/knlp).

A workload is a paged packed KV cache filled by the library's own
quantize/append kernel from seeded bf16/fp32 N(0,1) K/V (1 % of the channels of
each kv head scaled x10 as outliers), a query batch, a block table and sequence
lengths.  K/V are generated and quantized chunk by chunk on the device, so the
5 GB caches never exist in floating point.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import ops

PAGE = 16


@dataclass
class Workload:
    name: str
    n_q_heads: int
    n_kv_heads: int  # kv heads held by THIS cache (after a head shard)
    head_dim: int
    k_mode: str  # "int4_asym" | "int4_sym" | "int8"
    v_mode: str  # "int4_asym" | "int4_sym"
    query: torch.Tensor
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    k_scales: torch.Tensor
    v_scales: torch.Tensor
    k_zeros: Optional[torch.Tensor]
    v_zeros: Optional[torch.Tensor]
    block_table: torch.Tensor
    seq_lens: torch.Tensor
    seq_lens_host: list = field(default_factory=list)
    max_seq_len: int = 0

    @property
    def n_seqs(self) -> int:
        return self.query.shape[0]

    def kv_bytes_per_token_head(self) -> int:
        d, ng = self.head_dim, self.head_dim // 32
        kb = d + 2 * ng if self.k_mode == "int8" else d // 2 + (4 * ng if self.k_mode == "int4_asym" else 2 * ng)
        vb = d + 2 * ng if self.v_mode == "int8" else d // 2 + (4 * ng if self.v_mode == "int4_asym" else 2 * ng)
        return kb + vb

    def algorithmic_bytes(self) -> int:
        """Bytes one decode step must move: every cached (token, kv head) row of
        codes, scales and zeros once, the queries in, the output out, and the
        page-table entries it walks."""
        toks = sum(self.seq_lens_host)
        qo = self.query.numel() * self.query.element_size() * 2
        pages = sum((L + PAGE - 1) // PAGE for L in self.seq_lens_host)
        return toks * self.n_kv_heads * self.kv_bytes_per_token_head() + qo + 4 * pages

    def planes(self):
        """The (K, V) cache planes as the C ABI takes them."""
        L = ops._lib
        if self.k_mode == "int8":
            kp = ops._plane(self.key_cache, self.k_scales, None, L.KV_INT8_G32)
        else:
            asym = self.k_mode == "int4_asym"
            kp = ops._plane(self.key_cache, self.k_scales, self.k_zeros if asym else None,
                            L.KV_INT4_ASYM if asym else L.KV_INT4_SYM)
        if self.v_mode == "int8":
            vp = ops._plane(self.value_cache, self.v_scales, None, L.KV_INT8_G32)
        else:
            asym = self.v_mode == "int4_asym"
            vp = ops._plane(self.value_cache, self.v_scales, self.v_zeros if asym else None,
                            L.KV_INT4_ASYM if asym else L.KV_INT4_SYM)
        return kp, vp

    def caches(self):
        return (self.key_cache, self.value_cache, self.k_scales, self.v_scales, self.k_zeros,
                self.v_zeros)

    def decode(self, **kw) -> torch.Tensor:
        if self.k_mode == "int8" and self.v_mode == "int8":
            return ops.kint8_vint8_decode(
                self.query, self.key_cache, self.value_cache, self.k_scales, self.v_scales,
                self.block_table, self.seq_lens, self.n_kv_heads, self.head_dim,
                max_seq_len=self.max_seq_len, **kw)
        if self.k_mode == "int8":
            return ops.kint8_vint4_decode(
                self.query, self.key_cache, self.value_cache, self.k_scales, self.v_scales,
                self.block_table, self.seq_lens, self.n_kv_heads, self.head_dim,
                v_zeros=self.v_zeros, asymmetric=self.v_mode == "int4_asym",
                max_seq_len=self.max_seq_len, **kw)
        asym = self.k_mode == "int4_asym"
        return ops.fused_int4_decode(
            self.query, self.key_cache, self.value_cache, self.k_scales, self.v_scales,
            self.block_table, self.seq_lens, self.n_kv_heads, self.head_dim,
            k_zeros=self.k_zeros, v_zeros=self.v_zeros, asymmetric=asym,
            max_seq_len=self.max_seq_len, **kw)


def outlier_channel_scale(n_kv_heads: int, head_dim: int, gen: torch.Generator,
                          frac: float = 0.01) -> torch.Tensor:
    """[n_kv_heads, head_dim] multiplier: x10 on ~1 % of the channels, at least one
    per head, chosen from the seed (CPU generator, so every rank draws the same)."""
    mask = torch.rand(n_kv_heads, head_dim, generator=gen) < frac
    for h in range(n_kv_heads):
        if not mask[h].any():
            mask[h, int(torch.randint(0, head_dim, (1,), generator=gen))] = True
    return torch.where(mask, torch.tensor(10.0), torch.tensor(1.0))


def alloc_cache(num_blocks: int, n_kv_heads: int, head_dim: int, k_mode: str, v_mode: str,
                device, page: int = PAGE):
    ng = head_dim // 32
    kw = head_dim if k_mode == "int8" else head_dim // 2
    kc = torch.zeros(num_blocks, page, n_kv_heads, kw, device=device,
                     dtype=torch.int8 if k_mode == "int8" else torch.uint8)
    vc = torch.zeros(num_blocks, page, n_kv_heads, head_dim if v_mode == "int8" else head_dim // 2,
                     device=device, dtype=torch.int8 if v_mode == "int8" else torch.uint8)
    mk = lambda: torch.zeros(num_blocks, page, n_kv_heads, ng, device=device, dtype=torch.float16)
    ks, vs = mk(), mk()
    kz = mk() if k_mode == "int4_asym" else None
    vz = mk() if v_mode == "int4_asym" else None
    return kc, vc, ks, vs, kz, vz


def append_tokens(w_or_caches, key, value, slots, k_mode, v_mode):
    kc, vc, ks, vs, kz, vz = w_or_caches
    if k_mode == "int8":
        ops.reshape_and_cache_k_int8(key, kc, ks, slots)
        if v_mode == "int8":
            ops.reshape_and_cache_v_int8(value, vc, vs, slots)
        else:
            ops.reshape_and_cache_v_only_int4(value, vc, vs, slots, vz,
                                              asymmetric=v_mode == "int4_asym")
    else:
        ops.reshape_and_cache_int4(key, value, kc, vc, ks, vs, slots, kz, vz,
                                   asymmetric=k_mode == "int4_asym")


def build(name: str, *, n_seqs: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
          seq_lens, seed: int, device, kv_dtype=torch.bfloat16, q_dtype=torch.bfloat16,
          k_mode: str = "int4_asym", v_mode: str = "int4_asym", shuffle_pages: bool = False,
          head_slice: Optional[slice] = None, extra_blocks_per_seq: int = 0,
          chunk_tokens: int = 32768, ctx_shard: Optional[tuple] = None) -> Workload:
    """Build one workload on ``device``.

    ``ctx_shard = (world, rank)`` keeps only the rank's contiguous, page-aligned token
    segment of every sequence (``shard.context_shard``): the cache of one rank of a
    context shard, holding exactly the values the unsharded cache holds there.

    ``head_slice`` keeps only those kv heads (and their q heads): the cache of one
    rank of a kv-head shard.  Values are drawn per (sequence, token chunk) from a
    generator seeded by (seed, sequence, chunk), for ALL heads, and sliced, so the
    shard of a rank holds exactly the values the unsharded cache would.
    """
    cpu_gen = torch.Generator().manual_seed(seed)
    glens = [int(x) for x in seq_lens]  # global lengths
    assert len(glens) == n_seqs
    if ctx_shard is not None:
        from .shard import context_shard
        segs = [context_shard(L, ctx_shard[0], ctx_shard[1], PAGE) for L in glens]
    else:
        segs = [(0, L) for L in glens]
    lens = [b - a for a, b in segs]  # lengths held by this cache
    n_rep = n_q_heads // n_kv_heads
    ch_scale = outlier_channel_scale(n_kv_heads, head_dim, cpu_gen)
    query_all = torch.randn(n_seqs, n_q_heads, head_dim, generator=cpu_gen)
    hs = head_slice if head_slice is not None else slice(0, n_kv_heads)
    heads = range(n_kv_heads)[hs]
    h_local = len(heads)
    qs = slice(heads[0] * n_rep, (heads[-1] + 1) * n_rep)
    query = query_all[:, qs].to(q_dtype).to(device)
    ch_scale_dev = ch_scale[hs].to(device)

    blocks_per_seq = [(L + PAGE - 1) // PAGE + extra_blocks_per_seq for L in lens]
    max_blocks = max(1, max(blocks_per_seq))
    total_blocks = sum(blocks_per_seq)
    if shuffle_pages:
        perm = torch.randperm(total_blocks, generator=cpu_gen).to(torch.int32)
    else:
        perm = torch.arange(total_blocks, dtype=torch.int32)
    bt = torch.zeros(n_seqs, max_blocks, dtype=torch.int32)
    o = 0
    for s, nb in enumerate(blocks_per_seq):
        bt[s, :nb] = perm[o:o + nb]
        o += nb
    caches = alloc_cache(total_blocks, h_local, head_dim, k_mode, v_mode, device)
    bt_dev = bt.to(device)

    dgen = torch.Generator(device=device)
    for s, L in enumerate(glens):
        a0, b0 = segs[s]
        for c0 in range(0, L, chunk_tokens):
            n = min(chunk_tokens, L - c0)
            lo, hi = max(a0, c0), min(b0, c0 + n)
            if hi <= lo:
                continue
            dgen.manual_seed((seed * 1000003 + s) * 4099 + c0 // chunk_tokens)
            kv = torch.randn(2, n, n_kv_heads, head_dim, generator=dgen, device=device,
                             dtype=torch.float32)
            k = (kv[0, lo - c0:hi - c0, hs] * ch_scale_dev).to(kv_dtype)
            v = (kv[1, lo - c0:hi - c0, hs] * ch_scale_dev).to(kv_dtype)
            pos = torch.arange(lo - a0, hi - a0, device=device)  # positions in this cache
            slots = bt_dev[s, pos // PAGE].to(torch.int64) * PAGE + (pos % PAGE)
            append_tokens(caches, k, v, slots, k_mode, v_mode)
    kc, vc, ks, vs, kz, vz = caches
    return Workload(name=name, n_q_heads=h_local * n_rep, n_kv_heads=h_local, head_dim=head_dim,
                    k_mode=k_mode, v_mode=v_mode, query=query, key_cache=kc, value_cache=vc,
                    k_scales=ks, v_scales=vs, k_zeros=kz, v_zeros=vz, block_table=bt_dev,
                    seq_lens=torch.tensor(lens, dtype=torch.int32, device=device),
                    seq_lens_host=lens, max_seq_len=max(lens) if lens else 0)


def config(name: str, device, *, seed: Optional[int] = None, scale: float = 1.0,
           head_slice: Optional[slice] = None, extra_blocks_per_seq: int = 0,
           ctx_shard: Optional[tuple] = None) -> Workload:
    """The named benchmark configurations.  ``scale`` < 1 shrinks context lengths
    (and nothing else) for tests; ``extra_blocks_per_seq`` reserves spare pages per
    sequence for tokens appended later.

      gpt2_mha_1k      12 heads MHA, d 64, batch 1, ctx 1024, fp32 q, fp32 K/V
      llama8b_b32_8k   32 q / 8 kv heads, d 128, batch 32, ctx 8192, bf16
      llama8b_b32_128k same at ctx 131072 (the headline)
      llama8b_b1_384k  batch 1, ctx 393216
      llama70b_ragged  64 q / 8 kv, batch 64, ctx ~ U[1024, 32768], shuffled pages
      mixed_k8v4       32 q / 8 kv, batch 128, ctx ~ U[512, 4096], K int8 + V int4
    """
    def ctx(n):
        return max(1, int(n * scale))

    if name == "gpt2_mha_1k":
        return build(name, n_seqs=1, n_q_heads=12, n_kv_heads=12, head_dim=64, seq_lens=[ctx(1024)],
                     seed=1000 if seed is None else seed, device=device, kv_dtype=torch.float32,
                     q_dtype=torch.float32, head_slice=head_slice, extra_blocks_per_seq=extra_blocks_per_seq,
                     ctx_shard=ctx_shard)
    import re
    m = re.fullmatch(r"llama8b_b(\d+)_(\d+)k", name)
    if m and name != "llama8b_b1_384k":
        # llama8b_b<batch>_<context in Ki tokens>k: uniform batch of the Llama-3-8B shape
        B, T = int(m.group(1)), int(m.group(2)) * 1024
        return build(name, n_seqs=B, n_q_heads=32, n_kv_heads=8, head_dim=128,
                     seq_lens=[ctx(T)] * B, seed=2000 if seed is None else seed, device=device,
                     head_slice=head_slice, extra_blocks_per_seq=extra_blocks_per_seq,
                     ctx_shard=ctx_shard)
    if name == "llama8b_b1_384k":
        return build(name, n_seqs=1, n_q_heads=32, n_kv_heads=8, head_dim=128,
                     seq_lens=[ctx(393216)], seed=3000 if seed is None else seed, device=device,
                     head_slice=head_slice, extra_blocks_per_seq=extra_blocks_per_seq,
                     ctx_shard=ctx_shard)
    if name == "llama70b_ragged":
        g = torch.Generator().manual_seed(4000 if seed is None else seed)
        lens = torch.randint(1024, 32769, (64,), generator=g).tolist()
        return build(name, n_seqs=64, n_q_heads=64, n_kv_heads=8, head_dim=128,
                     seq_lens=[ctx(L) for L in lens], seed=4000 if seed is None else seed,
                     device=device, shuffle_pages=True, head_slice=head_slice, extra_blocks_per_seq=extra_blocks_per_seq,
                     ctx_shard=ctx_shard)
    if name == "mixed_k8v4":
        g = torch.Generator().manual_seed(5000 if seed is None else seed)
        lens = torch.randint(512, 4097, (128,), generator=g).tolist()
        return build(name, n_seqs=128, n_q_heads=32, n_kv_heads=8, head_dim=128,
                     seq_lens=[ctx(L) for L in lens], seed=5000 if seed is None else seed,
                     device=device, k_mode="int8", v_mode="int4_asym", shuffle_pages=True,
                     head_slice=head_slice, extra_blocks_per_seq=max(4, extra_blocks_per_seq),
                     ctx_shard=ctx_shard)
    if name == "k8v8":
        # the mixed workload's batch with both planes INT8 (kint8_vint8_decode)
        g = torch.Generator().manual_seed(5000 if seed is None else seed)
        lens = torch.randint(512, 4097, (128,), generator=g).tolist()
        return build(name, n_seqs=128, n_q_heads=32, n_kv_heads=8, head_dim=128,
                     seq_lens=[ctx(L) for L in lens], seed=5000 if seed is None else seed,
                     device=device, k_mode="int8", v_mode="int8", shuffle_pages=True,
                     head_slice=head_slice, extra_blocks_per_seq=max(4, extra_blocks_per_seq),
                     ctx_shard=ctx_shard)
    raise ValueError(f"unknown workload {name}")
