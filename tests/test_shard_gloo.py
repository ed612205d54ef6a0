"""World-size-2 (and 4) gloo tests of the multi-GPU plumbing on CPU: ownership
arithmetic, the single all-gather of packed partials, the head gather.  The
per-rank attention is computed by the CPU oracle here (the CUDA kernels are
covered by the GPU tests); what is under test is that sharding + gather + merge
reproduces the unsharded result."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from knlp_b200 import shard
from oracle import kv_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _data(seed=0, S=3, Hq=8, Hkv=4, d=64, lens=(100, 37, 257)):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((S, Hq, d)).astype(np.float32)
    ks = [rng.standard_normal((L, Hkv, d)).astype(np.float32) for L in lens]
    vs = [rng.standard_normal((L, Hkv, d)).astype(np.float32) for L in lens]
    return q, ks, vs, list(lens)


def _reference(q, ks, vs):
    return np.stack([O.attend_one(q[s], ks[s], vs[s])[0] for s in range(q.shape[0])])


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, ks, vs, lens = _data()
        S, Hq, d = q.shape
        Hkv = ks[0].shape[1]
        if mode == "context":
            packed = np.zeros((S, Hq, d + 2), np.float32)
            for s in range(S):
                a, b = shard.context_shard(lens[s], world, rank, page=16)
                o, m, l = O.attend_one(q[s], ks[s][a:b], vs[s][a:b])
                packed[s, :, :d] = o * l[:, None]  # un-normalised
                packed[s, :, d] = m
                packed[s, :, d + 1] = l
            g = shard.all_gather_packed(torch.from_numpy(packed)).numpy()  # [G, S, Hq, d+2]
            assert g.shape == (world, S, Hq, d + 2)
            out = O.combine_partials(np.moveaxis(g[..., d], 0, -1), np.moveaxis(g[..., d + 1], 0, -1),
                                     np.moveaxis(g[..., :d], 0, -2))
        else:
            kv = shard.head_shard(Hkv, world, rank)
            qs = shard.q_heads_of(kv, Hq // Hkv)
            loc = np.stack([O.attend_one(q[s][qs], ks[s][:, kv], vs[s][:, kv])[0] for s in range(S)])
            out = shard.gather_heads(torch.from_numpy(loc)).numpy()
        ref = _reference(q, ks, vs)
        ret[rank] = float(np.abs(out - ref).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("mode", ["context", "heads"])
def test_sharded_equals_unsharded(world, mode):
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world
    assert max(ret.values()) < 5e-6


def test_ownership_arithmetic():
    assert shard.head_shard(8, 4, 1) == slice(2, 4)
    assert shard.q_heads_of(slice(2, 4), 4) == slice(8, 16)
    with pytest.raises(ValueError):
        shard.head_shard(8, 3, 0)
    # context segments: page aligned, disjoint, covering
    for L in (0, 1, 15, 16, 17, 1000, 393216):
        for G in (1, 2, 3, 8):
            seg = [shard.context_shard(L, G, r, 16) for r in range(G)]
            assert seg[0][0] == 0 and seg[-1][1] == L
            for (a, b), (c, e) in zip(seg, seg[1:]):
                assert b == c and a <= b
            assert all(a % 16 == 0 for a, _ in seg if a < L)
    assert shard.context_shard_lens([100, 16], 2, 1, 16) == [36, 0]


def test_single_process_passthrough():
    x = torch.zeros(2, 4, 66)
    assert shard.all_gather_packed(x).shape == (1, 2, 4, 66)
    y = torch.zeros(2, 4, 64)
    assert shard.gather_heads(y).shape == (2, 4, 64)
