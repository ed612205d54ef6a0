"""Routed (block-sparse) decode over the packed cache against the reference's own torch
implementation (routing/fused_routed_attention.py:496-548) run over the dequantized cache:
fixtures tests/golden/routed_*.npz from make_golden.py --only-routed.  The CPU test pins the
oracle; the GPU tests run knlp_b200.routing.fused_routed_decode through the C ABI."""

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import kv_oracle as O

CASES = ["routed_gqa4_d128_p16", "routed_gqa2_d64_p32", "routed_mha_d128_p64"]
ATOL, RTOL = 2e-3, 1e-3
DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def _f16(bits):
    return np.ascontiguousarray(bits).view(np.float16)


def _close(out, ref, what):
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    err = np.abs(out - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{what}: max abs err {err.max():.3e}"


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", ["asym", "sym"])
def test_oracle_matches_reference_routed_decode(case, mode):
    G = load_golden(case)
    asym = mode == "asym"
    kd = O.dequant_int4(G[f"{mode}_k_cache"], _f16(G[f"{mode}_k_scales"]),
                        _f16(G["asym_k_zeros"]) if asym else None)
    vd = O.dequant_int4(G[f"{mode}_v_cache"], _f16(G[f"{mode}_v_scales"]),
                        _f16(G["asym_v_zeros"]) if asym else None)
    out = O.routed_decode(G["query"], kd, vd, G["block_tables"], G["block_counts"])
    np.testing.assert_allclose(out, G[f"{mode}_out"], rtol=2e-5, atol=2e-6)
    # a head with nothing selected yields zeros
    empty = np.argwhere(G["block_counts"] == 0)
    n_rep = G["query"].shape[1] // G["block_counts"].shape[1]
    for b, h in empty:
        assert not out[b, h * n_rep:(h + 1) * n_rep].any()


def _planes(G, mode, dev):
    from knlp_b200 import _lib, ops
    asym = mode == "asym"
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    h = lambda bits: t(np.ascontiguousarray(bits).view(np.int16)).view(torch.float16)
    kc, vc = t(G[f"{mode}_k_cache"]), t(G[f"{mode}_v_cache"])
    ks, vs = h(G[f"{mode}_k_scales"]), h(G[f"{mode}_v_scales"])
    kz = h(G["asym_k_zeros"]) if asym else None
    vz = h(G["asym_v_zeros"]) if asym else None
    m = _lib.KV_INT4_ASYM if asym else _lib.KV_INT4_SYM
    keep = (kc, vc, ks, vs, kz, vz)
    return ops._plane(kc, ks, kz, m), ops._plane(vc, vs, vz, m), keep


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", ["asym", "sym"])
def test_routed_decode_matches_reference(case, mode, cuda_device):
    from knlp_b200 import routing
    G = load_golden(case)
    kp, vp, keep = _planes(G, mode, cuda_device)
    q = torch.from_numpy(G["query"]).to(DT[str(G["q_dtype"])]).to(cuda_device)
    tables = torch.from_numpy(G["block_tables"]).to(cuda_device)
    counts = torch.from_numpy(G["block_counts"]).to(cuda_device)
    hkv, P = int(G["num_kv_heads"]), int(G["block_size"])
    out = routing.fused_routed_decode(q, kp, vp, int(G["num_blocks"]), P, hkv, tables, counts,
                                      out_dtype=torch.float32)
    assert out.shape == q.shape
    _close(out.cpu().numpy(), G[f"{mode}_out"], f"{case}/{mode}")
    # int64 tables as torch.topk yields them, and the default output dtype
    out2 = routing.fused_routed_decode(q, kp, vp, int(G["num_blocks"]), P, hkv, tables.long(),
                                       counts)
    assert out2.dtype == q.dtype
    # rounded to the query dtype: half an ulp of bf16 (2^-9) or fp16 (2^-12) on top
    np.testing.assert_allclose(out2.float().cpu().numpy(), G[f"{mode}_out"], rtol=5e-3, atol=3e-3)
    # the workspace counters are left zero for the next call
    out3 = routing.fused_routed_decode(q, kp, vp, int(G["num_blocks"]), P, hkv, tables, counts,
                                       out_dtype=torch.float32)
    _close(out3.cpu().numpy(), G[f"{mode}_out"], f"{case}/{mode} (second call)")


@pytest.mark.gpu
def test_routed_equals_dense_when_every_block_is_selected(cuda_device):
    """Selecting all blocks of a sequence, in order, for every head is ordinary decode."""
    from knlp_b200 import ops, routing, workloads
    w = workloads.build("routed_dense", n_seqs=5, n_q_heads=16, n_kv_heads=4, head_dim=128,
                        seq_lens=[16 * 40, 16 * 3, 16 * 17, 16 * 64, 16], device=cuda_device,
                        seed=11, shuffle_pages=True)
    kp, vp = w.planes()
    P = 16
    dense = ops.decode_attention(w.query, kp, vp, w.key_cache.shape[0], w.block_table, w.seq_lens,
                                 w.n_kv_heads, 128, P, out_dtype=torch.float32)
    tables = w.block_table[:, None, :].expand(-1, w.n_kv_heads, -1).contiguous()
    counts = (w.seq_lens // P)[:, None].expand(-1, w.n_kv_heads).contiguous().to(torch.int32)
    routed = routing.fused_routed_decode(w.query, kp, vp, w.key_cache.shape[0], P, w.n_kv_heads,
                                         tables, counts, out_dtype=torch.float32)
    torch.testing.assert_close(routed, dense, rtol=1e-4, atol=1e-5)
    # the partial form merges back to the same output
    part = routing.fused_routed_decode(w.query, kp, vp, w.key_cache.shape[0], P, w.n_kv_heads,
                                       tables, counts, emit_partial=True)
    o = part[..., :128] / part[..., 129:130]
    torch.testing.assert_close(o, dense, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_select_top_k_blocks(cuda_device):
    from knlp_b200 import routing
    prior = torch.rand(3, 4, 20, device=cuda_device)
    tables, counts = routing.select_top_k_blocks(prior, 6)
    assert tables.shape == (3, 4, 6) and counts.shape == (3, 4) and int(counts.min()) == 6
    assert torch.equal(tables, torch.topk(prior, 6, dim=-1).indices)
    tables, counts = routing.select_top_k_blocks(prior, 50)
    assert tables.shape == (3, 4, 20) and int(counts.max()) == 20


@pytest.mark.gpu
@pytest.mark.parametrize("k_mode,v_mode", [("int8", "int4_asym"), ("int8", "int8"),
                                           ("int4_sym", "int4_sym"), ("fp16", "int4_asym"),
                                           ("bf16", "int8")])
def test_routed_other_modes_equal_dense(k_mode, v_mode, cuda_device):
    """Every K / V mode pair of the dense kernel also runs with per-kv-head block tables:
    selecting all blocks of a sequence in order reproduces the dense decode."""
    from knlp_b200 import _lib, ops, routing, workloads
    fp = k_mode in ("fp16", "bf16")
    w = workloads.build("routed_modes", n_seqs=4, n_q_heads=8, n_kv_heads=2, head_dim=128,
                        seq_lens=[16 * 21, 16 * 5, 16 * 64, 16], device=cuda_device, seed=23,
                        shuffle_pages=True, v_mode=v_mode,
                        k_mode=k_mode if not fp else ("int8" if v_mode == "int8" else "int4_asym"))
    kp, vp = w.planes()
    nb, P = w.key_cache.shape[0], 16
    if fp:  # an unquantized K cache of its own in the same pages
        g = torch.Generator(device=cuda_device).manual_seed(3)
        kfp = torch.randn(nb, P, 2, 128, device=cuda_device, generator=g).to(
            torch.float16 if k_mode == "fp16" else torch.bfloat16)
        kp = ops._fp_plane(kfp)
    dense = ops.decode_attention(w.query, kp, vp, nb, w.block_table, w.seq_lens, 2, 128, P,
                                 out_dtype=torch.float32)
    tables = w.block_table[:, None, :].expand(-1, 2, -1).contiguous()
    counts = (w.seq_lens // P)[:, None].expand(-1, 2).contiguous().to(torch.int32)
    routed = routing.fused_routed_decode(w.query, kp, vp, nb, P, 2, tables, counts,
                                         out_dtype=torch.float32)
    torch.testing.assert_close(routed, dense, rtol=2e-4, atol=2e-5)
    # a different selection per head: only the first half of the blocks for head 1
    counts2 = counts.clone()
    counts2[:, 1] = torch.clamp(counts[:, 1] // 2, min=1)
    routed2 = routing.fused_routed_decode(w.query, kp, vp, nb, P, 2, tables, counts2,
                                          out_dtype=torch.float32)
    half = ops.decode_attention(w.query, kp, vp, nb, w.block_table,
                                (counts2[:, 1] * P).contiguous(), 2, 128, P,
                                out_dtype=torch.float32)
    torch.testing.assert_close(routed2[:, :4], dense[:, :4], rtol=2e-4, atol=2e-5)
    torch.testing.assert_close(routed2[:, 4:], half[:, 4:], rtol=2e-4, atol=2e-5)
    # counts beyond the table's width are cut at the width, as the reference's loop does
    short = tables[:, :, :3].contiguous()
    over = routing.fused_routed_decode(w.query, kp, vp, nb, P, 2, short,
                                       torch.full_like(counts, 50), out_dtype=torch.float32)
    exact = routing.fused_routed_decode(w.query, kp, vp, nb, P, 2, short,
                                        torch.full_like(counts, 3), out_dtype=torch.float32)
    torch.testing.assert_close(over, exact, rtol=2e-4, atol=2e-5)
