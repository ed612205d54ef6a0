"""GPU parity tests: the CUDA path, called through the C ABI (via the operator
wrappers of knlp_b200.ops, which only marshal pointers), against the CPU oracle
and the golden outputs of the reference kernels.

Bars: packed bytes / int8 codes / fp16 scales / fp16 zeros bit-exact; attention
output (read from an fp32 output buffer) within 2e-3 absolute + 1e-3 relative of
the fp32 dequantize-then-attend oracle.
"""

import numpy as np
import pytest
import torch

from conftest import alloc_cache_np, load_golden
from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-3  # the stated tolerance of the decode path (fp32 accumulate)
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
WRITE_CASES = ["write_f32_d64", "write_bf16_d128", "write_f16_d128"]
DECODE_CASES = ["decode_mha_f32_d64", "decode_gqa4_bf16_d128", "decode_gqa8_f16_d128"]


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def zeros_equal(a, b):
    # the sign of a zero minimum is not defined by the reference (see test_oracle_golden)
    return bool(np.all((a == b) | (((a | b) & 0x7FFF) == 0)))


def dev_cache(nb, P, h, d, dev, int8_k=False):
    ng = d // 32
    kc = torch.zeros(nb, P, h, d if int8_k else d // 2, device=dev,
                     dtype=torch.int8 if int8_k else torch.uint8)
    vc = torch.zeros(nb, P, h, d // 2, device=dev, dtype=torch.uint8)
    mk = lambda: torch.zeros(nb, P, h, ng, device=dev, dtype=torch.float16)
    return kc, vc, mk(), mk(), mk(), mk()


def assert_close(out, ref, what=""):
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(out - ref)
    bound = ATOL + RTOL * np.abs(ref)
    assert np.all(err <= bound), (
        f"{what}: max abs err {err.max():.3e}, worst excess {np.max(err - bound):.3e}, "
        f"ref absmax {np.abs(ref).max():.3e}")


# ---------------------------------------------------------------- write path
@pytest.mark.parametrize("case", WRITE_CASES)
def test_quant_append_matches_reference_bits(case, cuda_device):
    from knlp_b200 import ops
    G = load_golden(case)
    dt = TDT[str(G["src_dtype"])]
    k = torch.from_numpy(G["key"]).to(dt).to(cuda_device)
    v = torch.from_numpy(G["value"]).to(dt).to(cuda_device)
    slots = torch.from_numpy(G["slot_mapping"]).to(cuda_device)
    n, h, d = k.shape
    nb, P = int(G["num_blocks"]), int(G["block_size"])

    kc, vc, ks, vs, kz, vz = dev_cache(nb, P, h, d, cuda_device)
    ops.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
    assert np.array_equal(kc.cpu().numpy(), G["asym_kc"])
    assert np.array_equal(vc.cpu().numpy(), G["asym_vc"])
    assert np.array_equal(bits(ks), G["asym_ks"]) and np.array_equal(bits(vs), G["asym_vs"])
    assert zeros_equal(bits(kz), G["asym_kz"]) and zeros_equal(bits(vz), G["asym_vz"])

    kc, vc, ks, vs, _, _ = dev_cache(nb, P, h, d, cuda_device)
    ops.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, asymmetric=False,
                               clip_ratio=float(G["clip_ratio"]))
    assert np.array_equal(kc.cpu().numpy(), G["sym_kc"])
    assert np.array_equal(vc.cpu().numpy(), G["sym_vc"])
    assert np.array_equal(bits(ks), G["sym_ks"]) and np.array_equal(bits(vs), G["sym_vs"])

    _, vc, _, vs, _, vz = dev_cache(nb, P, h, d, cuda_device)
    ops.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
    assert np.array_equal(vc.cpu().numpy(), G["vonly_vc"])
    assert np.array_equal(bits(vs), G["vonly_vs"]) and zeros_equal(bits(vz), G["vonly_vz"])

    kc8, _, ks, _, _, _ = dev_cache(nb, P, h, d, cuda_device, int8_k=True)
    ops.reshape_and_cache_k_int8(k, kc8, ks, slots)
    assert np.array_equal(kc8.cpu().numpy(), G["int8_kc"])
    assert np.array_equal(bits(ks), G["int8_ks"])


@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("strided", [False, True])
def test_quant_append_random_bit_exact_vs_oracle(dt, strided, cuda_device):
    """2 000 tokens x 8 heads x 128 with outlier channels, shuffled slots, padding
    tokens; also through a non-contiguous source view (scalar-load path) and a
    head-major cache view (byte-store path)."""
    from knlp_b200 import ops
    g = torch.Generator().manual_seed(11)
    n, h, d, P = 2000, 8, 128, 16
    nb = (n + P - 1) // P + 2
    k = torch.randn(n, h, d, generator=g)
    v = torch.randn(n, h, d, generator=g) * 0.5 + 0.2
    k[:, :, 7] *= 10
    v[:, :, 100] *= 10
    tdt = TDT[dt]
    k, v = k.to(tdt), v.to(tdt)
    slots = torch.randperm(nb * P, generator=g)[:n].to(torch.int64)
    slots[::97] = -1
    if strided:
        big_k = torch.zeros(n, h, d + 3, dtype=tdt)
        big_k[:, :, 1:d + 1] = k
        kd = big_k.to(cuda_device)[:, :, 1:d + 1]
        vd = v.to(cuda_device)
        mk_u8 = lambda w, t: torch.zeros(nb, h, P, w, device=cuda_device, dtype=t).permute(0, 2, 1, 3)
        mk_f = lambda: torch.zeros(nb, h, P, d // 32, device=cuda_device,
                                   dtype=torch.float16).permute(0, 2, 1, 3)
        kc, vc = mk_u8(d // 2, torch.uint8), mk_u8(d // 2, torch.uint8)
        ks, vs, kz, vz = mk_f(), mk_f(), mk_f(), mk_f()
        kc8 = mk_u8(d, torch.int8)
        ks8 = mk_f()
    else:
        kd, vd = k.to(cuda_device), v.to(cuda_device)
        kc, vc, ks, vs, kz, vz = dev_cache(nb, P, h, d, cuda_device)
        kc8, _, ks8, _, _, _ = dev_cache(nb, P, h, d, cuda_device, int8_k=True)
    sd = slots.to(cuda_device)
    kf, vf = k.float().numpy(), v.float().numpy()

    ops.reshape_and_cache_int4(kd, vd, kc, vc, ks, vs, sd, kz, vz, asymmetric=True)
    okc, ovc, oks, ovs, okz, ovz = alloc_cache_np(nb, P, h, d)
    O.reshape_and_cache_int4(kf, vf, okc, ovc, oks, ovs, slots.numpy(), okz, ovz, asymmetric=True)
    assert np.array_equal(kc.cpu().numpy(), okc) and np.array_equal(vc.cpu().numpy(), ovc)
    assert np.array_equal(bits(ks.contiguous()), oks.view(np.uint16))
    assert np.array_equal(bits(vs.contiguous()), ovs.view(np.uint16))
    assert zeros_equal(bits(kz.contiguous()), okz.view(np.uint16))
    assert zeros_equal(bits(vz.contiguous()), ovz.view(np.uint16))

    kc.zero_(); vc.zero_(); ks.zero_(); vs.zero_()
    ops.reshape_and_cache_int4(kd, vd, kc, vc, ks, vs, sd, asymmetric=False)
    okc, ovc, oks, ovs, _, _ = alloc_cache_np(nb, P, h, d)
    O.reshape_and_cache_int4(kf, vf, okc, ovc, oks, ovs, slots.numpy(), asymmetric=False)
    assert np.array_equal(kc.cpu().numpy(), okc) and np.array_equal(vc.cpu().numpy(), ovc)
    assert np.array_equal(bits(ks.contiguous()), oks.view(np.uint16))
    assert np.array_equal(bits(vs.contiguous()), ovs.view(np.uint16))

    ops.reshape_and_cache_k_int8(kd, kc8, ks8, sd)
    okc8, _, oks8, _, _, _ = alloc_cache_np(nb, P, h, d, int8_k=True)
    O.reshape_and_cache_k_int8(kf, okc8, oks8, slots.numpy())
    assert np.array_equal(kc8.cpu().numpy(), okc8)
    assert np.array_equal(bits(ks8.contiguous()), oks8.view(np.uint16))


def test_quant_append_empty_and_all_padding(cuda_device):
    from knlp_b200 import ops
    kc, vc, ks, vs, kz, vz = dev_cache(2, 16, 2, 64, cuda_device)
    k = torch.zeros(0, 2, 64, device=cuda_device, dtype=torch.bfloat16)
    ops.reshape_and_cache_int4(k, k, kc, vc, ks, vs, torch.zeros(0, dtype=torch.int64, device=cuda_device),
                               kz, vz, asymmetric=True)
    k = torch.randn(5, 2, 64, device=cuda_device, dtype=torch.bfloat16)
    ops.reshape_and_cache_int4(k, k, kc, vc, ks, vs,
                               torch.full((5,), -1, dtype=torch.int64, device=cuda_device),
                               kz, vz, asymmetric=True)
    torch.cuda.synchronize()
    assert int(kc.sum()) == 0 and float(ks.abs().sum()) == 0.0


# ---------------------------------------------------------------- decode
def _golden_decode_setup(G, mode, dev):
    from knlp_b200 import ops
    dt = TDT[str(G["q_dtype"])]
    hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    k = torch.from_numpy(G["key"]).to(dt).to(dev)
    v = torch.from_numpy(G["value"]).to(dt).to(dev)
    q = torch.from_numpy(G["query"]).to(dt).to(dev)
    slots = torch.from_numpy(G["slot_mapping"]).to(dev)
    bt = torch.from_numpy(G["block_table"]).to(dev)
    sl = torch.from_numpy(G["seq_lens"]).to(dev)
    if mode == "k8v4":
        kc, vc, ks, vs, _, vz = dev_cache(nb, P, hkv, d, dev, int8_k=True)
        ops.reshape_and_cache_k_int8(k, kc, ks, slots)
        ops.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)

        def run(**kw):
            return ops.kint8_vint4_decode(q, kc, vc, ks, vs, bt, sl, hkv, d, v_zeros=vz,
                                          asymmetric=True, **kw)

        def oracle():
            return O.kint8_vint4_decode(G["query"], kc.cpu().numpy(), vc.cpu().numpy(),
                                        ks.cpu().numpy(), vs.cpu().numpy(), G["block_table"],
                                        G["seq_lens"], hkv, d, v_zeros=vz.cpu().numpy(),
                                        asymmetric=True)
    else:
        asym = mode == "asym"
        kc, vc, ks, vs, kz, vz = dev_cache(nb, P, hkv, d, dev)
        ops.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=asym)

        def run(**kw):
            return ops.fused_int4_decode(q, kc, vc, ks, vs, bt, sl, hkv, d,
                                         k_zeros=kz if asym else None,
                                         v_zeros=vz if asym else None, asymmetric=asym, **kw)

        def oracle():
            return O.fused_int4_decode(G["query"], kc.cpu().numpy(), vc.cpu().numpy(),
                                       ks.cpu().numpy(), vs.cpu().numpy(), G["block_table"],
                                       G["seq_lens"], hkv, d,
                                       k_zeros=kz.cpu().numpy() if asym else None,
                                       v_zeros=vz.cpu().numpy() if asym else None, asymmetric=asym)
    return run, oracle


@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("mode", ["asym", "sym", "k8v4"])
@pytest.mark.parametrize("generic", [False, "tma", True])
def test_decode_golden(case, mode, generic, cuda_device):
    G = load_golden(case)
    run, oracle = _golden_decode_setup(G, mode, cuda_device)
    ref = oracle()
    if generic is False:  # the default path: balanced one-launch kernel
        outb = run(out_dtype=torch.float32, max_seq_len=int(G["seq_lens"].max()))
        assert_close(outb.cpu().numpy(), ref, f"{case}/{mode}/balanced")
    for n_splits in (1, 3):
        out = run(out_dtype=torch.float32, n_splits=n_splits, force_generic=generic,
                  max_seq_len=int(G["seq_lens"].max()))
        assert_close(out.cpu().numpy(), ref, f"{case}/{mode}/splits={n_splits}")
    # against the reference kernel's own output, at ITS output resolution
    gold = G[f"{mode}_out"]
    rtol = {"f32": 6e-4, "f16": 6e-4, "bf16": 8e-3}[str(G["q_dtype"])]
    np.testing.assert_allclose(out.cpu().numpy(), gold, atol=ATOL, rtol=rtol + RTOL)
    # query-dtype output (the reference's return type)
    out_q = run(force_generic=generic)
    assert out_q.dtype == TDT[str(G["q_dtype"])]
    ulp = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[str(G["q_dtype"])]
    np.testing.assert_allclose(out_q.float().cpu().numpy(), ref, atol=ATOL, rtol=RTOL + ulp)


def _workload_oracle(w, seqs=None):
    args = dict(dtype=np.float32, seqs=seqs)
    q = w.query.float().cpu().numpy()
    bt, sl = w.block_table.cpu().numpy(), w.seq_lens.cpu().numpy()
    if w.k_mode == "int8":
        return O.kint8_vint4_decode(q, w.key_cache.cpu().numpy(), w.value_cache.cpu().numpy(),
                                    w.k_scales.cpu().numpy(), w.v_scales.cpu().numpy(), bt, sl,
                                    w.n_kv_heads, w.head_dim,
                                    v_zeros=None if w.v_zeros is None else w.v_zeros.cpu().numpy(),
                                    asymmetric=w.v_mode == "int4_asym", **args)
    asym = w.k_mode == "int4_asym"
    return O.fused_int4_decode(q, w.key_cache.cpu().numpy(), w.value_cache.cpu().numpy(),
                               w.k_scales.cpu().numpy(), w.v_scales.cpu().numpy(), bt, sl,
                               w.n_kv_heads, w.head_dim,
                               k_zeros=w.k_zeros.cpu().numpy() if asym else None,
                               v_zeros=w.v_zeros.cpu().numpy() if asym else None,
                               asymmetric=asym, **args)


def test_config1_gpt2_mha_exact_shape(cuda_device):
    """12 heads MHA, d 64, batch 1, ctx 1024, fp32 query, asymmetric INT4."""
    from knlp_b200 import workloads
    w = workloads.config("gpt2_mha_1k", cuda_device)
    ref = _workload_oracle(w)
    for generic in (False, "tma", True):
        out = w.decode(out_dtype=torch.float32, force_generic=generic)
        assert_close(out.cpu().numpy(), ref, f"gpt2 generic={generic}")


@pytest.mark.parametrize("name,scale", [("llama8b_b32_8k", 0.25), ("llama70b_ragged", 0.06),
                                        ("mixed_k8v4", 0.5), ("llama8b_b1_384k", 0.02)])
def test_configs_scaled_full_compare(name, scale, cuda_device):
    """Every benchmark configuration at reduced context, every sequence compared."""
    from knlp_b200 import workloads
    w = workloads.config(name, cuda_device, scale=scale)
    ref = _workload_oracle(w)
    out = w.decode(out_dtype=torch.float32)
    assert_close(out.cpu().numpy(), ref, name)
    out1 = w.decode(out_dtype=torch.float32, n_splits=1)
    assert_close(out1.cpu().numpy(), ref, name + "/1 split")
    outg = w.decode(out_dtype=torch.float32, force_generic=True)
    assert_close(outg.cpu().numpy(), ref, name + "/generic")
    outc = w.decode(out_dtype=torch.float32, force_generic="tma")
    assert_close(outc.cpu().numpy(), ref, name + "/TMA staging")
    # determinism of the fixed-split path: same launch twice gives identical bits
    assert torch.equal(out1, w.decode(out_dtype=torch.float32, n_splits=1))
    # the default is the balanced one-launch kernel; the split-context kernel followed by
    # the combine kernel (two launches, planner's split count) must agree with it
    out2 = w.decode(out_dtype=torch.float32, two_launches=True)
    assert_close(out2.cpu().numpy(), ref, name + "/two launches")
    assert torch.equal(out2, w.decode(out_dtype=torch.float32, two_launches=True))
    # (the balanced kernel hands chunks out dynamically, so the summation order, and with
    # it the last bits, may differ from run to run; its ticket counters must be back at zero)
    for _ in range(3):
        assert_close(w.decode(out_dtype=torch.float32).cpu().numpy(), ref, name + "/rerun")


@pytest.mark.parametrize("length", [0, 1, 15, 16, 17, 31, 63, 64, 65, 127, 128, 129, 1000])
def test_decode_edge_lengths(length, cuda_device):
    from knlp_b200 import workloads
    lens = [length, 40, max(length - 1, 0)]
    w = workloads.build("edge", n_seqs=3, n_q_heads=8, n_kv_heads=2, head_dim=128, seq_lens=lens,
                        seed=77 + length, device=cuda_device, shuffle_pages=True,
                        extra_blocks_per_seq=1)
    ref = _workload_oracle(w)
    for kw in (dict(), dict(n_splits=4), dict(force_generic="tma"), dict(force_generic=True)):
        out = w.decode(out_dtype=torch.float32, **kw).cpu().numpy()
        assert_close(out, ref, f"len={length} {kw}")
        if length == 0:
            assert np.all(out[0] == 0)


@pytest.mark.parametrize("n_kv,n_rep", [(1, 4), (2, 4), (3, 2), (4, 8), (8, 1), (12, 1)])
def test_decode_kv_heads_per_cta(n_kv, n_rep, cuda_device):
    """1, 2 or 4 kv heads per CTA (a stage is then 4, 2 or 1 sixteen-token blocks), long
    enough that most stages go through the loop without end-of-sequence tests, ragged
    so that the last stages do not; shuffled pages."""
    from knlp_b200 import workloads
    w = workloads.build("few_heads", n_seqs=3, n_q_heads=n_kv * n_rep, n_kv_heads=n_kv,
                        head_dim=128, seq_lens=[2500, 1031, 64], seed=500 + n_kv,
                        device=cuda_device, shuffle_pages=True)
    ref = _workload_oracle(w)
    for kw in (dict(), dict(n_splits=1), dict(n_splits=3), dict(force_generic="tma")):
        out = w.decode(out_dtype=torch.float32, **kw).cpu().numpy()
        assert_close(out, ref, f"kv heads {n_kv} x rep {n_rep} {kw}")


def test_head_major_cache_view_goes_generic(cuda_device):
    """A [block, head, token, d/2] cache viewed as [block, token, head, d/2] has a
    16-byte-aligned but permuted layout; both kernels must address it."""
    from knlp_b200 import ops
    g = torch.Generator().manual_seed(5)
    S, Hq, Hkv, d, P, L = 2, 8, 4, 64, 16, 90
    nb = S * ((L + P - 1) // P)
    mk = lambda w, t: torch.zeros(nb, Hkv, P, w, device=cuda_device, dtype=t).permute(0, 2, 1, 3)
    kc, vc = mk(d // 2, torch.uint8), mk(d // 2, torch.uint8)
    ks, vs, kz, vz = (mk(d // 32, torch.float16) for _ in range(4))
    k = torch.randn(S * L, Hkv, d, generator=g).to(torch.float16).to(cuda_device)
    v = torch.randn(S * L, Hkv, d, generator=g).to(torch.float16).to(cuda_device)
    q = torch.randn(S, Hq, d, generator=g).to(torch.float16).to(cuda_device)
    bt = torch.arange(nb, dtype=torch.int32).reshape(S, -1).to(cuda_device)
    pos = torch.arange(L)
    slots = torch.cat([(bt[s].cpu()[pos // P].long() * P + pos % P) for s in range(S)]).to(cuda_device)
    ops.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
    sl = torch.tensor([L, L - 7], dtype=torch.int32, device=cuda_device)
    ref = O.fused_int4_decode(q.float().cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(),
                              ks.cpu().numpy(), vs.cpu().numpy(), bt.cpu().numpy(), sl.cpu().numpy(),
                              Hkv, d, k_zeros=kz.cpu().numpy(), v_zeros=vz.cpu().numpy(), asymmetric=True)
    for generic in (False, True):
        out = ops.fused_int4_decode(q, kc, vc, ks, vs, bt, sl, Hkv, d, k_zeros=kz, v_zeros=vz,
                                    asymmetric=True, out_dtype=torch.float32, force_generic=generic)
        assert_close(out.cpu().numpy(), ref, f"head-major generic={generic}")


def test_combine_vs_oracle(cuda_device):
    from knlp_b200 import ops
    rng = np.random.default_rng(9)
    rows, n, d = 37, 11, 128
    pm = rng.standard_normal((rows, n)).astype(np.float32) * 3
    pl = (rng.random((rows, n)).astype(np.float32) + 0.1) * 50
    po = rng.standard_normal((rows, n, d)).astype(np.float32) * 10
    pl[:, 3] = 0; pm[:, 3] = -np.inf; po[:, 3] = 0     # an empty split
    pl[5] = 0; pm[5] = -np.inf; po[5] = 0              # a row with no tokens at all
    ref = O.combine_partials(pm, pl, po)
    t = lambda a: torch.from_numpy(a).to(cuda_device)
    out = ops.combine_partials(t(pm), t(pl), t(po))
    np.testing.assert_allclose(out.cpu().numpy(), ref, atol=1e-5, rtol=1e-5)
    assert np.all(out.cpu().numpy()[5] == 0)
    # parts-first layout (what an all-gather produces) and partial emission
    out2 = ops.combine_partials(t(np.ascontiguousarray(pm.T)), t(np.ascontiguousarray(pl.T)),
                                t(np.ascontiguousarray(po.transpose(1, 0, 2))), parts_dim=0)
    np.testing.assert_allclose(out2.cpu().numpy(), ref, atol=1e-5, rtol=1e-5)
    m, l, o = ops.combine_partials(t(pm[:, :6].copy()), t(pl[:, :6].copy()), t(po[:, :6].copy()),
                                   emit_partial=True)
    m2, l2, o2 = ops.combine_partials(t(pm[:, 6:].copy()), t(pl[:, 6:].copy()), t(po[:, 6:].copy()),
                                      emit_partial=True)
    out3 = ops.combine_partials(torch.stack([m, m2]), torch.stack([l, l2]), torch.stack([o, o2]),
                                parts_dim=0)
    np.testing.assert_allclose(out3.cpu().numpy(), ref, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("world", [2, 8])
def test_context_shard_on_one_gpu(world, cuda_device):
    """The context-shard path with the ranks emulated one after the other on one
    GPU: every 'rank' decodes its contiguous, page-aligned token segment (its own
    view of the block table and local lengths), packs ONE partial per (sequence,
    q head); the stacked partials (what the all-gather would deliver) are merged."""
    from knlp_b200 import ops, shard, workloads
    w = workloads.config("llama8b_b1_384k", cuda_device, scale=0.03)  # 11 796 tokens
    w2 = workloads.build("ragged", n_seqs=3, n_q_heads=32, n_kv_heads=8, head_dim=128,
                         seq_lens=[5000, 17, 900], seed=9, device=cuda_device, shuffle_pages=True)
    for wl in (w, w2):
        ref = _workload_oracle(wl)
        kp = ops._plane(wl.key_cache, wl.k_scales, wl.k_zeros, ops._lib.KV_INT4_ASYM)
        vp = ops._plane(wl.value_cache, wl.v_scales, wl.v_zeros, ops._lib.KV_INT4_ASYM)
        packed = []
        for r in range(world):
            segs = [shard.context_shard(L, world, r, 16) for L in wl.seq_lens_host]
            first_page = [a // 16 for a, _ in segs]
            max_pages = max((b - a + 15) // 16 for a, b in segs) or 1
            bt = torch.zeros(wl.n_seqs, max_pages, dtype=torch.int32)
            full = wl.block_table.cpu()
            for s, (a, b) in enumerate(segs):
                n = (b - a + 15) // 16
                bt[s, :n] = full[s, first_page[s]:first_page[s] + n]
            lens = torch.tensor([b - a for a, b in segs], dtype=torch.int32, device=cuda_device)
            pm, pl, po = ops.decode_partials(wl.query, kp, vp, wl.key_cache.shape[0],
                                             bt.to(cuda_device), lens, wl.n_kv_heads, wl.head_dim, 16,
                                             max_seq_len=int(max(b - a for a, b in segs)))
            packed.append(ops.combine_to_packed(pm, pl, po))
            # the same partial straight from the balanced kernel (what shard.py sends)
            direct = ops.decode_attention(wl.query, kp, vp, wl.key_cache.shape[0],
                                          bt.to(cuda_device), lens, wl.n_kv_heads, wl.head_dim, 16,
                                          max_seq_len=int(max(b - a for a, b in segs)),
                                          emit_partial=True)
            both = ops.combine_packed(torch.stack([packed[-1], direct]))
            one = ops.combine_packed(packed[-1].unsqueeze(0))
            # merging a partial with itself leaves the normalised result unchanged
            np.testing.assert_allclose(both.cpu().numpy(), one.cpu().numpy(), atol=2e-5, rtol=1e-4)
        out = ops.combine_packed(torch.stack(packed))
        assert_close(out.cpu().numpy(), ref, f"context shard x{world}")


def test_bounded_wait_gives_up_and_reports(cuda_device):
    """The TMA staging waits on its "stage landed" barriers for at most 2 ms.  With the test
    flag the first stage of every CTA announces 16 bytes that never come (every copy that is
    issued still lands, nothing faults): the wait runs out, the kernel reports its splits as
    empty, sets the status word and RETURNS; the context stays usable."""
    from knlp_b200 import ops, workloads
    w = workloads.build("stall", n_seqs=2, n_q_heads=32, n_kv_heads=8, head_dim=128,
                        seq_lens=[300, 100], seed=3, device=cuda_device)
    ref = _workload_oracle(w)
    assert ops.device_status() == 0
    out = w.decode(out_dtype=torch.float32, force_generic="tma_stall", n_splits=2)
    assert ops.device_status() == 1      # synchronises: the kernel came back
    assert ops.device_status() == 0      # reading it cleared it
    assert torch.isfinite(out).all()     # empty splits, not garbage
    # and the same launch without the flag is right again
    out = w.decode(out_dtype=torch.float32, force_generic="tma", n_splits=2)
    assert_close(out.cpu().numpy(), ref, "after a give-up")
    assert ops.device_status() == 0


def test_zz_device_status_is_clean(cuda_device):
    """No kernel of this session gave up on a barrier wait."""
    from knlp_b200 import ops
    assert ops.device_status() == 0


def test_cpu_tensor_is_refused():
    from knlp_b200 import ops
    q = torch.zeros(1, 4, 64)
    c = torch.zeros(1, 16, 4, 32, dtype=torch.uint8)
    s = torch.zeros(1, 16, 4, 2, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        ops.fused_int4_decode(q, c, c, s, s, torch.zeros(1, 1, dtype=torch.int32),
                              torch.ones(1, dtype=torch.int32), 4, 64)
