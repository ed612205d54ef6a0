"""Generate the golden fixtures in this directory by running the REFERENCE's own
kernels (mcgrof/knlp, fused-quant/fused_int4.v0.1.0.py) on CPU tensors under the
Triton interpreter.

Run once, where a checkout of the reference is available:

    TRITON_INTERPRET=1 KNLP_REFERENCE=/path/to/knlp python tests/golden/make_golden.py

The fixtures (.npz, a few hundred KB in total) are committed; tests read only
them, never the reference checkout.  Inputs are stored as fp32 arrays holding
values exactly representable in the named source dtype.
"""

import importlib.util
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("KNLP_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set KNLP_REFERENCE to a checkout of mcgrof/knlp")

DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def load_reference():
    path = os.path.join(REF, "fused-quant", "fused_int4.v0.1.0.py")
    spec = importlib.util.spec_from_file_location("knlp_ref_fused_int4", path)
    m = importlib.util.module_from_spec(spec)
    sys.modules["knlp_ref_fused_int4"] = m
    spec.loader.exec_module(m)
    return m


def make_kv(g, n, h, d, dtype, outlier=True, special_rows=True):
    k = torch.randn(n, h, d, generator=g)
    v = torch.randn(n, h, d, generator=g) + 0.3
    if outlier:
        k[:, :, 5] *= 10.0
        v[:, :, d - 3] *= 10.0
    if special_rows and n >= 6:
        # all-zero row, constant row, exact .5 ties (range 15 -> scale 1),
        # tiny range, symmetric ties (amax 7 -> scale 1)
        k[0] = 0.0
        v[0] = 0.0
        k[1] = 1.25
        v[1] = -3.0
        ramp = torch.arange(32, dtype=torch.float32) * 0.5
        ramp[-1] = 15.0
        k[2, :, :32] = ramp
        v[2, :, :32] = ramp - 4.0
        k[3] = k[3] * 1e-6
        v[3] = v[3] * 1e-9
        sym = (torch.arange(32, dtype=torch.float32) - 16.0) * 0.5
        sym[0] = -7.0
        sym[-1] = 7.0
        k[4, :, :32] = sym
        v[4, :, :32] = sym
        k[5, :, :32] = 0.0
        k[5, :, 7] = 400.0  # one extreme outlier in an otherwise zero group
        v[5, :, :32] = torch.linspace(-1, 1, 32)
        v[5, :, 9] = -400.0
    return k.to(dtype), v.to(dtype)


def alloc_cache(nb, P, h, d, int8_k=False):
    ng = d // 32
    kc = torch.zeros(nb, P, h, d if int8_k else d // 2, dtype=torch.int8 if int8_k else torch.uint8)
    vc = torch.zeros(nb, P, h, d // 2, dtype=torch.uint8)
    mk = lambda: torch.zeros(nb, P, h, ng, dtype=torch.float16)
    return kc, vc, mk(), mk(), mk(), mk()


def f16_bits(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def gen_write_cases(m, out):
    P = 16
    for name, dtype, d, h, n in (("f32_d64", "f32", 64, 3, 24), ("bf16_d128", "bf16", 128, 2, 20),
                                 ("f16_d128", "f16", 128, 2, 12)):
        g = torch.Generator().manual_seed(1000 + d + n)
        k, v = make_kv(g, n, h, d, DT[dtype])
        nb = 4
        perm = torch.randperm(nb * P, generator=g)[:n].to(torch.int64)
        slots = perm.clone()
        slots[n // 2] = -1
        rec = dict(key=k.float().numpy(), value=v.float().numpy(), slot_mapping=slots.numpy(),
                   src_dtype=dtype, block_size=P, num_blocks=nb)
        # asymmetric K+V
        kc, vc, ks, vs, kz, vz = alloc_cache(nb, P, h, d)
        m.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
        rec.update(asym_kc=kc.numpy().copy(), asym_vc=vc.numpy().copy(), asym_ks=f16_bits(ks),
                   asym_vs=f16_bits(vs), asym_kz=f16_bits(kz), asym_vz=f16_bits(vz))
        # symmetric K+V with the default outlier clip
        kc, vc, ks, vs, _, _ = alloc_cache(nb, P, h, d)
        m.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, asymmetric=False)
        rec.update(sym_kc=kc.numpy().copy(), sym_vc=vc.numpy().copy(), sym_ks=f16_bits(ks),
                   sym_vs=f16_bits(vs), clip_ratio=float(m.OUTLIER_CLIP_RATIO))
        # V only, asymmetric
        _, vc, _, vs, _, vz = alloc_cache(nb, P, h, d)
        m.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
        rec.update(vonly_vc=vc.numpy().copy(), vonly_vs=f16_bits(vs), vonly_vz=f16_bits(vz))
        # K int8 group-32
        kc8, _, ks, _, _, _ = alloc_cache(nb, P, h, d, int8_k=True)
        m.reshape_and_cache_k_int8(k, kc8, ks, slots)
        rec.update(int8_kc=kc8.numpy().copy(), int8_ks=f16_bits(ks))
        out[f"write_{name}"] = rec
        print("write", name, "done", flush=True)


def gen_decode_cases(m, out):
    P = 16
    cases = (
        # name, q dtype, Hq, Hkv, d, seq lens
        ("mha_f32_d64", "f32", 3, 3, 64, (100, 37)),
        ("gqa4_bf16_d128", "bf16", 8, 2, 128, (37, 16, 130)),
        ("gqa8_f16_d128", "f16", 8, 1, 128, (65, 1)),
    )
    for name, dtype, hq, hkv, d, lens in cases:
        g = torch.Generator().manual_seed(2000 + hq * 7 + d)
        S = len(lens)
        max_blocks = max((L + P - 1) // P for L in lens)
        nb = S * max_blocks + 3
        perm = torch.randperm(nb, generator=g)
        bt = torch.zeros(S, max_blocks, dtype=torch.int32)
        slots, toks = [], 0
        for s, L in enumerate(lens):
            bt[s] = perm[s * max_blocks:(s + 1) * max_blocks].to(torch.int32)
            for n in range(L):
                slots.append(int(bt[s, n // P]) * P + n % P)
            toks += L
        slots = torch.tensor(slots, dtype=torch.int64)
        kvdt = DT[dtype]
        k, v = make_kv(g, toks, hkv, d, kvdt, special_rows=False)
        q = torch.randn(S, hq, d, generator=g).to(kvdt)
        seq_lens = torch.tensor(lens, dtype=torch.int32)
        rec = dict(query=q.float().numpy(), key=k.float().numpy(), value=v.float().numpy(),
                   slot_mapping=slots.numpy(), block_table=bt.numpy(), seq_lens=seq_lens.numpy(),
                   q_dtype=dtype, block_size=P, num_blocks=nb, num_kv_heads=hkv, head_size=d)
        for mode, asym in (("asym", True), ("sym", False)):
            kc, vc, ks, vs, kz, vz = alloc_cache(nb, P, hkv, d)
            m.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz if asym else None,
                                     vz if asym else None, asymmetric=asym)
            o = m.fused_int4_decode(q, kc, vc, ks, vs, bt, seq_lens, hkv, d, block_n=64,
                                    k_zeros=kz if asym else None, v_zeros=vz if asym else None,
                                    asymmetric=asym)
            rec[f"{mode}_out"] = o.float().numpy()
            rec[f"{mode}_out_dtype"] = str(o.dtype)
        kc8, vc, ks, vs, _, vz = alloc_cache(nb, P, hkv, d, int8_k=True)
        m.reshape_and_cache_k_int8(k, kc8, ks, slots)
        m.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
        o = m.kint8_vint4_decode(q, kc8, vc, ks, vs, bt, seq_lens, hkv, d, block_n=64,
                                 v_zeros=vz, asymmetric=True)
        rec["k8v4_out"] = o.float().numpy()
        out[f"decode_{name}"] = rec
        print("decode", name, "done", flush=True)


def gen_plugin_cases(out):
    """Plugin-level simulated quantizers (backends/quant.py:23-86), run as they are on
    CPU tensors of each dtype.  Values are stored as fp32 views (exact)."""
    sys.path.insert(0, REF)
    from backends import quant as Q  # noqa: E402  (the reference module itself)

    rec = {}
    for dt_name, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        for D in (64, 80):  # 80: the int4 block quantizer pads the last block
            g = torch.Generator().manual_seed(4000 + D)
            x = torch.randn(2, 3, 13, D, generator=g)
            x[0, 0, 1] *= 50.0          # a large row
            x[0, 1, 2] *= 1e-3          # a small row
            x[1, 2, 5, :7] = 0.5        # ties after scaling are possible here
            if dt == torch.float32:
                x[1, 0, 0] = 0.0        # all-zero row: the 1e-8 floor (fp32 only: in
                                        # fp16 the floor rounds to 0 and the row is 0/0)
            x = x.to(dt)
            q8, s8 = Q.quantize_int8_symmetric(x)
            d8 = Q.dequantize_int8_symmetric(q8, s8)
            q4, s4 = Q.quantize_int4_block(x, 32)
            d4 = Q.dequantize_int4_block(q4, s4, 32)
            key = f"{dt_name}_d{D}"
            rec[key + "_x"] = x.float().numpy()
            rec[key + "_q8"] = q8.numpy()
            rec[key + "_s8"] = s8.float().numpy()
            rec[key + "_d8"] = d8.float().numpy()
            rec[key + "_q4"] = q4.numpy()
            rec[key + "_s4"] = s4.float().numpy()
            rec[key + "_d4"] = d4.float().numpy()
            assert s8.dtype == dt and s4.dtype == dt and d8.dtype == torch.float32
    out["plugin_quant"] = rec
    print("plugin quantizers done", flush=True)


def gen_v8_cases(m, out):
    """INT8 V: reshape_and_cache_v_int8 (:1619-1645) and kint8_vint8_decode (:1796-1843) on
    the inputs of the write and decode cases above (read back from their files)."""
    rec = {}
    for name in ("write_f32_d64", "write_bf16_d128", "write_f16_d128"):
        G = np.load(os.path.join(HERE, name + ".npz"))
        dt = DT[str(G["src_dtype"])]
        v = torch.from_numpy(G["value"]).to(dt)
        slots = torch.from_numpy(G["slot_mapping"])
        n, h, d = v.shape
        nb, P = int(G["num_blocks"]), int(G["block_size"])
        vc8 = torch.zeros(nb, P, h, d, dtype=torch.int8)
        vs = torch.zeros(nb, P, h, d // 32, dtype=torch.float16)
        m.reshape_and_cache_v_int8(v, vc8, vs, slots)
        rec[name + "_vc8"] = vc8.numpy().copy()
        rec[name + "_vs8"] = f16_bits(vs)
        print("v8 write", name, "done", flush=True)
    for name in ("decode_mha_f32_d64", "decode_gqa4_bf16_d128", "decode_gqa8_f16_d128"):
        G = np.load(os.path.join(HERE, name + ".npz"))
        dt = DT[str(G["q_dtype"])]
        q = torch.from_numpy(G["query"]).to(dt)
        k = torch.from_numpy(G["key"]).to(dt)
        v = torch.from_numpy(G["value"]).to(dt)
        slots = torch.from_numpy(G["slot_mapping"])
        bt = torch.from_numpy(G["block_table"])
        seq_lens = torch.from_numpy(G["seq_lens"])
        nb, P = int(G["num_blocks"]), int(G["block_size"])
        hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
        kc8 = torch.zeros(nb, P, hkv, d, dtype=torch.int8)
        vc8 = torch.zeros(nb, P, hkv, d, dtype=torch.int8)
        ks = torch.zeros(nb, P, hkv, d // 32, dtype=torch.float16)
        vs = torch.zeros(nb, P, hkv, d // 32, dtype=torch.float16)
        m.reshape_and_cache_k_int8(k, kc8, ks, slots)
        m.reshape_and_cache_v_int8(v, vc8, vs, slots)
        o = m.kint8_vint8_decode(q, kc8, vc8, ks, vs, bt, seq_lens, hkv, d, block_n=64)
        rec[name + "_k8v8_out"] = o.float().numpy()
        print("v8 decode", name, "done", flush=True)
    out["v8_modes"] = rec


def gen_kfp16_cases(m, out):
    """Unquantized K: kfp16_vint4_decode (:1159-1224) and kfp16_vint8_decode (:1975-2028) on
    the inputs of the decode cases (read back from their files).  The K cache holds the
    keys in the query dtype (fp16 for the fp32 case); it is stored as an fp32 view."""
    rec = {}
    for name in ("decode_mha_f32_d64", "decode_gqa4_bf16_d128", "decode_gqa8_f16_d128"):
        G = np.load(os.path.join(HERE, name + ".npz"))
        dt = DT[str(G["q_dtype"])]
        kdt = torch.float16 if dt == torch.float32 else dt
        q = torch.from_numpy(G["query"]).to(dt)
        k = torch.from_numpy(G["key"]).to(kdt)
        v = torch.from_numpy(G["value"]).to(dt)
        slots = torch.from_numpy(G["slot_mapping"])
        bt = torch.from_numpy(G["block_table"])
        seq_lens = torch.from_numpy(G["seq_lens"])
        nb, P = int(G["num_blocks"]), int(G["block_size"])
        hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
        kcache = torch.zeros(nb, P, hkv, d, dtype=kdt)
        kcache.view(nb * P, hkv, d)[slots] = k
        _, vc, _, vs, _, vz = alloc_cache(nb, P, hkv, d)
        m.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
        o4 = m.kfp16_vint4_decode(q, kcache, vc, vs, bt, seq_lens, hkv, d, block_n=64,
                                  v_zeros=vz, asymmetric=True)
        vc8 = torch.zeros(nb, P, hkv, d, dtype=torch.int8)
        vs8 = torch.zeros(nb, P, hkv, d // 32, dtype=torch.float16)
        m.reshape_and_cache_v_int8(v, vc8, vs8, slots)
        o8 = m.kfp16_vint8_decode(q, kcache, vc8, vs8, bt, seq_lens, hkv, d, block_n=64)
        rec[name + "_kcache"] = kcache.float().numpy()
        rec[name + "_kdtype"] = "f16" if kdt == torch.float16 else "bf16"
        rec[name + "_kf16v4_out"] = o4.float().numpy()
        rec[name + "_kf16v8_out"] = o8.float().numpy()
        print("kfp16 decode", name, "done", flush=True)
    out["kfp16_modes"] = rec


def gen_contig_cases(out):
    """The contiguous head-major symmetric cache of the reference's kernel benches:
    quantize_and_pack_int4, dequant_int4 and pipeline_A of scripts/v29_flash_bench.py
    (:40-97), run on CPU tensors (the module imports without a GPU; its shape constants are
    14 query / 2 kv heads, head_dim 64)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "v29_flash_bench", os.path.join(REF, "scripts", "v29_flash_bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    g = torch.Generator().manual_seed(29)
    B, T, hd = 2, 96, m.HEAD_DIM
    k = torch.randn(B, m.N_KV_HEADS, T, hd, generator=g).to(torch.float16)
    v = (torch.randn(B, m.N_KV_HEADS, T, hd, generator=g) * 0.7 + 0.1).to(torch.float16)
    k[..., 5] *= 10  # an outlier channel
    k[0, 0, 3] = 0   # an all-zero row
    v[1, 1, 7] = torch.arange(hd, dtype=torch.float16) * 0.5  # exact ties after scaling
    q = torch.randn(B, m.N_HEADS, 1, hd, generator=g).to(torch.float16)
    kp, ks = m.quantize_and_pack_int4(k)
    vp, vs = m.quantize_and_pack_int4(v)
    # pipeline_A's arithmetic (dequantize, repeat the kv heads, SDPA) carried out in fp32:
    # the packed tensors and the dequantized values are the contract, the fp16 rounding of
    # its SDPA is not
    kd, vd = m.dequant_int4(kp, ks), m.dequant_int4(vp, vs)
    n_rep = m.N_HEADS // m.N_KV_HEADS
    o = torch.nn.functional.scaled_dot_product_attention(
        q.float(), kd.float().repeat_interleave(n_rep, dim=1),
        vd.float().repeat_interleave(n_rep, dim=1), is_causal=False)
    out["contig_sym"] = dict(
        key=k.float().numpy(), value=v.float().numpy(), query=q.float().numpy(),
        k_packed=kp.numpy(), v_packed=vp.numpy(),
        k_scales=ks.view(torch.int16).numpy().view(np.uint16),
        v_scales=vs.view(torch.int16).numpy().view(np.uint16),
        k_dequant=kd.float().numpy(), v_dequant=vd.float().numpy(), out=o.numpy(),
        n_heads=np.int32(m.N_HEADS), n_kv_heads=np.int32(m.N_KV_HEADS))
    print("contiguous symmetric case done", flush=True)


def gen_routed_cases(m, out):
    """Routed decode (routing/fused_routed_attention.py): the reference's own torch
    implementation ``reference_routed_decode`` (:496-548) over the DEQUANTIZED contents of a
    packed cache that the reference's write kernel filled; the dequantization is the
    reference's ``_cpu_dequant_slot`` (:150-195), slot by slot."""
    spec = importlib.util.spec_from_file_location(
        "knlp_ref_routed", os.path.join(REF, "routing", "fused_routed_attention.py"))
    r = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(r)
    cases = (
        # name, dtype, Hq, Hkv, d, block size, blocks in the cache, batch, max selected
        ("gqa4_d128_p16", "bf16", 8, 2, 128, 16, 24, 2, 9),
        ("gqa2_d64_p32", "f16", 4, 2, 64, 32, 10, 3, 4),
        ("mha_d128_p64", "f16", 2, 2, 128, 64, 6, 1, 5),
    )
    for name, dtype, hq, hkv, d, P, nb, B, max_sel in cases:
        g = torch.Generator().manual_seed(4100 + d + P)
        kvdt = DT[dtype]
        k, v = make_kv(g, nb * P, hkv, d, kvdt, special_rows=False)
        slots = torch.arange(nb * P, dtype=torch.int64)
        q = torch.randn(B, hq, d, generator=g).to(kvdt)
        tables = torch.zeros(B, hkv, max_sel, dtype=torch.int32)
        counts = torch.zeros(B, hkv, dtype=torch.int32)
        for b in range(B):
            for h in range(hkv):
                n = int(torch.randint(1, max_sel + 1, (1,), generator=g))
                counts[b, h] = n
                tables[b, h, :n] = torch.randperm(nb, generator=g)[:n].to(torch.int32)
        counts[0, 0] = max_sel
        tables[0, 0] = torch.randperm(nb, generator=g)[:max_sel].to(torch.int32)
        if B > 1:
            counts[1, hkv - 1] = 0  # a head with nothing selected: zeros
        rec = dict(query=q.float().numpy(), block_tables=tables.numpy(), block_counts=counts.numpy(), q_dtype=dtype,
                   block_size=P, num_blocks=nb, num_kv_heads=hkv, head_size=d)
        for mode, asym in (("asym", True), ("sym", False)):
            kc, vc, ks, vs, kz, vz = alloc_cache(nb, P, hkv, d)
            m.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz if asym else None,
                                     vz if asym else None, asymmetric=asym)
            kd = torch.zeros(nb, P, hkv, d)
            vd = torch.zeros(nb, P, hkv, d)
            for blk in range(nb):
                for off in range(P):
                    for h in range(hkv):
                        kd[blk, off, h] = torch.tensor(m._cpu_dequant_slot(
                            kc, ks, blk, off, h, d, n_values=d, zeros=kz if asym else None))
                        vd[blk, off, h] = torch.tensor(m._cpu_dequant_slot(
                            vc, vs, blk, off, h, d, n_values=d, zeros=vz if asym else None))
            o = r.reference_routed_decode(q.float(), kd, vd, tables.long(), counts)
            rec[f"{mode}_out"] = o.float().numpy()
            rec[f"{mode}_k_cache"], rec[f"{mode}_v_cache"] = kc.numpy(), vc.numpy()
            rec[f"{mode}_k_scales"], rec[f"{mode}_v_scales"] = f16_bits(ks), f16_bits(vs)
            if asym:
                rec["asym_k_zeros"], rec["asym_v_zeros"] = f16_bits(kz), f16_bits(vz)
        out[f"routed_{name}"] = rec
        print("routed", name, "done", flush=True)


def gen_lowrank_cases(out):
    """Low-rank-V decode: the reference's own torch implementations ``lowrank_decode_ref`` and
    ``dense_decode`` (pos_quant_v/kernel/vlowrank_kernel.py:157-174) on CPU tensors; the basis
    is orthonormal (QR of a seeded matrix), the coefficients are proj = V B as the method
    defines them."""
    spec = importlib.util.spec_from_file_location(
        "knlp_ref_vlowrank", os.path.join(REF, "pos_quant_v", "kernel", "vlowrank_kernel.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    rec = {}
    cases = (("gqa4_d128_bf16", 2, 4, 300, 128, "bf16"), ("gqa8_d64_f16", 3, 8, 70, 64, "f16"),
             ("one_token_bf16", 1, 1, 1, 128, "bf16"), ("gqa5_d128_f16", 2, 5, 517, 128, "f16"))
    for name, hkv, nq, T, dh, dt in cases:
        g = torch.Generator().manual_seed(5100 + T + dh)
        Q = torch.randn(hkv, nq, dh, generator=g).to(DT[dt])
        K = (torch.randn(hkv, T, dh, generator=g) * 1.3).to(DT[dt])
        V = torch.randn(hkv, T, dh, generator=g)
        B = torch.linalg.qr(torch.randn(hkv, dh, 32, generator=g)).Q.contiguous()
        proj = torch.bmm(V, B).contiguous()
        rec[name + "_q"], rec[name + "_k"] = f16_bits(Q), f16_bits(K)  # raw 16-bit patterns
        rec[name + "_proj"], rec[name + "_basis"] = proj.numpy(), B.numpy()
        rec[name + "_out"] = m.lowrank_decode_ref(Q, K, proj, B).numpy()
        rec[name + "_dense_of_lifted_v"] = m.dense_decode(Q, K, torch.bmm(proj, B.transpose(1, 2))).numpy()
        rec[name + "_dtype"] = dt
        print("lowrank", name, "done", flush=True)
    out["lowrank"] = rec


def main():
    out = {}
    if "--only-lowrank" in sys.argv:
        gen_lowrank_cases(out)
        for name, rec in out.items():
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
            print("saved", name)
        return
    if "--only-routed" in sys.argv:
        gen_routed_cases(load_reference(), out)
        for name, rec in out.items():
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
            print("saved", name)
        return
    if "--only-contig" in sys.argv:
        gen_contig_cases(out)
        for name, rec in out.items():
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
            print("saved", name)
        return
    if "--only-kfp16" in sys.argv:
        gen_kfp16_cases(load_reference(), out)
        for name, rec in out.items():
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
            print("saved", name)
        return
    if "--only-plugin" in sys.argv:
        gen_plugin_cases(out)
    elif "--only-v8" in sys.argv:
        gen_v8_cases(load_reference(), out)
    else:
        m = load_reference()
        gen_write_cases(m, out)
        gen_decode_cases(m, out)
        gen_plugin_cases(out)
        for name, rec in out.items():  # gen_v8_cases reads the files written so far
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        gen_v8_cases(m, out)
    for name, rec in out.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print("saved", name)


if __name__ == "__main__":
    main()
