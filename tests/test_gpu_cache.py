"""knlp_b200.cache.PackedKVCache: the cache write, the five-way decode dispatch and the
one-launch decode step against the oracle (reference do_kv_cache_update :2483-2546,
_fused_decode :2851-2928)."""

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3
P = 16


def _close(out, ref, what):
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    err = np.abs(out - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{what}: max abs err {err.max():.3e}"


@pytest.mark.parametrize("kp,vp,asym", [("int4", "int4", True), ("int4", "int4", False),
                                        ("int8", "int4", True), ("int8", "int8", False),
                                        ("fp16", "int4", True), ("fp16", "int8", False)])
def test_write_decode_and_step(kp, vp, asym, cuda_device):
    from knlp_b200 import cache as KC
    dev = cuda_device
    rng = np.random.default_rng(7)
    S, Hq, Hkv, d = 3, 16, 4, 128
    lens = [50, 16, 133]
    nb = sum((L + 1 + P - 1) // P for L in lens) + 1
    bt = np.zeros((S, max((L + 1 + P - 1) // P for L in lens)), np.int32)
    perm = rng.permutation(nb)
    o = 0
    for s, L in enumerate(lens):
        n = (L + 1 + P - 1) // P
        bt[s, :n] = perm[o:o + n]
        o += n
    c = KC.PackedKVCache(Hkv, d, kp, vp, asym)
    c.ensure(nb, P, dev)
    # oracle caches
    ng = d // 32
    kc = np.zeros((nb, P, Hkv, d if kp == "int8" else d // 2), np.int8 if kp == "int8" else np.uint8)
    vc = np.zeros((nb, P, Hkv, d if vp == "int8" else d // 2), np.int8 if vp == "int8" else np.uint8)
    ks, vs, kz, vz = (np.zeros((nb, P, Hkv, ng), np.float16) for _ in range(4))
    kfp = np.zeros((nb, P, Hkv, d), np.float32)
    kfp_d = torch.zeros(nb, P, Hkv, d, dtype=torch.float16, device=dev)

    def write(k_h, v_h, slots):
        kf, vf = k_h.float().numpy(), v_h.float().numpy()
        if kp == "int8":
            O.reshape_and_cache_k_int8(kf, kc, ks, slots)
        elif kp == "int4":
            O.reshape_and_cache_int4(kf, vf, kc, np.zeros_like(kc), ks, np.zeros_like(ks), slots,
                                     kz if asym else None, np.zeros_like(kz) if asym else None,
                                     asymmetric=asym)
        else:
            kfp.reshape(nb * P, Hkv, d)[slots] = kf
            kfp_d.view(nb * P, Hkv, d)[torch.from_numpy(slots).to(dev)] = k_h.to(dev)
        if vp == "int8":
            O.reshape_and_cache_v_int8(vf, vc, vs, slots)
        else:
            O.reshape_and_cache_v_only_int4(vf, vc, vs, slots, vz if asym else None, asymmetric=asym)

    def oracle(q, L):
        qf = q.float().numpy()
        la = np.array(L, np.int32)
        if kp == "fp16":
            f = O.kfp16_vint8_decode if vp == "int8" else O.kfp16_vint4_decode
            kw = {} if vp == "int8" else dict(v_zeros=vz if asym else None, asymmetric=asym)
            return f(qf, kfp, vc, vs, bt, la, Hkv, d, **kw)
        if kp == "int8" and vp == "int8":
            return O.kint8_vint8_decode(qf, kc, vc, ks, vs, bt, la, Hkv, d)
        if kp == "int8":
            return O.kint8_vint4_decode(qf, kc, vc, ks, vs, bt, la, Hkv, d,
                                        v_zeros=vz if asym else None, asymmetric=asym)
        return O.fused_int4_decode(qf, kc, vc, ks, vs, bt, la, Hkv, d, k_zeros=kz if asym else None,
                                   v_zeros=vz if asym else None, asymmetric=asym)

    h16 = lambda a: torch.from_numpy(a.astype(np.float32)).to(torch.float16)
    # prefill through cache.write
    for s, L in enumerate(lens):
        k_h, v_h = h16(rng.standard_normal((L, Hkv, d))), h16(rng.standard_normal((L, Hkv, d)))
        pos = np.arange(L)
        slots = bt[s, pos // P].astype(np.int64) * P + pos % P
        write(k_h, v_h, slots)
        c.write(None if kp == "fp16" else k_h.to(dev), v_h.to(dev), torch.from_numpy(slots).to(dev))
    bt_d = torch.from_numpy(bt).to(dev)
    q = h16(rng.standard_normal((S, Hq, d)))
    out = c.decode(q.to(dev), bt_d, torch.tensor(lens, dtype=torch.int32, device=dev),
                   key_cache_fp16=kfp_d if kp == "fp16" else None, out_dtype=torch.float32)
    _close(out.cpu().numpy(), oracle(q, lens), f"decode {kp}/{vp}")
    # one decode step: new token in, attention over it
    k_h, v_h = h16(rng.standard_normal((S, Hkv, d))), h16(rng.standard_normal((S, Hkv, d)))
    la = np.array(lens)
    slots = bt[np.arange(S), la // P].astype(np.int64) * P + la % P
    write(k_h, v_h, slots)
    if kp == "fp16":
        pass  # the framework's K cache was updated in write()
    new_lens = [L + 1 for L in lens]
    meta = KC.AttentionMetadata(num_actual_tokens=S, max_query_len=1, query_start_loc=None,
                                max_seq_len=max(new_lens),
                                seq_lens=torch.tensor(new_lens, dtype=torch.int32, device=dev),
                                block_table=bt_d, slot_mapping=torch.from_numpy(slots).to(dev))
    out = c.decode_step(q.to(dev), k_h.to(dev), v_h.to(dev), meta,
                        key_cache_fp16=kfp_d if kp == "fp16" else None, out_dtype=torch.float32)
    _close(out.cpu().numpy(), oracle(q, new_lens), f"decode_step {kp}/{vp}")
    assert c.actual_bytes_per_block() == c.expected_bytes_per_block()
