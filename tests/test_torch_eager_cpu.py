"""The PyTorch-eager CPU baseline (oracle/torch_eager.py) against the numpy oracle."""

import numpy as np
import torch

from conftest import alloc_cache_np
from oracle import kv_oracle as O
from oracle import torch_eager as TE


def _case(int8_k, asym, seed=3):
    rng = np.random.default_rng(seed)
    S, Hq, Hkv, d, P = 2, 8, 2, 64, 16
    lens = np.array([37, 100], np.int32)
    nb = int(sum((L + P - 1) // P for L in lens)) + 1
    kc, vc, ks, vs, kz, vz = alloc_cache_np(nb, P, Hkv, d, int8_k=int8_k)
    perm = rng.permutation(nb)
    bt = np.zeros((S, 8), np.int32)
    o = 0
    slots = []
    for s, L in enumerate(lens):
        n = (L + P - 1) // P
        bt[s, :n] = perm[o:o + n]
        o += n
        pos = np.arange(L)
        slots.append(bt[s, pos // P].astype(np.int64) * P + pos % P)
    slots = np.concatenate(slots)
    k = rng.standard_normal((len(slots), Hkv, d)).astype(np.float32)
    v = rng.standard_normal((len(slots), Hkv, d)).astype(np.float32)
    q = rng.standard_normal((S, Hq, d)).astype(np.float32)
    if int8_k:
        O.reshape_and_cache_k_int8(k, kc, ks, slots)
        O.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz if asym else None, asymmetric=asym)
        ref = O.kint8_vint4_decode(q, kc, vc, ks, vs, bt, lens, Hkv, d,
                                   v_zeros=vz if asym else None, asymmetric=asym)
    else:
        O.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz if asym else None,
                                 vz if asym else None, asymmetric=asym)
        ref = O.fused_int4_decode(q, kc, vc, ks, vs, bt, lens, Hkv, d,
                                  k_zeros=kz if asym else None, v_zeros=vz if asym else None,
                                  asymmetric=asym)
    t = torch.from_numpy
    out = TE.decode(t(q), t(kc), t(vc), t(ks), t(vs), t(bt), t(lens), Hkv, d,
                    k_zeros=t(kz) if (asym and not int8_k) else None,
                    v_zeros=t(vz) if asym else None, k_int8=int8_k)
    return out.numpy(), ref


def test_torch_eager_matches_numpy_oracle():
    for int8_k, asym in ((False, True), (False, False), (True, True)):
        out, ref = _case(int8_k, asym)
        np.testing.assert_allclose(out, ref, atol=2e-5, rtol=1e-5)
