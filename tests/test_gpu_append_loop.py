"""Benchmark configuration 5 as it is stated: every step appends one new token per sequence
to the packed cache (quantize-append) and then attends over the full cache, for 64
consecutive steps (reference flow: fused-quant/fused_int4.v0.1.0.py:2661-2689, the cache
write, then :2901-2914, the decode).  The appended rows must be bit-identical to the
oracle's, the attention output within the stated tolerance at steps that cross page
boundaries and at the last one."""

import numpy as np
import pytest
import torch

from conftest import alloc_cache_np
from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-3
P = 16
CHECK_STEPS = (0, 1, 15, 16, 17, 31, 32, 63)


def _close(out, ref, what):
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    err = np.abs(out - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{what}: max abs err {err.max():.3e}"


def _zeros_equal(a, b):
    # the sign of a zero minimum is not defined by the reference (see test_oracle_golden)
    a, b = a.view(np.uint16), b.view(np.uint16)
    return bool(np.all((a == b) | (((a | b) & 0x7FFF) == 0)))


@pytest.mark.parametrize("mode", ["k8v4", "int4", "k8v4_two_calls", "k8v4_fused", "int4_fused"])
def test_append_then_attend_64_steps(mode, cuda_device):
    from knlp_b200 import ops
    dev = cuda_device
    rng = np.random.default_rng(50)
    Hq, Hkv, d, n_steps = 32, 8, 128, 64
    # lengths that put the appended token on every position of a page over the 64 steps,
    # first and last slot of a page included, and that move the end of the sequence through
    # the balanced kernel's chunk (64 tokens) and the fixed splits' boundaries
    lens0 = [15, 16, 31, 100, 257, 1000, 1, 2047, 0]
    S = len(lens0)
    k8 = mode.startswith("k8v4")
    fused = mode.endswith("_fused")  # the step's token is appended by the decode launch itself
    pages = [(L + n_steps + P - 1) // P for L in lens0]
    nb = sum(pages) + 3
    perm = rng.permutation(nb)
    bt = np.zeros((S, max(pages)), np.int32)
    o = 0
    for s, n in enumerate(pages):
        bt[s, :n] = perm[o:o + n]
        o += n
    kc, vc, ks, vs, kz, vz = alloc_cache_np(nb, P, Hkv, d, int8_k=k8)
    chs = np.where(rng.random((Hkv, d)) < 0.02, 10.0, 1.0).astype(np.float32)

    def bf16(a):  # the bench's tokens are bf16
        return torch.from_numpy(a).to(torch.bfloat16)

    # device mirrors
    t = lambda a: torch.from_numpy(a).to(dev)
    kc_d, vc_d, ks_d, vs_d, kz_d, vz_d = (t(a) for a in (kc, vc, ks, vs, kz, vz))
    bt_d = t(bt)
    L = ops._lib
    if k8:
        kp = ops._plane(kc_d, ks_d, None, L.KV_INT8_G32)
    else:
        kp = ops._plane(kc_d, ks_d, kz_d, L.KV_INT4_ASYM)
    vp = ops._plane(vc_d, vs_d, vz_d, L.KV_INT4_ASYM)

    def append(k_b, v_b, slots):
        kf, vf = k_b.float().numpy(), v_b.float().numpy()
        if k8:
            O.reshape_and_cache_k_int8(kf, kc, ks, slots)
            O.reshape_and_cache_v_only_int4(vf, vc, vs, slots, vz, asymmetric=True)
        else:
            O.reshape_and_cache_int4(kf, vf, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
        sl = torch.from_numpy(slots).to(dev)
        if mode == "k8v4_two_calls":  # the reference's own two operators
            ops.reshape_and_cache_k_int8(k_b.to(dev), kc_d, ks_d, sl)
            ops.reshape_and_cache_v_only_int4(v_b.to(dev), vc_d, vs_d, sl, vz_d, asymmetric=True)
        else:  # both planes in one launch
            ops.quant_append(k_b.to(dev), v_b.to(dev), kp, vp, sl, P)

    # prefill
    for s, n in enumerate(lens0):
        if n == 0:
            continue
        k_b = bf16(rng.standard_normal((n, Hkv, d)).astype(np.float32) * chs)
        v_b = bf16(rng.standard_normal((n, Hkv, d)).astype(np.float32) * chs)
        pos = np.arange(n)
        append(k_b, v_b, bt[s, pos // P].astype(np.int64) * P + pos % P)

    lens = np.array(lens0, np.int32)
    for step in range(n_steps):
        q = bf16(rng.standard_normal((S, Hq, d)).astype(np.float32))
        k_b = bf16(rng.standard_normal((S, Hkv, d)).astype(np.float32) * chs)
        v_b = bf16(rng.standard_normal((S, Hkv, d)).astype(np.float32) * chs)
        slots = bt[np.arange(S), lens // P].astype(np.int64) * P + lens % P
        if fused:
            # oracle: write, then attend; GPU: ONE launch given the lengths before the append
            kf, vf = k_b.float().numpy(), v_b.float().numpy()
            if k8:
                O.reshape_and_cache_k_int8(kf, kc, ks, slots)
                O.reshape_and_cache_v_only_int4(vf, vc, vs, slots, vz, asymmetric=True)
            else:
                O.reshape_and_cache_int4(kf, vf, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
            out = ops.decode_attention(q.to(dev), kp, vp, nb, bt_d, torch.from_numpy(lens).to(dev),
                                       Hkv, d, P, out_dtype=torch.float32,
                                       max_seq_len=int(lens.max()) + 1,
                                       new_key=k_b.to(dev), new_value=v_b.to(dev))
            lens = lens + 1
            lens_d = torch.from_numpy(lens).to(dev)
        else:
            append(k_b, v_b, slots)
            lens = lens + 1
            lens_d = torch.from_numpy(lens).to(dev)
            # every step runs on the GPU (the loop is the point); the oracle checks some
            out = ops.decode_attention(q.to(dev), kp, vp, nb, bt_d, lens_d, Hkv, d, P,
                                       out_dtype=torch.float32, max_seq_len=int(lens.max()))
        if step in CHECK_STEPS:
            qf = q.float().numpy()
            if k8:
                ref = O.kint8_vint4_decode(qf, kc, vc, ks, vs, bt, lens, Hkv, d, v_zeros=vz,
                                           asymmetric=True)
            else:
                ref = O.fused_int4_decode(qf, kc, vc, ks, vs, bt, lens, Hkv, d, k_zeros=kz,
                                          v_zeros=vz, asymmetric=True)
            _close(out.cpu().numpy(), ref, f"{mode} step {step}")
            # the fixed-split path on the same cache
            pm, pl, po = ops.decode_partials(q.to(dev), kp, vp, nb, bt_d, lens_d, Hkv, d, P,
                                             max_seq_len=int(lens.max()))
            _close(ops.combine_partials(pm, pl, po).cpu().numpy(), ref, f"{mode} step {step} splits")

    # every appended row, bit for bit
    assert np.array_equal(kc_d.cpu().numpy(), kc)
    assert np.array_equal(vc_d.cpu().numpy(), vc)
    assert np.array_equal(ks_d.cpu().numpy().view(np.uint16), ks.view(np.uint16))
    assert np.array_equal(vs_d.cpu().numpy().view(np.uint16), vs.view(np.uint16))
    assert _zeros_equal(vz_d.cpu().numpy(), vz)
    if not k8:
        assert _zeros_equal(kz_d.cpu().numpy(), kz)
