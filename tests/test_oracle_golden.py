"""Pin the CPU oracle against outputs of the reference's own kernels
(tests/golden/*.npz, produced by tests/golden/make_golden.py under the Triton
interpreter).  Write path: bit-exact.  Decode: to the resolution of the
reference's output, which is its fp32 accumulator rounded through fp16 into the
query dtype (fused_int4.v0.1.0.py:891-894, :932).
"""

import numpy as np
import pytest

from conftest import alloc_cache_np, load_golden
from oracle import kv_oracle as O

WRITE_CASES = ["write_f32_d64", "write_bf16_d128", "write_f16_d128"]
DECODE_CASES = ["decode_mha_f32_d64", "decode_gqa4_bf16_d128", "decode_gqa8_f16_d128"]


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def zeros_equal(a_bits, b_bits):
    """fp16 zero-points equal bit for bit, except that +0.0 and -0.0 are not told
    apart: for a group holding zeros of both signs the reference's minimum is
    whichever sign its reduction meets last (the golden run shows both), so the
    sign of a zero minimum is not defined by the reference."""
    a_bits, b_bits = np.asarray(a_bits), np.asarray(b_bits)
    return bool(np.all((a_bits == b_bits) | (((a_bits | b_bits) & 0x7FFF) == 0)))


@pytest.mark.parametrize("case", WRITE_CASES)
def test_write_asym_bit_exact(case):
    G = load_golden(case)
    k, v, slots = G["key"], G["value"], G["slot_mapping"]
    n, h, d = k.shape
    kc, vc, ks, vs, kz, vz = alloc_cache_np(int(G["num_blocks"]), int(G["block_size"]), h, d)
    O.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=True)
    assert np.array_equal(kc, G["asym_kc"]) and np.array_equal(vc, G["asym_vc"])
    assert np.array_equal(bits(ks), G["asym_ks"]) and np.array_equal(bits(vs), G["asym_vs"])
    assert zeros_equal(bits(kz), G["asym_kz"]) and zeros_equal(bits(vz), G["asym_vz"])


@pytest.mark.parametrize("case", WRITE_CASES)
def test_write_sym_clip_bit_exact(case):
    G = load_golden(case)
    k, v, slots = G["key"], G["value"], G["slot_mapping"]
    n, h, d = k.shape
    kc, vc, ks, vs, _, _ = alloc_cache_np(int(G["num_blocks"]), int(G["block_size"]), h, d)
    O.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, asymmetric=False,
                             clip_ratio=float(G["clip_ratio"]))
    assert np.array_equal(kc, G["sym_kc"]) and np.array_equal(vc, G["sym_vc"])
    assert np.array_equal(bits(ks), G["sym_ks"]) and np.array_equal(bits(vs), G["sym_vs"])


@pytest.mark.parametrize("case", WRITE_CASES)
def test_write_v_only_and_k_int8_bit_exact(case):
    G = load_golden(case)
    k, v, slots = G["key"], G["value"], G["slot_mapping"]
    n, h, d = k.shape
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    _, vc, _, vs, _, vz = alloc_cache_np(nb, P, h, d)
    O.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
    assert np.array_equal(vc, G["vonly_vc"])
    assert np.array_equal(bits(vs), G["vonly_vs"]) and zeros_equal(bits(vz), G["vonly_vz"])
    kc8, _, ks, _, _, _ = alloc_cache_np(nb, P, h, d, int8_k=True)
    O.reshape_and_cache_k_int8(k, kc8, ks, slots)
    assert np.array_equal(kc8, G["int8_kc"]) and np.array_equal(bits(ks), G["int8_ks"])


def _tol(q_dtype):
    # (atol, rtol).  The reference casts its fp32 accumulator to fp16 before the
    # store whatever the query dtype (half-ulp 4.9e-4 relative), and a bf16 query
    # then converts that to bf16 (ulp 7.8e-3; the measured gap is 7.1e-3): the comparison cannot be finer.
    return {"f32": (2e-6, 6e-4), "f16": (2e-6, 6e-4), "bf16": (2e-6, 8e-3)}[str(q_dtype)]


@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("mode", ["asym", "sym", "k8v4"])
def test_decode_matches_reference_kernel(case, mode):
    G = load_golden(case)
    k, v, slots = G["key"], G["value"], G["slot_mapping"]
    hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    q, bt, sl = G["query"], G["block_table"], G["seq_lens"]
    if mode == "k8v4":
        kc8, vc, ks, vs, _, vz = alloc_cache_np(nb, P, hkv, d, int8_k=True)
        O.reshape_and_cache_k_int8(k, kc8, ks, slots)
        O.reshape_and_cache_v_only_int4(v, vc, vs, slots, vz, asymmetric=True)
        out = O.kint8_vint4_decode(q, kc8, vc, ks, vs, bt, sl, hkv, d, v_zeros=vz, asymmetric=True)
    else:
        asym = mode == "asym"
        kc, vc, ks, vs, kz, vz = alloc_cache_np(nb, P, hkv, d)
        O.reshape_and_cache_int4(k, v, kc, vc, ks, vs, slots, kz, vz, asymmetric=asym)
        out = O.fused_int4_decode(q, kc, vc, ks, vs, bt, sl, hkv, d,
                                  k_zeros=kz if asym else None, v_zeros=vz if asym else None,
                                  asymmetric=asym)
    ref = G[f"{mode}_out"]
    atol, rtol = _tol(G["q_dtype"])
    np.testing.assert_allclose(out, ref, atol=atol, rtol=rtol)


def test_round_half_away_fp32_add():
    y = np.array([0.5 - 2.0 ** -25, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.49999994, -0.49999994],
                 dtype=np.float32)
    r = O.round_half_away(y)
    assert r.tolist() == [1.0, 1.0, 2.0, 3.0, -1.0, -2.0, -3.0, 0.0, -0.0]


def test_combine_equals_unsplit():
    rng = np.random.default_rng(3)
    T, Hq, Hkv, d = 300, 8, 2, 64
    q = rng.standard_normal((Hq, d)).astype(np.float32)
    k = rng.standard_normal((T, Hkv, d)).astype(np.float32)
    v = rng.standard_normal((T, Hkv, d)).astype(np.float32)
    full, _, _ = O.attend_one(q, k, v)
    for n in (1, 2, 7, 400):  # 400 > T: some parts are empty
        pm, pl, po = O.partials_one(q, k, v, n)
        np.testing.assert_allclose(O.combine_partials(pm, pl, po), full, atol=2e-6, rtol=1e-5)


def test_plugin_quantizers_match_reference_functions():
    # backends/quant.py:23-72 on fp32 input: round-half-even, clamp, scale shapes
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 2, 5, 64)).astype(np.float32)
    x[0, 0, 0, :] = 0.0
    q8, s8 = O.plugin_quantize_int8_symmetric(x)
    assert q8.dtype == np.int8 and s8.shape == (1, 2, 5, 1)
    assert np.abs(q8.astype(np.float32) * s8 - x).max() <= s8.max() * 0.5 + 1e-7
    q4, s4 = O.plugin_quantize_int4_block(x, 32)
    assert q4.shape == x.shape and s4.shape == (1, 2, 5, 2)
    assert q4.min() >= -8 and q4.max() <= 7
