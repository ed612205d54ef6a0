"""Unquantized K: kfp16_vint4_decode and kfp16_vint8_decode.

Golden outputs (tests/golden/kfp16_modes.npz) come from the reference's own kernels run
under the Triton interpreter (tests/golden/make_golden.py --only-kfp16)."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import kv_oracle as O

DECODE_CASES = ["decode_mha_f32_d64", "decode_gqa4_bf16_d128", "decode_gqa8_f16_d128"]
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
ATOL, RTOL = 2e-3, 1e-3


def _oracle_inputs(G, K):
    """numpy caches for the oracle: V INT4 asym and V INT8 quantized by the oracle itself."""
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
    vc = np.zeros((nb, P, hkv, d // 2), np.uint8)
    vs = np.zeros((nb, P, hkv, d // 32), np.float16)
    vz = np.zeros_like(vs)
    O.reshape_and_cache_v_only_int4(G["value"], vc, vs, G["slot_mapping"], vz, asymmetric=True)
    vc8 = np.zeros((nb, P, hkv, d), np.int8)
    vs8 = np.zeros((nb, P, hkv, d // 32), np.float16)
    O.reshape_and_cache_v_int8(G["value"], vc8, vs8, G["slot_mapping"])
    return vc, vs, vz, vc8, vs8, hkv, d


@pytest.mark.parametrize("case", DECODE_CASES)
def test_oracle_kfp16_decodes_vs_reference(case):
    G, K = load_golden(case), load_golden("kfp16_modes")
    vc, vs, vz, vc8, vs8, hkv, d = _oracle_inputs(G, K)
    kcache = K[case + "_kcache"]
    ulp = {"f32": 6e-4, "f16": 6e-4, "bf16": 8e-3}[str(G["q_dtype"])]
    o4 = O.kfp16_vint4_decode(G["query"], kcache, vc, vs, G["block_table"], G["seq_lens"], hkv, d,
                              v_zeros=vz, asymmetric=True)
    np.testing.assert_allclose(o4, K[case + "_kf16v4_out"], atol=2e-6, rtol=ulp)
    o8 = O.kfp16_vint8_decode(G["query"], kcache, vc8, vs8, G["block_table"], G["seq_lens"], hkv, d)
    np.testing.assert_allclose(o8, K[case + "_kf16v8_out"], atol=2e-6, rtol=ulp)


@pytest.mark.gpu
@pytest.mark.parametrize("case", DECODE_CASES)
def test_kfp16_decodes_golden(case, cuda_device):
    from knlp_b200 import ops
    G, K = load_golden(case), load_golden("kfp16_modes")
    dev = cuda_device
    vc, vs, vz, vc8, vs8, hkv, d = _oracle_inputs(G, K)
    kdt = TDT[str(K[case + "_kdtype"])]
    q = torch.from_numpy(G["query"]).to(TDT[str(G["q_dtype"])]).to(dev)
    kcache = torch.from_numpy(K[case + "_kcache"]).to(kdt).to(dev)
    bt = torch.from_numpy(G["block_table"]).to(dev)
    sl = torch.from_numpy(G["seq_lens"]).to(dev)
    t = lambda a: torch.from_numpy(a).to(dev)
    ulp = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[str(G["q_dtype"])]

    ref4 = O.kfp16_vint4_decode(G["query"], K[case + "_kcache"], vc, vs, G["block_table"],
                                G["seq_lens"], hkv, d, v_zeros=vz, asymmetric=True)
    out4 = ops.kfp16_vint4_decode(q, kcache, t(vc), t(vs), bt, sl, hkv, d, v_zeros=t(vz),
                                  asymmetric=True, out_dtype=torch.float32)
    err = np.abs(out4.cpu().numpy() - ref4)
    assert np.all(err <= ATOL + RTOL * np.abs(ref4)), f"v4: max abs err {err.max():.3e}"
    out4q = ops.kfp16_vint4_decode(q, kcache, t(vc), t(vs), bt, sl, hkv, d, v_zeros=t(vz),
                                   asymmetric=True)
    np.testing.assert_allclose(out4q.float().cpu().numpy(), K[case + "_kf16v4_out"], atol=ATOL,
                               rtol=RTOL + ulp)

    ref8 = O.kfp16_vint8_decode(G["query"], K[case + "_kcache"], vc8, vs8, G["block_table"],
                                G["seq_lens"], hkv, d)
    out8 = ops.kfp16_vint8_decode(q, kcache, t(vc8), t(vs8), bt, sl, hkv, d,
                                  out_dtype=torch.float32, n_splits=3)
    err = np.abs(out8.cpu().numpy() - ref8)
    assert np.all(err <= ATOL + RTOL * np.abs(ref8)), f"v8: max abs err {err.max():.3e}"
    out8q = ops.kfp16_vint8_decode(q, kcache, t(vc8), t(vs8), bt, sl, hkv, d)
    np.testing.assert_allclose(out8q.float().cpu().numpy(), K[case + "_kf16v8_out"], atol=ATOL,
                               rtol=RTOL + ulp)


def test_unquantized_plane_is_refused_where_it_has_no_meaning():
    """fp16 K is a decode-side K plane only: the write path and the V side reject it on the
    host (no launch), and fp32 caches are refused by the wrapper."""
    import ctypes as C
    from knlp_b200 import _lib, ops
    lib = _lib.load()
    p = C.c_void_p(0x1000)
    st2 = (C.c_int64 * 2)(64, 64)
    pk = _lib.KvPlane(); pk.codes = p.value; pk.mode = _lib.KV_F16
    pv = _lib.KvPlane(); pv.codes = p.value; pv.scales = p.value; pv.mode = _lib.KV_INT4_SYM
    assert lib.knlp_b200_quant_append(p, st2, p, st2, 1, C.byref(pk), C.byref(pv), p, 1, 1, 64, 16,
                                      0.0, None) == -4
    assert lib.knlp_b200_decode_splitk(p, 0, st2, C.byref(pv), C.byref(pk), p, 1, p, 1, 1, 4, 4,
                                       64, 16, 1, 16, p, p, p, 0, None) == -4
    with pytest.raises(TypeError):
        ops._fp_plane(torch.zeros(1, 16, 1, 64))


@pytest.mark.gpu
@pytest.mark.parametrize("kdt,qdt,hq,hkv,d,v8", [
    (torch.float16, torch.float16, 32, 8, 128, False),   # GQA-4, four kv heads per CTA
    (torch.bfloat16, torch.bfloat16, 32, 8, 128, True),  # bf16 product, INT8 V
    (torch.bfloat16, torch.float32, 8, 2, 128, False),   # q split into two bf16 parts
    (torch.float16, torch.float32, 6, 6, 64, False),     # MHA, d 64, two kv heads per CTA
    (torch.float16, torch.bfloat16, 16, 2, 128, True),   # GQA-8: one column per q head
    (torch.bfloat16, torch.bfloat16, 8, 1, 128, False),  # GQA-8 with bf16 (exact for bf16 q)
    (torch.bfloat16, torch.float16, 8, 1, 128, False),   # GQA-8, bf16 K, fp16 q: generic kernel
])
def test_kfp16_tensor_core_path_vs_generic_and_oracle(kdt, qdt, hq, hkv, d, v8, cuda_device):
    """Ragged lengths over shuffled pages: the balanced tensor-core launch (default) against
    the stride-generic CUDA-core kernel (a given split count selects it) and the oracle."""
    from knlp_b200 import ops
    dev, P = cuda_device, 16
    g = torch.Generator().manual_seed(hq * 131 + d + int(v8))
    lens = [700, 33, 1, 1500, 64, 257, 16, 0]
    S = len(lens)
    blocks = [(L + P - 1) // P for L in lens]
    nb = sum(blocks) + 3
    perm = torch.randperm(nb, generator=g).to(torch.int32)
    bt = torch.zeros(S, max(blocks), dtype=torch.int32)
    slots, o = [], 0
    for s, L in enumerate(lens):
        bt[s, :blocks[s]] = perm[o:o + blocks[s]]
        o += blocks[s]
        slots += [int(bt[s, n // P]) * P + n % P for n in range(L)]
    slots = torch.tensor(slots, dtype=torch.int64)
    T = int(slots.numel())
    k = (torch.randn(T, hkv, d, generator=g) * 1.5).to(kdt)
    k[:, :, 3] *= 8  # an outlier channel
    v = torch.randn(T, hkv, d, generator=g).to(kdt)
    q = torch.randn(S, hq, d, generator=g).to(qdt)
    kcache = torch.zeros(nb, P, hkv, d, dtype=kdt)
    kcache.view(nb * P, hkv, d)[slots] = k
    vcache = torch.zeros(nb, P, hkv, d if v8 else d // 2, dtype=torch.int8 if v8 else torch.uint8,
                         device=dev)
    vs = torch.zeros(nb, P, hkv, d // 32, dtype=torch.float16, device=dev)
    vz = torch.zeros_like(vs)
    if v8:
        ops.reshape_and_cache_v_int8(v.to(dev), vcache, vs, slots.to(dev))
    else:
        ops.reshape_and_cache_v_only_int4(v.to(dev), vcache, vs, slots.to(dev), vz, asymmetric=True)
    qd, kd, btd = q.to(dev), kcache.to(dev), bt.to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)

    def run(**kw):
        if v8:
            return ops.kfp16_vint8_decode(qd, kd, vcache, vs, btd, sl, hkv, d,
                                          out_dtype=torch.float32, **kw)
        return ops.kfp16_vint4_decode(qd, kd, vcache, vs, btd, sl, hkv, d, v_zeros=vz,
                                      asymmetric=True, out_dtype=torch.float32, **kw)

    fast, generic = run(), run(n_splits=2)
    kn, qn = kcache.float().numpy(), q.float().numpy()
    if v8:
        ref = O.kfp16_vint8_decode(qn, kn, vcache.cpu().numpy(), vs.cpu().numpy(), bt.numpy(),
                                   np.asarray(lens, np.int32), hkv, d)
    else:
        ref = O.kfp16_vint4_decode(qn, kn, vcache.cpu().numpy(), vs.cpu().numpy(), bt.numpy(),
                                   np.asarray(lens, np.int32), hkv, d,
                                   v_zeros=vz.cpu().numpy(), asymmetric=True)
    for name, out in (("tensor-core", fast), ("generic", generic)):
        err = np.abs(out.cpu().numpy() - ref)
        assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{name}: max abs err {err.max():.3e}"
    assert not fast[-1].any()  # the sequence without tokens
