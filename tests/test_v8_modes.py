"""INT8 V: reshape_and_cache_v_int8 and kint8_vint8_decode.

Golden outputs (tests/golden/v8_modes.npz) come from the reference's own kernels run under
the Triton interpreter on the inputs of the write_* and decode_* fixtures
(tests/golden/make_golden.py --only-v8)."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import kv_oracle as O

WRITE_CASES = ["write_f32_d64", "write_bf16_d128", "write_f16_d128"]
DECODE_CASES = ["decode_mha_f32_d64", "decode_gqa4_bf16_d128", "decode_gqa8_f16_d128"]
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
ATOL, RTOL = 2e-3, 1e-3


def _bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


# ------------------------------------------------------------------ oracle vs reference (CPU)
@pytest.mark.parametrize("case", WRITE_CASES)
def test_oracle_v_int8_write_bit_exact(case):
    G, V8 = load_golden(case), load_golden("v8_modes")
    v, slots = G["value"], G["slot_mapping"]
    n, h, d = v.shape
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    vc = np.zeros((nb, P, h, d), np.int8)
    vs = np.zeros((nb, P, h, d // 32), np.float16)
    O.reshape_and_cache_v_int8(v, vc, vs, slots)
    assert np.array_equal(vc, V8[case + "_vc8"])
    assert np.array_equal(vs.view(np.uint16), V8[case + "_vs8"])


@pytest.mark.parametrize("case", DECODE_CASES)
def test_oracle_k8v8_decode_vs_reference(case):
    G, V8 = load_golden(case), load_golden("v8_modes")
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
    kc = np.zeros((nb, P, hkv, d), np.int8)
    vc = np.zeros((nb, P, hkv, d), np.int8)
    ks = np.zeros((nb, P, hkv, d // 32), np.float16)
    vs = np.zeros((nb, P, hkv, d // 32), np.float16)
    O.reshape_and_cache_k_int8(G["key"], kc, ks, G["slot_mapping"])
    O.reshape_and_cache_v_int8(G["value"], vc, vs, G["slot_mapping"])
    out = O.kint8_vint8_decode(G["query"], kc, vc, ks, vs, G["block_table"], G["seq_lens"], hkv, d)
    # the reference stores its fp32 accumulator through fp16, then the query dtype
    ulp = {"f32": 6e-4, "f16": 6e-4, "bf16": 8e-3}[str(G["q_dtype"])]
    np.testing.assert_allclose(out, V8[case + "_k8v8_out"], atol=2e-6, rtol=ulp)


# ------------------------------------------------------------------ CUDA path vs both (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("case", WRITE_CASES)
def test_v_int8_write_matches_reference_bits(case, cuda_device):
    from knlp_b200 import ops
    G, V8 = load_golden(case), load_golden("v8_modes")
    dt = TDT[str(G["src_dtype"])]
    v = torch.from_numpy(G["value"]).to(dt).to(cuda_device)
    slots = torch.from_numpy(G["slot_mapping"]).to(cuda_device)
    n, h, d = v.shape
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    vc = torch.zeros(nb, P, h, d, dtype=torch.int8, device=cuda_device)
    vs = torch.zeros(nb, P, h, d // 32, dtype=torch.float16, device=cuda_device)
    ops.reshape_and_cache_v_int8(v, vc, vs, slots)
    assert np.array_equal(vc.cpu().numpy(), V8[case + "_vc8"])
    assert np.array_equal(_bits(vs), V8[case + "_vs8"])


def _k8v8_setup(G, dev):
    from knlp_b200 import ops
    dt = TDT[str(G["q_dtype"])]
    q = torch.from_numpy(G["query"]).to(dt).to(dev)
    k = torch.from_numpy(G["key"]).to(dt).to(dev)
    v = torch.from_numpy(G["value"]).to(dt).to(dev)
    slots = torch.from_numpy(G["slot_mapping"]).to(dev)
    bt = torch.from_numpy(G["block_table"]).to(dev)
    sl = torch.from_numpy(G["seq_lens"]).to(dev)
    nb, P = int(G["num_blocks"]), int(G["block_size"])
    hkv, d = int(G["num_kv_heads"]), int(G["head_size"])
    kc = torch.zeros(nb, P, hkv, d, dtype=torch.int8, device=dev)
    vc = torch.zeros(nb, P, hkv, d, dtype=torch.int8, device=dev)
    ks = torch.zeros(nb, P, hkv, d // 32, dtype=torch.float16, device=dev)
    vs = torch.zeros(nb, P, hkv, d // 32, dtype=torch.float16, device=dev)
    ops.reshape_and_cache_k_int8(k, kc, ks, slots)
    ops.reshape_and_cache_v_int8(v, vc, vs, slots)
    return q, kc, vc, ks, vs, bt, sl, hkv, d


@pytest.mark.gpu
@pytest.mark.parametrize("case", DECODE_CASES)
@pytest.mark.parametrize("generic", [False, True])
def test_k8v8_decode_golden(case, generic, cuda_device):
    from knlp_b200 import ops
    G, V8 = load_golden(case), load_golden("v8_modes")
    q, kc, vc, ks, vs, bt, sl, hkv, d = _k8v8_setup(G, cuda_device)
    ref = O.kint8_vint8_decode(G["query"], kc.cpu().numpy(), vc.cpu().numpy(), ks.cpu().numpy(),
                               vs.cpu().numpy(), G["block_table"], G["seq_lens"], hkv, d)
    out = ops.kint8_vint8_decode(q, kc, vc, ks, vs, bt, sl, hkv, d, out_dtype=torch.float32,
                                 force_generic=generic)
    err = np.abs(out.cpu().numpy() - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"max abs err {err.max():.3e}"
    # and, in the query dtype, the reference kernel's own output
    out_q = ops.kint8_vint8_decode(q, kc, vc, ks, vs, bt, sl, hkv, d, force_generic=generic)
    ulp = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[str(G["q_dtype"])]
    np.testing.assert_allclose(out_q.float().cpu().numpy(), V8[case + "_k8v8_out"], atol=ATOL,
                               rtol=RTOL + ulp)


@pytest.mark.gpu
@pytest.mark.parametrize("n_kv,n_rep", [(8, 4), (2, 8), (1, 4)])
def test_k8v8_decode_long_ragged(n_kv, n_rep, cuda_device):
    """Long, ragged, shuffled pages, several splits; every sequence compared."""
    from knlp_b200 import ops
    g = torch.Generator().manual_seed(31 + n_kv)
    lens = [2100, 517, 16, 0]
    P, d = 16, 128
    S, hq = len(lens), n_kv * n_rep
    max_blocks = max((L + P - 1) // P for L in lens) + 1
    nb = S * max_blocks + 5
    perm = torch.randperm(nb, generator=g)
    bt = torch.zeros(S, max_blocks, dtype=torch.int32)
    slots = []
    for s, L in enumerate(lens):
        bt[s] = perm[s * max_blocks:(s + 1) * max_blocks].to(torch.int32)
        slots += [int(bt[s, t // P]) * P + t % P for t in range(L)]
    toks = sum(lens)
    k = torch.randn(toks, n_kv, d, generator=g)
    v = torch.randn(toks, n_kv, d, generator=g) + 0.3
    k[:, :, 5] *= 10
    v[:, :, 100] *= 10
    q = torch.randn(S, hq, d, generator=g)
    dev = cuda_device
    kd, vd, qd = (t.to(torch.bfloat16).to(dev) for t in (k, v, q))
    kc = torch.zeros(nb, P, n_kv, d, dtype=torch.int8, device=dev)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(nb, P, n_kv, d // 32, dtype=torch.float16, device=dev)
    vs = torch.zeros_like(ks)
    sd = torch.tensor(slots, dtype=torch.int64, device=dev)
    ops.reshape_and_cache_k_int8(kd, kc, ks, sd)
    ops.reshape_and_cache_v_int8(vd, vc, vs, sd)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    ref = O.kint8_vint8_decode(qd.float().cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(),
                               ks.cpu().numpy(), vs.cpu().numpy(), bt.numpy(), np.array(lens),
                               n_kv, d)
    for kw in (dict(), dict(n_splits=1), dict(n_splits=5), dict(force_generic=True)):
        out = ops.kint8_vint8_decode(qd, kc, vc, ks, vs, bt.to(dev), sl, n_kv, d,
                                     out_dtype=torch.float32, max_seq_len=max(lens), **kw)
        err = np.abs(out.cpu().numpy() - ref)
        assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{kw}: max abs err {err.max():.3e}"
        assert np.all(out.cpu().numpy()[3] == 0)
