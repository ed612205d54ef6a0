"""The contiguous head-major symmetric INT4 cache of the reference's kernel benches
(scripts/v29_flash_bench.py:40-97): quantizer bit-exact against the reference's own
function (golden fixture made by running it), decode against its dequantize-then-SDPA."""

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3


def _close(out, ref, what):
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    err = np.abs(out - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{what}: max abs err {err.max():.3e}"


def test_quantize_and_pack_matches_reference_bits(cuda_device):
    from knlp_b200 import contiguous as C
    G = load_golden("contig_sym")
    k = torch.from_numpy(G["key"]).to(torch.float16).to(cuda_device)
    v = torch.from_numpy(G["value"]).to(torch.float16).to(cuda_device)
    kp, ks = C.quantize_and_pack_int4(k)
    vp, vs = C.quantize_and_pack_int4(v)
    assert kp.dtype == torch.uint8 and ks.dtype == torch.float16
    assert np.array_equal(kp.cpu().numpy(), G["k_packed"])
    assert np.array_equal(vp.cpu().numpy(), G["v_packed"])
    assert np.array_equal(ks.cpu().view(torch.int16).numpy().view(np.uint16), G["k_scales"])
    assert np.array_equal(vs.cpu().view(torch.int16).numpy().view(np.uint16), G["v_scales"])
    np.testing.assert_array_equal(C.dequant_int4(kp, ks).float().cpu().numpy(), G["k_dequant"])
    np.testing.assert_array_equal(C.dequant_int4(vp, vs).float().cpu().numpy(), G["v_dequant"])


@pytest.mark.parametrize("tokens", [96, 80, 37])
def test_decode_contiguous_vs_reference_pipeline(tokens, cuda_device):
    """96 and 80 tokens: pages of 16, tensor-core kernel; 37: strided view, generic kernel."""
    from knlp_b200 import contiguous as C
    G = load_golden("contig_sym")
    t = lambda a: torch.from_numpy(a).to(cuda_device)
    q = t(G["query"]).to(torch.float16)
    T = G["k_packed"].shape[2]
    kp, vp = t(G["k_packed"]), t(G["v_packed"])
    ks = t(G["k_scales"].view(np.int16)).view(torch.float16)
    vs = t(G["v_scales"].view(np.int16)).view(torch.float16)
    if tokens == T:
        ref = G["out"]
        out = C.fused_int4_decode_contiguous(q, kp, vp, ks, vs, out_dtype=torch.float32)
    else:
        # a shorter cache: the first tokens of every (batch, head), re-laid contiguously
        kp, vp, ks, vs = (x[:, :, :tokens].contiguous() for x in (kp, vp, ks, vs))
        n_rep = int(G["n_heads"]) // int(G["n_kv_heads"])
        kd = torch.from_numpy(G["k_dequant"])[:, :, :tokens].repeat_interleave(n_rep, dim=1)
        vd = torch.from_numpy(G["v_dequant"])[:, :, :tokens].repeat_interleave(n_rep, dim=1)
        ref = torch.nn.functional.scaled_dot_product_attention(
            torch.from_numpy(G["query"]), kd, vd, is_causal=False).numpy()
        out = C.fused_int4_decode_contiguous(q, kp, vp, ks, vs, out_dtype=torch.float32)
    assert out.shape == q.shape
    _close(out.cpu().numpy(), ref, f"contiguous decode, {tokens} tokens")
    # a prefix of the cache through seq_len
    part = C.fused_int4_decode_contiguous(q, kp, vp, ks, vs, seq_len=20, out_dtype=torch.float32)
    n_rep = int(G["n_heads"]) // int(G["n_kv_heads"])
    kd = torch.from_numpy(G["k_dequant"])[:, :, :20].repeat_interleave(n_rep, dim=1)
    vd = torch.from_numpy(G["v_dequant"])[:, :, :20].repeat_interleave(n_rep, dim=1)
    ref20 = torch.nn.functional.scaled_dot_product_attention(
        torch.from_numpy(G["query"]), kd, vd, is_causal=False).numpy()
    _close(part.cpu().numpy(), ref20, "contiguous decode, seq_len 20")
