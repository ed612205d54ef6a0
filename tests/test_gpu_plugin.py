"""Plugin surface on the GPU: the CUDA quantizers against vectors produced by the
reference's own functions, and QuantBackend.run_decode over a small random GPT-2."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from conftest import load_golden

pytestmark = pytest.mark.gpu

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
CASES = [(dt, D) for dt in ("f32", "f16", "bf16") for D in (64, 80)]


@pytest.mark.parametrize("dt,D", CASES)
def test_plugin_quantizers_bit_exact_vs_reference(dt, D, cuda_device):
    from knlp_b200 import backends as B
    G = load_golden("plugin_quant")
    key = f"{dt}_d{D}"
    x = torch.from_numpy(G[key + "_x"]).to(TORCH_DT[dt]).to(cuda_device)
    q8, s8 = B.quantize_int8_symmetric(x)
    assert q8.dtype == torch.int8 and s8.dtype == x.dtype and s8.shape == x.shape[:-1] + (1,)
    assert np.array_equal(q8.cpu().numpy(), G[key + "_q8"])
    assert np.array_equal(s8.float().cpu().numpy(), G[key + "_s8"])
    d8 = B.dequantize_int8_symmetric(q8, s8)
    assert d8.dtype == torch.float32 and np.array_equal(d8.cpu().numpy(), G[key + "_d8"])
    q4, s4 = B.quantize_int4_block(x, 32)
    assert s4.shape == x.shape[:-1] + ((D + 31) // 32,)
    assert np.array_equal(q4.cpu().numpy(), G[key + "_q4"])
    assert np.array_equal(s4.float().cpu().numpy(), G[key + "_s4"])
    assert np.array_equal(B.dequantize_int4_block(q4, s4, 32).cpu().numpy(), G[key + "_d4"])


def test_plugin_quantizers_large_random_vs_oracle(cuda_device):
    from knlp_b200 import backends as B
    g = torch.Generator().manual_seed(77)
    x32 = torch.randn(2, 8, 257, 128, generator=g) * torch.rand(2, 8, 257, 1, generator=g) * 20
    for dt in ("f32", "f16", "bf16"):
        x = x32.to(TORCH_DT[dt]).to(cuda_device)
        xn = x.float().cpu().numpy()
        rt = O.PLUGIN_ROUNDERS[dt]
        q8, s8 = B.quantize_int8_symmetric(x[:, :, ::2])  # a non-contiguous view
        rq8, rs8 = O.plugin_quantize_int8_symmetric(xn[:, :, ::2], rt)
        assert np.array_equal(q8.cpu().numpy(), rq8)
        assert np.array_equal(s8.float().cpu().numpy(), rs8)
        q4, s4 = B.quantize_int4_block(x, 32)
        rq4, rs4 = O.plugin_quantize_int4_block(xn, 32, rt)
        assert np.array_equal(q4.cpu().numpy(), rq4)
        assert np.array_equal(s4.float().cpu().numpy(), rs4)
        # block sizes other than 32 and empty tensors
        q, s = B.quantize_int4_block(x[:, :, :5], 16)
        rq, rs = O.plugin_quantize_int4_block(xn[:, :, :5], 16, rt)
        assert np.array_equal(q.cpu().numpy(), rq) and np.array_equal(s.float().cpu().numpy(), rs)
        q, s = B.quantize_int8_symmetric(x[:, :, :0])
        assert q.shape == (2, 8, 0, 128) and s.shape == (2, 8, 0, 1)


def test_zero_row_in_fp16_is_defined(cuda_device):
    """The reference divides 0 by 0 here (its 1e-8 floor rounds to 0 in fp16) and its NaN
    becomes code 0 in the int8 conversion; the kernel gives scale 0 and code 0 as well."""
    from knlp_b200 import backends as B
    x = torch.zeros(1, 1, 2, 64, dtype=torch.float16, device=cuda_device)
    x[0, 0, 1] = 1.0
    q, s = B.quantize_int8_symmetric(x)
    assert float(s[0, 0, 0, 0]) == 0.0 and int(q[0, 0, 0].abs().max()) == 0
    assert int(q[0, 0, 1, 0]) == 127


def _tiny_gpt2(device):
    from transformers import GPT2Config, GPT2LMHeadModel
    cfg = GPT2Config(n_layer=3, n_head=4, n_embd=128, vocab_size=300, n_positions=512)
    torch.manual_seed(11)
    model = GPT2LMHeadModel(cfg).eval().to(device)
    mc = dict(n_layers=3, n_kv_heads=4, head_dim=32)
    return model, mc


@pytest.mark.parametrize("bits", [8, 4])
def test_quant_backend_run_decode_matches_oracle_cache(bits, cuda_device):
    """run_decode with the CUDA quantizers against the same decode over a cache whose far
    segment was quantized and dequantized by the oracle on the CPU."""
    from transformers.cache_utils import DynamicCache
    from knlp_b200 import backends as B
    model, mc = _tiny_gpt2(cuda_device)
    g = torch.Generator().manual_seed(5)
    prefix = torch.randint(0, 300, (1, 96), generator=g).to(cuda_device)
    cont = torch.randint(0, 300, (1, 6), generator=g).to(cuda_device)

    b = B.get_backend("quant")
    b.configure(96, mc, W_min=32, W_sink=4)
    b.calibrated, b.layer_bits = True, [bits] * 3  # skip calibrate(): fixed widths
    logits, stats = b.run_decode(model, prefix, cont, str(cuda_device), 512)
    assert logits.shape == (1, 7, 300) and len(stats) == 6
    assert stats[0].n_compressed == 96 - 32 - 4 and stats[0].n_full == 32 + 4 + 1
    assert stats[0].compress_ms > 0 and stats[1].compress_ms == 0
    assert stats[0].kv_bytes_compressed == b._compressed_bytes(60)
    assert stats[-1].kv_kept == 96 + 6

    # the same with the oracle's quantizers on the far segment [4, 64)
    with torch.no_grad():
        out = model(prefix, use_cache=True)
        past = out.past_key_values
        ref_logits = [out.logits[:, -1:, :]]
        cache = DynamicCache()
        for li in range(3):
            kv = []
            for t in (past.layers[li].keys, past.layers[li].values):
                far = t[:, :, 4:64, :].float().cpu().numpy()
                if bits == 8:
                    q, s = O.plugin_quantize_int8_symmetric(far)
                    hat = O.plugin_dequantize_int8_symmetric(q, s)
                else:
                    q, s = O.plugin_quantize_int4_block(far, 32)
                    hat = O.plugin_dequantize_int4_block(q, s, 32)
                hat = torch.from_numpy(hat).to(t.dtype).to(cuda_device)
                kv.append(torch.cat([t[:, :, :4], hat, t[:, :, 64:]], dim=2))
            cache.update(kv[0], kv[1], li)
        pos = 96
        for step in range(6):
            out = model(cont[:, step:step + 1], past_key_values=cache, use_cache=True,
                        position_ids=torch.tensor([[pos]], device=cuda_device))
            cache = out.past_key_values
            ref_logits.append(out.logits)
            pos += 1
    ref = torch.cat(ref_logits, dim=1)
    assert torch.allclose(logits, ref, atol=1e-5, rtol=1e-5)

    # and the dense control differs from it (the quantization is really applied)
    d = B.get_backend("dense")
    d.configure(96, mc)
    dl, ds = d.run_decode(model, prefix, cont, str(cuda_device), 512)
    assert ds[0].kv_bytes_total == 97 * 2 * 4 * 32 * 2 * 3
    assert (dl - logits).abs().max() > 1e-4


def test_quant_backend_calibrate_picks_bits(cuda_device):
    from knlp_b200 import backends as B
    model, mc = _tiny_gpt2(cuda_device)
    tokens = np.random.RandomState(3).randint(0, 300, size=4000)
    b = B.get_backend("quant")
    b.configure(128, mc, W_min=32)
    b.calibrate(model, tokens, 128, str(cuda_device), mc)
    assert b.calibrated and len(b.layer_bits) == 3 and set(b.layer_bits) <= {4, 8}
    f = B.get_backend("quant_int4")
    f.configure(128, mc, W_min=32)
    f.calibrate(model, tokens, 128, str(cuda_device), mc)
    assert f.layer_bits == [4, 4, 4] and f.compression_ratio() == 0.25


@pytest.mark.parametrize("bits,hd", [(4, 32), (8, 32), (4, 64)])
def test_packed_backend_run_decode_matches_oracle_cache(bits, hd, cuda_device):
    """quant_packed: the far segment lives in a REAL packed cache read by the decode kernel
    inside the model's attention.  Against the same decode over a float cache whose far
    segment the kv oracle quantized (INT4 asymmetric / INT8, group 32) and dequantized on
    the CPU: the logits must agree to the precision of the attention path."""
    from transformers import GPT2Config, GPT2LMHeadModel
    from transformers.cache_utils import DynamicCache
    from knlp_b200 import backends as B
    from oracle import kv_oracle as KO
    n_head = 4
    cfg = GPT2Config(n_layer=3, n_head=n_head, n_embd=n_head * hd, vocab_size=300, n_positions=512)
    torch.manual_seed(11)
    model = GPT2LMHeadModel(cfg).eval().to(cuda_device)
    mc = dict(n_layers=3, n_kv_heads=n_head, head_dim=hd)
    g = torch.Generator().manual_seed(5)
    prefix = torch.randint(0, 300, (1, 120), generator=g).to(cuda_device)
    cont = torch.randint(0, 300, (1, 6), generator=g).to(cuda_device)
    W_min, W_sink, L = 32, 4, 120
    far_end = L - W_min

    b = B.get_backend("quant_packed")
    b.configure(L, mc, W_min=W_min, W_sink=W_sink)
    b.calibrated, b.layer_bits = True, [bits] * 3
    logits, stats = b.run_decode(model, prefix, cont, str(cuda_device), 512)
    assert logits.shape == (1, 7, 300) and len(stats) == 6
    n_far = far_end - W_sink
    assert stats[0].n_compressed == n_far and stats[0].n_full == W_min + W_sink + 1
    # real bytes: per (token, kv head) 2 x (hd/2 + 4 hd/32) for INT4 asym, 2 x (hd + 2 hd/32) INT8
    per_tok = n_head * (2 * (hd // 2 + 4 * hd // 32) if bits == 4 else 2 * (hd + 2 * hd // 32))
    assert stats[0].kv_bytes_compressed == n_far * per_tok * 3
    assert model.config._attn_implementation != "knlp_b200_packed"  # restored

    with torch.no_grad():
        out = model(prefix, use_cache=True)
        past = out.past_key_values
        ref_logits = [out.logits[:, -1:, :]]
        cache = DynamicCache()
        for li in range(3):
            kv = []
            for t in (past.layers[li].keys, past.layers[li].values):
                far = t[0, :, W_sink:far_end, :].permute(1, 0, 2).float().cpu().numpy()  # [T, H, D]
                if bits == 4:
                    packed, sc, zp = KO.quant_int4_asym(far)
                    hat = KO.dequant_int4(packed, sc, zp)
                else:
                    codes, sc = KO.quant_int8_group(far)
                    hat = KO.dequant_int8(codes, sc)
                hat = torch.from_numpy(np.ascontiguousarray(hat)).permute(1, 0, 2)[None]
                hat = hat.to(t.dtype).to(cuda_device)
                kv.append(torch.cat([t[:, :, :W_sink], hat, t[:, :, far_end:]], dim=2))
            cache.update(kv[0], kv[1], li)
        pos = L
        for step in range(6):
            out = model(cont[:, step:step + 1], past_key_values=cache, use_cache=True,
                        position_ids=torch.tensor([[pos]], device=cuda_device))
            cache = out.past_key_values
            ref_logits.append(out.logits)
            pos += 1
    ref = torch.cat(ref_logits, dim=1)
    assert torch.allclose(logits, ref, atol=2e-3, rtol=1e-3), (logits - ref).abs().max()

    d = B.get_backend("dense")
    d.configure(L, mc)
    dl, _ = d.run_decode(model, prefix, cont, str(cuda_device), 512)
    assert (dl - logits).abs().max() > 1e-4  # the quantization is really applied
