"""Plugin surface without a GPU: the oracle's restatement of the reference quantizers
against vectors produced by the reference functions themselves
(tests/golden/make_golden.py --only-plugin), and the host logic of the backend classes."""
import dataclasses

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from conftest import load_golden

CASES = [(dt, D) for dt in ("f32", "f16", "bf16") for D in (64, 80)]


@pytest.mark.parametrize("dt,D", CASES)
def test_oracle_plugin_quantizers_bit_exact_vs_reference(dt, D):
    G = load_golden("plugin_quant")
    key = f"{dt}_d{D}"
    x = G[key + "_x"]
    rt = O.PLUGIN_ROUNDERS[dt]
    q8, s8 = O.plugin_quantize_int8_symmetric(x, rt)
    assert np.array_equal(q8, G[key + "_q8"]) and np.array_equal(s8, G[key + "_s8"])
    assert np.array_equal(O.plugin_dequantize_int8_symmetric(q8, s8), G[key + "_d8"])
    q4, s4 = O.plugin_quantize_int4_block(x, 32, rt)
    assert np.array_equal(q4, G[key + "_q4"]) and np.array_equal(s4, G[key + "_s4"])
    assert np.array_equal(O.plugin_dequantize_int4_block(q4, s4, 32), G[key + "_d4"])
    assert s4.shape[-1] == (D + 31) // 32 and s8.shape[-1] == 1


def test_rounders():
    a = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8], np.float32)
    assert np.array_equal(O.round_to_f16(a), a.astype(np.float16).astype(np.float32))
    b = torch.tensor(a).to(torch.bfloat16).float().numpy()
    assert np.array_equal(O.round_to_bf16(a), b)
    assert O.round_to_f16(np.float32(1e-8)) == 0.0  # the amax floor vanishes in fp16


def test_interface_matches_reference_names():
    from knlp_b200 import backends as B
    fields = [f.name for f in dataclasses.fields(B.V14StepStats)]
    assert fields == ["kv_kept", "kv_bytes_full", "kv_bytes_compressed", "kv_bytes_total",
                      "compress_ms", "decompress_ms", "gate_ms", "n_full", "n_compressed"]
    assert B.CompressionBackend.W_min == 1024 and B.CompressionBackend.W_sink == 4
    for name in ("name", "configure", "calibrate", "run_decode", "compression_ratio",
                 "description"):
        assert hasattr(B.CompressionBackend, name)
    with pytest.raises(TypeError):
        B.CompressionBackend()  # abstract
    assert B.get_backend("dense").name == "dense"
    assert B.get_backend("quant").name == "quant"
    assert B.get_backend("quant_int4").name == "quant_int4"
    with pytest.raises(ValueError):
        B.get_backend("lowrank")
    for fn in ("quantize_int8_symmetric", "dequantize_int8_symmetric", "quantize_int4_block",
               "dequantize_int4_block"):
        assert callable(getattr(B, fn))


def test_quantizers_refuse_cpu_tensors():
    from knlp_b200 import backends as B
    x = torch.randn(1, 2, 3, 64)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        B.quantize_int8_symmetric(x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        B.quantize_int4_block(x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        B.dequantize_int8_symmetric(torch.zeros(2, 4, dtype=torch.int8), torch.ones(2, 1))


def test_quant_backend_accounting_and_descriptions():
    from knlp_b200 import backends as B
    mc = dict(n_layers=4, n_kv_heads=2, head_dim=64)
    b = B.QuantBackend()
    b.configure(8192, mc, W_min=256, W_sink=4)
    assert (b.W_min, b.W_sink, b.default_bits, b.block_size) == (256, 4, 8, 32)
    assert not b.calibrated and b.compression_ratio() == 0.5
    assert b.description() == "quant (default=8bit)"
    # all layers at 8 bits: int8 payload + one fp16 scale per (k|v, head)
    b.calibrated, b.layer_bits = True, [8, 8, 8, 8]
    assert b._compressed_bytes(100) == int(100 * (2 * 2 * 64 * 1 + 2 * 2 * 2) * 4)
    assert b.compression_ratio() == 0.5
    # all at 4 bits: half a byte per element + an fp16 scale per block of 32
    b.layer_bits = [4, 4, 4, 4]
    assert b._compressed_bytes(100) == int(100 * (2 * 2 * 64 * 0.5 + 2 * 2 * (64 / 32) * 2) * 4)
    assert b.compression_ratio() == 0.25 and b.description() == "quant (4xINT4 + 0xINT8)"
    # mixed: the average bit width prices the payload, overhead as in the 8-bit branch
    b.layer_bits = [4, 8, 8, 8]
    assert b._compressed_bytes(10) == int(10 * (2 * 2 * 64 * (7 / 8) + 2 * 2 * 2) * 4)
    # a calibration survives configure()
    b.configure(4096, mc)
    assert b.calibrated and b.layer_bits == [4, 8, 8, 8]
    with pytest.raises(ValueError, match="too short"):
        B.QuantBackend._text_window(np.arange(10), 16, np.random.RandomState(0))
    w = B.QuantBackend._text_window(np.arange(1000), 16, np.random.RandomState(42))
    assert w.shape == (1, 16) and w.dtype == torch.int64
    assert int(w[0, 0]) == int(np.random.RandomState(42).randint(0, 984, size=1)[0])
