"""Cache shapes and byte accounting of knlp_b200.cache against the reference's formulae
(fused-quant/fused_int4.v0.1.0.py:2123-2158 shape, :2451-2470 bytes per block)."""

import pytest
import torch

from knlp_b200 import cache as KC


def test_kv_cache_shape():
    assert KC.get_kv_cache_shape(100, 16, 8, 128) == (2, 100, 16, 8, 128)
    assert KC.get_kv_cache_shape(7, 32, 2, 64, replace_cache=True) == (1, 7, 32, 2, 64)


@pytest.mark.parametrize("kp,vp,asym", [("int4", "int4", True), ("int4", "int4", False),
                                        ("int8", "int4", True), ("int8", "int8", False),
                                        ("fp16", "int4", True), ("fp16", "int8", False)])
def test_bytes_per_block_match_the_allocation(kp, vp, asym):
    bs, h, d = 16, 8, 128
    c = KC.PackedKVCache(h, d, kp, vp, asym)
    c.ensure(5, bs, "cpu")
    assert c.actual_bytes_per_block() == c.expected_bytes_per_block()
    # the figures the benchmark configurations quote, per (token, kv head)
    per_tok_head = c.expected_bytes_per_block() / (bs * h)
    want = {("int4", "int4", True): 160, ("int4", "int4", False): 144, ("int8", "int4", True): 216,
            ("int8", "int8", False): 272, ("fp16", "int4", True): 80, ("fp16", "int8", False): 136}
    assert per_tok_head == want[(kp, vp, asym)]
    # growing re-allocates, shrinking does not
    old = c.value_cache
    c.ensure(3, bs, "cpu")
    assert c.value_cache is old
    c.ensure(9, bs, "cpu")
    assert c.value_cache.shape[0] == 9


def test_bad_arguments():
    with pytest.raises(ValueError):
        KC.PackedKVCache(8, 100)
    with pytest.raises(ValueError):
        KC.PackedKVCache(8, 128, "int3", "int4")
    with pytest.raises(ValueError):
        KC.shadow_bytes_per_block(16, 8, 128, "int4", "fp16", False)


def test_backend_facade_and_metadata_builder():
    """Names and answers of the reference's backend class (:2096-2176) and the builder's
    field-for-field hand-over (:2241-2251)."""
    from types import SimpleNamespace
    import torch
    from knlp_b200 import cache as C
    B = C.AttentionBackend
    assert B.get_name() == "FUSED_INT4" and B.get_builder_cls() is C.AttentionMetadataBuilder
    assert B.get_cache_cls() is C.PackedKVCache
    assert B.supports_kv_cache_dtype(None) and B.supports_kv_cache_dtype("int4_fused")
    assert not B.supports_kv_cache_dtype("fp8")
    assert B.supports_head_size(128) and B.supports_head_size(96)
    assert not B.supports_head_size(80) and not B.supports_head_size(0)
    assert B.get_kv_cache_shape(10, 16, 8, 128) == (2, 10, 16, 8, 128)
    assert torch.bfloat16 in B.supported_dtypes and not B.forward_includes_kv_cache_update
    common = SimpleNamespace(num_actual_tokens=3, max_query_len=1,
                             query_start_loc=torch.arange(4, dtype=torch.int32), max_seq_len=77,
                             seq_lens=torch.tensor([5, 77, 20], dtype=torch.int32),
                             block_table_tensor=torch.zeros(3, 5, dtype=torch.int32),
                             slot_mapping=torch.tensor([4, 76, 19]), num_reqs=3)
    meta = C.AttentionMetadataBuilder(16, 8, 128).build(0, common)
    assert isinstance(meta, C.AttentionMetadata)
    assert meta.max_seq_len == 77 and meta.num_actual_tokens == 3 and meta.max_query_len == 1
    assert meta.seq_lens is common.seq_lens and meta.block_table is common.block_table_tensor
    assert meta.slot_mapping is common.slot_mapping and meta.query_start_loc is common.query_start_loc
