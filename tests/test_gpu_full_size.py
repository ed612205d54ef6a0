"""The benchmark's full sizes (batch 32 x 131 072 tokens, 5.4 GB of packed KV; 1 Mi tokens
through the write path), checked through properties that do not need the whole oracle:

* sampled (sequence, kv head) pairs against the CPU oracle over their FULL 128K context;
* the tensor-core kernel against the stride-generic kernel (a different algorithm) everywhere;
* other split counts give the same attention; reruns are bit-identical;
* attention is linear in V: doubling the V scales and zero-points (exact in fp16) doubles the
  fp32 output, to 1e-4 (softmax weight x scale products in the fp16 subnormal range round
  differently after the doubling, nothing else does);
* the context cut in two segments, decoded separately and merged, equals the whole;
* write path: the 16-element kernel and the 4-element kernel fill 1 Mi tokens identically, and
  sampled rows equal the oracle's bytes.
"""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3


def _close(out, ref, what):
    out, ref = np.asarray(out, np.float64), np.asarray(ref, np.float64)
    err = np.abs(out - ref)
    assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"{what}: max abs err {err.max():.3e}"


def test_decode_at_full_size(cuda_device):
    from knlp_b200 import ops, shard, workloads
    w = workloads.config("llama8b_b32_128k", cuda_device)
    assert w.seq_lens_host == [131072] * 32 and w.n_kv_heads == 8 and w.head_dim == 128
    n_rep = w.n_q_heads // w.n_kv_heads
    out = w.decode(out_dtype=torch.float32)
    assert torch.isfinite(out).all()
    # The balanced kernel hands chunks out dynamically: the order of summation, and with it
    # the last bits, may differ between runs.  The fixed-split path is bitwise repeatable.
    _close(w.decode(out_dtype=torch.float32).cpu().numpy(), out.cpu().numpy(), "rerun")
    fixed = w.decode(out_dtype=torch.float32, two_launches=True)
    assert torch.equal(fixed, w.decode(out_dtype=torch.float32, two_launches=True))
    _close(fixed.cpu().numpy(), out.cpu().numpy(), "balanced vs fixed splits")

    # sampled rows against the oracle over the whole context
    pages = 131072 // 16
    for s, h in ((0, 0), (13, 5), (31, 7)):
        idx = w.block_table[s, :pages].long()
        take = lambda t: t[idx][:, :, h:h + 1].contiguous().cpu().numpy()
        ref = O.fused_int4_decode(
            w.query[s:s + 1, h * n_rep:(h + 1) * n_rep].float().cpu().numpy(),
            take(w.key_cache), take(w.value_cache), take(w.k_scales), take(w.v_scales),
            np.arange(pages, dtype=np.int32)[None], np.array([131072], np.int32), 1, w.head_dim,
            k_zeros=take(w.k_zeros), v_zeros=take(w.v_zeros), asymmetric=True)
        _close(out[s:s + 1, h * n_rep:(h + 1) * n_rep].cpu().numpy(), ref, f"oracle seq {s} head {h}")

    # a different algorithm, every row
    gen = w.decode(out_dtype=torch.float32, force_generic=True)
    _close(out.cpu().numpy(), gen.cpu().numpy(), "tensor-core vs generic kernel")
    # other split counts
    for n in (8, 64):
        _close(w.decode(out_dtype=torch.float32, n_splits=n).cpu().numpy(), out.cpu().numpy(),
               f"{n} splits")

    # linearity in V: scales and zero-points x 2 -> output x 2
    vs, vz = w.v_scales, w.v_zeros
    assert float(vs.abs().max()) < 3e4 and float(vz.abs().max()) < 3e4
    # (tight on the fixed-split path, whose order of summation does not change between the
    # two runs; the balanced path within the parity tolerance)
    w.v_scales, w.v_zeros = vs * 2, vz * 2
    doubled = w.decode(out_dtype=torch.float32)
    doubled_fixed = w.decode(out_dtype=torch.float32, two_launches=True)
    w.v_scales, w.v_zeros = vs, vz
    lin = (doubled_fixed - fixed * 2).abs().max().item()
    assert lin <= 1e-4 * max(1.0, out.abs().max().item()), f"V linearity off by {lin:.3e}"
    _close(doubled.cpu().numpy(), (out * 2).cpu().numpy(), "V linearity, balanced path")

    # two context segments decoded on their own and merged
    kp = ops._plane(w.key_cache, w.k_scales, w.k_zeros, ops._lib.KV_INT4_ASYM)
    vp = ops._plane(w.value_cache, w.v_scales, w.v_zeros, ops._lib.KV_INT4_ASYM)
    packed = []
    for r in range(2):
        a, b = shard.context_shard(131072, 2, r, 16)
        bt = w.block_table[:, a // 16:(b + 15) // 16].contiguous()
        lens = torch.full((32,), b - a, dtype=torch.int32, device=cuda_device)
        pm, pl, po = ops.decode_partials(w.query, kp, vp, w.key_cache.shape[0], bt, lens,
                                         w.n_kv_heads, w.head_dim, 16, max_seq_len=b - a)
        packed.append(ops.combine_to_packed(pm, pl, po))
    merged = ops.combine_packed(torch.stack(packed))
    _close(merged.float().cpu().numpy(), out.cpu().numpy(), "two context segments")


def test_write_path_at_full_size(cuda_device):
    from knlp_b200 import ops
    n, h, d, P = 1 << 20, 8, 128, 16
    g = torch.Generator(device=cuda_device).manual_seed(5)
    # one spare element in front: the view that starts there is 2-byte aligned only, which
    # takes the 4-elements-per-lane kernel; the copy of it is aligned and takes the wide one
    buf_k = torch.empty(n * h * d + 1, device=cuda_device, dtype=torch.bfloat16)
    buf_v = torch.empty(n * h * d + 1, device=cuda_device, dtype=torch.bfloat16)
    buf_k[1:].normal_(generator=g)
    buf_v[1:].normal_(generator=g)
    k_odd, v_odd = buf_k[1:].view(n, h, d), buf_v[1:].view(n, h, d)
    k_odd[:, :, 9] *= 11
    k, v = k_odd.clone(), v_odd.clone()
    assert k.data_ptr() % 16 == 0 and k_odd.data_ptr() % 16 != 0
    slots = torch.randperm(n, device=cuda_device, generator=g).to(torch.int64)
    nb = n // P
    sample = torch.randperm(n, device=cuda_device, generator=g)[:512]

    def caches(width, dtype):
        return (torch.zeros(nb, P, h, width, device=cuda_device, dtype=dtype),
                torch.zeros(nb, P, h, width, device=cuda_device, dtype=dtype))

    def scales():
        return tuple(torch.zeros(nb, P, h, d // 32, device=cuda_device, dtype=torch.float16)
                     for _ in range(4))

    for asym in (True, False):
        res = []
        for kk, vv in ((k, v), (k_odd, v_odd)):
            kc, vc = caches(d // 2, torch.uint8)
            ks, vs, kz, vz = scales()
            ops.reshape_and_cache_int4(kk, vv, kc, vc, ks, vs, slots, kz if asym else None,
                                       vz if asym else None, asymmetric=asym)
            res.append((kc, vc, ks, vs, kz, vz))
        for a, b in zip(*res):
            assert torch.equal(a, b), "wide and narrow kernels differ"
        # sampled tokens against the oracle
        kc, vc, ks, vs, kz, vz = res[0]
        okc = np.zeros((len(sample) // P, P, h, d // 2), np.uint8); ovc = np.zeros_like(okc)
        oks = np.zeros((len(sample) // P, P, h, d // 32), np.float16)
        ovs, okz, ovz = np.zeros_like(oks), np.zeros_like(oks), np.zeros_like(oks)
        O.reshape_and_cache_int4(k[sample].float().cpu().numpy(), v[sample].float().cpu().numpy(),
                                 okc, ovc, oks, ovs, np.arange(len(sample)),
                                 okz if asym else None, ovz if asym else None, asymmetric=asym)
        sl = slots[sample]
        rows = lambda t: t.view(nb * P, h, -1)[sl].cpu().numpy()
        assert np.array_equal(rows(kc), okc.reshape(len(sample), h, -1))
        assert np.array_equal(rows(vc), ovc.reshape(len(sample), h, -1))
        assert np.array_equal(rows(ks).view(np.uint16), oks.reshape(len(sample), h, -1).view(np.uint16))
        assert np.array_equal(rows(vs).view(np.uint16), ovs.reshape(len(sample), h, -1).view(np.uint16))
        del res, kc, vc, ks, vs, kz, vz
        torch.cuda.empty_cache()

    # INT8 K and V: both kernels over the whole cache, sampled rows against the oracle
    res = []
    for kk, vv in ((k, v), (k_odd, v_odd)):
        kc, vc = caches(d, torch.int8)
        ks, vs, _, _ = scales()
        ops.reshape_and_cache_k_int8(kk, kc, ks, slots)
        ops.reshape_and_cache_v_int8(vv, vc, vs, slots)
        res.append((kc, vc, ks, vs))
    for a, b in zip(*res):
        assert torch.equal(a, b), "wide and narrow INT8 kernels differ"
    kc, vc, ks, vs = res[0]
    okc = np.zeros((len(sample) // P, P, h, d), np.int8)
    oks = np.zeros((len(sample) // P, P, h, d // 32), np.float16)
    O.reshape_and_cache_k_int8(k[sample].float().cpu().numpy(), okc, oks, np.arange(len(sample)))
    sl = slots[sample]
    rows = lambda t: t.view(nb * P, h, -1)[sl].cpu().numpy()
    assert np.array_equal(rows(kc), okc.reshape(len(sample), h, -1))
    assert np.array_equal(rows(ks).view(np.uint16), oks.reshape(len(sample), h, -1).view(np.uint16))
