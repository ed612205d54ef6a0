"""Block sizes other than 16: powers of two above and below the 16-token tile (tensor-core
kernel, general loop) and a non-power-of-two (stride-generic kernel), write path included."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3


def _build(P, n_kv, n_rep, d, lens, dev, seed):
    from knlp_b200 import ops
    g = torch.Generator().manual_seed(seed)
    S, hq = len(lens), n_kv * n_rep
    max_blocks = max((L + P - 1) // P for L in lens) + 1
    nb = S * max_blocks + 3
    perm = torch.randperm(nb, generator=g)
    bt = torch.zeros(S, max_blocks, dtype=torch.int32)
    slots = []
    for s, L in enumerate(lens):
        bt[s] = perm[s * max_blocks:(s + 1) * max_blocks].to(torch.int32)
        slots += [int(bt[s, t // P]) * P + t % P for t in range(L)]
    toks = sum(lens)
    k = torch.randn(toks, n_kv, d, generator=g)
    v = torch.randn(toks, n_kv, d, generator=g) * 0.7 + 0.2
    k[:, :, 3] *= 10
    q = torch.randn(S, hq, d, generator=g)
    kd, vd, qd = (t.to(torch.bfloat16).to(dev) for t in (k, v, q))
    mk = lambda w, dt: torch.zeros(nb, P, n_kv, w, dtype=dt, device=dev)
    kc, vc = mk(d // 2, torch.uint8), mk(d // 2, torch.uint8)
    ks, vs, kz, vz = (mk(d // 32, torch.float16) for _ in range(4))
    sd = torch.tensor(slots, dtype=torch.int64, device=dev)
    ops.reshape_and_cache_int4(kd, vd, kc, vc, ks, vs, sd, kz, vz, asymmetric=True)
    # the write path against the oracle, bit for bit
    okc = np.zeros((nb, P, n_kv, d // 2), np.uint8); ovc = np.zeros_like(okc)
    oks = np.zeros((nb, P, n_kv, d // 32), np.float16)
    ovs, okz, ovz = np.zeros_like(oks), np.zeros_like(oks), np.zeros_like(oks)
    O.reshape_and_cache_int4(kd.float().cpu().numpy(), vd.float().cpu().numpy(), okc, ovc, oks,
                             ovs, np.array(slots), okz, ovz, asymmetric=True)
    assert np.array_equal(kc.cpu().numpy(), okc) and np.array_equal(vc.cpu().numpy(), ovc)
    assert np.array_equal(ks.cpu().numpy().view(np.uint16), oks.view(np.uint16))
    return qd, kc, vc, ks, vs, kz, vz, bt, okc, ovc, oks, ovs, okz, ovz


@pytest.mark.parametrize("P", [8, 32, 64, 48])
@pytest.mark.parametrize("n_kv,n_rep,d", [(8, 4, 128), (2, 4, 128), (4, 1, 64)])
def test_decode_other_block_sizes(P, n_kv, n_rep, d, cuda_device):
    from knlp_b200 import ops
    lens = [1500, 257, P, 1]
    qd, kc, vc, ks, vs, kz, vz, bt, okc, ovc, oks, ovs, okz, ovz = _build(
        P, n_kv, n_rep, d, lens, cuda_device, seed=900 + P + n_kv)
    ref = O.fused_int4_decode(qd.float().cpu().numpy(), okc, ovc, oks, ovs, bt.numpy(),
                              np.array(lens), n_kv, d, k_zeros=okz, v_zeros=ovz, asymmetric=True)
    sl = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    for kw in (dict(), dict(n_splits=1), dict(n_splits=4), dict(force_generic=True)):
        out = ops.fused_int4_decode(qd, kc, vc, ks, vs, bt.to(cuda_device), sl, n_kv, d,
                                    k_zeros=kz, v_zeros=vz, asymmetric=True,
                                    out_dtype=torch.float32, max_seq_len=max(lens), **kw)
        err = np.abs(out.cpu().numpy() - ref)
        assert np.all(err <= ATOL + RTOL * np.abs(ref)), f"P={P} {kw}: max abs err {err.max():.3e}"
