"""Low-rank-V decode against the reference's own torch implementation
(pos_quant_v/kernel/vlowrank_kernel.py:166-174), fixtures tests/golden/lowrank.npz from
make_golden.py --only-lowrank.  CPU: the oracle is pinned.  GPU: knlp_b200.lowrank through
the C ABI."""

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import kv_oracle as O

CASES = ["gqa4_d128_bf16", "gqa8_d64_f16", "one_token_bf16", "gqa5_d128_f16"]
TDT = {"f16": torch.float16, "bf16": torch.bfloat16}


def _inputs(G, name):
    dt = TDT[str(G[name + "_dtype"])]
    bits = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(dt)
    return bits(G[name + "_q"]), bits(G[name + "_k"]), torch.from_numpy(G[name + "_proj"]), \
        torch.from_numpy(G[name + "_basis"])


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_lowrank(name):
    G = load_golden("lowrank")
    Q, K, proj, B = _inputs(G, name)
    o, za = O.lowrank_decode(Q.float().numpy(), K.float().numpy(), proj.numpy(), B.numpy())
    np.testing.assert_allclose(o, G[name + "_out"], rtol=2e-5, atol=2e-6)
    # an orthonormal basis: aggregating the coefficients and lifting equals dense attention
    # over the lifted values
    np.testing.assert_allclose(o, G[name + "_dense_of_lifted_v"], rtol=1e-4, atol=1e-5)
    assert za.shape == Q.shape[:2] + (32,)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_lowrank_decode_matches_reference(name, cuda_device):
    from knlp_b200 import lowrank
    G = load_golden("lowrank")
    Q, K, proj, B = (t.to(cuda_device) for t in _inputs(G, name))
    o, za = lowrank.lowrank_decode(Q, K, proj, B, return_coefficients=True)
    ref = G[name + "_out"]
    err = np.abs(o.cpu().numpy() - ref)
    assert np.all(err <= 2e-3 + 1e-3 * np.abs(ref)), f"max abs err {err.max():.3e}"
    _, za_ref = O.lowrank_decode(Q.float().cpu().numpy(), K.float().cpu().numpy(),
                                 proj.cpu().numpy(), B.cpu().numpy())
    np.testing.assert_allclose(za.cpu().numpy(), za_ref, rtol=1e-3, atol=2e-3)
    o2 = lowrank.lowrank_decode(Q, K, proj, B)  # the workspace is reused
    torch.testing.assert_close(o2, o, rtol=0, atol=0)


@pytest.mark.gpu
@pytest.mark.parametrize("dt,hkv,nq,T,dh", [(torch.bfloat16, 8, 4, 20000, 128),
                                            (torch.float16, 2, 8, 4097, 64),
                                            (torch.bfloat16, 1, 1, 63, 128)])
def test_lowrank_decode_many_splits_vs_oracle(dt, hkv, nq, T, dh, cuda_device):
    """Long contexts are cut into many splits (ragged last split, last tile partly masked)."""
    from knlp_b200 import lowrank
    g = torch.Generator().manual_seed(T + dh)
    Q = torch.randn(hkv, nq, dh, generator=g).to(dt)
    K = torch.randn(hkv, T, dh, generator=g).to(dt)
    proj = torch.randn(hkv, T, 32, generator=g)
    B = torch.linalg.qr(torch.randn(hkv, dh, 32, generator=g)).Q.contiguous()
    ref, _ = O.lowrank_decode(Q.float().numpy(), K.float().numpy(), proj.numpy(), B.numpy())
    o = lowrank.lowrank_decode(Q.to(cuda_device), K.to(cuda_device), proj.to(cuda_device),
                               B.to(cuda_device))
    err = np.abs(o.cpu().numpy() - ref)
    assert np.all(err <= 2e-3 + 1e-3 * np.abs(ref)), f"max abs err {err.max():.3e}"


@pytest.mark.gpu
def test_lowrank_decode_refuses_what_is_not_built(cuda_device):
    from knlp_b200 import lowrank
    Q = torch.zeros(1, 2, 128, dtype=torch.float16, device=cuda_device)
    K = torch.zeros(1, 8, 128, dtype=torch.float16, device=cuda_device)
    with pytest.raises(NotImplementedError):
        lowrank.lowrank_decode(Q, K, torch.zeros(1, 8, 16, device=cuda_device),
                               torch.zeros(1, 128, 16, device=cuda_device))
    with pytest.raises(TypeError):
        lowrank.lowrank_decode(Q.float(), K.float(), torch.zeros(1, 8, 32, device=cuda_device),
                               torch.zeros(1, 128, 32, device=cuda_device))
