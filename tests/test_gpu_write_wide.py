"""Write path at every head_dim the 16-elements-per-lane kernel takes (32 ... 512) and one it
does not (96: 4-elements-per-lane kernel), all quantizers, bit for bit against the oracle.
Row counts that do not fill the last warp, padding tokens, ties at .5 and saturating values."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu
TDT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _bits(t):
    return t.contiguous().cpu().numpy().view(np.uint16)


def _zeros_equal(a, b):
    # +0 and -0 zero-points are the same number
    return np.array_equal(np.where(a == 0x8000, 0, a), np.where(b == 0x8000, 0, b))


def _inputs(n, h, d, dt, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(n, h, d, generator=g)
    v = torch.randn(n, h, d, generator=g) * 0.5 + 0.2
    k[:, :, 5] *= 12                    # an outlier channel: the clip of the symmetric mode acts
    v[:, :, d - 3] *= 9
    # rows built to land on rounding ties and on the clamps: multiples of amax / 14 and / 254
    lin = torch.arange(d, dtype=torch.float32) - d / 2
    k[1, 0] = lin / 14 * 7
    v[1, 0] = lin / 30 * 15
    k[2, 0] = lin / 254 * 127
    k[3, 0] = 0                         # all-zero row: the 1e-8 floor of the range
    v[3, 0] = 3.25                      # constant row: zero range, asymmetric
    return k.to(TDT[dt]), v.to(TDT[dt])


@pytest.mark.parametrize("dt", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("d", [32, 64, 128, 256, 512, 96])
def test_write_path_head_dims(d, dt, cuda_device):
    from knlp_b200 import ops
    n, h, P = 203, 3, 16
    nb = (n + P - 1) // P + 1
    k, v = _inputs(n, h, d, dt, seed=40 + d)
    g = torch.Generator().manual_seed(d)
    slots = torch.randperm(nb * P, generator=g)[:n].to(torch.int64)
    slots[::31] = -1
    kd, vd, sd = k.to(cuda_device), v.to(cuda_device), slots.to(cuda_device)
    kf, vf, sn = k.float().numpy(), v.float().numpy(), slots.numpy()

    def dev(w, t):
        return torch.zeros(nb, P, h, w, dtype=t, device=cuda_device)

    def host(w, t):
        return np.zeros((nb, P, h, w), t)

    for asym, clip in ((True, 0.0), (False, 0.0), (False, O.OUTLIER_CLIP_RATIO), (False, 2.5)):
        kc, vc = dev(d // 2, torch.uint8), dev(d // 2, torch.uint8)
        ks, vs, kz, vz = (dev(d // 32, torch.float16) for _ in range(4))
        okc, ovc = host(d // 2, np.uint8), host(d // 2, np.uint8)
        oks, ovs, okz, ovz = (host(d // 32, np.float16) for _ in range(4))
        if asym:
            ops.reshape_and_cache_int4(kd, vd, kc, vc, ks, vs, sd, kz, vz, asymmetric=True)
            O.reshape_and_cache_int4(kf, vf, okc, ovc, oks, ovs, sn, okz, ovz, asymmetric=True)
            assert _zeros_equal(_bits(kz), okz.view(np.uint16))
            assert _zeros_equal(_bits(vz), ovz.view(np.uint16))
        else:
            ops.reshape_and_cache_int4(kd, vd, kc, vc, ks, vs, sd, asymmetric=False,
                                       clip_ratio=clip)
            O.reshape_and_cache_int4(kf, vf, okc, ovc, oks, ovs, sn, asymmetric=False,
                                     clip_ratio=clip)
        what = f"d={d} {dt} asym={asym} clip={clip}"
        assert np.array_equal(kc.cpu().numpy(), okc), what
        assert np.array_equal(vc.cpu().numpy(), ovc), what
        assert np.array_equal(_bits(ks), oks.view(np.uint16)), what
        assert np.array_equal(_bits(vs), ovs.view(np.uint16)), what

    kc8, vc8 = dev(d, torch.int8), dev(d, torch.int8)
    ks, vs = dev(d // 32, torch.float16), dev(d // 32, torch.float16)
    ops.reshape_and_cache_k_int8(kd, kc8, ks, sd)
    ops.reshape_and_cache_v_int8(vd, vc8, vs, sd)
    okc8, ovc8 = host(d, np.int8), host(d, np.int8)
    oks, ovs = host(d // 32, np.float16), host(d // 32, np.float16)
    O.reshape_and_cache_k_int8(kf, okc8, oks, sn)
    O.reshape_and_cache_v_int8(vf, ovc8, ovs, sn)
    assert np.array_equal(kc8.cpu().numpy(), okc8) and np.array_equal(vc8.cpu().numpy(), ovc8)
    assert np.array_equal(_bits(ks), oks.view(np.uint16))
    assert np.array_equal(_bits(vs), ovs.view(np.uint16))

    ovc, ovs, ovz = host(d // 2, np.uint8), host(d // 32, np.float16), host(d // 32, np.float16)
    vc, vs, vz = dev(d // 2, torch.uint8), dev(d // 32, torch.float16), dev(d // 32, torch.float16)
    ops.reshape_and_cache_v_only_int4(vd, vc, vs, sd, vz, asymmetric=True)
    O.reshape_and_cache_v_only_int4(vf, ovc, ovs, sn, ovz, asymmetric=True)
    assert np.array_equal(vc.cpu().numpy(), ovc) and np.array_equal(_bits(vs), ovs.view(np.uint16))
