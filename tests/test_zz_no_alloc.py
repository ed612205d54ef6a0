"""knlp_b200_decode_noalloc: decode attention with the partials in the library's
fixed device array.  Called straight through the C ABI and compared with the
existing split-k + combine entry points on the same inputs.

The file name keeps this module last in collection order, so it runs after the
other GPU tests have used the device; it must also pass alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

ATOL, RTOL = 2e-3, 1e-3  # the decode parity tolerance of the other GPU tests

_MODE = {"int4_asym": 2, "int4_sym": 1, "int8": 3}
ERR_TOO_LARGE = -9
MAX_FLOATS = 8 << 20  # KNLP_NOALLOC_MAX_FLOATS


def _planes(w):
    from knlp_b200 import ops
    kp = ops._plane(w.key_cache, w.k_scales, w.k_zeros if w.k_mode == "int4_asym" else None,
                    _MODE[w.k_mode])
    vp = ops._plane(w.value_cache, w.v_scales, w.v_zeros if w.v_mode == "int4_asym" else None,
                    _MODE[w.v_mode])
    return kp, vp


def _noalloc(w, out, n_splits=0, out_dtype=None):
    """One raw C-ABI call on torch's current stream; returns the status code."""
    from knlp_b200 import _lib, ops, workloads
    lib = _lib.load()
    kp, vp = _planes(w)
    S, Hq, d = w.query.shape
    page = workloads.PAGE
    max_len = int(w.max_seq_len)  # what Workload.decode passes: same split boundaries
    with torch.cuda.device(w.query.device):
        return lib.knlp_b200_decode_noalloc(
            w.query.data_ptr(), ops._dt(w.query), ops._stride2(w.query), C.byref(kp), C.byref(vp),
            w.block_table.data_ptr(), w.block_table.stride(0), w.seq_lens.data_ptr(),
            int(w.key_cache.shape[0]), S, Hq, w.n_kv_heads, d, page, n_splits, max_len,
            out.data_ptr(), _lib.F32 if out_dtype is None else out_dtype, d,
            torch.cuda.current_stream(w.query.device).cuda_stream)


def _check(out, ref, what):
    out, ref = out.cpu().numpy(), ref.cpu().numpy()
    assert np.isfinite(out).all(), what
    np.testing.assert_allclose(out, ref, atol=ATOL, rtol=RTOL, err_msg=what)


@pytest.mark.gpu
def test_noalloc_matches_splitk_twice_in_a_row(cuda_device):
    from knlp_b200 import workloads
    # two shapes with different split counts and row counts, so that the second call
    # finds the first one's partials at other offsets of the shared array
    wa = workloads.build("noalloc_a", n_seqs=4, n_q_heads=32, n_kv_heads=8, head_dim=128,
                         seq_lens=[3000, 17, 0, 2049], seed=901, device=cuda_device,
                         shuffle_pages=True)
    wb = workloads.build("noalloc_b", n_seqs=2, n_q_heads=12, n_kv_heads=12, head_dim=64,
                         seq_lens=[1024, 700], seed=902, device=cuda_device, shuffle_pages=True,
                         q_dtype=torch.float32, k_mode="int4_sym", v_mode="int4_sym")
    ref_a = wa.decode(out_dtype=torch.float32, two_launches=True)
    ref_b = wb.decode(out_dtype=torch.float32, two_launches=True)
    torch.cuda.synchronize()

    out_a = torch.full_like(ref_a, float("nan"))
    out_b = torch.full_like(ref_b, float("nan"))
    held = torch.cuda.memory_allocated(cuda_device)
    assert _noalloc(wa, out_a) == 0            # first call on the device: looks the array up
    assert _noalloc(wb, out_b) == 0            # second call, straight after, other shape
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(cuda_device) == held
    _check(out_a, ref_a, "first call")
    _check(out_b, ref_b, "second call")

    # the same inputs again, with explicit split counts, over whatever the calls above left
    for n in (1, 3, 8):
        again = torch.full_like(ref_a, float("nan"))
        assert _noalloc(wa, again, n_splits=n) == 0
        torch.cuda.synchronize()
        _check(again, ref_a, f"repeat with {n} splits")
        # bit-identical to the same two kernels run through the workspace entry points
        assert torch.equal(again, wa.decode(out_dtype=torch.float32, n_splits=n,
                                            two_launches=True))


@pytest.mark.gpu
def test_noalloc_rejects_what_the_array_cannot_hold(cuda_device):
    from knlp_b200 import _lib, workloads
    w = workloads.build("noalloc_big", n_seqs=2, n_q_heads=32, n_kv_heads=8, head_dim=128,
                        seq_lens=[256, 100], seed=903, device=cuda_device)
    ref = w.decode(out_dtype=torch.float32, two_launches=True)
    per_split = 2 * 32 * (128 + 2)
    too_many = MAX_FLOATS // per_split + 1
    out = torch.full_like(ref, 7.0)
    rc = _noalloc(w, out, n_splits=too_many)
    torch.cuda.synchronize()
    assert rc == ERR_TOO_LARGE
    assert b"capacity" in _lib.load().knlp_b200_strerror(rc).lower() or \
        b"large" in _lib.load().knlp_b200_strerror(rc).lower()
    assert torch.all(out == 7.0)               # nothing was launched
    # an output type the merge would refuse is refused before anything is launched, too
    rc = _noalloc(w, out, n_splits=2, out_dtype=99)
    torch.cuda.synchronize()
    assert rc < 0 and torch.all(out == 7.0)
    # the largest count that fits is accepted and right
    assert _noalloc(w, out, n_splits=too_many - 1) == 0
    torch.cuda.synchronize()
    _check(out, ref, "largest split count that fits")
