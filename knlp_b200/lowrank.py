"""Low-rank-V decode attention.

Host-side mirror of mcgrof/knlp's ``pos_quant_v/kernel/vlowrank_kernel.py``:

    lowrank_decode      :139-156   o = B (sum_i softmax(q.k_i)_i proj_i): scores against the
                                   full K, values aggregated in rank r, lifted once
                                   (kernel _lowrank_decode :25-75)

The value side is stored as coefficients ``proj_i = B^T v_i`` (rank r = 32 against a head
dimension of 128) with a per-head basis ``B``; the kernel reads K and the coefficients, not
V.  Same tensors and result as the reference function; the kernels are this library's
(``knlp_b200_lowrank_decode``: tensor-core scores over the unquantized K tile, the r-wide
accumulation on the CUDA cores, the lift inside the second launch).
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib, ops

_workspaces = {}  # (device index, stream) -> float workspace


def lowrank_decode(Q: torch.Tensor, K: torch.Tensor, proj: torch.Tensor, Bbasis: torch.Tensor,
                   BLOCK_T: int = 128, return_coefficients: bool = False):
    """Q [Hkv, nq, dh] and K [Hkv, T, dh] fp16 / bf16 (one dtype), proj [Hkv, T, r] fp32,
    Bbasis [Hkv, dh, r] fp32 -> o [Hkv, nq, dh] fp32 (``return_coefficients``: also za
    [Hkv, nq, r], the aggregate before the lift, which is what the reference's kernel
    writes).  ``BLOCK_T`` is the reference's tuning hint; ignored."""
    dev = ops._need_cuda(Q, K, proj, Bbasis)
    Hkv, nq, dh = Q.shape
    T, r = K.shape[1], proj.shape[2]
    if K.shape != (Hkv, T, dh) or proj.shape != (Hkv, T, r) or Bbasis.shape != (Hkv, dh, r):
        raise ValueError("expected Q [Hkv,nq,dh], K [Hkv,T,dh], proj [Hkv,T,r], Bbasis [Hkv,dh,r]")
    if Q.dtype != K.dtype or Q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("Q and K must both be float16 or both bfloat16")
    if proj.dtype != torch.float32 or Bbasis.dtype != torch.float32:
        raise TypeError("proj and Bbasis must be float32")
    if r != 32 or dh not in (64, 128) or nq > 8:
        raise NotImplementedError("built for rank 32, head_dim 64 / 128, at most 8 queries per head")
    if T == 0:  # no token to attend to
        o = torch.zeros((Hkv, nq, dh), dtype=torch.float32, device=dev)
        return (o, torch.zeros((Hkv, nq, r), dtype=torch.float32, device=dev)) \
            if return_coefficients else o
    Q, K, proj, Bbasis = (t if t.is_contiguous() else t.contiguous() for t in (Q, K, proj, Bbasis))
    lib = _lib.load()
    need = C.c_int64(0)
    with ops._on(dev):
        _lib.check(lib.knlp_b200_lowrank_decode_workspace(Hkv, nq, T, C.byref(need)),
                   "knlp_b200_lowrank_decode_workspace")
        key = (dev.index, ops._stream(dev))
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < need.value:
            ws = _workspaces[key] = torch.empty(max(need.value, 1 << 18), dtype=torch.float32,
                                                device=dev)
        out = torch.empty((Hkv, nq, dh), dtype=torch.float32, device=dev)
        za = torch.empty((Hkv, nq, r), dtype=torch.float32, device=dev) if return_coefficients else None
        rc = lib.knlp_b200_lowrank_decode(
            Q.data_ptr(), K.data_ptr(), ops._dt(Q), proj.data_ptr(), Bbasis.data_ptr(), Hkv, nq, T,
            dh, r, ws.data_ptr(), ws.numel(), za.data_ptr() if za is not None else None,
            out.data_ptr(), ops._stream(dev))
    _lib.check(rc, "knlp_b200_lowrank_decode")
    return (out, za) if return_coefficients else out
