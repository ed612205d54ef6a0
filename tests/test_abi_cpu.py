"""CPU checks of the C-ABI library: it loads, exports every function that
include/knlp_b200.h declares, and rejects bad arguments on the host with the
documented status codes (no kernel is launched in this file)."""

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from knlp_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "knlp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(knlp_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from knlp_b200 import _lib
    names = declared_functions()
    assert names, "no declarations parsed"
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.SYMBOLS), "python binding list and header disagree"


def test_abi_version_and_strerror(lib):
    assert lib.knlp_b200_abi_version() == 2
    assert lib.knlp_b200_strerror(0) == b"ok"
    for code in range(-9, 0):
        assert len(lib.knlp_b200_strerror(code)) > 3


def test_argument_errors_are_reported_on_the_host(lib):
    from knlp_b200 import _lib
    null = None
    # NULL query
    rc = lib.knlp_b200_decode_splitk(null, 0, null, null, null, null, 0, null, 1, 1, 4, 4, 64, 16,
                                     1, 16, null, null, null, 0, null)
    assert rc == -1
    # bad dtype
    st2 = (C.c_int64 * 2)(64, 64)
    buf = C.create_string_buffer(64)
    p = C.cast(buf, C.c_void_p)
    rc = lib.knlp_b200_decode_splitk(p, 7, st2, null, null, p, 1, p, 1, 1, 4, 4, 64, 16, 1, 16,
                                     p, p, p, 0, null)
    assert rc == -3
    # heads do not divide
    rc = lib.knlp_b200_decode_splitk(p, 0, st2, null, null, p, 1, p, 1, 1, 5, 4, 64, 16, 1, 16,
                                     p, p, p, 0, null)
    assert rc == -2
    # head_dim not supported
    rc = lib.knlp_b200_decode_splitk(p, 0, st2, null, null, p, 1, p, 1, 1, 4, 4, 48, 16, 1, 16,
                                     p, p, p, 0, null)
    assert rc == -2
    # missing plane
    rc = lib.knlp_b200_decode_splitk(p, 0, st2, null, null, p, 1, p, 1, 1, 4, 4, 64, 16, 1, 16,
                                     p, p, p, 0, null)
    assert rc == -1
    # asymmetric plane without zeros; unknown mode
    pl = _lib.KvPlane()
    pl.codes = p.value
    pl.scales = p.value
    pl.mode = _lib.KV_INT4_ASYM
    rc = lib.knlp_b200_decode_splitk(p, 0, st2, C.byref(pl), C.byref(pl), p, 1, p, 1, 1, 4, 4, 64,
                                     16, 1, 16, p, p, p, 0, null)
    assert rc == -1
    pk = _lib.KvPlane(); pk.codes = p.value; pk.scales = p.value; pk.mode = _lib.KV_INT4_SYM
    pv = _lib.KvPlane(); pv.codes = p.value; pv.scales = p.value; pv.mode = 7  # no such mode
    rc = lib.knlp_b200_decode_splitk(p, 0, st2, C.byref(pk), C.byref(pv), p, 1, p, 1, 1, 4, 4, 64,
                                     16, 1, 16, p, p, p, 0, null)
    assert rc == -4
    # n_splits < 1
    rc = lib.knlp_b200_decode_splitk(p, 0, st2, C.byref(pk), C.byref(pk), p, 1, p, 1, 1, 4, 4, 64,
                                     16, 0, 16, p, p, p, 0, null)
    assert rc == -6
    # quant_append: bad dtype / odd head_dim; nothing to do is OK
    assert lib.knlp_b200_quant_append(p, st2, p, st2, 9, C.byref(pk), C.byref(pk), p, 1, 1, 64, 16,
                                      0.0, null) == -3
    assert lib.knlp_b200_quant_append(p, st2, p, st2, 0, C.byref(pk), C.byref(pk), p, 1, 1, 40, 16,
                                      0.0, null) == -2
    assert lib.knlp_b200_quant_append(null, null, null, null, 0, null, null, null, 5, 1, 64, 16,
                                      0.0, null) == 0
    # combine
    assert lib.knlp_b200_combine(null, null, null, 1, 1, 1, 1, 1, null, 0, 1, null, null, 0, 1, 64,
                                 null) == -1
    assert lib.knlp_b200_combine(p, p, p, 0, 1, 1, 1, 1, p, 0, 1, null, null, 0, 1, 64, null) == -2
    assert lib.knlp_b200_combine(p, p, p, 1, 1, 1, 1, 1, p, 1, 1, p, p, 1, 1, 64, null) == -3


def test_host_side_checks_of_the_routed_and_lowrank_entry_points(lib):
    """Argument errors are found on the host, before anything is launched."""
    from knlp_b200 import _lib
    null = None
    p = C.c_void_p(0x1000)
    st2 = (C.c_int64 * 2)(128, 128)
    pk = _lib.KvPlane(); pk.codes = p.value; pk.scales = p.value; pk.mode = _lib.KV_INT4_SYM
    R = lib.knlp_b200_routed_decode_attention
    args = lambda out, flags, max_sel: (p, 2, st2, C.byref(pk), C.byref(pk), p, 4, p, 8, 1, 4, 1, 128,
                                        16, max_sel, p, 1 << 20, p, 64, out, 2, 128, flags, null)
    assert R(*args(null, 0, 4)) == -1            # no output
    assert R(*args(p, 8, 4)) == -4               # fixed splits have no per-head tables
    assert R(*args(p, 0, -1)) == -2
    L = lib.knlp_b200_lowrank_decode
    assert L(null, p, 2, p, p, 1, 1, 8, 128, 32, p, 1 << 20, null, p, null) == -1
    assert L(p, p, 0, p, p, 1, 1, 8, 128, 32, p, 1 << 20, null, p, null) == -3   # fp32 q / K
    assert L(p, p, 2, p, p, 1, 9, 8, 128, 32, p, 1 << 20, null, p, null) == -2   # > 8 queries
    assert L(p, p, 2, p, p, 1, 1, 8, 128, 16, p, 1 << 20, null, p, null) == -2   # rank != 32
    assert L(p, p, 2, p, p, 1, 1, 0, 128, 32, p, 1 << 20, null, p, null) == -2   # no token
    assert L(C.c_void_p(0x1004), p, 2, p, p, 1, 1, 8, 128, 32, p, 1 << 20, null, p, null) == -5
    n = C.c_int64(0)
    assert lib.knlp_b200_lowrank_decode_workspace(1, 9, 8, C.byref(n)) == -2
    assert lib.knlp_b200_lowrank_decode_workspace(1, 1, 8, null) == -1


def test_decode_plan_fills_waves(lib):
    n = C.c_int(0)
    ws = C.c_int64(0)
    # batch 32 x 128K, 8 kv heads: 32 CTAs per split, 296 slots on 148 SMs
    assert lib.knlp_b200_decode_plan(32, 32, 8, 128, 16, 131072, 2, 2, C.byref(n), C.byref(ws)) == 0
    assert n.value >= 9 and (32 * n.value) % 296 <= 296  # sane
    waves = -(-32 * n.value // 296)
    assert 32 * n.value / (waves * 296) > 0.9
    assert ws.value == 32 * 32 * n.value * 130
    # short context: one split
    assert lib.knlp_b200_decode_plan(4, 8, 2, 128, 16, 100, 2, 2, C.byref(n), C.byref(ws)) == 0
    assert n.value == 1
    assert lib.knlp_b200_decode_plan(4, 9, 2, 128, 16, 100, 2, 2, C.byref(n), C.byref(ws)) == -2


def test_ops_refuse_cpu_tensors_and_missing_library(monkeypatch):
    import torch
    from knlp_b200 import _lib, ops
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.reshape_and_cache_k_int8(torch.zeros(1, 1, 32), torch.zeros(1, 16, 1, 32, dtype=torch.int8),
                                     torch.zeros(1, 16, 1, 1, dtype=torch.float16),
                                     torch.zeros(1, dtype=torch.int64))
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libknlp_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
