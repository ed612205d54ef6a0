"""ctypes binding of libknlp_b200.so (the C ABI declared in include/knlp_b200.h).

There is no fallback: if the library is missing or does not export a symbol, the
import of the operators fails with an error that says how to build it.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# KNLP_B200_LIB points the binding at another build of the same library.
LIB_PATH = os.environ.get("KNLP_B200_LIB") or os.path.join(_PKG, "libknlp_b200.so")

ABI_VERSION = 2

# dtype / mode codes of include/knlp_b200.h
F32, F16, BF16 = 0, 1, 2
KV_NONE, KV_INT4_SYM, KV_INT4_ASYM, KV_INT8_G32 = 0, 1, 2, 3
KV_F16, KV_BF16 = 4, 5  # unquantized K plane of the kfp16_* decodes
DECODE_FORCE_GENERIC = 1
DECODE_USE_TMA = 2
DECODE_EMIT_PARTIAL = 4
DECODE_FIXED_SPLITS = 8
DECODE_DEBUG_STALL = 16

SYMBOLS = (
    "knlp_b200_abi_version",
    "knlp_b200_debug_status",
    "knlp_b200_strerror",
    "knlp_b200_quant_append",
    "knlp_b200_decode_plan",
    "knlp_b200_decode_splitk",
    "knlp_b200_decode_attention",
    "knlp_b200_decode_workspace",
    "knlp_b200_decode_append_attention",
    "knlp_b200_routed_decode_attention",
    "knlp_b200_lowrank_decode_workspace",
    "knlp_b200_lowrank_decode",
    "knlp_b200_combine",
    "knlp_b200_decode_noalloc",
    "knlp_b200_plugin_quantize",
    "knlp_b200_plugin_dequantize",
)


class KvPlane(C.Structure):
    """knlp_kv_plane"""

    _fields_ = [
        ("codes", C.c_void_p),
        ("scales", C.c_void_p),
        ("zeros", C.c_void_p),
        ("codes_stride", C.c_int64 * 3),
        ("scales_stride", C.c_int64 * 3),
        ("zeros_stride", C.c_int64 * 3),
        ("mode", C.c_int32),
        ("reserved", C.c_int32),
    ]


class NewTokens(C.Structure):
    """knlp_new_tokens"""

    _fields_ = [
        ("key", C.c_void_p),
        ("value", C.c_void_p),
        ("key_stride", C.c_int64 * 2),
        ("value_stride", C.c_int64 * 2),
        ("dtype", C.c_int32),
        ("clip_ratio", C.c_float),
    ]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build the CUDA library first with "
            "`python -m knlp_b200.build` (needs nvcc; no GPU needed to build). "
            "knlp_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for s in SYMBOLS:
        if not hasattr(lib, s):
            raise RuntimeError(f"{LIB_PATH} does not export {s}; rebuild it")
    I64P = C.POINTER(C.c_int64)
    PL = C.POINTER(KvPlane)
    lib.knlp_b200_abi_version.restype = C.c_int
    lib.knlp_b200_abi_version.argtypes = []
    lib.knlp_b200_debug_status.restype = C.c_int
    lib.knlp_b200_debug_status.argtypes = []
    lib.knlp_b200_strerror.restype = C.c_char_p
    lib.knlp_b200_strerror.argtypes = [C.c_int]
    lib.knlp_b200_quant_append.restype = C.c_int
    lib.knlp_b200_quant_append.argtypes = [
        C.c_void_p, I64P, C.c_void_p, I64P, C.c_int, PL, PL, C.c_void_p,
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p]
    lib.knlp_b200_decode_plan.restype = C.c_int
    lib.knlp_b200_decode_plan.argtypes = [
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.POINTER(C.c_int), C.POINTER(C.c_int64)]
    lib.knlp_b200_decode_splitk.restype = C.c_int
    lib.knlp_b200_decode_splitk.argtypes = [
        C.c_void_p, C.c_int, I64P, PL, PL, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_void_p]
    lib.knlp_b200_decode_attention.restype = C.c_int
    lib.knlp_b200_decode_attention.argtypes = [
        C.c_void_p, C.c_int, I64P, PL, PL, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
        C.c_uint, C.c_void_p]
    lib.knlp_b200_decode_append_attention.restype = C.c_int
    lib.knlp_b200_decode_append_attention.argtypes = [
        C.c_void_p, C.c_int, I64P, PL, PL, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
        C.c_uint, C.POINTER(NewTokens), C.c_void_p]
    lib.knlp_b200_routed_decode_attention.restype = C.c_int
    lib.knlp_b200_routed_decode_attention.argtypes = [
        C.c_void_p, C.c_int, I64P, PL, PL, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
        C.c_uint, C.c_void_p]
    lib.knlp_b200_lowrank_decode_workspace.restype = C.c_int
    lib.knlp_b200_lowrank_decode_workspace.argtypes = [C.c_int, C.c_int, C.c_int,
                                                       C.POINTER(C.c_int64)]
    lib.knlp_b200_lowrank_decode.restype = C.c_int
    lib.knlp_b200_lowrank_decode.argtypes = [
        C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
        C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.knlp_b200_decode_workspace.restype = C.c_int
    lib.knlp_b200_decode_workspace.argtypes = [
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    lib.knlp_b200_combine.restype = C.c_int
    lib.knlp_b200_combine.argtypes = [
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
        C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int,
        C.c_void_p]
    lib.knlp_b200_decode_noalloc.restype = C.c_int
    lib.knlp_b200_decode_noalloc.argtypes = [
        C.c_void_p, C.c_int, I64P, PL, PL, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
        C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
    lib.knlp_b200_plugin_quantize.restype = C.c_int
    lib.knlp_b200_plugin_quantize.argtypes = [
        C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
        C.c_void_p]
    lib.knlp_b200_plugin_dequantize.restype = C.c_int
    lib.knlp_b200_plugin_dequantize.argtypes = [
        C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    if lib.knlp_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libknlp_b200.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().knlp_b200_strerror(status).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {status})")
