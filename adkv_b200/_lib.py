"""ctypes binding of ``libadkv_b200.so`` (the C ABI in ``include/adkv_b200.h``).

There is no CPU fallback: if the library has not been built, importing the kernels fails
with instructions instead of silently computing something else.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

c_void_p, c_int, c_float, c_uint, c_longlong = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float,
                                                 ctypes.c_uint, ctypes.c_longlong)

FLAG_FAST_REPLAY = 1
FLAG_HALF_STATE = 2
FLAG_TAIL_KEEP = 4
FLAG_SPLIT_CHANNELS = 8
FLAG_NO_SPLIT_CHANNELS = 16
FLAG_SELFTEST_MUTE_K = 0x80000000
ABI_VERSION = 2


def flags(fast: bool = False, half_state: bool = False, tail_keep: bool = False,
          split_channels: bool | None = None) -> int:
    """``split_channels``: None = the library decides from the size of the launch."""
    return (FLAG_FAST_REPLAY if fast else 0) | (FLAG_HALF_STATE if half_state else 0) | \
        (FLAG_TAIL_KEEP if tail_keep else 0) | \
        (0 if split_channels is None else FLAG_SPLIT_CHANNELS if split_channels else FLAG_NO_SPLIT_CHANNELS)

# name -> argument types (return type is int unless listed in _RESTYPE); mirrors include/adkv_b200.h
SIGNATURES = {
    "adkv_abi_version": [],
    "adkv_strerror": [c_int],
    "adkv_encode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                    c_float, c_float, c_void_p],
    "adkv_encode_kv": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "adkv_append_kv": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "adkv_encode_kv_flags": [c_void_p] * 10 + [c_int] * 9 + [c_float, c_float, c_uint, c_void_p],
    "adkv_append_kv_flags": [c_void_p] * 10 + [c_int] * 8 + [c_float, c_float, c_uint, c_void_p],
    "adkv_encode_kv_layers": [c_void_p, c_int] + [c_int] * 7 + [c_float, c_float, c_void_p],
    "adkv_append_kv_layers": [c_void_p, c_int] + [c_int] * 6 + [c_float, c_float, c_void_p],
    "adkv_encode_kv_ckpt": [c_void_p] * 10 + [c_int] * 9 + [c_float, c_float, c_void_p],
    "adkv_append_kv_ckpt": [c_void_p] * 10 + [c_int] * 8 + [c_float, c_float, c_void_p],
    "adkv_decode_attn_ckpt_scratch_bytes": [c_int, c_int, c_int, c_int, c_int],
    "adkv_decode_attn_ckpt": [c_void_p] * 11 + [c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_uint,
                              c_void_p],
    "adkv_decode_attn_ckpt_static": [c_void_p] * 11 + [c_int, c_int, c_void_p, c_longlong, c_void_p,
                                     c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float,
                                     c_uint, c_void_p],
    "adkv_append": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                    c_float, c_float, c_void_p],
    "adkv_forward_qk": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_float, c_float, c_uint, c_void_p],
    "adkv_forward_ov": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_float, c_float, c_uint, c_void_p],
    "adkv_decode_attn": [c_void_p] * 10 + [c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_float, c_float, c_float, c_uint, c_void_p],
    "adkv_decode_attn_varlen": [c_void_p] * 11 + [c_int] * 6 + [c_float, c_float, c_float, c_uint, c_void_p],
    "adkv_device_status": [c_void_p, c_void_p],
    "adkv_selftest_wait_timeout": [c_int, c_void_p],
}
_RESTYPE = {"adkv_strerror": ctypes.c_char_p, "adkv_decode_attn_ckpt_scratch_bytes": c_longlong}


class Params(ctypes.Structure):
    """``adkv_params``: five fp16 ``[Hkv, D]`` device pointers."""
    _fields_ = [("zp_init", c_void_p), ("scale_init", c_void_p), ("alpha", c_void_p),
                ("beta", c_void_p), ("target", c_void_p)]


class LayerKV(ctypes.Structure):
    """``adkv_layer_kv``: K and V of one layer for the layered calls."""
    _fields_ = [("k_cache", c_void_p), ("k", c_void_p), ("kp", Params), ("k_tail", c_void_p),
                ("v_cache", c_void_p), ("v", c_void_p), ("vp", Params), ("v_tail", c_void_p)]


_lib = None


def library_path() -> str:
    return _build.LIB


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is missing (no fallback path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m adkv_b200.build` (needs nvcc). "
            "adkv_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(path)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _RESTYPE.get(name, c_int)
    if lib.adkv_abi_version() != ABI_VERSION:
        raise RuntimeError("libadkv_b200.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().adkv_strerror(code).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what}: {strerror(code)} (code {code})")
