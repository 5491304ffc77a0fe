"""ctypes front end of ``adkv_oracle.c`` (TEST INFRASTRUCTURE: checker and timed CPU baseline only)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "adkv_oracle.c")
LIB = os.path.join(HERE, "liboracle_adkv.so")


def build(force: bool = False) -> str:
    """Compile the C restatement (gcc, no FMA contraction, OpenMP)."""
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
                               SRC, "-o", LIB, "-lm"])
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = ctypes.CDLL(LIB)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _params(p, H, D):
    out = np.ascontiguousarray(np.stack([np.asarray(a, dtype=np.float32).reshape(H * D) for a in p]))
    assert out.shape == (5, H * D)
    return out


def num_threads() -> int:
    return lib().oracle_num_threads()


def use_all_cores() -> int:
    """Let OpenMP use every core this process may run on (launchers often export OMP_NUM_THREADS=1)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(n)
    return num_threads()


def encode(cache: np.ndarray, x16: np.ndarray, params, bits, smin, smax, want_tail=False):
    """cache uint8 [B,H,ns,D/4,4,4] (in place), x16 float16 [B,H,T,D]."""
    B, H, T, D = x16.shape
    x16 = np.ascontiguousarray(x16, dtype=np.float16)
    assert cache.flags.c_contiguous and cache.dtype == np.uint8
    tail = np.empty((B, H, 2, D), np.float32) if want_tail else None
    pr = _params(params, H, D)
    rc = lib().oracle_encode(_p(cache), _p(x16), _p(pr), B, H, T, D, cache.shape[2], bits,
                             ctypes.c_float(smin), ctypes.c_float(smax), _p(tail))
    if rc:
        raise RuntimeError("oracle_encode: capacity too small")
    return tail


def decode_attn(q16, k_cache, v_cache, k_new16, v_new16, kparams, vparams, T, scaling, bits, smin, smax,
                mask=None, first_stream=0, n_streams=-1):
    """q16 [B,Hq,D] float16; caches uint8 tiles (in place append); returns out [B,Hq,D] float32."""
    B, Hq, D = q16.shape
    Hkv = k_cache.shape[1]
    q16 = np.ascontiguousarray(q16, dtype=np.float16)
    k_new16 = np.ascontiguousarray(k_new16, dtype=np.float16)
    v_new16 = np.ascontiguousarray(v_new16, dtype=np.float16)
    out = np.zeros((B, Hq, D), np.float32)
    kp, vp = _params(kparams, Hkv, D), _params(vparams, Hkv, D)
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.float32).reshape(B, T + 1)
    rc = lib().oracle_decode_attn(_p(q16), _p(k_cache), _p(v_cache), _p(k_new16), _p(v_new16), _p(kp), _p(vp),
                                  _p(mask), _p(out), B, Hq, Hkv, T, D, k_cache.shape[2], bits,
                                  ctypes.c_float(scaling), ctypes.c_float(smin), ctypes.c_float(smax),
                                  first_stream, n_streams)
    if rc:
        raise RuntimeError("oracle_decode_attn: capacity too small")
    return out
