"""Shared helpers of the GPU parity tests: build inputs on CPU, run the oracle, ship to the device."""
from __future__ import annotations

import numpy as np
import torch

from adkv_b200 import synth
from oracle import adkv_oracle as orc

SMIN, SMAX = synth.SCALE_MIN, synth.SCALE_MAX


def np_params(params):
    return tuple(p.float().cpu().numpy() for p in params)


def make_case(seed, B, Hq, Hkv, T, bits, D=128, outlier_mode="scale", random_params=False):
    """Inputs for one decode step with T cached tokens (+1 new), on CPU."""
    k = synth.gen_kv(seed, B, Hkv, T + 1, D, outlier_mode=outlier_mode)
    v = synth.gen_kv(seed + 1, B, Hkv, T + 1, D, outlier_mode=outlier_mode)
    q = synth.gen_q(seed + 2, B, Hq, D)
    if random_params:
        g = torch.Generator().manual_seed(seed + 3)

        def rp():
            return tuple(t.half() for t in (
                torch.randn(Hkv, D, generator=g) * 0.5, torch.rand(Hkv, D, generator=g) * 2 + 0.05,
                torch.rand(Hkv, D, generator=g) * 0.3, torch.rand(Hkv, D, generator=g) * 0.1,
                torch.rand(Hkv, D, generator=g) * (2 ** (bits - 1)) * 0.6 + 0.2))
        kp, vp = rp(), rp()
    else:
        kp, vp = synth.gen_params(seed + 3, Hkv, D, bits), synth.gen_params(seed + 4, Hkv, D, bits)
    return dict(k=k, v=v, q=q, kp=kp, vp=vp, B=B, Hq=Hq, Hkv=Hkv, T=T, bits=bits, D=D)


def oracle_prefill(case, extra_super=1):
    """Packed caches holding tokens [0, T) as the oracle encodes them (numpy uint8)."""
    B, Hkv, T, bits, D = case["B"], case["Hkv"], case["T"], case["bits"], case["D"]
    ns = orc.n_super_for(T + 1, bits) + extra_super
    kc = np.zeros(orc.cache_shape(B, Hkv, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    orc.encode_kv(kc, case["k"][:, :, :T].numpy(), np_params(case["kp"]), bits, SMIN, SMAX)
    orc.encode_kv(vc, case["v"][:, :, :T].numpy(), np_params(case["vp"]), bits, SMIN, SMAX)
    return kc, vc


def dev(t, device="cuda"):
    if isinstance(t, np.ndarray):
        t = torch.from_numpy(t)
    if isinstance(t, (tuple, list)):
        return tuple(dev(x, device) for x in t)
    return t.to(device).contiguous()


def code_mismatch(a: np.ndarray, b: np.ndarray, T: int, bits: int):
    """(fraction of differing codes over tokens [0,T), max |difference|) between two packed caches."""
    ca, cb = orc.unpack_codes(a, T, bits).astype(np.int32), orc.unpack_codes(b, T, bits).astype(np.int32)
    d = np.abs(ca - cb)
    return float((d != 0).mean()), int(d.max()) if d.size else 0
