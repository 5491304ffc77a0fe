"""Digest of the reference's own torch path on the CPU-runnable benchmark case, full size.

    TORCH_COMPILE_DISABLE=1 python tests/golden/make_golden_config1.py /path/to/reference

The case: batch 1, 32 heads, head dim 128, 1024 tokens, 4-bit codes; K and V from the seeded
generator of ``adkv_b200.synth`` (both outlier modes), parameters from ``synth.gen_params``.  The
script EXECUTES the reference's ``_adkv_chunk_forward`` (``src/adkv/train/train_model.py:46-86``,
eagerly, through ``make_golden.load_reference``) on K and on V, then computes single-query attention
in fp32 torch over the dequantised values and over the unquantised ones.

The 4 M codes per tensor are too large for a fixture, so what is stored is size-independent: the
SHA-256 of the inputs (to detect a host whose generator produces other values), one SHA-256 per head
of the int8 codes ``[T, D]``, the final state, both attention outputs ``[1, 32, 128]`` fp32 and the
reference's wall time.  One small ``.npz`` per outlier mode under ``tests/golden/config1/``.
"""
from __future__ import annotations

import hashlib
import math
import os
import sys
import time

os.environ.setdefault("TORCH_COMPILE_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)

B, H, T, D, BITS, SEED = 1, 32, 1024, 128, 4, 1000


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def head_digests(codes: np.ndarray):
    """codes [1,H,T,D] int8 -> one digest per head."""
    return np.array([sha(codes[0, h]) for h in range(codes.shape[1])])


def inputs(mode: str):
    """The case's tensors; the test regenerates them with this same function."""
    from adkv_b200 import synth
    k = synth.gen_kv(SEED, B, H, T, D, outlier_mode=mode)
    v = synth.gen_kv(SEED + 1, B, H, T, D, outlier_mode=mode)
    q = synth.gen_q(SEED + 2, B, H, D)
    kp = synth.gen_params(SEED + 3, H, D, BITS)
    vp = synth.gen_params(SEED + 4, H, D, BITS)
    return k, v, q, kp, vp


def attention(q, k, v):
    """q [B,H,1,D], k/v [B,H,T,D] fp32 -> [B,H,D] fp32 (scaling 1/sqrt(D), fp32 softmax)."""
    logits = torch.einsum("bhqd,bhtd->bhqt", q, k) * (1.0 / math.sqrt(q.shape[-1]))
    return torch.einsum("bhqt,bhtd->bhqd", torch.softmax(logits, dim=-1), v)[:, :, 0]


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden_config1.py /path/to/reference")
    import make_golden as mg
    tm, recorded = mg.load_reference(sys.argv[1])
    smin, smax = math.exp(-4.0), math.exp(4.0)
    os.makedirs(os.path.join(HERE, "config1"), exist_ok=True)
    for mode in ("scale", "persistent"):
        k, v, q, kp, vp = inputs(mode)
        t0 = time.perf_counter()
        rk = mg.run_case(tm, recorded, k, tuple(p.float() for p in kp), BITS, smin, smax)
        rv = mg.run_case(tm, recorded, v, tuple(p.float() for p in vp), BITS, smin, smax)
        qf = q.float()
        out_q = attention(qf, torch.from_numpy(rk["x_hat"]), torch.from_numpy(rv["x_hat"]))
        wall = time.perf_counter() - t0
        out_d = attention(qf, k.float(), v.float())
        d = dict(
            mode=mode, seed=np.int64(SEED), bits=np.int32(BITS), shape=np.array([B, H, T, D]),
            sha_k=sha(k.numpy()), sha_v=sha(v.numpy()), sha_q=sha(q.numpy()),
            sha_kparams=sha(np.stack([p.numpy() for p in kp])), sha_vparams=sha(np.stack([p.numpy() for p in vp])),
            k_code_sha=head_digests(rk["codes"]), v_code_sha=head_digests(rv["codes"]),
            k_zp_final=rk["zp_final"], k_s_final=rk["s_final"], v_zp_final=rv["zp_final"], v_s_final=rv["s_final"],
            attn_quantised=out_q.numpy().astype(np.float32), attn_dense=out_d.numpy().astype(np.float32),
            reference_wall_s=np.float64(wall), reference_threads=np.int32(torch.get_num_threads()),
        )
        path = os.path.join(HERE, "config1", f"config1_{mode}_b{BITS}.npz")
        np.savez_compressed(path, **d)
        rel = float((out_q - out_d).norm() / out_d.norm())
        print(mode, "rel-Frobenius error of attention vs unquantised:", rel, "max abs:",
              float((out_q - out_d).abs().max()), "wall s:", round(wall, 2), os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
