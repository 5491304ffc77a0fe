"""The CPU-runnable benchmark case at full size (batch 1, 32 heads, 1024 tokens, head dim 128, 4-bit).

The expected values come from EXECUTING the reference's torch code on the same seeded inputs
(``tests/golden/make_golden_config1.py``): one SHA-256 per head of the integer codes, the final
states, and the fp32 attention output over the dequantised cache.  The oracles are checked against
them on CPU, the CUDA path on the GPU; the quality against unquantised attention is report-only.
"""
import glob
import hashlib
import math
import os
import sys

import numpy as np
import pytest
import torch

from oracle import adkv_oracle as orc
from oracle import c_oracle
from tests.util import SMAX, SMIN, dev, np_params

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden_config1 as c1  # noqa: E402  (only its seeded input generator and digest helpers)

FIXTURES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "config1", "*.npz")))
RTOL, ATOL = 2e-3, 2e-3
SCALING = 1.0 / math.sqrt(c1.D)


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _case(path):
    d = np.load(path)
    k, v, q, kp, vp = c1.inputs(str(d["mode"]))
    same = (_sha(k.numpy()) == str(d["sha_k"]) and _sha(v.numpy()) == str(d["sha_v"])
            and _sha(q.numpy()) == str(d["sha_q"])
            and _sha(np.stack([p.numpy() for p in kp])) == str(d["sha_kparams"])
            and _sha(np.stack([p.numpy() for p in vp])) == str(d["sha_vparams"]))
    if not same:
        pytest.skip("this host's torch generates other values for the seeded inputs than the fixture's host did")
    return d, k, v, q, kp, vp


def test_fixtures_present():
    assert len(FIXTURES) == 2


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_oracles_reproduce_reference_codes_and_attention(path):
    d, k, v, q, kp, vp = _case(path)
    B, H, T, D, bits = c1.B, c1.H, c1.T, c1.D, c1.BITS
    ns = orc.n_super_for(T, bits)
    caches = {}
    for name, x, p in (("k", k, kp), ("v", v, vp)):
        want = d[f"{name}_code_sha"]
        # numpy oracle
        c_np = np.zeros(orc.cache_shape(B, H, ns, D), np.uint8)
        _, st = orc.encode_kv(c_np, x.numpy(), np_params(p), bits, SMIN, SMAX)
        assert np.array_equal(c1.head_digests(orc.unpack_codes(c_np, T, bits)), want)
        assert np.array_equal(st.zp.view(np.uint32), d[f"{name}_zp_final"].view(np.uint32))
        assert np.array_equal(st.s.view(np.uint32), d[f"{name}_s_final"].view(np.uint32))
        # C oracle
        c_c = np.zeros_like(c_np)
        tail = c_oracle.encode(c_c, x.numpy(), np_params(p), bits, SMIN, SMAX, want_tail=True)
        assert np.array_equal(c_c, c_np)
        assert np.array_equal(tail[:, :, 1].view(np.uint32), d[f"{name}_s_final"].view(np.uint32))
        caches[name] = c_np
    # Decode step of the oracle = attention over the 1024 dequantised tokens: cache of 1023 + the last as new.
    kc = np.zeros_like(caches["k"])
    vc = np.zeros_like(kc)
    orc.encode_kv(kc, k[:, :, :T - 1].numpy(), np_params(kp), bits, SMIN, SMAX)
    orc.encode_kv(vc, v[:, :, :T - 1].numpy(), np_params(vp), bits, SMIN, SMAX)
    out = c_oracle.decode_attn(q.numpy()[:, :, 0], kc, vc, k[:, :, T - 1].numpy(), v[:, :, T - 1].numpy(),
                               np_params(kp), np_params(vp), T - 1, SCALING, bits, SMIN, SMAX)
    assert np.array_equal(kc, caches["k"]) and np.array_equal(vc, caches["v"])     # append == one-shot encode
    np.testing.assert_allclose(out, d["attn_quantised"], rtol=1e-4, atol=1e-4)
    dense = orc.dense_attn(q.numpy()[:, :, 0].astype(np.float32), k.float().numpy(), v.float().numpy(), SCALING)
    np.testing.assert_allclose(dense, d["attn_dense"], rtol=1e-4, atol=1e-4)
    rel = np.linalg.norm(out - d["attn_dense"]) / np.linalg.norm(d["attn_dense"])
    print(f"\n[config 1, {d['mode']}] attention rel-Frobenius error vs unquantised {rel:.4f}, "
          f"max abs {np.abs(out - d['attn_dense']).max():.3f}; reference torch path took "
          f"{float(d['reference_wall_s']):.2f} s on {int(d['reference_threads'])} threads when the fixture was made")


@pytest.mark.gpu
@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_cuda_path_reproduces_reference_codes_and_attention(path):
    from adkv_b200 import gemv
    d, k, v, q, kp, vp = _case(path)
    B, H, T, D, bits = c1.B, c1.H, c1.T, c1.D, c1.BITS
    ns = orc.n_super_for(T, bits)
    # one-shot encode of all 1024 tokens: codes and final state equal the reference's
    for name, x, p in (("k", k, kp), ("v", v, vp)):
        cache = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
        tail = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
        gemv.encode_kv(cache, dev(x), *dev(p), SMIN, SMAX, bits=bits, tail=tail)
        assert np.array_equal(c1.head_digests(orc.unpack_codes(cache.cpu().numpy(), T, bits)), d[f"{name}_code_sha"])
        t = tail.cpu().numpy()
        assert np.array_equal(t[:, :, 0].view(np.uint32), d[f"{name}_zp_final"].view(np.uint32))
        assert np.array_equal(t[:, :, 1].view(np.uint32), d[f"{name}_s_final"].view(np.uint32))
    # 1023 cached tokens + fused decode step with token 1023 as the new one
    kc = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    gemv.encode_kv(kc, dev(k[:, :, :T - 1]), *dev(kp), SMIN, SMAX, bits=bits)
    gemv.encode_kv(vc, dev(v[:, :, :T - 1]), *dev(vp), SMIN, SMAX, bits=bits)
    out = gemv.decode_attn(dev(q), kc, vc, dev(k[:, :, T - 1:]), dev(v[:, :, T - 1:]), dev(kp), dev(vp), T - 1,
                           SCALING, SMIN, SMAX, bits=bits)
    for name, cache in (("k", kc), ("v", vc)):
        assert np.array_equal(c1.head_digests(orc.unpack_codes(cache.cpu().numpy(), T, bits)), d[f"{name}_code_sha"])
    got = out.float().cpu().numpy().reshape(B, H, D)
    np.testing.assert_allclose(got, d["attn_quantised"], rtol=RTOL, atol=ATOL)
    # the reference's three calls (unscaled logits -> caller's softmax -> weighted sum), same bar
    kc2 = torch.zeros_like(kc)
    vc2 = torch.zeros_like(kc)
    gemv.encode_kv(kc2, dev(k[:, :, :T - 1]), *dev(kp), SMIN, SMAX, bits=bits)
    gemv.encode_kv(vc2, dev(v[:, :, :T - 1]), *dev(vp), SMIN, SMAX, bits=bits)
    logits = gemv.forward_qk(dev(q), kc2, dev(k[:, :, T - 1:]), *dev(kp), T - 1, SMIN, SMAX, bits=bits)
    w = torch.softmax(logits.float() * SCALING, dim=-1).to(torch.float16)
    out3 = gemv.forward_ov(w, vc2, dev(v[:, :, T - 1:]), *dev(vp), SMIN, SMAX, bits=bits)
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)
    np.testing.assert_allclose(out3.float().cpu().numpy().reshape(B, H, D), d["attn_quantised"], rtol=3e-2, atol=3e-2)
    assert gemv.device_status() == 0
