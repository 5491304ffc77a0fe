"""CPU checks of the numpy restatement of the reference CUDA kernels' fp16-state arithmetic.

Its bit-for-bit pin against those kernels needs a GPU (``tests/test_gpu_half_state.py``); here: internal
consistency, the documented special cases, and how far it is from the fp32 recurrence.
"""
import numpy as np
import pytest

from adkv_b200 import synth
from oracle import adkv_oracle as orc
from oracle import adkv_oracle_half as orh


def _p16(seed, H, bits=4):
    return tuple(t.numpy() for t in synth.gen_params(seed, H, 128, bits))


@pytest.mark.parametrize("bits", [4, 2])
def test_replay_of_codes_reproduces_encoder_values_and_state(bits):
    x = synth.gen_kv(1, 2, 3, 61, 128).numpy()
    zp0, s0, alpha, beta, target = _p16(2, 3, bits)
    st_e = orh.init_state(2, zp0, s0)
    codes, xhat = orh.encode_scan(x, st_e, alpha, beta, target, bits)
    lo, hi = orc.quant_limits(bits)
    assert codes.min() >= lo and codes.max() <= hi
    st_d = orh.init_state(2, zp0, s0)
    xhat_d = orh.decode_scan(codes, st_d, alpha, beta, target)
    assert np.array_equal(xhat.view(np.uint16), xhat_d.view(np.uint16))
    assert np.array_equal(st_e.zp.view(np.uint16), st_d.zp.view(np.uint16))
    assert np.array_equal(st_e.sc.view(np.uint16), st_d.sc.view(np.uint16))


def test_one_minus_beta_target_is_rounded_once():
    beta = np.array([[0.05, 0.0999, 0.013]], np.float16)
    target = np.array([[3.5, 6.77, 1.3]], np.float16)
    got = orh.one_minus_bt(beta, target)
    want = (1.0 - beta.astype(np.float64) * target.astype(np.float64)).astype(np.float16)
    twice = (np.float16(1) - (beta * target)).astype(np.float16)          # product rounded first: not what is used
    assert np.array_equal(got, want)
    assert got.dtype == np.float16 and twice.dtype == np.float16


def test_frozen_state_equals_fp32_recurrence():
    """alpha = beta = 0 freezes both recurrences; their quantisers then agree code for code."""
    x = synth.gen_kv(3, 1, 2, 40, 128).numpy()
    g = np.random.default_rng(0)
    zp0 = (g.standard_normal((2, 128)) * 0.5).astype(np.float16)
    s0 = (g.random((2, 128)) * 1.7 + 0.3).astype(np.float16)
    z = np.zeros((2, 128), np.float16)
    p = (zp0, s0, z, z, np.full((2, 128), 3.5, np.float16))
    a = np.zeros(orc.cache_shape(1, 2, orc.n_super_for(40, 4), 128), np.uint8)
    b = np.zeros_like(a)
    orh.encode_kv(a, x, p, 4)
    orc.encode_kv(b, x, tuple(t.astype(np.float32) for t in p), 4)
    assert np.array_equal(a, b)


def test_live_state_drifts_from_fp32_recurrence_by_a_few_percent_of_codes():
    x = synth.gen_kv(4, 1, 4, 256, 128).numpy()
    p = _p16(5, 4)
    a = np.zeros(orc.cache_shape(1, 4, orc.n_super_for(256, 4), 128), np.uint8)
    b = np.zeros_like(a)
    orh.encode_kv(a, x, p, 4)
    orc.encode_kv(b, x, tuple(t.astype(np.float32) for t in p), 4)
    frac = (orc.unpack_codes(a, 256, 4) != orc.unpack_codes(b, 256, 4)).mean()
    assert 1e-4 < frac < 0.1, frac        # why the fp16-state arithmetic is not the parity target


def test_zero_scale_saturates_and_zero_over_zero_gives_code_zero():
    zp0 = np.zeros((1, 128), np.float16)
    s0 = np.zeros((1, 128), np.float16)
    p = (zp0, s0, np.full((1, 128), 0.1, np.float16), np.full((1, 128), 0.05, np.float16), np.full((1, 128), 3.5, np.float16))
    x = np.zeros((1, 1, 1, 128), np.float16)
    x[..., :40] = 1.0
    x[..., 40:80] = -1.0
    st = orh.init_state(1, zp0, s0)
    codes, _ = orh.encode_scan(x, st, p[2], p[3], p[4], 4)
    assert (codes[..., :40] == 7).all() and (codes[..., 40:80] == -8).all() and (codes[..., 80:] == 0).all()


def test_decode_step_appends_and_attends_over_all_tokens():
    B, Hq, Hkv, T = 1, 4, 2, 20
    k = synth.gen_kv(6, B, Hkv, T + 1, 128).numpy()
    v = synth.gen_kv(7, B, Hkv, T + 1, 128).numpy()
    q = synth.gen_q(8, B, Hq, 128).numpy()[:, :, 0]
    kp, vp = _p16(9, Hkv), _p16(10, Hkv)
    ns = orc.n_super_for(T + 1, 4)
    kc = np.zeros(orc.cache_shape(B, Hkv, ns, 128), np.uint8)
    vc = np.zeros_like(kc)
    orh.encode_kv(kc, k[:, :, :T], kp, 4)
    orh.encode_kv(vc, v[:, :, :T], vp, 4)
    full_k = np.zeros_like(kc)
    orh.encode_kv(full_k, k, kp, 4)
    out, logits = orh.decode_attn(q, kc, vc, k[:, :, T], v[:, :, T], kp, vp, T, 0.0884, 4)
    assert np.array_equal(kc, full_k)                      # append == encoding one more token
    assert out.shape == (B, Hq, 128) and logits.shape == (B, Hq, T + 1) and np.isfinite(out).all()
