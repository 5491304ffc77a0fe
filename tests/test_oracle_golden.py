"""The numpy oracle against the fixtures produced by executing the reference's torch code."""
import glob
import os

import numpy as np
import pytest

from oracle import adkv_oracle as orc

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _load(path):
    d = np.load(path)
    params = tuple(d[k].astype(np.float32) for k in ("zp_init", "scale_init", "alpha", "beta", "target"))
    return d, params, int(d["bits"]), float(d["scale_min"]), float(d["scale_max"])


def test_fixtures_present():
    assert len(GOLDEN) >= 4


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_encode_scan_bit_exact(path):
    d, params, bits, smin, smax = _load(path)
    x = d["x"].astype(np.float32)
    st = orc.init_state(x.shape[0], params[0], params[1])
    codes, xhat = orc.encode_scan(x, st, params[2], params[3], params[4], bits, smin, smax)
    assert np.array_equal(codes, d["codes"])
    assert np.array_equal(xhat.view(np.uint32), d["x_hat"].view(np.uint32))
    assert np.array_equal(st.zp.view(np.uint32), d["zp_final"].view(np.uint32))
    assert np.array_equal(st.s.view(np.uint32), d["s_final"].view(np.uint32))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_decode_scan_replays_reference(path):
    """Replaying the reference's codes rebuilds the reference's x_hat and final state bit for bit."""
    d, params, bits, smin, smax = _load(path)
    st = orc.init_state(d["x"].shape[0], params[0], params[1])
    xhat = orc.decode_scan(d["codes"], st, params[2], params[3], params[4], smin, smax)
    assert np.array_equal(xhat.view(np.uint32), d["x_hat"].view(np.uint32))
    assert np.array_equal(st.s.view(np.uint32), d["s_final"].view(np.uint32))


def test_clamp_and_ties_are_exercised():
    d, params, bits, smin, smax = _load([p for p in GOLDEN if "clamp" in p][0])
    assert np.isclose(d["s_final"].min(), smin) and np.isclose(d["s_final"].max(), smax)
    ties = d["codes"][0, 0, 0, 64:96]
    # round-half-to-even of -8.0, -7.5, ... 7.5 then clamp to [-8, 7]
    want = np.clip(np.rint((np.arange(32) - 16) * 0.5), -8, 7)
    assert np.array_equal(ties, want.astype(np.int8))


@pytest.mark.parametrize("bits", [4, 2])
def test_pack_roundtrip_and_layout(bits):
    rng = np.random.default_rng(0)
    lo, hi = orc.quant_limits(bits)
    T = 37
    codes = rng.integers(lo, hi + 1, size=(2, 3, T, 128)).astype(np.int8)
    cache = orc.pack_codes(codes, bits)
    assert cache.shape == (2, 3, orc.n_super_for(T, bits), 32, 4, 4)
    assert np.array_equal(orc.unpack_codes(cache, T, bits), codes)
    if bits == 4:
        # token 5 of channel 4*7+2: supergroup 0, vector 7, word 2, byte 2, high nibble (gemv.cu:266-295)
        b = cache[1, 2, 0, 7, 2, 2]
        assert (b >> 4) == codes[1, 2, 5, 30] + 8
        assert (b & 15) == codes[1, 2, 4, 30] + 8
    # unused fields of the last word are zero
    tpw = orc.tokens_per_word(bits)
    words = orc.cache_words(cache)
    used = T % tpw
    assert np.all(words[:, :, -1, :] >> np.uint32(bits * used) == 0)


def test_append_matches_longer_encode():
    rng = np.random.default_rng(1)
    B, H, T, D = 1, 2, 21, 128
    x = rng.standard_normal((B, H, T + 1, D)).astype(np.float16).astype(np.float32)
    params = (np.zeros((H, D), np.float32), np.ones((H, D), np.float32),
              np.full((H, D), 0.05, np.float32), np.full((H, D), 0.05, np.float32),
              np.full((H, D), 3.5, np.float32))
    full = np.zeros(orc.cache_shape(B, H, 4, D), np.uint8)
    orc.encode_kv(full, x, params, 4)
    part = np.zeros_like(full)
    _, st = orc.encode_kv(part, x[:, :, :T], params, 4)
    orc.append_token(part, x[:, :, T], st, T, params, 4)
    assert np.array_equal(full, part)
