"""The C restatement against the numpy oracle (which is pinned to the reference's fixtures)."""
import numpy as np
import pytest

from adkv_b200 import synth
from oracle import adkv_oracle as orc
from oracle import c_oracle


def _np(ts):
    return tuple(t.float().numpy() for t in ts)


@pytest.mark.parametrize("bits,T", [(4, 77), (4, 8), (2, 50), (2, 1)])
def test_c_encode_matches_numpy(bits, T):
    B, H, D = 2, 3, 128
    x = synth.gen_kv(5, B, H, T, D).numpy()
    p = _np(synth.gen_params(6, H, D, bits))
    ns = orc.n_super_for(T, bits) + 1
    c1 = np.zeros(orc.cache_shape(B, H, ns, D), np.uint8)
    c2 = np.zeros_like(c1)
    _, st = orc.encode_kv(c1, x, p, bits)
    tail = c_oracle.encode(c2, x, p, bits, orc.SCALE_MIN, orc.SCALE_MAX, want_tail=True)
    assert np.array_equal(c1, c2)
    assert np.array_equal(tail[:, :, 0], st.zp) and np.array_equal(tail[:, :, 1], st.s)


@pytest.mark.parametrize("bits,Hq,Hkv,T", [(4, 2, 2, 45), (2, 4, 2, 33), (4, 2, 2, 0)])
def test_c_decode_matches_numpy(bits, Hq, Hkv, T):
    B, D = 2, 128
    k = synth.gen_kv(1, B, Hkv, T + 1, D).numpy()
    v = synth.gen_kv(2, B, Hkv, T + 1, D).numpy()
    q = synth.gen_q(3, B, Hq, D).numpy()[:, :, 0]
    kp, vp = _np(synth.gen_params(4, Hkv, D, bits)), _np(synth.gen_params(5, Hkv, D, bits))
    ns = orc.n_super_for(T + 1, bits)
    kc = np.zeros(orc.cache_shape(B, Hkv, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    orc.encode_kv(kc, k[:, :, :T], kp, bits)
    orc.encode_kv(vc, v[:, :, :T], vp, bits)
    kc2, vc2 = kc.copy(), vc.copy()
    mask = np.zeros((B, 1, T + 1), np.float32)
    mask[1, 0, : T // 2] = -1e4
    want = orc.decode_attn(q, kc, vc, k[:, :, T], v[:, :, T], kp, vp, T, 0.0884, mask=mask, bits=bits)
    got = c_oracle.decode_attn(q, kc2, vc2, k[:, :, T], v[:, :, T], kp, vp, T, 0.0884, bits,
                               orc.SCALE_MIN, orc.SCALE_MAX, mask=mask[:, 0])
    assert np.array_equal(kc, kc2) and np.array_equal(vc, vc2)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
