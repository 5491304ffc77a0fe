"""Head dims 256 and 512 (the reference's channel-split configurations, gemv.cu:336-353, 857-874, 1208-1225)."""
import numpy as np
import pytest
import torch

from adkv_b200 import gemv, synth
from oracle import adkv_oracle as orc
from tests.util import SMAX, SMIN, dev, make_case, np_params, oracle_prefill

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 2e-3

WIDE = [  # D, Hq, Hkv, T, bits
    (256, 2, 2, 0, 4), (256, 2, 2, 33, 4), (256, 4, 2, 205, 4), (256, 2, 2, 77, 2), (256, 4, 2, 130, 2),
    (512, 2, 2, 1, 4), (512, 2, 2, 100, 4), (512, 4, 2, 65, 4), (512, 1, 1, 47, 2),
]


@pytest.mark.parametrize("D", [256, 512])
@pytest.mark.parametrize("bits", [4, 2])
def test_encode_chunks_and_appends_wide(D, bits):
    B, H, T = 2, 2, 75
    x = synth.gen_kv(40 + D, B, H, T, D)
    p = synth.gen_params(41, H, D, bits)
    ns = orc.n_super_for(T, bits) + 1
    want = np.zeros(orc.cache_shape(B, H, ns, D), np.uint8)
    _, st = orc.encode_kv(want, x.numpy(), np_params(p), bits, SMIN, SMAX)
    one = torch.zeros(want.shape, dtype=torch.uint8, device="cuda")
    tail = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    gemv.encode_kv(one, dev(x), *dev(p), SMIN, SMAX, bits=bits, tail=tail)
    assert np.array_equal(one.cpu().numpy(), want)
    t = tail.cpu().numpy()
    assert np.array_equal(t[:, :, 0].view(np.uint32), st.zp.view(np.uint32))
    assert np.array_equal(t[:, :, 1].view(np.uint32), st.s.view(np.uint32))
    parts = torch.zeros_like(one)
    tk, tv = torch.empty_like(tail), torch.empty_like(tail)
    other = torch.zeros_like(one)
    gemv.encode_kv_pair(parts, dev(x[:, :, :29]), dev(p), other, dev(x[:, :, :29]), dev(p), SMIN, SMAX, bits=bits,
                        k_tail=tk, v_tail=tv)
    gemv.encode_kv(parts, dev(x[:, :, 29:70]), *dev(p), SMIN, SMAX, bits=bits, tail=tk, t_start=29)
    for tt in range(70, T):
        gemv.append_kv(parts, dev(x[:, :, tt:tt + 1]), *dev(p), tk, tt, SMIN, SMAX, bits=bits)
    assert torch.equal(parts, one) and torch.equal(tk.view(torch.int32), tail.view(torch.int32))


@pytest.mark.parametrize("fast", [False, True], ids=["exact", "fast"])
@pytest.mark.parametrize("D,Hq,Hkv,T,bits", WIDE)
def test_decode_entry_points_wide(D, Hq, Hkv, T, bits, fast):
    B = 2
    case = make_case(800 + T + D, B, Hq, Hkv, T, bits, D=D, random_params=(T % 2 == 1))
    kc, vc = oracle_prefill(case)
    scaling = D ** -0.5
    mask = torch.zeros(B, 1, 1, T + 1)
    mask[0, ..., : (T + 1) // 4] = torch.finfo(torch.float16).min
    q, kn, vn = dev(case["q"]), dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1])
    # fused
    wk, wv = kc.copy(), vc.copy()
    want = orc.decode_attn(case["q"][:, :, 0].numpy(), wk, wv, case["k"][:, :, T].numpy(), case["v"][:, :, T].numpy(),
                           np_params(case["kp"]), np_params(case["vp"]), T, scaling, mask=mask[:, 0].numpy(), bits=bits,
                           scale_min=SMIN, scale_max=SMAX)
    dk, dv = dev(kc), dev(vc)
    got = gemv.decode_attn(q, dk, dv, kn, vn, dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX,
                           mask=dev(mask), bits=bits, fast=fast)
    assert gemv.device_status() == 0
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    if not fast:
        assert np.array_equal(dk.cpu().numpy(), wk) and np.array_equal(dv.cpu().numpy(), wv)
    # the reference's two calls
    ak, av = dev(kc), dev(vc)
    wk2 = kc.copy()
    want_l = orc.forward_qk(case["q"][:, :, 0].numpy(), wk2, case["k"][:, :, T].numpy(), np_params(case["kp"]), T, bits,
                            SMIN, SMAX)
    logits = gemv.forward_qk(q, ak, kn, *dev(case["kp"]), T, SMIN, SMAX, bits=bits, fast=fast)
    assert logits.shape == (B, Hq, T + 1)
    np.testing.assert_allclose(logits.float().cpu().numpy(), want_l, rtol=RTOL, atol=ATOL * max(1.0, np.abs(want_l).max()))
    g = torch.Generator().manual_seed(T)
    attn = torch.softmax(torch.randn(B, Hq, T + 1, generator=g) * 2, dim=-1).half()
    wv2 = vc.copy()
    want_o = orc.forward_ov(attn.float().numpy(), wv2, case["v"][:, :, T].numpy(), np_params(case["vp"]), bits, SMIN, SMAX)
    out = gemv.forward_ov(dev(attn), av, vn, *dev(case["vp"]), SMIN, SMAX, bits=bits, fast=fast)
    np.testing.assert_allclose(out.float().cpu().numpy(), want_o, rtol=RTOL, atol=ATOL)
    assert gemv.device_status() == 0
    if not fast:
        assert np.array_equal(ak.cpu().numpy(), wk2) and np.array_equal(av.cpu().numpy(), wv2)


def test_unsupported_wide_combinations_raise():
    D, H = 256, 2
    p = dev(synth.gen_params(1, H, D))
    cache = torch.zeros(1, H, 4, D // 4, 4, 4, dtype=torch.uint8, device="cuda")
    q8 = torch.zeros(1, 8, 1, D, dtype=torch.float16, device="cuda")        # group size 4 with head_dim 256
    kn = torch.zeros(1, H, 1, D, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="invalid sizes"):
        gemv.decode_attn(q8, cache, cache.clone(), kn, kn, p, p, 3, 0.1, SMIN, SMAX)
    sl = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="head dim"):
        gemv.decode_attn_varlen(q8[:, :2], cache, cache.clone(), kn, kn, p, p, sl, 0.1, SMIN, SMAX)
