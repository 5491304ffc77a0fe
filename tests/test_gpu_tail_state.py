"""Decode steps next to a persisted tail state (called through the C ABI) against the oracle.  Needs a B200.

The reference quantises the token it appends with the state its replay of the whole cache ends in
(src/adkv/kernel/gemv.cu:744-764).  Here the state after the last token is kept between steps, so the appended
code comes from it -- bit-identical to the encoder -- while the replay runs in the contracted arithmetic:
codes, caches and tails must equal the oracle's bit for bit, attention outputs within rtol 2e-3 / atol 2e-3.
"""
import numpy as np
import pytest
import torch

from adkv_b200 import gemv, synth
from oracle import adkv_oracle as orc
from tests.util import SMAX, SMIN, dev, make_case, np_params

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-3, 2e-3      # tolerance stated for fp16 attention outputs; used as is, not scaled


def _status_ok():
    assert gemv.device_status() == 0, "a kernel gave up on a bounded wait"


def _bits_equal(t: torch.Tensor, a: np.ndarray) -> bool:
    return np.array_equal(t.cpu().numpy().view(np.uint32), np.ascontiguousarray(a, np.float32).view(np.uint32))


def _oracle_tail(st) -> np.ndarray:
    """Oracle state -> the [B, H, 2, D] layout of a tail tensor."""
    return np.stack([st.zp, st.s], axis=2).astype(np.float32)


def _prefill(case, capacity_tokens, **kw):
    """Prefill on the GPU with tails; oracle caches and states for the same tokens."""
    B, Hkv, T, bits, D = case["B"], case["Hkv"], case["T"], case["bits"], case["D"]
    ns = orc.n_super_for(capacity_tokens, bits)
    dk = torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    dv = torch.zeros_like(dk)
    tk = torch.zeros(B, Hkv, 2, D, dtype=torch.float32, device="cuda")
    tv = torch.zeros_like(tk)
    gemv.encode_kv_pair(dk, dev(case["k"][:, :, :T]), dev(case["kp"]), dv, dev(case["v"][:, :, :T]), dev(case["vp"]),
                        SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv, **kw)
    ok_ = np.zeros(orc.cache_shape(B, Hkv, ns, D), np.uint8)
    ov_ = np.zeros_like(ok_)
    _, sk = orc.encode_kv(ok_, case["k"][:, :, :T].numpy(), np_params(case["kp"]), bits, SMIN, SMAX)
    _, sv = orc.encode_kv(ov_, case["v"][:, :, :T].numpy(), np_params(case["vp"]), bits, SMIN, SMAX)
    if T:
        assert np.array_equal(dk.cpu().numpy(), ok_) and np.array_equal(dv.cpu().numpy(), ov_)
    assert _bits_equal(tk, _oracle_tail(sk)) and _bits_equal(tv, _oracle_tail(sv))
    return dk, dv, tk, tv, ok_, ov_, sk, sv


CASES = [
    # B, Hq, Hkv, T, bits
    (2, 2, 2, 0, 4), (2, 2, 2, 1, 4), (1, 3, 3, 31, 4), (2, 2, 2, 32, 4), (2, 2, 2, 33, 4), (2, 4, 4, 205, 4),
    (1, 2, 2, 1031, 4), (2, 2, 2, 0, 2), (1, 2, 2, 15, 2), (2, 2, 2, 16, 2), (2, 3, 3, 200, 2),
    (2, 4, 2, 77, 4), (1, 8, 2, 130, 2), (1, 8, 1, 40, 4),
]


@pytest.mark.parametrize("split", [False, True], ids=["whole_head", "split_head"])
@pytest.mark.parametrize("B,Hq,Hkv,T,bits", CASES)
def test_decode_from_tail_state(B, Hq, Hkv, T, bits, split):
    case = make_case(300 + T, B, Hq, Hkv, T, bits, random_params=(T % 2 == 1))
    dk, dv, tk, tv, ok_, ov_, sk, sv = _prefill(case, T + 1)
    kn, vn = case["k"][:, :, T], case["v"][:, :, T]
    want = orc.decode_attn(case["q"][:, :, 0].numpy(), ok_, ov_, kn.numpy(), vn.numpy(), np_params(case["kp"]),
                           np_params(case["vp"]), T, 0.09, bits=bits, scale_min=SMIN, scale_max=SMAX)
    # the oracle's states after the appended token
    orc.append_token(ok_.copy(), kn.numpy(), sk, T, np_params(case["kp"]), bits, SMIN, SMAX)
    orc.append_token(ov_.copy(), vn.numpy(), sv, T, np_params(case["vp"]), bits, SMIN, SMAX)
    tk0, tv0 = tk.clone(), tv.clone()
    args = (dev(case["q"]), dk, dv, dev(kn[:, :, None]), dev(vn[:, :, None]), dev(case["kp"]), dev(case["vp"]), T, 0.09,
            SMIN, SMAX)
    # tail_keep: same result and same code, tails untouched; the call can be repeated
    for _ in range(2):
        got = gemv.decode_attn(*args, bits=bits, k_tail=tk, v_tail=tv, tail_keep=True, split_channels=split)
        np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
        assert torch.equal(tk.view(torch.int32), tk0.view(torch.int32)) and torch.equal(tv.view(torch.int32), tv0.view(torch.int32))
        assert np.array_equal(dk.cpu().numpy(), ok_) and np.array_equal(dv.cpu().numpy(), ov_)
    got = gemv.decode_attn(*args, bits=bits, k_tail=tk, v_tail=tv, split_channels=split)   # contracted replay by default
    _status_ok()
    assert got.shape == (B, Hq, 128) and got.dtype == torch.float16
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert np.array_equal(dk.cpu().numpy(), ok_) and np.array_equal(dv.cpu().numpy(), ov_)    # whole caches, bit for bit
    assert _bits_equal(tk, _oracle_tail(sk)) and _bits_equal(tv, _oracle_tail(sv))            # advanced canonically


@pytest.mark.parametrize("variant", ["dense", "dense_whole_head", "dense_exact", "varlen", "ckpt", "static"])
@pytest.mark.parametrize("bits", [4, 2])
def test_generation_chain_from_tail_state(variant, bits):
    """Prefill, then 40 decode steps that carry the tails; caches and tails stay bit-identical to the oracle's,
    through every fused entry point."""
    B, Hq, Hkv, T0, steps, D, iv = 2, 4, 2, 21, 40, 128, 32
    case = make_case(17 + bits, B, Hq, Hkv, T0 + steps, bits)
    case_pre = dict(case, T=T0)
    kw = {}
    if variant in ("ckpt", "static"):
        kck = gemv.alloc_ckpt(B, Hkv, D, T0 + steps + 1, iv, "cuda")
        vck = gemv.alloc_ckpt(B, Hkv, D, T0 + steps + 1, iv, "cuda")
        kw = dict(k_ckpt=kck, v_ckpt=vck, ckpt_interval=iv)
    dk, dv, tk, tv, ok_, ov_, sk, sv = _prefill(case_pre, T0 + steps + 1, **kw)
    kp, vp = dev(case["kp"]), dev(case["vp"])
    g = torch.Generator().manual_seed(5)
    lens = torch.full((B,), T0, dtype=torch.int32, device="cuda")
    out = torch.empty(B, Hq, D, dtype=torch.float16, device="cuda")
    for s in range(steps):
        T = T0 + s
        q = torch.randn(B, Hq, 1, D, generator=g).half()
        kn, vn = case["k"][:, :, T], case["v"][:, :, T]
        want = orc.decode_attn(q[:, :, 0].numpy(), ok_, ov_, kn.numpy(), vn.numpy(), np_params(case["kp"]),
                               np_params(case["vp"]), T, 0.1, bits=bits, scale_min=SMIN, scale_max=SMAX)
        args = (dev(q), dk, dv, dev(kn[:, :, None]), dev(vn[:, :, None]), kp, vp)
        if variant == "varlen":
            got = gemv.decode_attn_varlen(*args, lens, 0.1, SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv)
            lens += 1
        elif variant == "static":
            got = gemv.decode_attn_static(*args, T, 0.1, SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv, out=out, **kw)
        else:
            # "dense": the library picks the layout (these few streams: heads split over two warp pairs)
            got = gemv.decode_attn(*args, T, 0.1, SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv,
                                   fast=False if variant == "dense_exact" else None,
                                   split_channels=False if variant == "dense_whole_head" else None, **kw)
        np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    _status_ok()
    assert np.array_equal(dk.cpu().numpy(), ok_) and np.array_equal(dv.cpu().numpy(), ov_)
    # the tails equal the state of a one-shot encode of all T0 + steps tokens
    Tn = T0 + steps
    _, sk = orc.encode_kv(np.zeros_like(ok_), case["k"][:, :, :Tn].numpy(), np_params(case["kp"]), bits, SMIN, SMAX)
    _, sv = orc.encode_kv(np.zeros_like(ov_), case["v"][:, :, :Tn].numpy(), np_params(case["vp"]), bits, SMIN, SMAX)
    assert _bits_equal(tk, _oracle_tail(sk)) and _bits_equal(tv, _oracle_tail(sv))
    if kw:      # checkpoints written by the decode steps equal those of a one-shot encode with checkpoints
        k2, v2 = gemv.alloc_ckpt(B, Hkv, D, Tn + 1, iv, "cuda"), gemv.alloc_ckpt(B, Hkv, D, Tn + 1, iv, "cuda")
        gemv.encode_kv_pair(torch.zeros_like(dk), dev(case["k"][:, :, :Tn]), kp, torch.zeros_like(dv),
                            dev(case["v"][:, :, :Tn]), vp, SMIN, SMAX, bits=bits, k_ckpt=k2, v_ckpt=v2, ckpt_interval=iv)
        n = Tn // iv
        assert torch.equal(kck[:, :, :n].view(torch.int32), k2[:, :, :n].view(torch.int32))
        assert torch.equal(vck[:, :, :n].view(torch.int32), v2[:, :, :n].view(torch.int32))


def test_tail_state_with_clamped_scales_and_wide_heads():
    """Scales pinned at both clamp bounds (the guarded replay path) and a 256-wide head, from tails."""
    for D, bits in ((128, 4), (256, 4), (128, 2)):
        B, H, T = 1, 2, 70
        case = make_case(41 + D, B, H, H, T, bits, D=D)
        zp, sc, al, be, tg = case["kp"]
        be = be.clone()
        be[:, ::2] = 0.45          # growth factors far from 1: scales hit scale_max / scale_min within a few tokens
        case["kp"] = (zp, sc, al, be, tg)
        case["vp"] = (case["vp"][0], case["vp"][1], case["vp"][2], be, case["vp"][4])
        dk, dv, tk, tv, ok_, ov_, sk, sv = _prefill(case, T + 1)
        kn, vn = case["k"][:, :, T], case["v"][:, :, T]
        want = orc.decode_attn(case["q"][:, :, 0].numpy(), ok_, ov_, kn.numpy(), vn.numpy(), np_params(case["kp"]),
                               np_params(case["vp"]), T, 0.05, bits=bits, scale_min=SMIN, scale_max=SMAX)
        got = gemv.decode_attn(dev(case["q"]), dk, dv, dev(kn[:, :, None]), dev(vn[:, :, None]), dev(case["kp"]),
                               dev(case["vp"]), T, 0.05, SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv)
        _status_ok()
        np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
        assert np.array_equal(dk.cpu().numpy(), ok_) and np.array_equal(dv.cpu().numpy(), ov_)


def test_tail_arguments_are_checked():
    case = make_case(5, 1, 2, 2, 8, 4)
    dk, dv, tk, tv, *_ = _prefill(case, 9)
    args = (dev(case["q"]), dk, dv, dev(case["k"][:, :, 8:9]), dev(case["v"][:, :, 8:9]), dev(case["kp"]),
            dev(case["vp"]), 8, 0.1, SMIN, SMAX)
    with pytest.raises(RuntimeError, match="go together"):
        gemv.decode_attn(*args, k_tail=tk)
    with pytest.raises(RuntimeError, match="fp32 arithmetic"):
        gemv.decode_attn(*args, k_tail=tk, v_tail=tv, half_state=True)
    with pytest.raises(RuntimeError, match="tail must be contiguous float32"):
        gemv.decode_attn(*args, k_tail=tk.half(), v_tail=tv)


@pytest.mark.parametrize("cfg", ["config2", "config5"])
def test_full_size_from_tail_state(cfg):
    """The two decode benchmark shapes through the tail path: a few distinct sequences replicated over the batch;
    every replica reproduces the C oracle's output (2e-3), appended codes and advanced tails (bit for bit)."""
    from oracle import c_oracle
    if cfg == "config2":
        B, Hq, Hkv, T, bits, D, R = 128, 32, 32, 4096, 4, 128, 2
    else:
        B, Hq, Hkv, T, bits, D, R = 32, 32, 8, 32768, 2, 128, 1
    case = make_case(911, R, Hq, Hkv, T, bits)
    ns = orc.n_super_for(T + 1, bits)
    kc = np.zeros(orc.cache_shape(R, Hkv, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    x = lambda t: t.numpy()
    c_oracle.encode(kc, x(case["k"][:, :, :T]), np_params(case["kp"]), bits, SMIN, SMAX)
    c_oracle.encode(vc, x(case["v"][:, :, :T]), np_params(case["vp"]), bits, SMIN, SMAX)
    # states after T + 1 tokens: what the tails must hold after the step
    tk_want = c_oracle.encode(np.zeros_like(kc), x(case["k"]), np_params(case["kp"]), bits, SMIN, SMAX, want_tail=True)
    tv_want = c_oracle.encode(np.zeros_like(vc), x(case["v"]), np_params(case["vp"]), bits, SMIN, SMAX, want_tail=True)
    rep = lambda t: dev(t).repeat(B // R, *([1] * (t.dim() - 1)))
    dk = torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    dv = torch.zeros_like(dk)
    tk = torch.empty(B, Hkv, 2, D, dtype=torch.float32, device="cuda")
    tv = torch.empty_like(tk)
    gemv.encode_kv_pair(dk, rep(case["k"][:, :, :T]), dev(case["kp"]), dv, rep(case["v"][:, :, :T]), dev(case["vp"]),
                        SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv)
    scaling = D ** -0.5
    want = c_oracle.decode_attn(x(case["q"][:, :, 0]), kc, vc, x(case["k"][:, :, T]), x(case["v"][:, :, T]),
                                np_params(case["kp"]), np_params(case["vp"]), T, scaling, bits, SMIN, SMAX)
    args = (rep(case["q"]), dk, dv, rep(case["k"][:, :, T:T + 1]), rep(case["v"][:, :, T:T + 1]), dev(case["kp"]),
            dev(case["vp"]), T, scaling, SMIN, SMAX)
    # the other layout of the heads over warps first (tails kept), then the one the library picks for this size
    auto_split = B * Hkv <= 160
    for kw in (dict(split_channels=not auto_split, tail_keep=True), dict()):
        out = gemv.decode_attn(*args, bits=bits, k_tail=tk, v_tail=tv, **kw)
        _status_ok()
        got = out.float().cpu().numpy().reshape(B // R, R, Hq, D)
        assert np.array_equal(got, np.broadcast_to(got[0], got.shape))
        np.testing.assert_allclose(got[0], want, rtol=RTOL, atol=ATOL)
        assert np.array_equal(dk[:R].cpu().numpy(), kc) and np.array_equal(dv[-R:].cpu().numpy(), vc)
    assert np.array_equal(dk[:R].cpu().numpy(), kc) and np.array_equal(dv[-R:].cpu().numpy(), vc)
    assert torch.equal(dk[:R], dk[-R:]) and torch.equal(dv[:R], dv[-R:])
    assert _bits_equal(tk[:R], tk_want) and _bits_equal(tv[-R:], tv_want)
