"""Parity of the CUDA path (called through the C ABI) against the oracle.  Needs a B200."""
import glob
import os

import numpy as np
import pytest
import torch

from adkv_b200 import gemv, synth
from oracle import adkv_oracle as orc
from tests.util import SMAX, SMIN, code_mismatch, dev, make_case, np_params, oracle_prefill

pytestmark = pytest.mark.gpu

# tolerance stated for fp16 attention outputs (|got - want| <= 2e-3 + 2e-3 |want|), applied as it stands to the
# outputs of decode_attn / forward_ov.  Only the unscaled fp16 logits of forward_qk get an absolute term scaled by
# their magnitude: they are not normalised, and half an fp16 ulp of a logit of size L is already L * 4.9e-4.
RTOL, ATOL = 2e-3, 2e-3
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _status_ok():
    assert gemv.device_status() == 0, "a kernel gave up on a bounded wait"


# ------------------------------------------------------------------------------- encode

@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("T", [1, 7, 8, 9, 16, 17, 77, 130])
def test_encode_bit_exact(bits, T):
    B, H, D = 2, 3, 128
    x = synth.gen_kv(11 + T, B, H, T, D)
    p = synth.gen_params(12, H, D, bits)
    ns = orc.n_super_for(T, bits) + 1
    want = np.zeros(orc.cache_shape(B, H, ns, D), np.uint8)
    _, st = orc.encode_kv(want, x.numpy(), np_params(p), bits, SMIN, SMAX)
    cache = torch.full(want.shape, 0xAB, dtype=torch.uint8, device="cuda")   # stale bytes must be overwritten
    tail = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    out = gemv.encode_kv(cache, dev(x), *dev(p), SMIN, SMAX, bits=bits, tail=tail)
    assert out is cache
    used = orc.n_super_for(T, bits)
    assert np.array_equal(cache.cpu().numpy()[:, :, :used], want[:, :, :used])
    assert np.all(cache.cpu().numpy()[:, :, used:] == 0xAB)          # untouched beyond the last word
    t = tail.cpu().numpy()
    assert np.array_equal(t[:, :, 0].view(np.uint32), st.zp.view(np.uint32))
    assert np.array_equal(t[:, :, 1].view(np.uint32), st.s.view(np.uint32))


_PARAM_NAMES = ("zp_init", "scale_init", "alpha", "beta", "target")


def _fp16_parameters(path) -> bool:
    """The kernel API takes fp16 parameters (as the reference's model file stores them): a fixture can go through the
    kernel only if its parameters are fp16 values.  (One fixture holds a scale_init of 1e-9 for the oracle's sake; its
    fp16 counterpart, with 0.0 as the only value below the guard, is guard_clamp_ties_fp16_b4.)"""
    d = np.load(path)
    return all(np.array_equal(d[k].astype(np.float16).astype(np.float32), d[k]) for k in _PARAM_NAMES)


GOLDEN_FP16 = [p for p in GOLDEN if _fp16_parameters(p)]


@pytest.mark.parametrize("path", GOLDEN_FP16, ids=[os.path.basename(p) for p in GOLDEN_FP16])
def test_encode_reproduces_reference_fixtures(path):
    """Codes written by the kernel equal the codes the reference's torch code produced: benchmark data, random
    parameters, and the two guard fixtures (eps guard from a zero initial scale, both clamps, exact .5 ties; scale
    decaying under the guard with scale_min = 0)."""
    d = np.load(path)
    bits = int(d["bits"])
    names = _PARAM_NAMES
    p16 = tuple(torch.from_numpy(d[k]).half() for k in names)
    x = torch.from_numpy(d["x"])
    B, H, T, D = x.shape
    cache = torch.zeros(orc.cache_shape(B, H, orc.n_super_for(T, bits), D), dtype=torch.uint8, device="cuda")
    tail = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    gemv.encode_kv(cache, dev(x), *dev(p16), float(d["scale_min"]), float(d["scale_max"]), bits=bits, tail=tail)
    got = orc.unpack_codes(cache.cpu().numpy(), T, bits)
    assert np.array_equal(got, d["codes"])
    assert np.array_equal(tail.cpu().numpy()[:, :, 1].view(np.uint32), d["s_final"].view(np.uint32))
    assert np.array_equal(tail.cpu().numpy()[:, :, 0].view(np.uint32), d["zp_final"].view(np.uint32))


@pytest.mark.parametrize("bits", [4, 2])
def test_chunked_encode_and_append_equal_one_shot(bits):
    B, H, D, T = 2, 2, 128, 61
    x = synth.gen_kv(21, B, H, T, D)
    p = dev(synth.gen_params(22, H, D, bits))
    ns = orc.n_super_for(T, bits)
    full = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    tail_full = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    gemv.encode_kv(full, dev(x), *p, SMIN, SMAX, bits=bits, tail=tail_full)
    part = torch.zeros_like(full)
    tail = torch.empty_like(tail_full)
    gemv.encode_kv(part, dev(x[:, :, :19]), *p, SMIN, SMAX, bits=bits, tail=tail)
    gemv.encode_kv(part, dev(x[:, :, 19:50]), *p, SMIN, SMAX, bits=bits, tail=tail, t_start=19)
    for t in range(50, T):
        gemv.append_kv(part, dev(x[:, :, t:t + 1]), *p, tail, t, SMIN, SMAX, bits=bits)
    assert torch.equal(full, part)
    assert torch.equal(tail_full.view(torch.int32), tail.view(torch.int32))


@pytest.mark.parametrize("bits", [4, 2])
def test_pair_launches_equal_single_tensor_launches(bits):
    B, H, D, T = 2, 3, 128, 45
    k, v = synth.gen_kv(31, B, H, T + 3, D), synth.gen_kv(32, B, H, T + 3, D)
    kp, vp = dev(synth.gen_params(33, H, D, bits)), dev(synth.gen_params(34, H, D, bits))
    ns = orc.n_super_for(T + 3, bits)
    mk = lambda: torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    mt = lambda: torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    k1, v1, k2, v2, tk1, tv1, tk2, tv2 = mk(), mk(), mk(), mk(), mt(), mt(), mt(), mt()
    gemv.encode_kv(k1, dev(k[:, :, :T]), *kp, SMIN, SMAX, bits=bits, tail=tk1)
    gemv.encode_kv(v1, dev(v[:, :, :T]), *vp, SMIN, SMAX, bits=bits, tail=tv1)
    gemv.encode_kv_pair(k2, dev(k[:, :, :T]), kp, v2, dev(v[:, :, :T]), vp, SMIN, SMAX, bits=bits, k_tail=tk2, v_tail=tv2)
    for t in range(T, T + 3):
        gemv.append_kv(k1, dev(k[:, :, t:t + 1]), *kp, tk1, t, SMIN, SMAX, bits=bits)
        gemv.append_kv(v1, dev(v[:, :, t:t + 1]), *vp, tv1, t, SMIN, SMAX, bits=bits)
        gemv.append_kv_pair(k2, dev(k[:, :, t:t + 1]), kp, tk2, v2, dev(v[:, :, t:t + 1]), vp, tv2, t, SMIN, SMAX, bits=bits)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.equal(tk1.view(torch.int32), tk2.view(torch.int32)) and torch.equal(tv1.view(torch.int32), tv2.view(torch.int32))


# ------------------------------------------------------------------------------- decode

CASES = [
    # B, Hq, Hkv, T, bits
    (2, 2, 2, 0, 4), (2, 2, 2, 1, 4), (1, 3, 3, 31, 4), (2, 2, 2, 32, 4), (2, 2, 2, 33, 4), (1, 2, 2, 64, 4),
    (2, 4, 4, 205, 4), (1, 2, 2, 1031, 4),
    (2, 2, 2, 0, 2), (1, 2, 2, 15, 2), (2, 2, 2, 16, 2), (1, 2, 2, 47, 2), (2, 3, 3, 200, 2),
    (2, 4, 2, 77, 4), (1, 8, 2, 130, 2), (1, 8, 1, 40, 4),
]


@pytest.mark.parametrize("fast", [False, True], ids=["exact", "fast"])
@pytest.mark.parametrize("B,Hq,Hkv,T,bits", CASES)
def test_forward_qk(B, Hq, Hkv, T, bits, fast):
    case = make_case(100 + T, B, Hq, Hkv, T, bits, random_params=(T % 2 == 1))
    kc, _ = oracle_prefill(case)
    want_cache = kc.copy()
    want = orc.forward_qk(case["q"][:, :, 0].numpy(), want_cache, case["k"][:, :, T].numpy(),
                          np_params(case["kp"]), T, bits, SMIN, SMAX)
    cache = dev(kc)
    got = gemv.forward_qk(dev(case["q"]), cache, dev(case["k"][:, :, T:T + 1]), *dev(case["kp"]), T, SMIN, SMAX,
                          bits=bits, fast=fast)
    _status_ok()
    assert got.shape == (B, Hq, T + 1) and got.dtype == torch.float16
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL * max(1.0, np.abs(want).max()))
    if not fast:
        assert np.array_equal(cache.cpu().numpy(), want_cache)          # appended code bit-exact
    else:
        # only the appended token can differ: at most one in 1e-4 of its codes (and one code at these sizes)
        frac, dmax = code_mismatch(cache.cpu().numpy(), want_cache, T + 1, bits)
        assert dmax <= 1 and frac * B * Hkv * 128 * (T + 1) <= 1 + 1e-4 * B * Hkv * 128


@pytest.mark.parametrize("fast", [False, True], ids=["exact", "fast"])
@pytest.mark.parametrize("B,Hq,Hkv,T,bits", CASES)
def test_forward_ov(B, Hq, Hkv, T, bits, fast):
    case = make_case(200 + T, B, Hq, Hkv, T, bits, random_params=(T % 2 == 1))
    _, vc = oracle_prefill(case)
    g = torch.Generator().manual_seed(T)
    attn = torch.softmax(torch.randn(B, Hq, T + 1, generator=g) * 2, dim=-1).half()
    want_cache = vc.copy()
    want = orc.forward_ov(attn.float().numpy(), want_cache, case["v"][:, :, T].numpy(), np_params(case["vp"]),
                          bits, SMIN, SMAX)
    cache = dev(vc)
    got = gemv.forward_ov(dev(attn), cache, dev(case["v"][:, :, T:T + 1]), *dev(case["vp"]), SMIN, SMAX,
                          bits=bits, fast=fast)
    _status_ok()
    assert got.shape == (B, Hq, 128) and got.dtype == torch.float16
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    if not fast:
        assert np.array_equal(cache.cpu().numpy(), want_cache)
    else:
        # only the appended token can differ: at most one in 1e-4 of its codes (and one code at these sizes)
        frac, dmax = code_mismatch(cache.cpu().numpy(), want_cache, T + 1, bits)
        assert dmax <= 1 and frac * B * Hkv * 128 * (T + 1) <= 1 + 1e-4 * B * Hkv * 128


@pytest.mark.parametrize("split", [False, True], ids=["whole_head", "split_head"])
@pytest.mark.parametrize("fast", [False, True], ids=["exact", "fast"])
@pytest.mark.parametrize("with_mask", [False, True], ids=["nomask", "mask"])
@pytest.mark.parametrize("B,Hq,Hkv,T,bits", CASES)
def test_decode_attn(B, Hq, Hkv, T, bits, with_mask, fast, split):
    case = make_case(300 + T, B, Hq, Hkv, T, bits, outlier_mode="persistent" if T % 3 == 0 else "scale")
    kc, vc = oracle_prefill(case)
    mask = None
    if with_mask:
        mask = torch.zeros(B, 1, 1, T + 1)
        mask[0, ..., : (T + 1) // 3] = torch.finfo(torch.float16).min      # HF-style additive mask (left padding)
        mask[-1, ..., T // 2] = -3.0
    scaling = 128 ** -0.5
    wk, wv = kc.copy(), vc.copy()
    want = orc.decode_attn(case["q"][:, :, 0].numpy(), wk, wv, case["k"][:, :, T].numpy(), case["v"][:, :, T].numpy(),
                           np_params(case["kp"]), np_params(case["vp"]), T, scaling,
                           mask=None if mask is None else mask[:, 0].numpy(), bits=bits,
                           scale_min=SMIN, scale_max=SMAX)
    dk, dv = dev(kc), dev(vc)
    got = gemv.decode_attn(dev(case["q"]), dk, dv, dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1]),
                           dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX,
                           mask=None if mask is None else dev(mask), bits=bits, fast=fast, split_channels=split)
    _status_ok()
    assert got.shape == (B, Hq, 128) and got.dtype == torch.float16
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    if not fast:
        assert np.array_equal(dk.cpu().numpy(), wk) and np.array_equal(dv.cpu().numpy(), wv)
    else:       # contracted replay without a tail state: the appended code may be off by one step, rarely
        for a, b in ((dk.cpu().numpy(), wk), (dv.cpu().numpy(), wv)):
            frac, dmax = code_mismatch(a, b, T + 1, bits)
            assert dmax <= 1 and frac * B * Hkv * 128 * (T + 1) <= 1 + 1e-4 * B * Hkv * 128


@pytest.mark.parametrize("split", [False, True], ids=["whole_head", "split_head"])
@pytest.mark.parametrize("bits", [4, 2])
def test_decode_with_scales_at_both_clamps(bits, split):
    """Channels whose scale sits at scale_min (all-zero input) or scale_max (saturating input) during the
    replay: the kernels' unguarded fast body must hand over to the guarded one without changing a bit."""
    B, H, T, D = 2, 2, 333, 128
    case = make_case(77, B, H, H, T, bits)
    for name in ("k", "v"):
        x = case[name].float()
        x[..., :16] = 0.0                       # q = 0 forever: scale decays to scale_min
        x[..., 16:32] *= 400.0                  # saturated codes: scale grows to scale_max
        x[..., 200:, 32:48] = 0.0               # decays only in the second part of the sequence
        case[name] = x.half()
    kc, vc = oracle_prefill(case)
    scaling = 0.05
    wk, wv = kc.copy(), vc.copy()
    want = orc.decode_attn(case["q"][:, :, 0].numpy(), wk, wv, case["k"][:, :, T].numpy(), case["v"][:, :, T].numpy(),
                           np_params(case["kp"]), np_params(case["vp"]), T, scaling, bits=bits,
                           scale_min=SMIN, scale_max=SMAX)
    _, st = orc.replay(vc, T, np_params(case["vp"]), bits, SMIN, SMAX)
    assert np.isclose(st.s.min(), SMIN) and np.isclose(st.s.max(), SMAX)      # both clamps really are active
    dk, dv = dev(kc), dev(vc)
    got = gemv.decode_attn(dev(case["q"]), dk, dv, dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1]),
                           dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX, bits=bits, split_channels=split)
    _status_ok()
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert np.array_equal(dk.cpu().numpy(), wk) and np.array_equal(dv.cpu().numpy(), wv)


@pytest.mark.parametrize("bits,Hq,Hkv", [(4, 2, 2), (2, 4, 2)])
def test_decode_varlen_ragged_batch(bits, Hq, Hkv):
    """Per-sequence lengths on the device: every sequence must match a fixed-length call on itself alone."""
    B, D, Tmax = 4, 128, 150
    lens = [0, 37, 150, 96]
    case = make_case(640, B, Hq, Hkv, Tmax, bits)
    kp, vp = dev(case["kp"]), dev(case["vp"])
    ns = orc.n_super_for(Tmax + 1, bits)
    kc = torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    for b, T in enumerate(lens):
        if T:
            gemv.encode_kv_pair(kc[b:b + 1], dev(case["k"][b:b + 1, :, :T]), kp, vc[b:b + 1],
                                dev(case["v"][b:b + 1, :, :T]), vp, SMIN, SMAX, bits=bits)
    k_ref, v_ref = kc.clone(), vc.clone()
    kn = torch.stack([case["k"][b, :, T:T + 1] for b, T in enumerate(lens)]).cuda()
    vn = torch.stack([case["v"][b, :, T:T + 1] for b, T in enumerate(lens)]).cuda()
    q = dev(case["q"])
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    got = gemv.decode_attn_varlen(q, kc, vc, kn, vn, kp, vp, sl, 0.09, SMIN, SMAX, bits=bits)
    for b, T in enumerate(lens):
        want = gemv.decode_attn(q[b:b + 1], k_ref[b:b + 1], v_ref[b:b + 1], kn[b:b + 1], vn[b:b + 1], kp, vp, T, 0.09,
                                SMIN, SMAX, bits=bits, split_channels=False)     # same kernel layout: bit-equal
        assert torch.equal(got[b:b + 1], want)
    assert torch.equal(kc, k_ref) and torch.equal(vc, v_ref)
    _status_ok()
    # a length beyond the cache is reported through the status word and that stream is left alone
    sl2 = torch.tensor([0, 37, ns * (32 // bits), 96], dtype=torch.int32, device="cuda")
    before = kc.clone()
    gemv.decode_attn_varlen(q, kc, vc, kn, vn, kp, vp, sl2, 0.09, SMIN, SMAX, bits=bits)
    assert gemv.device_status() == 6
    assert torch.equal(kc[2], before[2])


def test_decode_with_infinite_mask_entries():
    """-inf mask entries (whole leading tiles masked, and a fully masked cache for one sequence) give the same
    result as dropping those tokens; no NaN from the online softmax."""
    B, H, T, bits, D = 2, 2, 100, 4, 128
    case = make_case(660, B, H, H, T, bits)
    kc, vc = oracle_prefill(case)
    mask = torch.zeros(B, T + 1)
    mask[0, :70] = float("-inf")                # two whole 32-token tiles and part of a third
    mask[1, :T] = float("-inf")                 # everything but the token being appended
    wk, wv = kc.copy(), vc.copy()
    want = orc.decode_attn(case["q"][:, :, 0].numpy(), wk, wv, case["k"][:, :, T].numpy(), case["v"][:, :, T].numpy(),
                           np_params(case["kp"]), np_params(case["vp"]), T, 0.1, mask=mask[:, None].numpy(), bits=bits,
                           scale_min=SMIN, scale_max=SMAX)
    assert np.isfinite(want).all()
    for kw in ({}, {"ckpt": True}):
        dk, dv = dev(kc), dev(vc)
        extra = {}
        if kw:
            kck, vck = gemv.alloc_ckpt(B, H, D, T + 1, 32, "cuda"), gemv.alloc_ckpt(B, H, D, T + 1, 32, "cuda")
            fk, fv = torch.zeros_like(dk), torch.zeros_like(dv)
            gemv.encode_kv_pair(fk, dev(case["k"][:, :, :T]), dev(case["kp"]), fv, dev(case["v"][:, :, :T]),
                                dev(case["vp"]), SMIN, SMAX, bits=bits, k_ckpt=kck, v_ckpt=vck, ckpt_interval=32)
            assert torch.equal(fk, dk) and torch.equal(fv, dv)
            extra = dict(k_ckpt=kck, v_ckpt=vck, ckpt_interval=32)
        got = gemv.decode_attn(dev(case["q"]), dk, dv, dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1]),
                               dev(case["kp"]), dev(case["vp"]), T, 0.1, SMIN, SMAX, mask=dev(mask), bits=bits, **extra)
        _status_ok()
        g = got.float().cpu().numpy()
        assert np.isfinite(g).all()
        np.testing.assert_allclose(g, want, rtol=RTOL, atol=ATOL)


def test_decode_steps_chain_like_generation():
    """Prefill with the kernel, then 40 fused decode steps; caches stay bit-identical to the oracle's."""
    B, H, T0, steps, bits, D = 2, 2, 21, 40, 4, 128
    case = make_case(7, B, H, H, T0 + steps, bits)
    kp, vp = dev(case["kp"]), dev(case["vp"])
    ns = orc.n_super_for(T0 + steps + 1, bits)
    dk = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    dv = torch.zeros_like(dk)
    gemv.encode_kv(dk, dev(case["k"][:, :, :T0]), *kp, SMIN, SMAX)
    gemv.encode_kv(dv, dev(case["v"][:, :, :T0]), *vp, SMIN, SMAX)
    ok_, ov_ = dk.cpu().numpy().copy(), dv.cpu().numpy().copy()
    g = torch.Generator().manual_seed(3)
    for s in range(steps):
        T = T0 + s
        q = torch.randn(B, H, 1, D, generator=g).half()
        want = orc.decode_attn(q[:, :, 0].numpy(), ok_, ov_, case["k"][:, :, T].numpy(), case["v"][:, :, T].numpy(),
                               np_params(case["kp"]), np_params(case["vp"]), T, 0.1, bits=bits,
                               scale_min=SMIN, scale_max=SMAX)
        got = gemv.decode_attn(dev(q), dk, dv, dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1]),
                               kp, vp, T, 0.1, SMIN, SMAX, bits=bits)
        np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    _status_ok()
    assert np.array_equal(dk.cpu().numpy(), ok_) and np.array_equal(dv.cpu().numpy(), ov_)


def test_unfused_trio_matches_fused():
    """forward_qk -> torch softmax -> forward_ov (the reference caller's sequence) vs the fused kernel."""
    case = make_case(55, 2, 4, 4, 300, 4)
    kc, vc = oracle_prefill(case)
    T, scaling = 300, 128 ** -0.5
    a_k, a_v, b_k, b_v = dev(kc), dev(vc), dev(kc), dev(vc)
    q, kn, vn = dev(case["q"]), dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1])
    logits = gemv.forward_qk(q, a_k, kn, *dev(case["kp"]), T, SMIN, SMAX)
    w = torch.softmax(logits.float() * scaling, dim=-1).to(torch.float16)
    o1 = gemv.forward_ov(w, a_v, vn, *dev(case["vp"]), SMIN, SMAX)
    o2 = gemv.decode_attn(q, b_k, b_v, kn, vn, dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX)
    assert torch.equal(a_k, b_k) and torch.equal(a_v, b_v)
    torch.testing.assert_close(o1.float(), o2.float(), rtol=4e-3, atol=4e-3 * float(o2.abs().max()))


def test_full_size_config2_properties():
    """The headline benchmark shape (B 128, H 32, T 4096, 4-bit): the batch is 2 distinct sequences replicated 64
    times, so every replica must reproduce the oracle's result for its sequence, and the appended slot must
    equal the oracle's.  Also checks that re-running the step with the same T overwrites the same slot."""
    B, H, T, bits, D, R = 128, 32, 4096, 4, 128, 2
    case = make_case(900, R, H, H, T, bits)
    from oracle import c_oracle
    ns = orc.n_super_for(T + 1, bits)
    kc = np.zeros(orc.cache_shape(R, H, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    c_oracle.encode(kc, case["k"][:, :, :T].numpy(), np_params(case["kp"]), bits, SMIN, SMAX)
    c_oracle.encode(vc, case["v"][:, :, :T].numpy(), np_params(case["vp"]), bits, SMIN, SMAX)
    # the kernel's own prefill must give the same caches
    dk = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    dv = torch.zeros_like(dk)
    rep = lambda t: dev(t).repeat(B // R, *([1] * (t.dim() - 1)))
    gemv.encode_kv(dk, rep(case["k"][:, :, :T]), *dev(case["kp"]), SMIN, SMAX)
    gemv.encode_kv(dv, rep(case["v"][:, :, :T]), *dev(case["vp"]), SMIN, SMAX)
    assert np.array_equal(dk[:R].cpu().numpy(), kc) and torch.equal(dk[:R], dk[-R:])
    assert np.array_equal(dv[:R].cpu().numpy(), vc)
    scaling = D ** -0.5
    want = c_oracle.decode_attn(case["q"][:, :, 0].numpy(), kc, vc, case["k"][:, :, T].numpy(),
                                case["v"][:, :, T].numpy(), np_params(case["kp"]), np_params(case["vp"]),
                                T, scaling, bits, SMIN, SMAX)
    for fast in (False, True):
        out = gemv.decode_attn(rep(case["q"]), dk, dv, rep(case["k"][:, :, T:T + 1]), rep(case["v"][:, :, T:T + 1]),
                               dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX, fast=fast)
        _status_ok()
        got = out.float().cpu().numpy().reshape(B // R, R, H, D)
        assert np.array_equal(got, np.broadcast_to(got[0], got.shape))        # replicas agree bit for bit
        np.testing.assert_allclose(got[0], want, rtol=RTOL, atol=ATOL)
        if not fast:
            assert np.array_equal(dk[:R].cpu().numpy(), kc) and np.array_equal(dv[-R:].cpu().numpy(), vc)
        else:
            frac, dmax = code_mismatch(dk[:R].cpu().numpy(), kc, T + 1, bits)
            assert dmax <= 1 and frac <= 1e-4


def test_full_size_config5_gqa_2bit_properties():
    """The long-context GQA benchmark shape (B 32, 32 q heads over 8 KV heads, T 32768, 2-bit): one distinct sequence
    replicated over the batch; every replica must reproduce the oracle's result and appended codes."""
    B, Hq, Hkv, T, bits, D = 32, 32, 8, 32768, 2, 128
    from oracle import c_oracle
    case = make_case(901, 1, Hq, Hkv, T, bits)
    ns = orc.n_super_for(T + 1, bits)
    kc = np.zeros(orc.cache_shape(1, Hkv, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    c_oracle.encode(kc, case["k"][:, :, :T].numpy(), np_params(case["kp"]), bits, SMIN, SMAX)
    c_oracle.encode(vc, case["v"][:, :, :T].numpy(), np_params(case["vp"]), bits, SMIN, SMAX)
    rep = lambda t: dev(t).repeat(B, *([1] * (t.dim() - 1)))
    dk = torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    dv = torch.zeros_like(dk)
    gemv.encode_kv(dk, rep(case["k"][:, :, :T]), *dev(case["kp"]), SMIN, SMAX, bits=bits)
    gemv.encode_kv(dv, rep(case["v"][:, :, :T]), *dev(case["vp"]), SMIN, SMAX, bits=bits)
    assert np.array_equal(dk[:1].cpu().numpy(), kc) and np.array_equal(dv[-1:].cpu().numpy(), vc)
    scaling = D ** -0.5
    want = c_oracle.decode_attn(case["q"][:, :, 0].numpy(), kc, vc, case["k"][:, :, T].numpy(),
                                case["v"][:, :, T].numpy(), np_params(case["kp"]), np_params(case["vp"]),
                                T, scaling, bits, SMIN, SMAX)
    out = gemv.decode_attn(rep(case["q"]), dk, dv, rep(case["k"][:, :, T:T + 1]), rep(case["v"][:, :, T:T + 1]),
                           dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX, bits=bits)
    _status_ok()
    got = out.float().cpu().numpy()
    assert np.array_equal(got, np.broadcast_to(got[:1], got.shape))
    np.testing.assert_allclose(got[:1], want, rtol=RTOL, atol=ATOL)
    assert np.array_equal(dk[:1].cpu().numpy(), kc) and np.array_equal(dv[-1:].cpu().numpy(), vc)
    assert torch.equal(dk[0], dk[-1]) and torch.equal(dv[0], dv[-1])
    # contracted replay over 32768 tokens: output within tolerance, appended codes within the 1e-4 allowance
    out_f = gemv.decode_attn(rep(case["q"]), dk, dv, rep(case["k"][:, :, T:T + 1]), rep(case["v"][:, :, T:T + 1]),
                             dev(case["kp"]), dev(case["vp"]), T, scaling, SMIN, SMAX, bits=bits, fast=True)
    _status_ok()
    np.testing.assert_allclose(out_f.float().cpu().numpy()[:1], want, rtol=RTOL, atol=ATOL)
    for got_c, want_c in ((dk[:1].cpu().numpy(), kc), (dv[:1].cpu().numpy(), vc)):
        a = orc.unpack_codes(got_c, T + 1, bits)[:, :, T].astype(np.int32)
        b = orc.unpack_codes(want_c, T + 1, bits)[:, :, T].astype(np.int32)
        d = np.abs(a - b)
        assert d.max() <= 1 and (d != 0).mean() <= 1e-4 + 1.5 / d.size, ((d != 0).sum(), d.size)


@pytest.mark.parametrize("bits", [4, 2])
def test_full_size_config3_prefill_properties(bits):
    """The prefill-quantise benchmark shape for one layer (B 16, H 32, T 8192): 2 distinct sequences replicated; every
    replica equals the oracle's codes and tail state; encoding in three chunks and appending the last 256
    tokens one by one gives the same cache as the one-shot prefill."""
    B, H, T, D, R, A = 16, 32, 8192, 128, 2, 256
    from oracle import c_oracle
    x = synth.gen_kv(902 + bits, R, H, T + A, D)
    p = synth.gen_params(903, H, D, bits)
    ns = orc.n_super_for(T + A, bits)
    want = np.zeros(orc.cache_shape(R, H, ns, D), np.uint8)
    tail_want = c_oracle.encode(want, x.numpy(), np_params(p), bits, SMIN, SMAX, want_tail=True)
    xd = dev(x).repeat(B // R, 1, 1, 1)
    pd = dev(p)
    one = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    t_one = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    gemv.encode_kv(one, xd, *pd, SMIN, SMAX, bits=bits, tail=t_one)
    assert np.array_equal(one[:R].cpu().numpy(), want) and torch.equal(one[:R], one[-R:])
    assert np.array_equal(t_one[:R].cpu().numpy().view(np.uint32), tail_want.view(np.uint32))
    parts = torch.zeros_like(one)
    t_parts = torch.empty_like(t_one)
    cuts = [0, 1000, 4099, T]                       # chunk boundaries inside words
    for a, b in zip(cuts[:-1], cuts[1:]):
        gemv.encode_kv(parts, xd[:, :, a:b].contiguous(), *pd, SMIN, SMAX, bits=bits, tail=t_parts, t_start=a)
    for t in range(T, T + A):
        gemv.append_kv(parts, xd[:, :, t:t + 1].contiguous(), *pd, t_parts, t, SMIN, SMAX, bits=bits)
    assert torch.equal(parts, one) and torch.equal(t_parts.view(torch.int32), t_one.view(torch.int32))


def test_bounded_wait_gives_up_and_reports():
    """A wait that nothing completes must end after its limit with a status code; the context stays usable."""
    import ctypes
    import time
    from adkv_b200 import _lib
    assert gemv.device_status() == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    _lib.check(_lib.load().adkv_selftest_wait_timeout(50, stream), "selftest")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.04 < dt < 1.0, dt
    assert gemv.device_status() == 7
    assert gemv.device_status() == 0                                   # reading clears it
    x = torch.arange(8, device="cuda")
    assert int((x * 2).sum()) == 56                                    # the device still answers


# ------------------------------------------------------------------------------- errors

def test_argument_errors_raise_runtime_error():
    H, D = 2, 128
    p = dev(synth.gen_params(1, H, D))
    cache = torch.zeros(1, H, 2, D // 4, 4, 4, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1, H, 16, D, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="kv_new must be float16"):
        gemv.encode_kv(cache, x.float(), *p, SMIN, SMAX)
    with pytest.raises(RuntimeError, match="kv_cache must be uint8"):
        gemv.encode_kv(cache.to(torch.int32), x, *p, SMIN, SMAX)
    with pytest.raises(RuntimeError, match="contiguous"):
        gemv.encode_kv(torch.zeros(1, H, 4, D // 4, 4, 4, dtype=torch.uint8, device="cuda")[:, :, ::2], x, *p, SMIN, SMAX)
    with pytest.raises(RuntimeError, match="capacity too small"):
        gemv.encode_kv(cache, torch.zeros(1, H, 17, D, dtype=torch.float16, device="cuda"), *p, SMIN, SMAX)
    q = torch.zeros(1, H, 1, D, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="no free supergroup"):
        gemv.forward_qk(q, cache, q, *p, 16, SMIN, SMAX)
    with pytest.raises(RuntimeError, match="non-negative"):
        gemv.forward_qk(q, cache, q, *p, -1, SMIN, SMAX)
    with pytest.raises(RuntimeError, match="k_zp must be float16"):
        gemv.forward_qk(q, cache, q, p[0].float(), *p[1:], 3, SMIN, SMAX)
    bad = torch.zeros(1, H, 2, 64 // 4, 4, 4, dtype=torch.uint8, device="cuda")        # head_dim 64
    with pytest.raises(RuntimeError, match="head dim"):
        gemv.forward_qk(torch.zeros(1, H, 1, 64, dtype=torch.float16, device="cuda"), bad,
                        torch.zeros(1, H, 1, 64, dtype=torch.float16, device="cuda"),
                        *[t[:, :64].contiguous() for t in p], 3, SMIN, SMAX)
    assert gemv.forward_qk(q, cache, q, *p, 15, SMIN, SMAX).shape == (1, H, 16)     # last legal slot


@pytest.mark.parametrize("bits,n_layers", [(4, 3), (2, 11)])
def test_layered_encode_and_append_equal_per_layer_calls(bits, n_layers):
    """adkv_encode_kv_layers / adkv_append_kv_layers (K and V of up to 8 layers per launch, 11 layers = two
    launches): caches and tails bit-identical to one call per layer, which the tests above hold to the oracle."""
    B, H, D, T, A = 2, 2, 128, 45, 5
    ns = orc.n_super_for(T + A, bits)
    mk = lambda: torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    tail = lambda: torch.zeros(B, H, 2, D, dtype=torch.float32, device="cuda")
    ks = [dev(synth.gen_kv(50 + 2 * l, B, H, T + A, D)) for l in range(n_layers)]
    vs = [dev(synth.gen_kv(51 + 2 * l, B, H, T + A, D)) for l in range(n_layers)]
    kps = [dev(synth.gen_params(70 + l, H, D, bits)) for l in range(n_layers)]
    vps = [dev(synth.gen_params(90 + l, H, D, bits)) for l in range(n_layers)]
    one = [(mk(), tail(), mk(), tail()) for _ in range(n_layers)]
    many = [(mk(), tail(), mk(), tail()) for _ in range(n_layers)]
    for l, (kc, kt, vc, vt) in enumerate(one):
        gemv.encode_kv_pair(kc, ks[l][:, :, :T], kps[l], vc, vs[l][:, :, :T], vps[l], SMIN, SMAX, bits=bits, k_tail=kt, v_tail=vt)
        for t in range(T, T + A):
            gemv.append_kv_pair(kc, ks[l][:, :, t:t + 1], kps[l], kt, vc, vs[l][:, :, t:t + 1], vps[l], vt, t, SMIN, SMAX, bits=bits)
    ls = gemv.LayerSet([(kc, kps[l], kt, vc, vps[l], vt) for l, (kc, kt, vc, vt) in enumerate(many)], bits=bits)
    gemv.encode_kv_layers(ls, [k[:, :, :T] for k in ks], [v[:, :, :T] for v in vs], SMIN, SMAX)
    for t in range(T, T + A):
        # the new tokens of all layers as one stacked buffer, the way a model step would leave them
        kn = torch.stack([k[:, :, t] for k in ks])
        vn = torch.stack([v[:, :, t] for v in vs])
        gemv.append_kv_layers(ls, kn, vn, t, SMIN, SMAX)
    _status_ok()
    for (kc1, kt1, vc1, vt1), (kc2, kt2, vc2, vt2) in zip(one, many):
        assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
        assert torch.equal(kt1.view(torch.int32), kt2.view(torch.int32)) and torch.equal(vt1.view(torch.int32), vt2.view(torch.int32))
    with pytest.raises(RuntimeError, match="no free supergroup"):
        gemv.append_kv_layers(ls, kn, vn, ns * (32 // bits), SMIN, SMAX)
