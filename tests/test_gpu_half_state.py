"""ADKV_FLAG_HALF_STATE: the arithmetic of the reference's CUDA kernels (fp16 state, gemv.cu:150-164).

Three parties are compared on a B200: this library's kernels with ``half_state=True``, the reference's own
kernels compiled for sm_100a (``oracle/_ref``, skipped when not built) and the numpy restatement
``oracle/adkv_oracle_half.py``.  Codes, appended codes and tail states must agree bit for bit (that is what
makes caches interchangeable); logits and outputs within fp16 accumulation error.
"""
import numpy as np
import pytest
import torch

from adkv_b200 import gemv, synth
from oracle import adkv_oracle as orc
from oracle import adkv_oracle_half as orh
from oracle import ref_cuda
from tests.util import SMAX, SMIN, np_params

pytestmark = pytest.mark.gpu
needs_ref = pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/adkv_gemv.so has not been built")

D = 128


def live_params(seed, H, bits=4, random=True):
    if not random:
        return synth.gen_params(seed, H, D, bits, device="cuda")
    g = torch.Generator().manual_seed(seed)
    p = (torch.randn(H, D, generator=g) * 0.5, torch.rand(H, D, generator=g) * 1.5 + 0.3,
         torch.rand(H, D, generator=g) * 0.2, torch.rand(H, D, generator=g) * 0.08,
         torch.rand(H, D, generator=g) * (2 ** (bits - 1)) * 0.6 + 0.2)
    return tuple(t.half().cuda() for t in p)


def np16(p):
    return tuple(t.cpu().numpy() for t in p)


def zeros_cache(B, H, tokens, bits, extra=0):
    return torch.zeros(orc.cache_shape(B, H, orc.n_super_for(tokens, bits) + extra, D), dtype=torch.uint8, device="cuda")


# ------------------------------------------------------------------------------------ encode

@needs_ref
@pytest.mark.parametrize("random", [False, True])
@pytest.mark.parametrize("T", [1, 7, 8, 9, 33, 64, 130, 1000, 4096])
def test_encode_codes_equal_reference_kernel(T, random):
    B, H = 2, 5
    ref = ref_cuda.module()
    x = synth.gen_kv(800 + T, B, H, T, D, outlier_mode="persistent" if T % 2 else "scale").cuda()
    p = live_params(T, H, random=random)
    mine, theirs = zeros_cache(B, H, T, 4), zeros_cache(B, H, T, 4)
    ref.encode_kv(theirs, x, *p, SMIN, SMAX)
    gemv.encode_kv(mine, x, *p, SMIN, SMAX, bits=4, half_state=True)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    assert gemv.device_status() == 0


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("T", [1, 9, 17, 77, 300])
def test_encode_codes_and_tail_equal_numpy_restatement(T, bits):
    B, H = 2, 3
    x = synth.gen_kv(810 + T, B, H, T, D)
    p = live_params(3 + T, H, bits)
    want = np.zeros(orc.cache_shape(B, H, orc.n_super_for(T, bits), D), np.uint8)
    _, st = orh.encode_kv(want, x.numpy(), np16(p), bits)
    mine = zeros_cache(B, H, T, bits)
    tail = torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda")
    gemv.encode_kv(mine, x.cuda(), *p, SMIN, SMAX, bits=bits, half_state=True, tail=tail)
    assert np.array_equal(mine.cpu().numpy(), want)
    t = tail.cpu().numpy()
    assert np.array_equal(t[:, :, 0], st.zp.astype(np.float32)) and np.array_equal(t[:, :, 1], st.sc.astype(np.float32))


@pytest.mark.parametrize("bits", [4, 2])
def test_chunked_encode_and_appends_equal_one_shot(bits):
    B, H, T = 2, 2, 93
    x = synth.gen_kv(820, B, H, T, D).cuda()
    kp, vp = live_params(5, H, bits), live_params(6, H, bits)
    full_k, full_v = zeros_cache(B, H, T, bits), zeros_cache(B, H, T, bits)
    tk, tv = (torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda") for _ in range(2))
    gemv.encode_kv_pair(full_k, x, kp, full_v, x.flip(2).contiguous(), vp, SMIN, SMAX, bits=bits, half_state=True,
                        k_tail=tk, v_tail=tv)
    pk, pv = torch.zeros_like(full_k), torch.zeros_like(full_v)
    ck, cv = torch.empty_like(tk), torch.empty_like(tv)
    xv = x.flip(2).contiguous()
    gemv.encode_kv_pair(pk, x[:, :, :21].contiguous(), kp, pv, xv[:, :, :21].contiguous(), vp, SMIN, SMAX, bits=bits,
                        half_state=True, k_tail=ck, v_tail=cv)
    gemv.encode_kv_pair(pk, x[:, :, 21:70].contiguous(), kp, pv, xv[:, :, 21:70].contiguous(), vp, SMIN, SMAX,
                        bits=bits, half_state=True, k_tail=ck, v_tail=cv, t_start=21)
    for t in range(70, T):
        if t % 2:
            gemv.append_kv_pair(pk, x[:, :, t:t + 1].contiguous(), kp, ck, pv, xv[:, :, t:t + 1].contiguous(), vp, cv, t,
                                SMIN, SMAX, bits=bits, half_state=True)
        else:
            gemv.append_kv(pk, x[:, :, t:t + 1].contiguous(), *kp, ck, t, SMIN, SMAX, bits=bits, half_state=True)
            gemv.append_kv(pv, xv[:, :, t:t + 1].contiguous(), *vp, cv, t, SMIN, SMAX, bits=bits, half_state=True)
    assert torch.equal(pk, full_k) and torch.equal(pv, full_v)
    assert torch.equal(ck, tk) and torch.equal(cv, tv)


def test_degenerate_scales_follow_the_reference_semantics():
    """Zero scale (division by zero: saturate, NaN -> code 0) and a scale that overflows fp16."""
    B, H, T = 1, 1, 40
    x = synth.gen_kv(830, B, H, T, D)
    x[0, 0, :, :8] = 0
    g = torch.Generator().manual_seed(1)
    p = [torch.zeros(H, D), torch.ones(H, D), torch.full((H, D), 0.1), torch.full((H, D), 0.05), torch.full((H, D), 3.5)]
    p[1][0, :16] = 0                    # zero scale: x = 0 gives 0/0, others x/0
    p[3][0, 16:32] = 8.0                # beta*|q| blows the scale up to inf within a few tokens
    p = tuple(t.half().cuda() for t in p)
    want = np.zeros(orc.cache_shape(B, H, orc.n_super_for(T, 4), D), np.uint8)
    orh.encode_kv(want, x.numpy(), np16(p), 4)
    mine = zeros_cache(B, H, T, 4)
    gemv.encode_kv(mine, x.cuda(), *p, SMIN, SMAX, bits=4, half_state=True)
    assert np.array_equal(mine.cpu().numpy(), want)
    if ref_cuda.available():
        theirs = zeros_cache(B, H, T, 4)
        ref_cuda.module().encode_kv(theirs, x.cuda(), *p, SMIN, SMAX)
        assert torch.equal(mine, theirs)


# ------------------------------------------------------------------------------------ decode

def _prefilled(seed, B, Hkv, T, bits, random=True):
    k = synth.gen_kv(seed, B, Hkv, T + 1, D, outlier_mode="persistent").cuda()
    v = synth.gen_kv(seed + 1, B, Hkv, T + 1, D, outlier_mode="persistent").cuda()
    kp, vp = live_params(seed + 2, Hkv, bits, random), live_params(seed + 3, Hkv, bits, random)
    kc, vc = zeros_cache(B, Hkv, T + 1, bits, 1), zeros_cache(B, Hkv, T + 1, bits, 1)
    if T:
        gemv.encode_kv_pair(kc, k[:, :, :T].contiguous(), kp, vc, v[:, :, :T].contiguous(), vp, SMIN, SMAX, bits=bits,
                            half_state=True)
    return k, v, kp, vp, kc, vc


@needs_ref
@pytest.mark.parametrize("T", [0, 1, 8, 9, 31, 32, 33, 77, 256, 1023])
def test_trio_appends_equal_reference_kernels_and_outputs_are_close(T):
    B, H = 2, 6
    ref = ref_cuda.module()
    k, v, kp, vp, kc, vc = _prefilled(900 + T, B, H, T, 4)
    q = synth.gen_q(950 + T, B, H, D).cuda()
    rk, rv = kc.clone(), vc.clone()
    kn, vn = k[:, :, T:].contiguous(), v[:, :, T:].contiguous()
    lt = ref.forward_qk(q, rk, kn, *kp, T, SMIN, SMAX)
    lm = gemv.forward_qk(q, kc, kn, *kp, T, SMIN, SMAX, bits=4, half_state=True)
    assert torch.equal(kc, rk)
    a, b = lm.float().cpu().numpy(), lt.float().cpu().numpy()
    np.testing.assert_allclose(b, a, rtol=2e-2, atol=2e-2 * max(1.0, np.abs(a).max()))
    attn = torch.softmax(lm.float() * D ** -0.5, dim=-1).half()
    ot = ref.forward_ov(attn, rv, vn, *vp, SMIN, SMAX)
    om = gemv.forward_ov(attn, vc, vn, *vp, SMIN, SMAX, bits=4, half_state=True)
    assert torch.equal(vc, rv)
    a, b = om.float().cpu().numpy().reshape(B * H, D), ot.float().cpu().numpy().reshape(B * H, D)
    np.testing.assert_allclose(b, a, rtol=2e-2, atol=2e-2 * max(1.0, np.abs(a).max()))
    assert gemv.device_status() == 0


CASES = [(2, 4, 4, 0, 4), (2, 4, 4, 5, 4), (2, 4, 4, 32, 4), (1, 4, 4, 100, 4), (2, 8, 2, 45, 4), (1, 8, 1, 70, 4),
         (2, 4, 4, 17, 2), (1, 4, 2, 130, 2), (1, 16, 2, 64, 2), (1, 2, 2, 700, 4)]


@pytest.mark.parametrize("B,Hq,Hkv,T,bits", CASES)
def test_fused_decode_against_numpy_restatement(B, Hq, Hkv, T, bits):
    k, v, kp, vp, kc, vc = _prefilled(1000 + T, B, Hkv, T, bits)
    q = synth.gen_q(1001 + T, B, Hq, D).cuda()
    mask = torch.zeros(B, T + 1)
    mask[0, : T // 3] = -1e4
    okc, ovc = kc.cpu().numpy().copy(), vc.cpu().numpy().copy()
    want, _ = orh.decode_attn(q[:, :, 0].cpu().numpy(), okc, ovc, k[:, :, T].cpu().numpy(), v[:, :, T].cpu().numpy(),
                              np16(kp), np16(vp), T, D ** -0.5, bits, mask=mask.numpy())
    got = gemv.decode_attn(q, kc, vc, k[:, :, T:].contiguous(), v[:, :, T:].contiguous(), kp, vp, T, D ** -0.5,
                           SMIN, SMAX, bits=bits, half_state=True, mask=mask.cuda())
    assert np.array_equal(kc.cpu().numpy(), okc) and np.array_equal(vc.cpu().numpy(), ovc)     # appended codes
    g = got.float().cpu().numpy()
    # logits are summed in fp16 over the 128 channels (as in the reference's kernel): tolerance of that sum
    np.testing.assert_allclose(g, want, rtol=2e-2, atol=2e-2 * max(1.0, np.abs(want).max()))
    assert gemv.device_status() == 0


@pytest.mark.parametrize("bits", [4, 2])
def test_trio_against_numpy_restatement(bits):
    B, Hq, Hkv, T = 2, 4, 2, 75
    k, v, kp, vp, kc, vc = _prefilled(1100, B, Hkv, T, bits)
    q = synth.gen_q(1101, B, Hq, D).cuda()
    okc, ovc = kc.cpu().numpy().copy(), vc.cpu().numpy().copy()
    want, want_logits = orh.decode_attn(q[:, :, 0].cpu().numpy(), okc, ovc, k[:, :, T].cpu().numpy(),
                                        v[:, :, T].cpu().numpy(), np16(kp), np16(vp), T, D ** -0.5, bits)
    logits = gemv.forward_qk(q, kc, k[:, :, T:].contiguous(), *kp, T, SMIN, SMAX, bits=bits, half_state=True)
    lg = logits.float().cpu().numpy()
    np.testing.assert_allclose(lg, want_logits, rtol=1e-2, atol=1e-2 * max(1.0, np.abs(want_logits).max()))
    attn = torch.softmax(torch.from_numpy(want_logits).cuda().float() * D ** -0.5, dim=-1).half()
    out = gemv.forward_ov(attn, vc, v[:, :, T:].contiguous(), *vp, SMIN, SMAX, bits=bits, half_state=True)
    assert np.array_equal(kc.cpu().numpy(), okc) and np.array_equal(vc.cpu().numpy(), ovc)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2 * max(1.0, np.abs(want).max()))


def test_varlen_equals_per_sequence_calls():
    B, H, bits = 3, 2, 4
    lens = [40, 7, 33]
    Tmax = max(lens)
    k, v, kp, vp, _, _ = _prefilled(1200, B, H, Tmax, bits)
    q = synth.gen_q(1201, B, H, D).cuda()
    kc, vc = zeros_cache(B, H, Tmax + 1, bits, 1), zeros_cache(B, H, Tmax + 1, bits, 1)
    for b, L in enumerate(lens):
        gemv.encode_kv_pair(kc[b:b + 1], k[b:b + 1, :, :L].contiguous(), kp, vc[b:b + 1], v[b:b + 1, :, :L].contiguous(),
                            vp, SMIN, SMAX, bits=bits, half_state=True)
    kc2, vc2 = kc.clone(), vc.clone()
    kn = torch.stack([k[b, :, L] for b, L in enumerate(lens)]).unsqueeze(2).contiguous()
    vn = torch.stack([v[b, :, L] for b, L in enumerate(lens)]).unsqueeze(2).contiguous()
    out = gemv.decode_attn_varlen(q, kc, vc, kn, vn, kp, vp, torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                  D ** -0.5, SMIN, SMAX, bits=bits, half_state=True)
    for b, L in enumerate(lens):
        o = gemv.decode_attn(q[b:b + 1], kc2[b:b + 1], vc2[b:b + 1], kn[b:b + 1], vn[b:b + 1], kp, vp, L, D ** -0.5,
                             SMIN, SMAX, bits=bits, half_state=True)
        assert torch.equal(o, out[b:b + 1])
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)


@pytest.mark.parametrize("bits,Hq,Hkv,T,interval", [(4, 4, 4, 200, 64), (4, 8, 2, 191, 32), (2, 4, 2, 300, 96), (4, 2, 2, 63, 64)])
def test_checkpointed_decode_equals_plain_decode(bits, Hq, Hkv, T, interval):
    """State checkpoints in the fp16-state arithmetic: the checkpoints the prefill writes are the states of the numpy
    restatement at those tokens, and the segment-parallel decode appends the same codes as the plain one."""
    B = 2
    k = synth.gen_kv(1700 + T, B, Hkv, T + 1, D, outlier_mode="persistent").cuda()
    v = synth.gen_kv(1701 + T, B, Hkv, T + 1, D, outlier_mode="persistent").cuda()
    q = synth.gen_q(1702 + T, B, Hq, D).cuda()
    kp, vp = live_params(T, Hkv, bits), live_params(T + 1, Hkv, bits)
    kc, vc = zeros_cache(B, Hkv, T + 1, bits, 1), zeros_cache(B, Hkv, T + 1, bits, 1)
    kck, vck = gemv.alloc_ckpt(B, Hkv, D, T + 1, interval, "cuda"), gemv.alloc_ckpt(B, Hkv, D, T + 1, interval, "cuda")
    gemv.encode_kv_pair(kc, k[:, :, :T].contiguous(), kp, vc, v[:, :, :T].contiguous(), vp, SMIN, SMAX, bits=bits,
                        half_state=True, k_ckpt=kck, v_ckpt=vck, ckpt_interval=interval)
    # checkpoint j = state before token (j+1)*interval, from the numpy restatement
    zp0, s0, alpha, beta, target = np16(kp)
    st = orh.init_state(B, zp0, s0)
    xs = k[:, :, :T].cpu().numpy()
    for j in range(T // interval):
        orh.encode_scan(xs[:, :, j * interval:(j + 1) * interval], st, alpha, beta, target, bits)
        got = kck[:, :, j].cpu().numpy()
        assert np.array_equal(got[:, :, 0], st.zp.astype(np.float32)) and np.array_equal(got[:, :, 1], st.sc.astype(np.float32))
    pk, pv = kc.clone(), vc.clone()
    kn, vn = k[:, :, T:].contiguous(), v[:, :, T:].contiguous()
    mask = torch.zeros(B, T + 1, device="cuda")
    mask[1, : T // 2] = -1e4
    plain = gemv.decode_attn(q, pk, pv, kn, vn, kp, vp, T, D ** -0.5, SMIN, SMAX, bits=bits, half_state=True, mask=mask)
    split = gemv.decode_attn(q, kc, vc, kn, vn, kp, vp, T, D ** -0.5, SMIN, SMAX, bits=bits, half_state=True, mask=mask,
                             k_ckpt=kck, v_ckpt=vck, ckpt_interval=interval)
    assert torch.equal(kc, pk) and torch.equal(vc, pv)
    a, b = plain.float(), split.float()
    torch.testing.assert_close(b, a, rtol=2e-2, atol=2e-2 * max(1.0, float(a.abs().max())))
    assert gemv.device_status() == 0


@pytest.mark.parametrize("bits", [4, 2])
def test_appends_keep_the_checkpoints_that_prefill_would_write(bits):
    B, H, T0, steps, interval = 2, 2, 40, 100, 32
    x = synth.gen_kv(1800, B, H, T0 + steps, D).cuda()
    kp, vp = live_params(31, H, bits), live_params(32, H, bits)
    cap = T0 + steps
    ck_full, cv_full = gemv.alloc_ckpt(B, H, D, cap, interval, "cuda"), gemv.alloc_ckpt(B, H, D, cap, interval, "cuda")
    fk, fv = zeros_cache(B, H, cap, bits), zeros_cache(B, H, cap, bits)
    gemv.encode_kv_pair(fk, x, kp, fv, x, vp, SMIN, SMAX, bits=bits, half_state=True, k_ckpt=ck_full, v_ckpt=cv_full,
                        ckpt_interval=interval)
    ck, cv = torch.zeros_like(ck_full), torch.zeros_like(cv_full)
    pk, pv = torch.zeros_like(fk), torch.zeros_like(fv)
    tk, tv = (torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda") for _ in range(2))
    gemv.encode_kv_pair(pk, x[:, :, :T0].contiguous(), kp, pv, x[:, :, :T0].contiguous(), vp, SMIN, SMAX, bits=bits,
                        half_state=True, k_tail=tk, v_tail=tv, k_ckpt=ck, v_ckpt=cv, ckpt_interval=interval)
    q = synth.gen_q(1801, B, H, D).cuda()
    for t in range(T0, T0 + steps):
        xn = x[:, :, t:t + 1].contiguous()
        if t % 3 == 0:    # a decode step maintains the checkpoints too (the tail state is not its business)
            gemv.decode_attn(q, pk, pv, xn, xn, kp, vp, t, D ** -0.5, SMIN, SMAX, bits=bits, half_state=True,
                             k_ckpt=ck, v_ckpt=cv, ckpt_interval=interval)
            sk, sv = pk.clone(), pv.clone()       # and the append kernel writes the same code and advances the tails
            gemv.append_kv_pair(sk, xn, kp, tk, sv, xn, vp, tv, t, SMIN, SMAX, bits=bits, half_state=True)
            assert torch.equal(sk, pk) and torch.equal(sv, pv)
        else:
            gemv.append_kv_pair(pk, xn, kp, tk, pv, xn, vp, tv, t, SMIN, SMAX, bits=bits, half_state=True,
                                k_ckpt=ck, v_ckpt=cv, ckpt_interval=interval)
    assert torch.equal(pk, fk) and torch.equal(pv, fv)
    assert torch.equal(ck, ck_full) and torch.equal(cv, cv_full)


@needs_ref
def test_generation_with_cache_object_leaves_the_reference_kernels_caches():
    """Prefill + 70 decode steps: the cache object in half_state mode (fused step) and a loop over the
    reference's own kernels end with identical buffers, and their step outputs stay close."""
    from adkv_b200.cache import KVCacheLayer
    ref = ref_cuda.module()
    B, H, T0, steps = 2, 4, 50, 70
    k = synth.gen_kv(1400, B, H, T0 + steps, D, outlier_mode="persistent").cuda()
    v = synth.gen_kv(1401, B, H, T0 + steps, D, outlier_mode="persistent").cuda()
    kp, vp = synth.gen_params(1402, H, D, 4, device="cuda"), synth.gen_params(1403, H, D, 4, device="cuda")
    g = torch.Generator().manual_seed(0)
    qs = [torch.randn(B, H, 1, D, generator=g).half().cuda() for _ in range(steps)]
    flat = lambda ps: tuple(p.reshape(-1) for p in ps)
    layer = KVCacheLayer(bits=4, fused=True, half_state=True, capacity_tokens=T0 + steps)
    layer.prefill(k[:, :, :T0], v[:, :, :T0], *flat(kp), *flat(vp))
    rk = torch.zeros_like(layer.key_states)
    rv = torch.zeros_like(layer.value_states)
    ref.encode_kv(rk, k[:, :, :T0].contiguous(), *kp, SMIN, SMAX)
    ref.encode_kv(rv, v[:, :, :T0].contiguous(), *vp, SMIN, SMAX)
    assert torch.equal(rk, layer.key_states) and torch.equal(rv, layer.value_states)
    scaling = D ** -0.5
    for s in range(steps):
        T = T0 + s
        kn, vn = k[:, :, T:T + 1].contiguous(), v[:, :, T:T + 1].contiguous()
        o, _ = layer.decode(qs[s], kn, vn, *flat(kp), *flat(vp), attention_mask=None, scaling=scaling)
        logits = ref.forward_qk(qs[s], rk, kn, *kp, T, SMIN, SMAX)
        attn = torch.softmax(logits.float() * scaling, dim=-1).half()
        ro = ref.forward_ov(attn, rv, vn, *vp, SMIN, SMAX).reshape(B, H, D)
        a, b = o.float().reshape(B, H, D), ro.float()
        torch.testing.assert_close(b, a, rtol=3e-2, atol=3e-2 * max(1.0, float(a.abs().max())))
    assert torch.equal(rk, layer.key_states) and torch.equal(rv, layer.value_states)


# ------------------------------------------------------------------------------------ head dims 256 / 512

def _wide_params(seed, H, Dw):
    g = torch.Generator().manual_seed(seed)
    p = (torch.randn(H, Dw, generator=g) * 0.5, torch.rand(H, Dw, generator=g) * 1.5 + 0.3,
         torch.rand(H, Dw, generator=g) * 0.2, torch.rand(H, Dw, generator=g) * 0.08,
         torch.rand(H, Dw, generator=g) * 4 + 0.5)
    return tuple(t.half().cuda() for t in p)


@needs_ref
@pytest.mark.parametrize("Dw", [256, 512])
@pytest.mark.parametrize("T", [0, 9, 77, 300])
def test_wide_heads_equal_reference_kernels(Dw, T):
    B, H = 2, 3
    ref = ref_cuda.module()
    k = synth.gen_kv(1500 + T, B, H, T + 1, Dw, outlier_mode="persistent").cuda()
    v = synth.gen_kv(1501 + T, B, H, T + 1, Dw, outlier_mode="persistent").cuda()
    q = synth.gen_q(1502 + T, B, H, Dw).cuda()
    kp, vp = _wide_params(T, H, Dw), _wide_params(T + 1, H, Dw)
    shape = orc.cache_shape(B, H, orc.n_super_for(T + 1, 4) + 1, Dw)
    kc, vc = (torch.zeros(shape, dtype=torch.uint8, device="cuda") for _ in range(2))
    rk, rv = torch.zeros_like(kc), torch.zeros_like(vc)
    if T:
        gemv.encode_kv_pair(kc, k[:, :, :T].contiguous(), kp, vc, v[:, :, :T].contiguous(), vp, SMIN, SMAX, half_state=True)
        ref.encode_kv(rk, k[:, :, :T].contiguous(), *kp, SMIN, SMAX)
        ref.encode_kv(rv, v[:, :, :T].contiguous(), *vp, SMIN, SMAX)
        assert torch.equal(kc, rk) and torch.equal(vc, rv)
    kn, vn = k[:, :, T:].contiguous(), v[:, :, T:].contiguous()
    fk, fv = kc.clone(), vc.clone()
    lt = ref.forward_qk(q, rk, kn, *kp, T, SMIN, SMAX)
    lm = gemv.forward_qk(q, kc, kn, *kp, T, SMIN, SMAX, half_state=True)
    assert torch.equal(kc, rk)
    a, b = lm.float().cpu().numpy(), lt.float().cpu().numpy()
    np.testing.assert_allclose(b, a, rtol=3e-2, atol=3e-2 * max(1.0, np.abs(a).max()))
    attn = torch.softmax(lm.float() * Dw ** -0.5, dim=-1).half()
    ot = ref.forward_ov(attn, rv, vn, *vp, SMIN, SMAX)
    om = gemv.forward_ov(attn, vc, vn, *vp, SMIN, SMAX, half_state=True)
    assert torch.equal(vc, rv)
    a, b = om.float().cpu().numpy().reshape(B * H, Dw), ot.float().cpu().numpy().reshape(B * H, Dw)
    np.testing.assert_allclose(b, a, rtol=3e-2, atol=3e-2 * max(1.0, np.abs(a).max()))
    # fused step: same appended codes, output close to the three calls
    of = gemv.decode_attn(q, fk, fv, kn, vn, kp, vp, T, Dw ** -0.5, SMIN, SMAX, half_state=True)
    assert torch.equal(fk, kc) and torch.equal(fv, vc)
    f = of.float().cpu().numpy().reshape(B * H, Dw)
    np.testing.assert_allclose(f, a, rtol=3e-2, atol=3e-2 * max(1.0, np.abs(a).max()))
    assert gemv.device_status() == 0


@needs_ref
def test_full_size_config2_equals_reference_kernels():
    """The headline workload (batch 128 x 32 heads x 4096 tokens, 4-bit) in the fp16-state arithmetic: the 1 GiB cache
    our prefill writes, and the codes the fused step appends, are byte for byte what the reference's kernels write."""
    ref = ref_cuda.module()
    B, H, T = 128, 32, 4096
    kp = synth.gen_params(1603, H, D, 4, device="cuda")
    ns = orc.n_super_for(T + 1, 4)
    mine = torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    theirs = torch.zeros_like(mine)
    for b0 in range(0, B, 16):
        x = synth.gen_kv(1600 + b0, 16, H, T, D, device="cuda")
        gemv.encode_kv(mine[b0:b0 + 16], x, *kp, SMIN, SMAX, half_state=True)
        ref.encode_kv(theirs[b0:b0 + 16], x, *kp, SMIN, SMAX)
        del x
    assert torch.equal(mine, theirs)
    q = synth.gen_q(1601, B, H, D, device="cuda")
    kn = synth.gen_kv(1602, B, H, 1, D, device="cuda", pos0=T)
    vmine, vtheirs = mine.clone(), theirs.clone()          # the same codes serve as the V cache
    out = gemv.decode_attn(q, mine, vmine, kn, kn, kp, kp, T, D ** -0.5, SMIN, SMAX, half_state=True)
    logits = ref.forward_qk(q, theirs, kn, *kp, T, SMIN, SMAX)
    attn = torch.softmax(logits.float() * D ** -0.5, dim=-1).half()
    ro = ref.forward_ov(attn, vtheirs, kn, *kp, SMIN, SMAX).reshape(B, H, D)
    assert torch.equal(mine, theirs) and torch.equal(vmine, vtheirs)
    a, b = out.float(), ro.float()
    torch.testing.assert_close(b, a, rtol=3e-2, atol=3e-2 * max(1.0, float(a.abs().max())))
    assert gemv.device_status() == 0
