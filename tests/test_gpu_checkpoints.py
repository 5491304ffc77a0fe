"""State checkpoints and the segment-parallel decode step (GPU)."""
import numpy as np
import pytest
import torch

from adkv_b200 import gemv, synth
from oracle import adkv_oracle as orc
from tests.util import SMAX, SMIN, dev, make_case, np_params, oracle_prefill

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 2e-3


def _oracle_states(x, params, bits, at):
    """Oracle states (zp, s) before each token index in `at`."""
    p = np_params(params)
    st = orc.init_state(x.shape[0], p[0], p[1])
    out, t0 = {}, 0
    for t in sorted(at):
        orc.encode_scan(x[:, :, t0:t].numpy().astype(np.float32), st, p[2], p[3], p[4], bits, SMIN, SMAX, want_xhat=False)
        out[t] = (st.zp.copy(), st.s.copy())
        t0 = t
    return out


@pytest.mark.parametrize("bits,Hq,Hkv,T0,steps,S", [(4, 2, 2, 150, 20, 64), (2, 4, 2, 100, 70, 32), (4, 2, 2, 63, 3, 64),
                                                    (4, 2, 2, 0, 40, 32)])
def test_checkpointed_generation_matches_plain(bits, Hq, Hkv, T0, steps, S):
    B, D = 2, 128
    case = make_case(500 + T0, B, Hq, Hkv, T0 + steps, bits)
    kp, vp = dev(case["kp"]), dev(case["vp"])
    Ttot = T0 + steps
    ns = orc.n_super_for(Ttot + 1, bits)
    mk = lambda: torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    k1, v1, k2, v2 = mk(), mk(), mk(), mk()
    kck = gemv.alloc_ckpt(B, Hkv, D, Ttot + 1, S, "cuda")
    vck = gemv.alloc_ckpt(B, Hkv, D, Ttot + 1, S, "cuda")
    if T0:
        gemv.encode_kv_pair(k1, dev(case["k"][:, :, :T0]), kp, v1, dev(case["v"][:, :, :T0]), vp, SMIN, SMAX, bits=bits)
        gemv.encode_kv_pair(k2, dev(case["k"][:, :, :T0]), kp, v2, dev(case["v"][:, :, :T0]), vp, SMIN, SMAX, bits=bits,
                            k_ckpt=kck, v_ckpt=vck, ckpt_interval=S)
    g = torch.Generator().manual_seed(1)
    mask = torch.zeros(B, Ttot + 1)
    mask[0, :5] = torch.finfo(torch.float16).min
    for s in range(steps):
        T = T0 + s
        q = dev(torch.randn(B, Hq, 1, D, generator=g).half())
        kn, vn = dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1])
        m = dev(mask[:, :T + 1])
        o1 = gemv.decode_attn(q, k1, v1, kn, vn, kp, vp, T, 0.09, SMIN, SMAX, bits=bits, mask=m)
        o2 = gemv.decode_attn(q, k2, v2, kn, vn, kp, vp, T, 0.09, SMIN, SMAX, bits=bits, mask=m,
                              k_ckpt=kck, v_ckpt=vck, ckpt_interval=S)
        torch.testing.assert_close(o2.float(), o1.float(), rtol=RTOL, atol=ATOL)
    assert gemv.device_status() == 0
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    # every checkpoint reached equals the oracle's state at that token, bit for bit
    n_ck = (Ttot) // S
    want = _oracle_states(case["k"][:, :, :Ttot], case["kp"], bits, [(k + 1) * S for k in range(n_ck)])
    got = kck.cpu().numpy()
    for k in range(n_ck):
        zp, s_ = want[(k + 1) * S]
        assert np.array_equal(got[:, :, k, 0].view(np.uint32), zp.view(np.uint32)), k
        assert np.array_equal(got[:, :, k, 1].view(np.uint32), s_.view(np.uint32)), k


def test_checkpointed_append_and_errors():
    B, H, D, T, S, bits = 1, 2, 128, 95, 32, 4
    x = synth.gen_kv(9, B, H, T + 2, D)
    p = dev(synth.gen_params(10, H, D, bits))
    ns = orc.n_super_for(T + 2, bits)
    mk = lambda: torch.zeros(orc.cache_shape(B, H, ns, D), dtype=torch.uint8, device="cuda")
    kc, vc = mk(), mk()
    kck, vck = gemv.alloc_ckpt(B, H, D, T + 2, S, "cuda"), gemv.alloc_ckpt(B, H, D, T + 2, S, "cuda")
    tk, tv = (torch.empty(B, H, 2, D, dtype=torch.float32, device="cuda") for _ in range(2))
    gemv.encode_kv_pair(kc, dev(x[:, :, :T]), p, vc, dev(x[:, :, :T]), p, SMIN, SMAX, bits=bits, k_tail=tk, v_tail=tv,
                        k_ckpt=kck, v_ckpt=vck, ckpt_interval=S)
    assert kck.shape[2] == 3 and float(kck[:, :, 2].abs().sum()) == 0.0          # checkpoint 96 not reached yet
    gemv.append_kv_pair(kc, dev(x[:, :, T:T + 1]), p, tk, vc, dev(x[:, :, T:T + 1]), p, tv, T, SMIN, SMAX, bits=bits,
                        k_ckpt=kck, v_ckpt=vck, ckpt_interval=S)
    assert torch.equal(kck[:, :, 2].view(torch.int32), tk.view(torch.int32))    # state before token 96 = tail after 95
    assert torch.equal(kck, vck)
    q = torch.zeros(B, H, 1, D, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 32"):
        gemv.decode_attn(q, kc, vc, q, q, p, p, T + 1, 0.1, SMIN, SMAX, k_ckpt=kck, v_ckpt=vck, ckpt_interval=48)
    with pytest.raises(RuntimeError, match="scratch"):
        gemv.decode_attn(q, kc, vc, q, q, p, p, T + 1, 0.1, SMIN, SMAX, k_ckpt=kck, v_ckpt=vck, ckpt_interval=S,
                         scratch=torch.empty(64, dtype=torch.uint8, device="cuda"))
    small = gemv.alloc_ckpt(B, H, D, 64, S, "cuda")
    with pytest.raises(RuntimeError, match="capacity"):
        gemv.decode_attn(q, kc, vc, q, q, p, p, T + 1, 0.1, SMIN, SMAX, k_ckpt=small, v_ckpt=small.clone(), ckpt_interval=S)


def test_segment_that_gives_up_marks_its_result():
    """Failure path of the checkpointed step, made on purpose without faulting anything: with the K warps muted no
    logits ever arrive, every V warp's bounded wait runs out (1 s), the kernels end normally and the context stays
    usable.  The status word names the wait, and the output is NaN everywhere -- not the previous call's result,
    which the scratch memory still held."""
    import ctypes
    import time

    from adkv_b200 import _lib
    B, H, T, bits, D, iv = 1, 2, 70, 4, 128, 32
    case = make_case(31, B, H, H, T, bits)
    kc, vc = oracle_prefill(case)
    dk, dv = dev(kc), dev(vc)
    kck, vck = gemv.alloc_ckpt(B, H, D, T + 1, iv, "cuda"), gemv.alloc_ckpt(B, H, D, T + 1, iv, "cuda")
    gemv.encode_kv_pair(torch.zeros_like(dk), dev(case["k"][:, :, :T]), dev(case["kp"]), torch.zeros_like(dv),
                        dev(case["v"][:, :, :T]), dev(case["vp"]), SMIN, SMAX, bits=bits, k_ckpt=kck, v_ckpt=vck,
                        ckpt_interval=iv)
    q, kn, vn = dev(case["q"]), dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1])
    kp, vp = dev(case["kp"]), dev(case["vp"])
    scratch = torch.empty(gemv.decode_scratch_bytes(B, H, H, T, iv), dtype=torch.uint8, device="cuda")
    good = gemv.decode_attn(q, dk, dv, kn, vn, kp, vp, T, 0.1, SMIN, SMAX, bits=bits, k_ckpt=kck, v_ckpt=vck,
                            ckpt_interval=iv, scratch=scratch)
    assert torch.isfinite(good).all() and gemv.device_status() == 0
    before_k = dk.clone()
    out = torch.zeros_like(good)
    P = lambda ps: _lib.Params(*[t.data_ptr() for t in ps])
    pk, pv = P(kp), P(vp)
    t0 = time.perf_counter()
    rc = _lib.load().adkv_decode_attn_ckpt(
        q.data_ptr(), dk.data_ptr(), dv.data_ptr(), kn.data_ptr(), vn.data_ptr(), ctypes.addressof(pk), ctypes.addressof(pv),
        None, None, kck.data_ptr(), vck.data_ptr(), iv, kck.shape[2], None, 0, out.data_ptr(), scratch.data_ptr(),
        scratch.numel(), B, H, H, T, D, dk.shape[2], bits, 0.1, SMIN, SMAX, _lib.FLAG_SELFTEST_MUTE_K,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert 0.9 < time.perf_counter() - t0 < 4.0
    assert gemv.device_status() == 3                               # the wait for logits ran out
    assert torch.isnan(out).all()                                  # marked, not stale
    assert torch.equal(dk, before_k)                               # the muted K warps appended nothing
    again = gemv.decode_attn(q, dk, dv, kn, vn, kp, vp, T, 0.1, SMIN, SMAX, bits=bits, k_ckpt=kck, v_ckpt=vck,
                             ckpt_interval=iv, scratch=scratch)
    assert torch.equal(again, good) and gemv.device_status() == 0  # the device still answers, and correctly
