"""The allocation-free decode entry point, checked against the entry point that takes caller-owned scratch.

Collected last on purpose (file name): a run that stops at the first failure has then already been through
every other test.  It passes on its own in a fresh process and after the rest of the suite: the only state it
touches is the library's built-in scratch array, which every call overwrites before reading.

Who this entry point is for: hosts that cannot allocate device memory at the time of the call -- a server
whose HBM is wholly owned by its own block pool, or a plugin that is only ever handed device pointers."""
import numpy as np
import pytest
import torch

from adkv_b200 import gemv
from oracle import adkv_oracle as orc
from tests.util import SMAX, SMIN, dev, make_case

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-3, 2e-3          # the tolerance of the other decode tests


def _setup(bits, Hq, Hkv, T0, S, B=2, D=128, extra=3):
    case = make_case(700 + T0, B, Hq, Hkv, T0 + extra, bits)
    kp, vp = dev(case["kp"]), dev(case["vp"])
    ns = orc.n_super_for(T0 + extra + 1, bits)
    mk = lambda: torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    ck = lambda: gemv.alloc_ckpt(B, Hkv, D, T0 + extra + 1, S, "cuda")
    a = dict(k=mk(), v=mk(), kck=ck(), vck=ck())
    b = dict(k=mk(), v=mk(), kck=ck(), vck=ck())
    for s in (a, b):
        gemv.encode_kv_pair(s["k"], dev(case["k"][:, :, :T0]), kp, s["v"], dev(case["v"][:, :, :T0]), vp, SMIN, SMAX,
                            bits=bits, k_ckpt=s["kck"], v_ckpt=s["vck"], ckpt_interval=S)
    return case, kp, vp, a, b


@pytest.mark.parametrize("bits,Hq,Hkv,T0,S", [(4, 2, 2, 127, 64), (2, 4, 2, 200, 32)])
def test_static_scratch_entry_point_matches_caller_scratch_entry_point(bits, Hq, Hkv, T0, S):
    B, D = 2, 128
    case, kp, vp, a, b = _setup(bits, Hq, Hkv, T0, S)
    g = torch.Generator().manual_seed(5)
    out_b = torch.empty(B, Hq, D, dtype=torch.float16, device="cuda")
    for step in range(2):                                     # two calls in a row share the built-in array
        T = T0 + step
        q = dev(torch.randn(B, Hq, 1, D, generator=g).half())
        kn, vn = dev(case["k"][:, :, T:T + 1]), dev(case["v"][:, :, T:T + 1])
        mask = torch.zeros(B, T + 1, dtype=torch.float32, device="cuda")
        mask[0, :7] = -1e4
        want = gemv.decode_attn(q, a["k"], a["v"], kn, vn, kp, vp, T, 0.11, SMIN, SMAX, bits=bits, mask=mask,
                                k_ckpt=a["kck"], v_ckpt=a["vck"], ckpt_interval=S)
        got = gemv.decode_attn_static(q, b["k"], b["v"], kn, vn, kp, vp, T, 0.11, SMIN, SMAX, bits=bits, mask=mask,
                                      k_ckpt=b["kck"], v_ckpt=b["vck"], ckpt_interval=S, out=out_b)
        torch.cuda.synchronize()
        assert got is out_b
        np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(), rtol=RTOL,
                                   atol=ATOL)
        assert torch.equal(a["k"], b["k"]) and torch.equal(a["v"], b["v"])                # same appended codes
        assert torch.equal(a["kck"], b["kck"]) and torch.equal(a["vck"], b["vck"])        # same checkpoints
    assert gemv.device_status() == 0


def test_static_scratch_entry_point_rejects_oversized_problems():
    """B * Hq * (T / interval + 1) segments-heads beyond the 16 MiB array: a clear error, nothing launched."""
    B, Hq, Hkv, D, S, bits = 4, 32, 8, 128, 32, 2
    T = 32 * 260                                              # 261 segments * 128 heads * 528 B > 16 MiB
    assert gemv.decode_scratch_bytes(B, Hq, Hkv, T, S) > gemv.STATIC_SCRATCH_BYTES
    ns = orc.n_super_for(T + 1, bits)
    k = torch.zeros(orc.cache_shape(B, Hkv, ns, D), dtype=torch.uint8, device="cuda")
    v = torch.zeros_like(k)
    kck = gemv.alloc_ckpt(B, Hkv, D, T + 1, S, "cuda")
    vck = torch.zeros_like(kck)
    p = tuple(torch.zeros(Hkv, D, dtype=torch.float16, device="cuda") for _ in range(5))
    q = torch.zeros(B, Hq, 1, D, dtype=torch.float16, device="cuda")
    kn = torch.zeros(B, Hkv, 1, D, dtype=torch.float16, device="cuda")
    out = torch.full((B, Hq, D), 7.0, dtype=torch.float16, device="cuda")
    before = k.clone()
    with pytest.raises(RuntimeError, match="built-in scratch"):
        gemv.decode_attn_static(q, k, v, kn, kn, p, p, T, 0.1, SMIN, SMAX, bits=bits, k_ckpt=kck, v_ckpt=vck,
                                ckpt_interval=S, out=out)
    torch.cuda.synchronize()
    assert torch.equal(k, before) and float(out.float().min()) == 7.0          # nothing ran
