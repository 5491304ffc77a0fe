"""The reference's own CUDA kernels (recompiled for sm_100a by ``oracle/build_ref.py``) against this library.

The reference's kernels keep the recurrence state in fp16 (``src/adkv/kernel/gemv.cu:158-164``), this
library follows the fp32 definition of ``src/adkv/train/train_model.py:70-81``, so codes differ once the state
moves.  With ``alpha = beta = 0`` the state is frozen in both, the quantiser of both is
``clamp(round_half_even((x - zp) / s))`` in fp32 (``gemv.cu:150-154``), and everything that is left is what
these tests pin BY EXECUTION of the reference: the packed layout (nibble order, offset, supergroup tiling,
zero fill), the in-place append at slot ``T``, the unscaled logits with the self logit last, and
``T = attn.size(2) - 1`` in the weighted sum.  Skipped when the extension has not been built.
"""
import numpy as np
import pytest
import torch

from adkv_b200 import gemv, synth
from oracle import adkv_oracle as orc
from oracle import ref_cuda
from tests.util import SMAX, SMIN

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/adkv_gemv.so has not been built")]

B, H, D = 3, 5, 128          # 15 streams: the reference packs 4 per CTA, so the last CTA is ragged


def frozen_params(seed):
    g = torch.Generator().manual_seed(seed)
    zp = (torch.randn(H, D, generator=g) * 0.5).half()
    sc = (torch.rand(H, D, generator=g) * 1.7 + 0.3).half()
    z = torch.zeros(H, D).half()
    return tuple(t.cuda() for t in (zp, sc, z, z.clone(), torch.full((H, D), 3.5).half()))


def caches(T, extra=0):
    ns = orc.n_super_for(T, 4) + extra
    shape = orc.cache_shape(B, H, max(ns, 1), D)
    return torch.zeros(shape, dtype=torch.uint8, device="cuda"), torch.zeros(shape, dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("T", [1, 2, 7, 8, 9, 16, 63, 64, 130, 1000])
def test_packed_layout_equals_reference_encode(T):
    ref = ref_cuda.module()
    x = synth.gen_kv(500 + T, B, H, T, D).cuda()
    x[0, 0, 0, :32] = ((torch.arange(32) - 16) * 0.5).half().cuda()       # exact ties at token 0 of one stream
    p = frozen_params(T)
    p[0][0, :32] = 0
    p[1][0, :32] = 1
    mine, theirs = caches(T)
    ref.encode_kv(theirs, x, *p, SMIN, SMAX)
    gemv.encode_kv(mine, x, *p, SMIN, SMAX, bits=4)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    # and the oracle's packer agrees with both
    want = np.zeros(tuple(mine.shape), np.uint8)
    orc.encode_kv(want, x.cpu().numpy(), tuple(t.float().cpu().numpy() for t in p), 4, SMIN, SMAX)
    assert np.array_equal(want, theirs.cpu().numpy())


@pytest.mark.parametrize("T", [0, 1, 8, 9, 77, 256])
def test_forward_qk_append_and_self_logit_equal_reference(T):
    ref = ref_cuda.module()
    k = synth.gen_kv(600 + T, B, H, T + 1, D).cuda()
    q = synth.gen_q(601 + T, B, H, D).cuda()
    p = frozen_params(10 + T)
    mine, theirs = caches(T + 1, extra=1)
    if T:
        gemv.encode_kv(mine, k[:, :, :T].contiguous(), *p, SMIN, SMAX, bits=4)
        theirs.copy_(mine)
    k_new = k[:, :, T:].contiguous()
    lt = ref.forward_qk(q, theirs, k_new, *p, T, SMIN, SMAX)
    lm = gemv.forward_qk(q, mine, k_new, *p, T, SMIN, SMAX, bits=4)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)                               # same nibble written at slot T
    assert lt.shape == lm.shape == (B, H, T + 1) and lt.dtype == lm.dtype == torch.float16
    # the reference accumulates the dot product and the cross-lane sum in fp16 (gemv.cu:644-686); ours in fp32
    a, b = lm.float().cpu().numpy(), lt.float().cpu().numpy()
    np.testing.assert_allclose(b, a, rtol=2e-2, atol=2e-2 * max(1.0, np.abs(a).max()))


@pytest.mark.parametrize("T", [0, 1, 8, 9, 77, 256])
def test_forward_ov_append_equals_reference(T):
    ref = ref_cuda.module()
    v = synth.gen_kv(700 + T, B, H, T + 1, D).cuda()
    p = frozen_params(20 + T)
    g = torch.Generator().manual_seed(T)
    attn = torch.softmax(torch.randn(B, H, T + 1, generator=g) * 2, dim=-1).half().cuda()
    mine, theirs = caches(T + 1, extra=1)
    if T:
        gemv.encode_kv(mine, v[:, :, :T].contiguous(), *p, SMIN, SMAX, bits=4)
        theirs.copy_(mine)
    v_new = v[:, :, T:].contiguous()
    ot = ref.forward_ov(attn, theirs, v_new, *p, SMIN, SMAX)
    om = gemv.forward_ov(attn, mine, v_new, *p, SMIN, SMAX, bits=4)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    a, b = om.float().cpu().numpy().reshape(B * H, D), ot.float().cpu().numpy().reshape(B * H, D)
    # fp16 accumulation over all tokens in the reference (gemv.cu:1087, 1096)
    np.testing.assert_allclose(b, a, rtol=2e-2, atol=2e-2 * max(1.0, np.abs(a).max()))
    assert gemv.device_status() == 0
