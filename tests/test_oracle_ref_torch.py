"""The reference's own torch recurrence, staged unchanged under oracle/_ref/src, against the numpy oracle: the CPU
baseline that bench.py times computes the same attention output as the oracle's decode step (and therefore as the
kernels, which are held to the oracle)."""
import numpy as np
import pytest
import torch

from adkv_b200 import synth
from oracle import adkv_oracle as orc
from oracle import ref_torch

pytestmark = pytest.mark.skipif(not ref_torch.available(), reason="oracle/_ref/src not staged (needs a reference checkout)")


@pytest.mark.parametrize("bits,Hq,Hkv", [(4, 2, 2), (2, 4, 2)])
def test_staged_torch_path_equals_oracle_decode(bits, Hq, Hkv):
    B, T, D = 2, 75, 128
    k, v = synth.gen_kv(1, B, Hkv, T + 1, D), synth.gen_kv(2, B, Hkv, T + 1, D)
    q = synth.gen_q(3, B, Hq, D)
    kp, vp = synth.gen_params(4, Hkv, D, bits), synth.gen_params(5, Hkv, D, bits)
    got = ref_torch.decode_attention(q, k, v, kp, vp, bits, D ** -0.5, synth.SCALE_MIN, synth.SCALE_MAX).numpy()
    npp = lambda p: tuple(t.float().numpy() for t in p)
    ns = orc.n_super_for(T + 1, bits)
    kc = np.zeros(orc.cache_shape(B, Hkv, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    orc.encode_kv(kc, k[:, :, :T].numpy(), npp(kp), bits, synth.SCALE_MIN, synth.SCALE_MAX)
    orc.encode_kv(vc, v[:, :, :T].numpy(), npp(vp), bits, synth.SCALE_MIN, synth.SCALE_MAX)
    want = orc.decode_attn(q[:, :, 0].numpy(), kc, vc, k[:, :, T].numpy(), v[:, :, T].numpy(), npp(kp), npp(vp), T,
                           D ** -0.5, bits=bits, scale_min=synth.SCALE_MIN, scale_max=synth.SCALE_MAX)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)       # fp32 softmax and sums against float64


def test_torch_compile_is_left_alone():
    """Importing the staged module neutralises torch.compile only for the duration of the import."""
    before = torch.compile
    ref_torch.module()
    assert torch.compile is before
