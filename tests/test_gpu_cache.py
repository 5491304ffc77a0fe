"""The cache object (mirror of the reference's KVCacheLayer_ADKV) on the GPU: growth boundaries, fused vs
the reference's three-call sequence, pre-sized capacity, grouped-query heads."""
import numpy as np
import pytest
import torch

from adkv_b200 import synth
from adkv_b200.cache import CAP_LEN, INIT_SEQ_LEN, KVCache, KVCacheLayer
from oracle import adkv_oracle as orc
from tests.util import SMAX, SMIN, np_params

pytestmark = pytest.mark.gpu


def _flat(params):
    return tuple(p.reshape(-1).cuda() for p in params)


def _run(layer, k, v, q_all, kp, vp, T0, steps, scaling):
    layer.prefill(k[:, :, :T0].cuda(), v[:, :, :T0].cuda(), *_flat(kp), *_flat(vp))
    outs = []
    for s in range(steps):
        T = T0 + s
        o, w = layer.decode(q_all[s].cuda(), k[:, :, T:T + 1].cuda(), v[:, :, T:T + 1].cuda(), *_flat(kp), *_flat(vp),
                            attention_mask=None, scaling=scaling)
        outs.append(o)
    return outs


@pytest.mark.parametrize("bits,Hq,Hkv", [(4, 2, 2), (2, 4, 2)])
def test_generation_across_growth_boundaries(bits, Hq, Hkv):
    B, D, T0, steps = 2, 128, 60, 75          # crosses the 64- and 128-token capacity steps
    k = synth.gen_kv(1, B, Hkv, T0 + steps, D)
    v = synth.gen_kv(2, B, Hkv, T0 + steps, D)
    kp, vp = synth.gen_params(3, Hkv, D, bits), synth.gen_params(4, Hkv, D, bits)
    g = torch.Generator().manual_seed(0)
    q_all = [torch.randn(B, Hq, 1, D, generator=g).half() for _ in range(steps)]
    fused = KVCacheLayer(bits=bits, fused=True)
    trio = KVCacheLayer(bits=bits, fused=False)
    sized = KVCacheLayer(bits=bits, fused=True, capacity_tokens=T0 + steps)
    o1 = _run(fused, k, v, q_all, kp, vp, T0, steps, 0.09)
    o2 = _run(trio, k, v, q_all, kp, vp, T0, steps, 0.09)
    o3 = _run(sized, k, v, q_all, kp, vp, T0, steps, 0.09)
    assert fused.get_seq_length() == T0 + steps and fused._cap_len >= T0 + steps
    assert fused._cap_len % CAP_LEN == 0 and INIT_SEQ_LEN == 64
    assert sized.key_states.shape[2] == orc.n_super_for(T0 + steps, bits)       # never reallocated
    n = fused.key_states.shape[2]
    assert torch.equal(fused.key_states, trio.key_states) and torch.equal(fused.value_states, trio.value_states)
    assert torch.equal(fused.key_states[:, :, :sized.key_states.shape[2]], sized.key_states[:, :, :n])
    # final caches equal the oracle's one-shot encode of the whole sequence (every append was canonical)
    want = np.zeros(orc.cache_shape(B, Hkv, n, D), np.uint8)
    orc.encode_kv(want, k.numpy(), np_params(kp), bits, SMIN, SMAX)
    assert np.array_equal(fused.key_states.cpu().numpy(), want)
    for a, b, c in zip(o1, o2, o3):
        assert torch.equal(a, c)
        # the three-call sequence rounds logits and weights to fp16 as the reference does; the fused step does not
        torch.testing.assert_close(a.float(), b.float(), rtol=3e-2, atol=3e-2 * float(a.abs().max()))


@pytest.mark.parametrize("half_state", [False, True])
def test_checkpointed_cache_object_matches_plain(half_state):
    B, H, D, T0, steps, bits = 2, 2, 128, 70, 40, 4
    k = synth.gen_kv(11, B, H, T0 + steps, D)
    v = synth.gen_kv(12, B, H, T0 + steps, D)
    kp, vp = synth.gen_params(13, H, D, bits), synth.gen_params(14, H, D, bits)
    g = torch.Generator().manual_seed(2)
    q_all = [torch.randn(B, H, 1, D, generator=g).half() for _ in range(steps)]
    plain = KVCacheLayer(bits=bits, capacity_tokens=T0 + steps, half_state=half_state)
    ck = KVCacheLayer(bits=bits, capacity_tokens=T0 + steps, checkpoint_interval=32, half_state=half_state)
    o1 = _run(plain, k, v, q_all, kp, vp, T0, steps, 0.09)
    o2 = _run(ck, k, v, q_all, kp, vp, T0, steps, 0.09)
    assert torch.equal(plain.key_states, ck.key_states) and torch.equal(plain.value_states, ck.value_states)
    tol = 2e-2 if half_state else 2e-3      # fp16 partial sums in the fp16-state arithmetic
    for a, b in zip(o1, o2):
        torch.testing.assert_close(a.float(), b.float(), rtol=tol, atol=tol * max(1.0, float(a.abs().max())))
    with pytest.raises(ValueError, match="capacity_tokens"):
        KVCacheLayer(checkpoint_interval=32)


def test_cache_object_errors_match_reference_behaviour():
    layer = KVCacheLayer()
    x = torch.zeros(1, 2, 4, 128, dtype=torch.float16, device="cuda")
    p = _flat(synth.gen_params(0, 2, 128))
    layer.prefill(x, x, *p, *p)
    with pytest.raises(NotImplementedError):
        layer.prefill(x, x, *p, *p)                        # chunked prefill (llama_adkv.py:195-197)
    with pytest.raises(ValueError, match="exactly one"):
        layer.decode(x, x, x, *p, *p)
    with pytest.raises(ValueError, match="different"):
        layer.decode(x[:, :1, :1], x[:, :1, :1], x[:, :1, :1], *p, *p)
    with pytest.raises(ValueError, match="head_dim"):
        KVCacheLayer().prefill(x[..., :64], x[..., :64], *p, *p)
    wide = KVCacheLayer()
    xw = torch.zeros(1, 2, 4, 256, dtype=torch.float16, device="cuda")
    pw = _flat(synth.gen_params(0, 2, 256))
    wide.prefill(xw, xw, *pw, *pw)                       # head_dim 256 is served (llama_adkv.py:97-99)
    assert wide.key_states.shape == (1, 2, 8, 64, 4, 4)
    assert KVCache(3)[2].get_mask_sizes(2) == (2, 0)
