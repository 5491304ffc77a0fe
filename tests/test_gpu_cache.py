"""The cache object (stand-in for the reference's KVCacheLayer_ADKV) on the GPU: growth boundaries, fused step vs
the reference's three-call sequence, pre-sized capacity, grouped-query heads, tail states, chunked prefill."""
import numpy as np
import pytest
import torch

from adkv_b200 import synth
from adkv_b200.cache import MIN_TOKENS, KVCache, KVCacheLayer
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
    B, D, T0, steps = 2, 128, 60, 75          # outgrows the first allocation (64 tokens) and its double (128)
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
    assert fused.get_seq_length() == T0 + steps and MIN_TOKENS == 64
    assert fused.capacity == 256 and trio.capacity == 256                       # 64 -> 128 -> 256: two copies in all
    assert sized.key_states.shape[2] == orc.n_super_for(T0 + steps, bits)       # never reallocated
    n = fused.key_states.shape[2]
    assert torch.equal(fused.key_states, trio.key_states) and torch.equal(fused.value_states, trio.value_states)
    assert torch.equal(fused.key_states[:, :, :sized.key_states.shape[2]], sized.key_states[:, :, :n])
    # final caches equal the oracle's one-shot encode of the whole sequence (every append was canonical)
    want = np.zeros(orc.cache_shape(B, Hkv, n, D), np.uint8)
    orc.encode_kv(want, k.numpy(), np_params(kp), bits, SMIN, SMAX)
    assert np.array_equal(fused.key_states.cpu().numpy(), want)
    # ... and the tails equal the state that encode leaves after the whole sequence
    _, st = orc.encode_kv(np.zeros_like(want), k.numpy(), np_params(kp), bits, SMIN, SMAX)
    kt, vt = fused.tails
    assert np.array_equal(kt.cpu().numpy()[:, :, 0].view(np.uint32), st.zp.view(np.uint32))
    assert np.array_equal(kt.cpu().numpy()[:, :, 1].view(np.uint32), st.s.view(np.uint32))
    assert trio.tails == (None, None)
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
    with pytest.raises(ValueError, match="multiple of 32"):
        KVCacheLayer(checkpoint_interval=48)
    grows = KVCacheLayer(bits=bits, checkpoint_interval=32, half_state=half_state)     # not pre-sized: regrown
    o3 = _run(grows, k, v, q_all, kp, vp, T0, steps, 0.09)
    assert torch.equal(grows.key_states[:, :, :ck.key_states.shape[2]], ck.key_states[:, :, :grows.key_states.shape[2]])
    for a, b in zip(o2, o3):
        assert torch.equal(a, b)


def test_chunked_prefill_and_per_head_mask_keep_the_tails_in_step():
    """Prefill in three pieces, a decode step with a per-head mask (which cannot use the fused kernel), then fused
    steps: buffers and tails equal those of a cache prefilled in one go and stepped with shared masks."""
    B, H, D, T0, steps, bits = 2, 2, 128, 90, 6, 4
    k, v = synth.gen_kv(31, B, H, T0 + steps, D), synth.gen_kv(32, B, H, T0 + steps, D)
    kp, vp = synth.gen_params(33, H, D, bits), synth.gen_params(34, H, D, bits)
    g = torch.Generator().manual_seed(4)
    q_all = [torch.randn(B, H, 1, D, generator=g).half() for _ in range(steps)]
    one, parts = KVCacheLayer(bits=bits), KVCacheLayer(bits=bits)
    outs = _run(one, k, v, q_all, kp, vp, T0, steps, 0.09)
    for a, b in ((0, 17), (17, 64), (64, T0)):
        parts.prefill(k[:, :, a:b].cuda(), v[:, :, a:b].cuda(), *_flat(kp), *_flat(vp))
    for s in range(steps):
        T = T0 + s
        mask = torch.zeros(B, H, 1, T + 1, device="cuda") if s == 1 else None       # per head: three-call path
        o, w = parts.decode(q_all[s].cuda(), k[:, :, T:T + 1].cuda(), v[:, :, T:T + 1].cuda(), *_flat(kp), *_flat(vp),
                            attention_mask=mask, scaling=0.09)
        assert (w is None) == (s != 1)
        torch.testing.assert_close(o.float(), outs[s].float(), rtol=3e-2, atol=3e-2 * float(o.abs().max()))
    used = orc.n_super_for(T0 + steps, bits)                  # the two objects grew differently: compare what is used
    assert torch.equal(one.key_states[:, :, :used], parts.key_states[:, :, :used])
    assert torch.equal(one.value_states[:, :, :used], parts.value_states[:, :, :used])
    for a, b in zip(one.tails, parts.tails):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))


def test_cache_object_errors():
    layer = KVCacheLayer(fused=False)
    x = torch.zeros(1, 2, 4, 128, dtype=torch.float16, device="cuda")
    p = _flat(synth.gen_params(0, 2, 128))
    layer.prefill(x, x, *p, *p)
    with pytest.raises(NotImplementedError):
        layer.prefill(x, x, *p, *p)                        # no tails in the reference's mode (llama_adkv.py:195-197)
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
