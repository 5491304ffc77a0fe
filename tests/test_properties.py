"""Property tests (hypothesis) of the oracle and the host logic, on CPU."""
import numpy as np
from hypothesis import given, settings, strategies as st

from adkv_b200 import gemv, sharding
from oracle import adkv_oracle as orc


@settings(max_examples=40, deadline=None)
@given(bits=st.sampled_from([2, 4]), T=st.integers(0, 70), seed=st.integers(0, 2**16))
def test_pack_unpack_roundtrip_and_zero_tail(bits, T, seed):
    rng = np.random.default_rng(seed)
    lo, hi = orc.quant_limits(bits)
    codes = rng.integers(lo, hi + 1, size=(1, 2, T, 128)).astype(np.int8)
    cache = orc.pack_codes(codes, bits, n_super_cap=orc.n_super_for(T, bits) + 1)
    assert np.array_equal(orc.unpack_codes(cache, T, bits), codes)
    tpw = orc.tokens_per_word(bits)
    words = orc.cache_words(cache)
    if T % tpw:
        assert np.all(words[:, :, T // tpw, :] >> np.uint32(bits * (T % tpw)) == 0)
    assert np.all(words[:, :, orc.n_super_for(T, bits):, :] == 0)
    assert gemv.n_super_for(T, bits) == orc.n_super_for(T, bits)


@settings(max_examples=15, deadline=None)
@given(bits=st.sampled_from([2, 4]), T=st.integers(1, 40), cut=st.integers(0, 40), seed=st.integers(0, 2**16))
def test_decoder_replay_reproduces_encoder_state_and_chunking_is_associative(bits, T, cut, seed):
    rng = np.random.default_rng(seed)
    H, D = 1, 128
    x = (rng.standard_normal((1, H, T, D)) * rng.choice([0.1, 1.0, 30.0])).astype(np.float16).astype(np.float32)
    p = (rng.standard_normal((H, D)).astype(np.float16).astype(np.float32),
         (rng.random((H, D)) * 2 + 0.01).astype(np.float16).astype(np.float32),
         (rng.random((H, D)) * 0.3).astype(np.float16).astype(np.float32),
         (rng.random((H, D)) * 0.1).astype(np.float16).astype(np.float32),
         (rng.random((H, D)) * 4).astype(np.float16).astype(np.float32))
    st_enc = orc.init_state(1, p[0], p[1])
    codes, xhat = orc.encode_scan(x, st_enc, p[2], p[3], p[4], bits)
    st_dec = orc.init_state(1, p[0], p[1])
    xhat2 = orc.decode_scan(codes, st_dec, p[2], p[3], p[4])
    assert np.array_equal(xhat.view(np.uint32), xhat2.view(np.uint32))
    assert np.array_equal(st_enc.zp.view(np.uint32), st_dec.zp.view(np.uint32))
    assert np.array_equal(st_enc.s.view(np.uint32), st_dec.s.view(np.uint32))
    lo, hi = orc.quant_limits(bits)
    assert codes.min() >= lo and codes.max() <= hi
    assert np.all(st_enc.s >= np.float32(orc.SCALE_MIN)) and np.all(st_enc.s <= np.float32(orc.SCALE_MAX))
    # encoding in two chunks from the carried state equals encoding in one go
    c = min(cut, T)
    st2 = orc.init_state(1, p[0], p[1])
    a, _ = orc.encode_scan(x[:, :, :c], st2, p[2], p[3], p[4], bits, want_xhat=False)
    b, _ = orc.encode_scan(x[:, :, c:], st2, p[2], p[3], p[4], bits, want_xhat=False)
    assert np.array_equal(np.concatenate([a, b], axis=2), codes)


@settings(max_examples=200, deadline=None)
@given(B=st.integers(1, 300), Hkv=st.integers(1, 64), world=st.sampled_from([1, 2, 4, 8]))
def test_sharding_plan_partitions_the_grid(B, Hkv, world):
    try:
        shards = sharding.plan(B, Hkv, world)
    except ValueError:
        assert all(pb > B or world // pb > Hkv for pb in range(1, world + 1) if world % pb == 0)
        return
    seen = np.zeros((B, Hkv), int)
    for s in shards:
        assert s.b1 > s.b0 and s.h1 > s.h0
        seen[s.b0:s.b1, s.h0:s.h1] += 1
    assert (seen == 1).all()


@settings(max_examples=15, deadline=None)
@given(bits=st.sampled_from([2, 4]), T=st.integers(1, 40), cut=st.integers(0, 40), seed=st.integers(0, 2**16))
def test_fp16_state_restatement_replays_and_chunks_like_the_fp32_one(bits, T, cut, seed):
    """The numpy restatement of the reference CUDA kernels' arithmetic: the decoder rebuilds the encoder's values and
    state from the codes, and encoding in two chunks with the state carried over equals encoding in one."""
    from oracle import adkv_oracle_half as orh
    rng = np.random.default_rng(seed)
    H, D = 1, 128
    x = (rng.standard_normal((1, H, T, D)) * rng.choice([0.1, 1.0, 30.0])).astype(np.float16)
    p = (rng.standard_normal((H, D)).astype(np.float16), (rng.random((H, D)) * 2 + 0.01).astype(np.float16),
         (rng.random((H, D)) * 0.3).astype(np.float16), (rng.random((H, D)) * 0.1).astype(np.float16),
         (rng.random((H, D)) * 4).astype(np.float16))
    st_enc = orh.init_state(1, p[0], p[1])
    codes, xhat = orh.encode_scan(x, st_enc, p[2], p[3], p[4], bits)
    st_dec = orh.init_state(1, p[0], p[1])
    xhat2 = orh.decode_scan(codes, st_dec, p[2], p[3], p[4])
    same = lambda a, b: np.array_equal(a.view(np.uint16), b.view(np.uint16))
    assert same(xhat, xhat2) and same(st_enc.zp, st_dec.zp) and same(st_enc.sc, st_dec.sc)
    c = min(cut, T)
    st2 = orh.init_state(1, p[0], p[1])
    c1, _ = orh.encode_scan(x[:, :, :c], st2, p[2], p[3], p[4], bits)
    c2, _ = orh.encode_scan(x[:, :, c:], st2, p[2], p[3], p[4], bits)
    assert np.array_equal(np.concatenate([c1, c2], axis=2), codes)
    assert same(st2.zp, st_enc.zp) and same(st2.sc, st_enc.sc)
