"""The reference's UNMODIFIED model file driving the three-function boundary, on CPU.

Runs on a checkout of the reference beside this repository or, where there is none, on the copy of the model file
that ``oracle/build_ref.py`` staged unchanged under ``oracle/_ref/src``.  A stand-in
for the kernel module with the reference's three signatures, backed by the numpy oracle, is registered as
``adkv.kernel.gemv`` before ``adkv.hf.llama_adkv`` is imported; a tiny random-init model then runs
``generate``.  What is checked is the CONTRACT the CUDA path is written against: which calls the model
makes, in which order, with which shapes, dtypes, strides and token counts, that the caches are mutated in
place and may be replaced by larger copies between calls, and that the same argument lists are accepted by
``adkv_b200.gemv`` (signature binding).  The numerics of the stand-in are the oracle's, so the run also
checks that the oracle's decode step composes into a working generation loop.
"""
import inspect
import os
import sys
import types

import numpy as np
import pytest
import torch

from adkv_b200 import gemv, hf_shim
from oracle import adkv_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("ADKV_REFERENCE_ROOT", os.path.join(ROOT, os.pardir, "reference"))


def _reference_src():
    """The reference's ``src`` folder: the checkout when it is there, else the unchanged copy of the files this test
    executes that oracle/build_ref.py staged under oracle/_ref/src (which travels to machines without a checkout)."""
    from oracle import build_ref
    if os.path.exists(os.path.join(REF, "src", "adkv", "hf", "llama_adkv.py")):
        return os.path.join(REF, "src")
    return build_ref.staged_src()


pytestmark = pytest.mark.skipif(_reference_src() is None,
                                reason="neither a reference checkout nor its staged copy is present")


def _np(ps):
    return tuple(p.float().numpy() for p in ps)


def make_standin(calls):
    mod = types.ModuleType("adkv.kernel.gemv")

    def encode_kv(kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max):
        inspect.signature(gemv.encode_kv).bind(kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max)
        assert kv_cache.dtype == torch.uint8 and kv_cache.is_contiguous() and kv_cache.dim() == 6
        assert kv_new.dtype == torch.float16 and kv_new.is_contiguous()
        assert all(p.dtype == torch.float16 and p.shape == (kv_new.shape[1], kv_new.shape[3]) for p in (kv_zp, kv_sc, kv_alpha, kv_beta, kv_t))
        calls.append(("encode_kv", tuple(kv_cache.shape), tuple(kv_new.shape)))
        cache = kv_cache.numpy()                                        # shares memory: written in place
        orc.encode_kv(cache, kv_new.numpy(), _np((kv_zp, kv_sc, kv_alpha, kv_beta, kv_t)), 4, scale_min, scale_max)
        return kv_cache

    def forward_qk(q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T, scale_min, scale_max):
        inspect.signature(gemv.forward_qk).bind(q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T, scale_min, scale_max)
        assert isinstance(T, int) and q.dtype == k_new.dtype == torch.float16 and q.shape[2] == k_new.shape[2] == 1
        assert k_cache.is_contiguous() and T // 8 < k_cache.shape[2]
        calls.append(("forward_qk", tuple(k_cache.shape), T))
        out = orc.forward_qk(q.numpy()[:, :, 0], k_cache.numpy(), k_new.numpy()[:, :, 0],
                             _np((k_zp, k_sc, k_alpha, k_beta, k_t)), T, 4, scale_min, scale_max)
        return torch.from_numpy(np.asarray(out, np.float32)).to(torch.float16)

    def forward_ov(attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max):
        inspect.signature(gemv.forward_ov).bind(attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max)
        assert attn.dtype == torch.float16 and attn.dim() == 3
        calls.append(("forward_ov", tuple(v_cache.shape), attn.shape[2] - 1))
        out = orc.forward_ov(attn.numpy(), v_cache.numpy(), v_new.numpy()[:, :, 0],
                             _np((v_zp, v_sc, v_alpha, v_beta, v_t)), 4, scale_min, scale_max)
        return torch.from_numpy(np.asarray(out, np.float32)).to(torch.float16)

    mod.encode_kv, mod.forward_qk, mod.forward_ov = encode_kv, forward_qk, forward_ov
    return mod


@pytest.fixture
def clean_reference_modules():
    yield
    for name in [m for m in sys.modules if m == "adkv" or m.startswith("adkv.")]:
        del sys.modules[name]


def test_reference_model_file_drives_the_boundary_as_documented(monkeypatch, clean_reference_modules):
    from transformers import LlamaConfig
    calls = []
    monkeypatch.syspath_prepend(_reference_src())
    for name in [m for m in sys.modules if m == "adkv" or m.startswith("adkv.")]:
        monkeypatch.delitem(sys.modules, name)
    import adkv.kernel as kernel_pkg                                   # the reference's package (empty __init__)
    standin = make_standin(calls)
    monkeypatch.setitem(sys.modules, "adkv.kernel.gemv", standin)
    monkeypatch.setattr(kernel_pkg, "gemv", standin, raising=False)
    import adkv.hf.llama_adkv as M                                     # unmodified reference model file
    hf_shim.patch_mask_sizes(M.KVCacheLayer_ADKV)

    torch.manual_seed(0)
    L, H, Dh, prompt, new = 2, 2, 128, 61, 6                           # 61 + 6 crosses the 64-token capacity step
    cfg = LlamaConfig(hidden_size=H * Dh, intermediate_size=256, num_hidden_layers=L, num_attention_heads=H,
                      num_key_value_heads=H, vocab_size=97, max_position_embeddings=256)
    model = M.LlamaForCausalLM_ADKV(cfg).eval()
    n = H * Dh
    rho = 0.9 + 0.099 * torch.rand(n)
    mk = lambda: M.ADKVConfig(torch.zeros(n), torch.ones(n), 1.0 - rho, torch.full((n,), 0.05), torch.full((n,), 3.5))
    model.load_adkv_config([(mk(), mk()) for _ in range(L)])
    ids = torch.randint(0, 97, (2, prompt))
    with torch.no_grad():
        out = model.generate(input_ids=ids, max_new_tokens=new, do_sample=False)
    assert out.shape == (2, prompt + new)

    enc = [c for c in calls if c[0] == "encode_kv"]
    qk = [c for c in calls if c[0] == "forward_qk"]
    ov = [c for c in calls if c[0] == "forward_ov"]
    assert len(enc) == 2 * L and all(c[2] == (2, H, prompt, Dh) for c in enc)          # K and V of every layer, once
    assert len(qk) == len(ov) == L * (new - 1)                                          # one pair per layer and decode step
    first_decode = calls.index(qk[0])
    assert all(c[0] == "encode_kv" for c in calls[:first_decode])                       # prefill first
    for i in range(0, len(qk)):
        a, b = calls[first_decode + 2 * i], calls[first_decode + 2 * i + 1]
        assert a[0] == "forward_qk" and b[0] == "forward_ov" and a[2] == b[2]           # same T for both halves of a step
    assert [c[2] for c in qk[::L]] == list(range(prompt, prompt + new - 1))             # T grows by one per step
    assert {c[1][2] for c in qk} == {8, 16}                                            # the caller replaced the caches by larger ones
