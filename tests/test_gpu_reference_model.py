"""The reference's UNMODIFIED model file running on this library's CUDA kernels.  Needs a B200.

``oracle/build_ref.py`` stages ``src/adkv/hf/llama_adkv.py`` of the reference, byte for byte, under
``oracle/_ref/src`` (a git-ignored build output that travels to the GPU box like the built libraries).  Here
``adkv_b200.hf_shim.install()`` registers the kernel module under the name that file imports
(``from adkv.kernel.gemv import encode_kv, forward_ov, forward_qk``, ``src/adkv/hf/llama_adkv.py:21``), the file is
imported as it is, and a random-init ``LlamaForCausalLM_ADKV`` runs HF ``generate`` on ``cuda`` across the
64-token capacity step of its cache object (``llama_adkv.py:104-123``).

Every call the model makes into the three entry points is executed by the CUDA kernels AND, on copies of the
same inputs, by the numpy oracle: outputs must agree within the stated tolerance and the packed caches bit
for bit after every single call -- at all layers, which a comparison of two independent generations could
not give (a 1e-3 difference in one layer's output changes the next layer's K/V in the last bit).
"""
import json
import os
import sys
import time

import numpy as np
import pytest
import torch

from adkv_b200 import gemv, hf_shim
from oracle import adkv_oracle as orc
from oracle import build_ref, ref_cuda

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(build_ref.staged_src() is None,
                                 reason="oracle/_ref/src not staged (run oracle/build_ref.py next to a reference checkout)")]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _np(ps):
    return tuple(p.float().cpu().numpy() for p in ps)


class CheckedKernels:
    """adkv_b200.gemv's three reference-facing functions, each call cross-checked against the oracle."""

    def __init__(self):
        self.calls = []
        self.max_logit_err = 0.0
        self.max_out_err = 0.0

    def encode_kv(self, kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max):
        assert kv_cache.is_cuda and kv_cache.dtype == torch.uint8 and kv_new.dtype == torch.float16
        want = kv_cache.cpu().numpy().copy()
        orc.encode_kv(want, kv_new.cpu().numpy(), _np((kv_zp, kv_sc, kv_alpha, kv_beta, kv_t)), 4, scale_min, scale_max)
        out = gemv.encode_kv(kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max)
        assert out is kv_cache
        assert np.array_equal(kv_cache.cpu().numpy(), want), "encode_kv: packed cache differs from the oracle's"
        self.calls.append(("encode_kv", tuple(kv_cache.shape), tuple(kv_new.shape)))
        return out

    def forward_qk(self, q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T, scale_min, scale_max):
        want_cache = k_cache.cpu().numpy().copy()
        want = orc.forward_qk(q.cpu().numpy()[:, :, 0], want_cache, k_new.cpu().numpy()[:, :, 0],
                              _np((k_zp, k_sc, k_alpha, k_beta, k_t)), T, 4, scale_min, scale_max)
        got = gemv.forward_qk(q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T, scale_min, scale_max)
        assert got.shape == want.shape and got.dtype == torch.float16
        g = got.float().cpu().numpy()
        # unscaled fp16 logits: half an fp16 ulp of the largest logit on top of the relative bound
        np.testing.assert_allclose(g, want, rtol=2e-3, atol=2e-3 * max(1.0, float(np.abs(want).max())))
        self.max_logit_err = max(self.max_logit_err, float(np.abs(g - want).max()))
        assert np.array_equal(k_cache.cpu().numpy(), want_cache), "forward_qk: appended code differs from the oracle's"
        self.calls.append(("forward_qk", tuple(k_cache.shape), T))
        return got

    def forward_ov(self, attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max):
        want_cache = v_cache.cpu().numpy().copy()
        want = orc.forward_ov(attn.float().cpu().numpy(), want_cache, v_new.cpu().numpy()[:, :, 0],
                              _np((v_zp, v_sc, v_alpha, v_beta, v_t)), 4, scale_min, scale_max)
        got = gemv.forward_ov(attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max)
        g = got.float().cpu().numpy()
        np.testing.assert_allclose(g, want, rtol=2e-3, atol=2e-3)
        self.max_out_err = max(self.max_out_err, float(np.abs(g - want).max()))
        assert np.array_equal(v_cache.cpu().numpy(), want_cache), "forward_ov: appended code differs from the oracle's"
        self.calls.append(("forward_ov", tuple(v_cache.shape), attn.shape[2] - 1))
        return got


class CheckedAgainstReferenceKernels:
    """The three entry points in the arithmetic of the reference's CUDA kernels (``hf_shim.install(half_state=True)``),
    each call repeated by the reference's own extension (``oracle/_ref/adkv_gemv.so``, its ``gemv.cu`` compiled for
    sm_100a) on copies of the same inputs: caches bit for bit, outputs within fp16 accumulation-order noise."""

    def __init__(self, ours, theirs):
        self.ours, self.theirs = ours, theirs
        self.n = 0
        self.max_logit_err = self.max_out_err = 0.0

    def encode_kv(self, kv_cache, kv_new, *rest):
        want = kv_cache.clone()
        self.theirs.encode_kv(want, kv_new, *rest)
        out = self.ours.encode_kv(kv_cache, kv_new, *rest)
        assert torch.equal(kv_cache, want), "encode_kv: packed cache differs from the reference kernel's"
        self.n += 1
        return out

    def forward_qk(self, q, k_cache, k_new, *rest):
        want_cache = k_cache.clone()
        want = self.theirs.forward_qk(q, want_cache, k_new, *rest).float()
        got = self.ours.forward_qk(q, k_cache, k_new, *rest)
        assert torch.equal(k_cache, want_cache), "forward_qk: appended code differs from the reference kernel's"
        assert got.shape == want.shape
        tol = 2e-2 * max(1.0, float(want.abs().max()))
        torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=tol)
        self.max_logit_err = max(self.max_logit_err, float((got.float() - want).abs().max()))
        self.n += 1
        return got

    def forward_ov(self, attn, v_cache, v_new, *rest):
        want_cache = v_cache.clone()
        want = self.theirs.forward_ov(attn, want_cache, v_new, *rest).view(attn.shape[0], attn.shape[1], -1).float()
        got = self.ours.forward_ov(attn, v_cache, v_new, *rest)
        assert torch.equal(v_cache, want_cache), "forward_ov: appended code differs from the reference kernel's"
        torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2 * max(1.0, float(want.abs().max())))
        self.max_out_err = max(self.max_out_err, float((got.float() - want).abs().max()))
        self.n += 1
        return got


class ReferenceKernels:
    """The reference's compiled extension behind the Python signatures of its ``adkv/kernel/gemv.py`` (a pass-through
    there too, ``src/adkv/kernel/gemv.py:16-132``; only ``forward_ov`` reshapes its result)."""

    def __init__(self, ext):
        self.ext = ext
        self.encode_kv, self.forward_qk = ext.encode_kv, ext.forward_qk

    def forward_ov(self, attn, *rest):
        return self.ext.forward_ov(attn, *rest).view(attn.shape[0], attn.shape[1], -1)


@pytest.fixture
def reference_model_module(monkeypatch):
    """The staged, unmodified ``adkv.hf.llama_adkv`` imported on top of ``adkv_b200.gemv``."""
    for name in [m for m in sys.modules if m == "adkv" or m.startswith("adkv.")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.syspath_prepend(build_ref.staged_src())
    hf_shim.install()
    assert sys.modules["adkv.kernel.gemv"] is gemv
    import adkv.hf.llama_adkv as M
    assert os.path.realpath(M.__file__).startswith(os.path.realpath(build_ref.staged_src()))
    assert M.forward_qk is gemv.forward_qk and M.forward_ov is gemv.forward_ov and M.encode_kv is gemv.encode_kv
    hf_shim.patch_mask_sizes(M.KVCacheLayer_ADKV)
    yield M
    for name in [m for m in sys.modules if m == "adkv" or m.startswith("adkv.")]:
        del sys.modules[name]


def _adkv_config(M, n, seed):
    g = torch.Generator().manual_seed(seed)
    rho = 0.9 + 0.099 * torch.rand(n, generator=g)
    return M.ADKVConfig(torch.zeros(n), torch.ones(n), 1.0 - rho, torch.full((n,), 0.05), torch.full((n,), 3.5))


def test_reference_model_file_generates_on_the_cuda_kernels(reference_model_module, monkeypatch):
    M = reference_model_module
    from transformers import LlamaConfig
    checked = CheckedKernels()
    for fn in ("encode_kv", "forward_qk", "forward_ov"):               # the names the model file bound at import
        monkeypatch.setattr(M, fn, getattr(checked, fn))
    torch.manual_seed(0)
    L, H, Dh, B, prompt, new = 3, 2, 128, 2, 61, 8                      # 61 + 8 crosses the 64-token capacity step
    cfg = LlamaConfig(hidden_size=H * Dh, intermediate_size=256, num_hidden_layers=L, num_attention_heads=H,
                      num_key_value_heads=H, vocab_size=97, max_position_embeddings=256)
    model = M.LlamaForCausalLM_ADKV(cfg).half().cuda().eval()
    model.load_adkv_config([(_adkv_config(M, H * Dh, 10 + i), _adkv_config(M, H * Dh, 20 + i)) for i in range(L)])
    ids = torch.randint(0, 97, (B, prompt), device="cuda")
    with torch.no_grad():
        out = model.generate(input_ids=ids, max_new_tokens=new, do_sample=False)
    torch.cuda.synchronize()
    assert gemv.device_status() == 0
    assert out.shape == (B, prompt + new) and out.is_cuda

    calls = checked.calls
    enc = [c for c in calls if c[0] == "encode_kv"]
    qk = [c for c in calls if c[0] == "forward_qk"]
    ov = [c for c in calls if c[0] == "forward_ov"]
    assert len(enc) == 2 * L and all(c[2] == (B, H, prompt, Dh) for c in enc)           # K and V of every layer, once
    assert len(qk) == len(ov) == L * (new - 1)                                          # one pair per layer and step
    first_decode = calls.index(qk[0])
    assert all(c[0] == "encode_kv" for c in calls[:first_decode])                       # prefill first
    for i in range(len(qk)):
        a, b = calls[first_decode + 2 * i], calls[first_decode + 2 * i + 1]
        assert a[0] == "forward_qk" and b[0] == "forward_ov" and a[2] == b[2]           # same T for both halves
    assert [c[2] for c in qk[::L]] == list(range(prompt, prompt + new - 1))             # T grows by one per step
    assert {c[1][2] for c in qk} == {8, 16}                                            # caches replaced by larger ones
    print(f"reference model file on CUDA kernels: {len(calls)} kernel calls checked, max |logit - oracle| "
          f"{checked.max_logit_err:.3e}, max |out - oracle| {checked.max_out_err:.3e}")


@pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/adkv_gemv.so has not been built")
def test_reference_model_file_writes_the_caches_its_own_kernels_write(reference_model_module, monkeypatch):
    """The same generation with ``hf_shim.install(half_state=True)``: every call the unmodified model file makes is
    repeated by the reference's own CUDA kernels; the packed caches must be identical bit for bit after each call."""
    M = reference_model_module
    from transformers import LlamaConfig
    checked = CheckedAgainstReferenceKernels(hf_shim.install(half_state=True), ReferenceKernels(ref_cuda.module()))
    for fn in ("encode_kv", "forward_qk", "forward_ov"):
        monkeypatch.setattr(M, fn, getattr(checked, fn))
    torch.manual_seed(1)
    L, H, Dh, B, prompt, new = 3, 4, 128, 3, 61, 8
    cfg = LlamaConfig(hidden_size=H * Dh, intermediate_size=256, num_hidden_layers=L, num_attention_heads=H,
                      num_key_value_heads=H, vocab_size=97, max_position_embeddings=256)
    model = M.LlamaForCausalLM_ADKV(cfg).half().cuda().eval()
    model.load_adkv_config([(_adkv_config(M, H * Dh, 30 + i), _adkv_config(M, H * Dh, 40 + i)) for i in range(L)])
    ids = torch.randint(0, 97, (B, prompt), device="cuda")
    with torch.no_grad():
        out = model.generate(input_ids=ids, max_new_tokens=new, do_sample=False)
    torch.cuda.synchronize()
    assert gemv.device_status() == 0
    assert out.shape == (B, prompt + new)
    assert checked.n == 2 * L + 2 * L * (new - 1)
    print(f"reference model file, reference-kernel arithmetic: {checked.n} calls equal the reference's own kernels "
          f"(caches bit for bit; max |logit diff| {checked.max_logit_err:.3e}, max |out diff| {checked.max_out_err:.3e})")


def test_reference_model_file_end_to_end_throughput(reference_model_module):
    """Decode tokens/s of the random-init Llama-2-7B architecture through the reference's unmodified model file
    (HF ``generate``, its cache object, qk -> torch softmax -> ov per layer) on this library's kernels: batch 128,
    prompt 1024, as the end-to-end benchmark configuration, with a short generation.  The decode rate is the
    difference of two runs (17 and 1 new tokens; method of the reference's tools/perf_e2e.py:102-113: wall
    time around ``generate``).  Report only; also written as JSON into the folder ``ADKV_RESULTS_DIR`` names, if set."""
    M = reference_model_module
    from transformers import LlamaConfig
    if torch.cuda.get_device_properties(0).total_memory < 100e9:
        pytest.skip("needs a GPU with room for the 7B-shaped model and its prefill")
    torch.manual_seed(0)
    L, H, Dh, B, prompt = 32, 32, 128, 128, 1024
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=11008, num_hidden_layers=L, num_attention_heads=H,
                      num_key_value_heads=H, vocab_size=32000, max_position_embeddings=2048)
    with torch.device("cuda"):
        torch.set_default_dtype(torch.float16)
        try:
            model = M.LlamaForCausalLM_ADKV(cfg).eval()
        finally:
            torch.set_default_dtype(torch.float32)
    n = H * Dh
    model.load_adkv_config([(_adkv_config(M, n, 10 + i), _adkv_config(M, n, 50 + i)) for i in range(L)])
    ids = torch.randint(0, 32000, (B, prompt), device="cuda")

    def run(new):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.no_grad():
            out = model.generate(input_ids=ids, max_new_tokens=new, do_sample=False)
        torch.cuda.synchronize()
        assert out.shape == (B, prompt + new)
        return time.perf_counter() - t0

    kernel_sets = {"adkv_b200, fp32 recurrence (forward_qk -> torch softmax -> forward_ov)": hf_shim.install(),
                   "adkv_b200, the reference kernels' arithmetic": hf_shim.install(half_state=True)}
    if ref_cuda.available():
        kernel_sets["the reference's own kernels compiled for sm_100a"] = ReferenceKernels(ref_cuda.module())
    res = {"what": "random-init Llama-2-7B architecture, HF generate through the reference's unmodified "
                   "src/adkv/hf/llama_adkv.py; only the three kernel entry points differ between the rows",
           "batch": B, "prompt": prompt, "rows": {}}
    for name, ks in kernel_sets.items():
        for fn in ("encode_kv", "forward_qk", "forward_ov"):
            setattr(M, fn, getattr(ks, fn))
        run(2)                                  # warm-up: allocator, cuBLAS handles
        t1, t17 = run(1), run(17)
        assert gemv.device_status() == 0
        step_ms = (t17 - t1) / 16 * 1e3
        assert step_ms > 0
        res["rows"][name] = {"decode_ms_per_step": step_ms, "decode_tokens_per_s": B / (step_ms * 1e-3),
                             "prefill_plus_first_token_s": t1}
    first = next(iter(res["rows"].values()))
    res.update(decode_ms_per_step=first["decode_ms_per_step"], decode_tokens_per_s=first["decode_tokens_per_s"],
               prefill_plus_first_token_s=first["prefill_plus_first_token_s"])
    print(json.dumps(res))
    out_dir = os.environ.get("ADKV_RESULTS_DIR", "")
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "e2e_reference_model_file.json"), "w") as f:
            json.dump(res, f)
