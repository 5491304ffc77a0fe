"""CPU-side checks of the drop-in boundary: the C-ABI library loads and exports every declared symbol;
the Python mirror refuses CPU tensors instead of falling back."""
import os
import re

import pytest
import torch

from adkv_b200 import _lib, gemv, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "adkv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(adkv_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/adkv_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of step with the header"
    assert lib.adkv_abi_version() == 2


def test_strerror_texts():
    assert _lib.strerror(0) == "success"
    for code in range(-7, 0):
        assert _lib.strerror(code).startswith("adkv:")


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib._build, "LIB", "/nonexistent/libadkv_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_cpu_tensors_are_refused():
    p = synth.gen_params(0, 2, 128)
    cache = torch.zeros(1, 2, 2, 32, 4, 4, dtype=torch.uint8)
    x = torch.zeros(1, 2, 8, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        gemv.encode_kv(cache, x, *p, synth.SCALE_MIN, synth.SCALE_MAX)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        gemv.forward_qk(x[:, :, :1], cache, x[:, :, :1], *p, 3, synth.SCALE_MIN, synth.SCALE_MAX)


def test_null_and_shape_errors_from_the_c_abi():
    lib = _lib.load()
    P = _lib.Params(16, 16, 16, 16, 16)
    import ctypes
    pp = ctypes.addressof(P)
    assert lib.adkv_encode(None, 16, pp, None, 1, 1, 8, 128, 1, 4, 0, 0.1, 1.0, None) == -1
    assert lib.adkv_encode(16, 16, pp, None, 1, 1, 8, 64, 1, 4, 0, 0.1, 1.0, None) == -2
    assert lib.adkv_encode(16, 16, pp, None, 1, 1, 8, 128, 1, 3, 0, 0.1, 1.0, None) == -3
    assert lib.adkv_encode(16, 16, pp, None, 1, 1, 9, 128, 1, 4, 0, 0.1, 1.0, None) == -5
    assert lib.adkv_encode(16, 16, pp, None, 1, 1, 4, 128, 1, 4, 4, 0.1, 1.0, None) == -7
    assert lib.adkv_forward_qk(16, 16, 16, pp, 16, 1, 3, 2, 4, 128, 1, 4, 0.1, 1.0, 0, None) == -4
    assert lib.adkv_forward_qk(16, 24, 16, pp, 16, 1, 2, 2, 4, 128, 1, 4, 0.1, 1.0, 0, None) == -6
    assert lib.adkv_decode_attn(16, 16, 16, 16, 16, pp, pp, None, None, None, 0, 16, 1, 2, 2, 8, 128, 1, 4,
                                0.1, 0.1, 1.0, 0, None) == -5
    # tail states: both or neither, and not with the fp16-state arithmetic
    da = lambda kt, vt, flags: lib.adkv_decode_attn(16, 16, 16, 16, 16, pp, pp, kt, vt, None, 0, 16, 1, 2, 2, 7, 128,
                                                    1, 4, 0.1, 0.1, 1.0, flags, None)
    assert da(16, None, 0) == -10
    assert da(16, 16, _lib.FLAG_HALF_STATE) == -10
    assert da(16, 24, 0) == -6


def test_argument_errors_of_the_flagged_entry_points():
    """adkv_encode_kv_flags / adkv_append_kv_flags validate before anything is launched, in both arithmetics."""
    import ctypes
    lib = _lib.load()
    P = _lib.Params(16, 16, 16, 16, 16)
    pp = ctypes.addressof(P)
    for flags in (0, _lib.FLAG_HALF_STATE):
        def enc(kc, k, kpp, kt, vc, v, vpp, vt, *dims, kck=None, vck=None, iv=0, cap=0):
            return lib.adkv_encode_kv_flags(kc, k, kpp, kt, kck, vc, v, vpp, vt, vck, iv, cap, *dims, 0.1, 1.0, flags, None)
        assert enc(None, 16, pp, None, None, None, None, None, 1, 1, 8, 128, 1, 4, 0) == -1
        assert enc(16, 16, pp, None, None, None, None, None, 1, 1, 8, 64, 1, 4, 0) == -2
        assert enc(16, 16, pp, None, None, None, None, None, 1, 1, 8, 128, 1, 3, 0) == -3
        assert enc(16, 16, pp, None, None, None, None, None, 1, 1, 9, 128, 1, 4, 0) == -5
        assert enc(16, 16, pp, None, None, None, None, None, 1, 1, 4, 128, 1, 4, 4) == -7      # t_start without tail
        assert enc(16, 16, pp, None, 16, None, pp, None, 1, 1, 8, 128, 1, 4, 0) == -1          # V tensor without data
        assert enc(16, 16, pp, None, None, None, None, None, 1, 1, 8, 128, 1, 4, 0, iv=32) == -4   # checkpoints: K and V
        assert enc(16, 16, pp, None, 16, 16, pp, None, 1, 1, 8, 128, 1, 4, 0, iv=48, kck=16, vck=16, cap=4) == -4
        assert enc(16, 16, pp, None, 16, 16, pp, None, 1, 1, 8, 128, 1, 4, 0, iv=32, cap=4) == -1  # no checkpoint tensors

        def app(kc, k, kpp, kt, vc, v, vpp, vt, *dims):
            return lib.adkv_append_kv_flags(kc, k, kpp, kt, None, vc, v, vpp, vt, None, 0, 0, *dims, 0.1, 1.0, flags, None)
        assert app(16, 16, pp, None, None, None, None, None, 1, 1, 3, 128, 1, 4) == -1         # no tail state
        assert app(16, 16, pp, 16, None, None, None, None, 1, 1, 8, 128, 1, 4) == -5
    assert _lib.strerror(-10).startswith("adkv:")


def test_parameter_struct_cache_is_bounded_and_pins_nothing(monkeypatch):
    """The per-layer parameter structs are cached by device address in an LRU that holds no tensors."""
    import gc
    import weakref

    class FakeParam:
        """Stands in for a CUDA tensor: the cache only looks at address, dtype, size, device and contiguity."""
        def __init__(self, addr):
            self.addr, self.dtype, self.is_cuda, self.device = addr, torch.float16, True, "cuda:0"
        def data_ptr(self): return self.addr
        def numel(self): return 2 * 128
        def is_contiguous(self): return True
        def contiguous(self): return self

    monkeypatch.setattr(gemv, "_PARAM_CACHE_MAX", 4)
    gemv._PARAM_CACHE.clear()
    sets = [tuple(FakeParam(1000 * (i + 1) + 16 * j) for j in range(5)) for i in range(7)]
    refs = [weakref.ref(s[0]) for s in sets]
    for s in sets:
        p, keep = gemv._params(("a", "b", "c", "d", "e"), s, 2, 128, "cuda:0")
        assert p.zp_init == s[0].addr and p.target == s[4].addr
    assert len(gemv._PARAM_CACHE) == 4                              # oldest entries dropped one at a time
    first = gemv._params(("a",) * 5, sets[6], 2, 128, "cuda:0")[0]
    assert first is gemv._params(("a",) * 5, sets[6], 2, 128, "cuda:0")[0]   # a hit returns the cached struct
    del sets, s, keep
    gc.collect()
    assert all(r() is None for r in refs)                           # nothing in the cache kept the tensors alive
    gemv._PARAM_CACHE.clear()
