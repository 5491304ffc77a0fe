"""The drop-in boundary: adkv_b200.gemv under the reference's module name, signature compatibility with
the reference's kernel module (checked against the reference checkout when it is present)."""
import importlib
import inspect
import os
import sys

import pytest

from adkv_b200 import gemv, hf_shim

# a checkout of the reference project, when one is available (the comparison is skipped otherwise)
REF = os.environ.get("ADKV_REFERENCE_ROOT",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.pardir, "reference"))


def test_install_registers_module_under_reference_name():
    saved = {k: sys.modules.get(k) for k in ("adkv", "adkv.kernel", "adkv.kernel.gemv")}
    try:
        hf_shim.install()
        mod = importlib.import_module("adkv.kernel.gemv")
        assert mod is gemv
        from adkv.kernel.gemv import encode_kv, forward_ov, forward_qk   # the reference model file's import line
        assert encode_kv is gemv.encode_kv and forward_qk is gemv.forward_qk and forward_ov is gemv.forward_ov
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def _ref_kernel_module_text():
    """Path of the reference's kernel module as text: the checkout when it is there, else the copy that
    oracle/build_ref.py staged (it travels to machines without a checkout), else None."""
    from oracle import build_ref
    for path in (os.path.join(REF, "src", "adkv", "kernel", "gemv.py"), build_ref.KERNEL_MODULE_TEXT):
        if os.path.exists(path):
            return path
    return None


def _ref_signatures():
    """Positional parameter names of the reference's three wrappers, parsed from its source text
    (importing it would JIT-build the reference's CUDA extension)."""
    import ast
    tree = ast.parse(open(_ref_kernel_module_text()).read())
    return {n.name: [a.arg for a in n.args.args] for n in tree.body if isinstance(n, ast.FunctionDef)}


@pytest.mark.skipif(_ref_kernel_module_text() is None, reason="neither a reference checkout nor its staged copy is present")
def test_positional_signatures_match_reference():
    ref = _ref_signatures()
    assert set(ref) == {"forward_qk", "forward_ov", "encode_kv"}
    for name, ref_args in ref.items():
        ours = inspect.signature(getattr(gemv, name))
        pos = [p.name for p in ours.parameters.values() if p.kind == p.POSITIONAL_OR_KEYWORD]
        assert pos == ref_args, f"{name}: {pos} != {ref_args}"
        extra = [p for p in ours.parameters.values() if p.kind == p.KEYWORD_ONLY]
        assert all(p.default is not inspect.Parameter.empty for p in extra)     # extensions are optional


def test_install_in_the_reference_kernels_arithmetic_keeps_the_positional_signatures():
    saved = {k: sys.modules.get(k) for k in ("adkv", "adkv.kernel", "adkv.kernel.gemv")}
    try:
        mod = hf_shim.install(half_state=True)
        assert importlib.import_module("adkv.kernel.gemv") is mod and mod is not gemv
        for name in ("encode_kv", "forward_qk", "forward_ov"):
            want = [p.name for p in inspect.signature(getattr(gemv, name)).parameters.values()
                    if p.kind == p.POSITIONAL_OR_KEYWORD]
            got = list(inspect.signature(getattr(mod, name)).parameters)
            assert got == want, f"{name}: {got} != {want}"          # nothing but the reference's own arguments
        assert hf_shim.install() is gemv                           # and the default registration comes back
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def test_patch_mask_sizes_accepts_int_and_tensor():
    import torch

    class Layer:
        def get_seq_length(self):
            return 5
    hf_shim.patch_mask_sizes(Layer)
    assert Layer().get_mask_sizes(3) == (8, 0)
    assert Layer().get_mask_sizes(torch.arange(2)) == (7, 0)
