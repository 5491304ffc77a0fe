"""Generate the golden fixtures in this folder by EXECUTING the reference's torch code.

Run in a container that has the reference checkout (it is not needed to run the tests):

    TORCH_COMPILE_DISABLE=1 python tests/golden/make_golden.py /path/to/reference [case ...]

(no case names: all of them).

The script imports ``adkv.train.train_model`` from ``<reference>/src`` unmodified and
calls its ``_adkv_chunk_forward`` (``src/adkv/train/train_model.py:46-86``) eagerly
(``TORCH_COMPILE_DISABLE=1``: the ``@torch.compile`` decorator would otherwise hand the
loop to Inductor, which is neither available for CPU here nor bit-faithful).  The
integer codes are observed by wrapping ``IntQuantSTE.apply`` (it returns ``(x_hat, q)``,
``train_model.py:22``) in the module namespace; the reference code itself is untouched.

Each ``*.npz`` holds the inputs (fp16 values as float16 / parameters as float32) and
the reference outputs: codes, dequantised values and the final state.
"""
from __future__ import annotations

import math
import os
import sys

os.environ.setdefault("TORCH_COMPILE_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def load_reference(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import adkv.train.train_model as tm  # noqa: E402  (the reference's module)

    recorded = []
    real = tm.IntQuantSTE

    class Observer:
        @staticmethod
        def apply(x, sc, upper, lower):
            x_hat, q = real.apply(x, sc, upper, lower)
            recorded.append(q.clone())
            return x_hat, q

    tm.IntQuantSTE = Observer
    return tm, recorded


def run_case(tm, recorded, x16, params, bits, smin, smax):
    """x16 [B,H,T,D] float16; params 5 x [H,D] float32 (fp16-representable or not)."""
    B, H, T, D = x16.shape
    C = H * D
    x = x16.float().permute(0, 2, 1, 3).reshape(B, T, C).contiguous()
    zp0, s0, alpha, beta, target = (p.reshape(C).float() for p in params)
    hi = 2 ** (bits - 1) - 1
    lo = -2 ** (bits - 1)
    recorded.clear()
    with torch.no_grad():
        out, zpT, sT, zp_seq, s_seq = tm._adkv_chunk_forward(
            x, zp0.expand(B, -1).contiguous(), s0.expand(B, -1).contiguous(),
            alpha, beta, target, hi, lo, smin, smax, True)
    q = torch.stack(recorded, dim=1)                     # [B,T,C]

    def back(t):  # [B,T,C] -> [B,H,T,D]
        return t.reshape(B, T, H, D).permute(0, 2, 1, 3).contiguous().numpy()

    return dict(
        x=x16.numpy(), bits=np.int32(bits), scale_min=np.float64(smin), scale_max=np.float64(smax),
        zp_init=params[0].numpy(), scale_init=params[1].numpy(), alpha=params[2].numpy(),
        beta=params[3].numpy(), target=params[4].numpy(),
        codes=back(q).astype(np.int8), x_hat=back(out).astype(np.float32),
        zp_final=zpT.reshape(B, H, D).numpy().astype(np.float32),
        s_final=sT.reshape(B, H, D).numpy().astype(np.float32),
    )


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    tm, recorded = load_reference(ref_root)
    from adkv_b200 import synth

    smin, smax = math.exp(-4.0), math.exp(4.0)
    cases = {}

    # 1/2: benchmark distribution, benchmark parameters, both bit widths
    for bits in (4, 2):
        x = synth.gen_kv(100 + bits, 1, 2, 77, 128)
        p = tuple(t.float() for t in synth.gen_params(103 + bits, 2, 128, bits))
        cases[f"synth_b{bits}"] = run_case(tm, recorded, x, p, bits, smin, smax)

    # 3: random parameters (non-zero zp_init, varied scale_init / beta / target), fp16-valued
    g = torch.Generator().manual_seed(7)
    H, D = 3, 128
    x = (torch.randn(1, H, 45, D, generator=g) * 3).half()
    p = (torch.randn(H, D, generator=g), torch.rand(H, D, generator=g) * 2 + 0.05,
         torch.rand(H, D, generator=g) * 0.3, torch.rand(H, D, generator=g) * 0.1,
         torch.rand(H, D, generator=g) * 4 + 1)
    p = tuple(t.half().float() for t in p)
    cases["randparam_b4"] = run_case(tm, recorded, x, p, 4, smin, smax)

    # 4: clamp at both ends, zero / tiny initial scale (eps guard), exact .5 ties at token 0
    H, D = 1, 128
    x = torch.zeros(1, H, 120, D)
    x[..., :32] = 0.0                                               # q = 0 forever: scale decays to scale_min
    x[..., 32:64] = torch.randn(1, H, 120, 32, generator=g) * 500   # saturated codes: scale grows to scale_max
    x[..., 64:96] = torch.randn(1, H, 120, 32, generator=g)
    x[..., 96:] = torch.randn(1, H, 120, 32, generator=g) * 0.01
    ties = (torch.arange(32).float() - 16) * 0.5                    # -8.0 .. 7.5 in steps of .5
    x[0, 0, 0, 64:96] = ties
    s0 = torch.ones(H, D)
    s0[0, 96:112] = 0.0                                             # below eps
    s0[0, 112:] = 1e-9
    p = (torch.zeros(H, D), s0, torch.full((H, D), 0.1), torch.full((H, D), 0.1), torch.full((H, D), 3.5))
    p = tuple(t.half().float() if i != 1 else t for i, t in enumerate(p))
    cases["clamp_eps_ties_b4"] = run_case(tm, recorded, x.half(), p, 4, smin, smax)

    # 5: case 4 with parameters the kernel API can take (fp16): the only fp16 value below the eps guard is 0.0
    # (the smallest fp16 subnormal, 5.96e-8, is already above 1e-8).  Guard, both clamps and exact ties.
    g5 = torch.Generator().manual_seed(55)
    x = torch.zeros(1, H, 120, D)
    x[..., 32:64] = torch.randn(1, H, 120, 32, generator=g5) * 500
    x[..., 64:96] = torch.randn(1, H, 120, 32, generator=g5)
    x[..., 96:] = torch.randn(1, H, 120, 32, generator=g5) * 0.01
    x[0, 0, 0, 64:96] = ties
    s0 = torch.ones(H, D)
    s0[0, 96:] = 0.0
    p = tuple(t.half().float() for t in (torch.zeros(H, D), s0, torch.full((H, D), 0.1), torch.full((H, D), 0.1),
                                          torch.full((H, D), 3.5)))
    cases["guard_clamp_ties_fp16_b4"] = run_case(tm, recorded, x.half(), p, 4, smin, smax)

    # 6: scale_min = 0, so nothing holds the scale up: on all-zero and on tiny inputs it decays below the eps guard
    # in mid-sequence (factor 1 - beta*target = 0.65 per token, 1e-8 after ~43 tokens) and the guard alone decides
    # the quotient from then on; later tokens are large again, so the scale has to climb back out.
    g6 = torch.Generator().manual_seed(66)
    x = torch.zeros(1, H, 120, D)
    x[..., 32:64] = torch.randn(1, H, 120, 32, generator=g6) * 3e-7      # fp16 subnormals
    x[..., 64:96] = torch.randn(1, H, 120, 32, generator=g6) * 1e-4
    x[..., 96:] = torch.randn(1, H, 120, 32, generator=g6)
    x[:, :, 80:, :64] = torch.randn(1, H, 40, 64, generator=g6) * 2.0
    p = tuple(t.half().float() for t in (torch.zeros(H, D), torch.ones(H, D), torch.full((H, D), 0.1),
                                          torch.full((H, D), 0.1), torch.full((H, D), 3.5)))
    cases["guard_decay_scale_min0_b4"] = run_case(tm, recorded, x.half(), p, 4, 0.0, smax)

    only = set(sys.argv[2:])
    for name, d in cases.items():
        if only and name not in only:
            continue
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **d)
        print(name, {k: getattr(v, "shape", v) for k, v in d.items() if k in ("x", "codes")},
              os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
