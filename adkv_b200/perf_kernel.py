"""Decode-step kernel micro-benchmark on the grid and with the methodology of the reference's own tool.

    python -m adkv_b200.perf_kernel [--impl trio,fused,fused-fast,fused-tail,trio-half,fused-half,reference] [--reference-so PATH]
                                    [--json out.json]

The reference measures one decode step of one layer (``forward_qk`` -> torch softmax -> ``forward_ov``) for
batch sizes 1..512 and 128..2048 cached tokens, Llama-2-7B heads (32 x 128), and reports
``B / (median step latency x 32 layers)`` requests per second (``tools/perf_kernel.py:12-16, 29-77, 91-104``;
its published table is for an L40).  This tool repeats that on the GPU it runs on for

* ``trio``       the same three calls through this library (drop-in signatures),
* ``fused``      the single-launch ``decode_attn`` that replaces them,
* ``fused-fast`` the same with the contracted replay of the fp32 recurrence (``fast=True``),
* ``fused-tail`` the same next to persisted tail states, as the cache object runs it: the appended code is quantised
                 from the tail (bit-exact) and the replay is contracted; the tails are kept unadvanced so that every
                 step overwrites slot T like the other columns,
* ``*-half``     both in the fp16-state arithmetic of the reference's CUDA kernels,
* ``reference``  the reference's own kernels, from the extension module given with ``--reference-so`` (the
                 ``adkv_gemv`` module the reference JIT-builds, or the one ``oracle/build_ref.py`` compiles for
                 sm_100a); skipped when none is given.

As there: caches filled with the byte 0x5A, q / k_new / v_new ~ 0.5 N(0,1) fp16, zp 0, scale 1, alpha 0.05,
beta 0, target 3.5; 3 warm-up steps; ``max(5, min(100, 2e6 / (B T)))`` timed steps, each bracketed by CUDA
events; the median; the new token overwrites slot T every step.
"""
from __future__ import annotations

import argparse
import importlib.machinery
import importlib.util
import json
import statistics
import sys

import torch

from . import gemv
from .synth import SCALE_MAX, SCALE_MIN

NH, DIM = 32, 128
BATCHES = [1, 4, 16, 32, 64, 128, 256, 512]
SEQ_LENS = [128, 256, 512, 1024, 2048]
LAYERS = 32
IMPLS = ("trio", "fused", "fused-fast", "fused-tail", "trio-half", "fused-half", "reference")


def load_extension(path: str):
    """The reference's torch extension (``forward_qk`` / ``forward_ov`` of ``src/adkv/kernel/gemv.cpp:28-33``) by path."""
    loader = importlib.machinery.ExtensionFileLoader("adkv_gemv", path)
    mod = importlib.util.module_from_spec(importlib.util.spec_from_loader("adkv_gemv", loader))
    loader.exec_module(mod)
    return mod


def make_step(impl: str, B: int, T: int, dev, ref=None):
    """Inputs of one (B, T) point and a callable that runs one decode step of one layer."""
    n_super = gemv.n_super_for(T + 1, 4) + 1
    kc = torch.full((B, NH, n_super, DIM // 4, 4, 4), 0x5A, dtype=torch.uint8, device=dev)
    vc = torch.full_like(kc, 0x5A)
    q, kn, vn = (torch.randn(B, NH, 1, DIM, dtype=torch.float16, device=dev) * 0.5 for _ in range(3))
    p = (torch.zeros(NH, DIM, dtype=torch.float16, device=dev), torch.ones(NH, DIM, dtype=torch.float16, device=dev),
         torch.full((NH, DIM), 0.05, dtype=torch.float16, device=dev),
         torch.zeros(NH, DIM, dtype=torch.float16, device=dev),
         torch.full((NH, DIM), 3.5, dtype=torch.float16, device=dev))
    half = impl.endswith("-half")
    if impl == "reference":
        if ref is None:
            return None

        def step():
            logits = ref.forward_qk(q, kc, kn, *p, T, SCALE_MIN, SCALE_MAX)
            ref.forward_ov(torch.softmax(logits, dim=-1), vc, vn, *p, SCALE_MIN, SCALE_MAX)
    elif impl.startswith("trio"):
        def step():
            logits = gemv.forward_qk(q, kc, kn, *p, T, SCALE_MIN, SCALE_MAX, half_state=half)
            gemv.forward_ov(torch.softmax(logits, dim=-1), vc, vn, *p, SCALE_MIN, SCALE_MAX, half_state=half)
    else:
        out = torch.empty(B, NH, DIM, dtype=torch.float16, device=dev)
        tails = {}
        if impl == "fused-tail":    # state after the cached tokens: zero point 0 (the codes are all 2: q * scale accumulates
            # with alpha, but any finite state does for timing), scale 1 (beta is 0 here)
            tk = torch.zeros(B, NH, 2, DIM, dtype=torch.float32, device=dev)
            tk[:, :, 1] = 1.0
            tails = dict(k_tail=tk, v_tail=tk.clone(), tail_keep=True)

        def step():
            gemv.decode_attn(q, kc, vc, kn, vn, p, p, T, 1.0, SCALE_MIN, SCALE_MAX, half_state=half,
                             fast=True if impl == "fused-fast" else None if impl == "fused-tail" else False, out=out,
                             **tails)
    return step


def median_ms(step, B: int, T: int) -> float:
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    iters = max(5, min(100, 2_000_000 // (B * T)))
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in ev)


def wake_gpu(dev, seconds: float = 0.5):
    """Bring the GPU out of its idle clocks before the small cases are timed."""
    import time
    a = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    b = torch.empty_like(a)
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        for _ in range(20):
            b.copy_(a)
        torch.cuda.synchronize()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--impl", default=",".join(IMPLS), help="comma-separated subset of " + ", ".join(IMPLS))
    ap.add_argument("--batches", default=",".join(map(str, BATCHES)))
    ap.add_argument("--seq-lens", default=",".join(map(str, SEQ_LENS)))
    ap.add_argument("--reference-so", default=None, help="path of the reference's adkv_gemv extension module")
    ap.add_argument("--json", default=None, help="also write the table as JSON to this file")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    impls = [s for s in a.impl.split(",") if s]
    batches = [int(s) for s in a.batches.split(",")]
    seq_lens = [int(s) for s in a.seq_lens.split(",")]
    ref = load_extension(a.reference_so) if a.reference_so else None
    wake_gpu(dev)
    table = {}
    for impl in impls:
        if impl not in IMPLS:
            sys.exit(f"unknown implementation {impl!r}")
        rows = {}
        for B in batches:
            row = {}
            for T in seq_lens:
                step = make_step(impl, B, T, dev, ref)
                if step is None:
                    break
                ms = median_ms(step, B, T)
                row[T] = {"ms": ms, "req_per_s": B / (ms * 1e-3 * LAYERS)}
                del step
                torch.cuda.empty_cache()
            if row:
                rows[B] = row
        if not rows:
            print(f"[{impl}] skipped: no --reference-so given")
            continue
        table[impl] = rows
        print(f"[{impl}] requests/s over {LAYERS} layers = B / (median step ms x {LAYERS}); heads {NH} x {DIM}, 4-bit")
        print("B\\T".ljust(8) + "".join(f"{t:>11}" for t in seq_lens))
        for B, row in rows.items():
            print(f"{B:<8}" + "".join(f"{row[t]['req_per_s']:11.1f}" for t in seq_lens))
        print()
    assert gemv.device_status(dev) == 0, "a kernel gave up on a bounded wait"
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"gpu": torch.cuda.get_device_name(dev), "layers": LAYERS, "heads": NH, "head_dim": DIM,
                       "table": table}, f)
    return table


if __name__ == "__main__":
    main()
