"""Benchmark of the ADKV decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one fused decode-attention pass (q.K^T, softmax, P.V and both appends, one launch) over one
batch of synthetic post-RoPE-outlier K/V held as packed ADKV codes.  The default workload is the
Llama-2-7B shape of the headline metric: 32 heads, head_dim 128, batch 128, 4096 cached tokens, 4-bit
codes.  With N > 1 (one process per GPU, launched by torch.distributed.run) the (batch, kv-head) streams
of that fixed workload are sharded over the ranks (``adkv_b200.sharding``: whole sequences first, KV heads
when the batch does not divide) with no collective on the data path: strong scaling.  ``--scaling weak``
gives every rank the whole workload instead; with the default the weak figure is measured too and printed
as the extra key ``weak_scaling``, and the same shards with state checkpoints as
``strong_with_checkpoints``.  Rank 0 prints one JSON line.

``value``  : packed-KV bytes processed per second by the whole job, inputs resident in HBM.
``e2e``    : the same through the public Python API with the step's q / k_new / v_new coming from
             pinned host memory and the output copied back, copies inside the timed region.
``roofline``: algorithmic bytes per launch / average launch time (CUDA events) against the measured
             HBM copy bandwidth of MEASURED_PEAKS.json.
``cpu_baseline``: the reference's own torch recurrence (staged unchanged under oracle/_ref/src by
             oracle/build_ref.py) + torch attention on the host cores, on a bounded sample of the same
             workload, and its time for the CPU-sized configuration (batch 1, 1024 tokens).  Where the staged
             file is absent: the C restatement (``kind: "port"``).
``cpu_baseline_port``: the C/OpenMP restatement of the same algorithm (oracle/), a much stricter CPU figure;
             it also checks the GPU result of its sample (``parity_check``).
             The baseline legs are the only code here that touches oracle/; they run after the timed
             regions, and ``--no-cpu`` skips them.
``--impl reference`` times the reference's CPU implementation alone, one bounded sample per step.
``reference_cuda``, ``unfused_trio``: for the record, the reference caller's three-call sequence
             (forward_qk, torch softmax, forward_ov) through the reference's own CUDA kernels recompiled for
             sm_100a (oracle/_ref, when built; they compute in fp16) and through this library's kernels.
``other_workloads``: one-GPU figures of the prefill-quantise configuration (4- and 2-bit) and of the long-context
             grouped-query configuration, a few steps each, so that one run records every benchmark shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

STRONG_CKPT_INTERVAL = 512     # tokens between state checkpoints in the `strong_with_checkpoints` figure

WORKLOADS = {
    # name: per-GPU batch, q heads, kv heads, head dim, cached tokens, bits
    "config2_llama2_7b_b128_t4096_4bit": dict(B=128, Hq=32, Hkv=32, D=128, T=4096, bits=4),
    "config5_llama3_8b_gqa_b32_t32768_2bit": dict(B=32, Hq=32, Hkv=8, D=128, T=32768, bits=2),
    "small_b8_t1024_4bit": dict(B=8, Hq=32, Hkv=32, D=128, T=1024, bits=4),
    # prefill quantise of one layer's K and V (config 3 has 32 such layers), then single-token appends
    "config3_prefill_b16_t8192_4bit": dict(kind="encode", B=16, Hq=32, Hkv=32, D=128, T=8192, bits=4, appends=256),
    "config3_prefill_b16_t8192_2bit": dict(kind="encode", B=16, Hq=32, Hkv=32, D=128, T=8192, bits=2, appends=256),
    "profile_prefill_b16_t2048_4bit": dict(kind="encode", B=16, Hq=32, Hkv=32, D=128, T=2048, bits=4, appends=8),
    "profile_prefill_b16_t2048_2bit": dict(kind="encode", B=16, Hq=32, Hkv=32, D=128, T=2048, bits=2, appends=8),
    # profiling-sized cases: same kernels and per-stream work, a few hundred MB on the device
    "profile_b16_t4096_4bit": dict(B=16, Hq=32, Hkv=32, D=128, T=4096, bits=4),
    "profile_b64_t4096_4bit": dict(B=64, Hq=32, Hkv=32, D=128, T=4096, bits=4),
    "profile_gqa_b8_t16384_2bit": dict(B=8, Hq=32, Hkv=8, D=128, T=16384, bits=2),
}
DEFAULT_WORKLOAD = "config2_llama2_7b_b128_t4096_4bit"
METRIC = "fused_adkv_decode_attn_packed_kv_bandwidth"
UNIT = "GB/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the fused kernel (bytes), from an ncu capture;
# None where no capture exists for the workload.
NCU_TRAFFIC_BYTES = {
    # 274.8 MB measured on a batch-16 capture of the same kernel (tail path); streams are independent, so traffic
    # scales with the batch: x8 for batch 128
    "config2_llama2_7b_b128_t4096_4bit": 8 * 274_810_624,
    "profile_b16_t4096_4bit": 274_810_624,
}


def algorithmic_bytes(w) -> int:
    """Bytes one step must move.  Decode: packed K and V, q and out, k_new and v_new, parameters.
    Encode (prefill quantise of K and V): fp16 in, packed codes out."""
    B, Hq, Hkv, D, T, bits = w["B"], w["Hq"], w["Hkv"], w["D"], w["T"], w["bits"]
    if w.get("kind") == "encode":
        return 2 * (B * Hkv * T * D * 2 + B * Hkv * T * D * bits // 8)
    return 2 * B * Hkv * T * D * bits // 8 + 2 * B * Hq * D * 2 + 2 * B * Hkv * D * 2 + 10 * Hkv * D * 2


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# --------------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read only) in a thread."""

    def __init__(self, index: int, pci_bus_id: str | None = None, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.mark = [], None
        self._stop = threading.Event()
        self._thr = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                self.h = pynvml.nvmlDeviceGetHandleByPciBusId(pci_bus_id.encode()) if pci_bus_id else \
                    pynvml.nvmlDeviceGetHandleByIndex(index)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _reasons(self, mask: int):
        nv = self.nv
        names = {"hw_slowdown": "nvmlClocksThrottleReasonHwSlowdown",
                 "hw_thermal_slowdown": "nvmlClocksThrottleReasonHwThermalSlowdown",
                 "sw_thermal_slowdown": "nvmlClocksThrottleReasonSwThermalSlowdown",
                 "sw_power_cap": "nvmlClocksThrottleReasonSwPowerCap"}
        return [k for k, v in names.items() if mask & getattr(nv, v, 0)]

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, mask))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self, t0: float, t1: float):
        if self.nv is None:
            return self._smi_fallback()
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mask = 0
        for s in inside:
            mask |= s[2]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.max_mhz,
                "reasons": self._reasons(mask), "samples": len(inside)}

    def _smi_fallback(self):
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.index),
                                  "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits"],
                                 capture_output=True, text=True, timeout=10).stdout.strip().split(",")
            return {"sm_mhz": float(out[0]), "sm_max_mhz": float(out[1]), "reasons": [], "samples": 1,
                    "note": "NVML unavailable: single nvidia-smi sample after the timed region"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


# --------------------------------------------------------------------------------------- CPU arm

def cpu_sample(w, n_streams: int, seed: int = 1234):
    """Inputs of `n_streams` (batch, kv head) streams of the workload, prefilled by the C restatement."""
    import numpy as np

    from adkv_b200 import synth
    from oracle import adkv_oracle as orc
    from oracle import c_oracle
    Hkv, G, D, T, bits = w["Hkv"], w["Hq"] // w["Hkv"], w["D"], w["T"], w["bits"]
    # the sample is laid out as a batch of n_streams sequences with one kv head each
    k = synth.gen_kv(seed, n_streams, 1, T + 1, D).numpy()
    v = synth.gen_kv(seed + 1, n_streams, 1, T + 1, D).numpy()
    q = synth.gen_q(seed + 2, n_streams, G, D).numpy()[:, :, 0]
    kp = tuple(t.float().numpy() for t in synth.gen_params(seed + 3, 1, D, bits))
    vp = tuple(t.float().numpy() for t in synth.gen_params(seed + 4, 1, D, bits))
    ns = orc.n_super_for(T + 1, bits)
    kc = np.zeros(orc.cache_shape(n_streams, 1, ns, D), np.uint8)
    vc = np.zeros_like(kc)
    c_oracle.encode(kc, k[:, :, :T], kp, bits, synth.SCALE_MIN, synth.SCALE_MAX)
    c_oracle.encode(vc, v[:, :, :T], vp, bits, synth.SCALE_MIN, synth.SCALE_MAX)
    return dict(k=k, v=v, q=q, kp=kp, vp=vp, kc=kc, vc=vc, n=n_streams)


def cpu_step(w, s):
    from adkv_b200 import synth
    from oracle import c_oracle
    T = w["T"]
    return c_oracle.decode_attn(s["q"], s["kc"], s["vc"], s["k"][:, :, T], s["v"][:, :, T], s["kp"], s["vp"], T,
                                w["D"] ** -0.5, w["bits"], synth.SCALE_MIN, synth.SCALE_MAX)


def sample_bytes(w, n_streams: int) -> int:
    ws = dict(w, B=n_streams, Hkv=1, Hq=w["Hq"] // w["Hkv"])
    return algorithmic_bytes(ws)


def pick_sample_streams(w, target_s: float) -> int:
    """Streams whose decode takes about `target_s` seconds of host time, from a 1-stream-per-thread probe."""
    from oracle import c_oracle
    c_oracle.build()
    thr = c_oracle.use_all_cores()
    probe = cpu_sample(w, thr)
    cpu_step(w, probe)
    t0 = time.perf_counter()
    cpu_step(w, probe)
    dt = max(time.perf_counter() - t0, 1e-4)
    n = int(target_s / dt) * thr
    return max(thr, min(n, w["B"] * w["Hkv"]))


def workload_config(name, w_rank, w_global, world, args) -> dict:
    """The ``config`` object of the JSON line; both arms print the same one for the same command line."""
    nbytes = algorithmic_bytes(w_rank)
    return dict(workload=name, per_gpu=w_rank, global_batch=w_global["B"], replay=args.replay,
                ckpt_interval=args.ckpt_interval,
                sharding="(batch, kv-head) streams split over one process per GPU, no collective on the data path",
                l2="inputs (packed K+V per step) larger than L2; no flush needed"
                if nbytes > 200e6 else "inputs smaller than L2: cache-resident timing")


def rank_workload(w, world, rank, scaling):
    """The slice of workload ``w`` that rank ``rank`` of ``world`` owns: all of it for weak scaling, its rectangle
    of the (batch, kv-head) grid for strong scaling."""
    if world == 1 or scaling == "weak":
        return dict(w)
    from adkv_b200 import sharding
    sh = sharding.plan(w["B"], w["Hkv"], world)[rank]
    G = w["Hq"] // w["Hkv"]
    return dict(w, B=sh.b1 - sh.b0, Hkv=sh.h1 - sh.h0, Hq=G * (sh.h1 - sh.h0))


# ---- the reference's torch recurrence (oracle/_ref/src, staged unchanged) on the host cores

def torch_reference_sample(w, n_seq: int, n_heads: int, tokens: int, seed: int = 4321):
    """Inputs of ``n_seq`` sequences x ``n_heads`` KV heads of the workload, the first ``tokens + 1`` tokens."""
    from adkv_b200 import synth
    G, D, bits = w["Hq"] // w["Hkv"], w["D"], w["bits"]
    return dict(k=synth.gen_kv(seed, n_seq, n_heads, tokens + 1, D), v=synth.gen_kv(seed + 1, n_seq, n_heads, tokens + 1, D),
                q=synth.gen_q(seed + 2, n_seq, G * n_heads, D), kp=synth.gen_params(seed + 3, n_heads, D, bits),
                vp=synth.gen_params(seed + 4, n_heads, D, bits), bits=bits, scaling=D ** -0.5, n_seq=n_seq,
                n_heads=n_heads, tokens=tokens)


def torch_reference_step(smp):
    from adkv_b200 import synth
    from oracle import ref_torch
    return ref_torch.decode_attention(smp["q"], smp["k"], smp["v"], smp["kp"], smp["vp"], smp["bits"], smp["scaling"],
                                      synth.SCALE_MIN, synth.SCALE_MAX)


def pick_torch_sample(w, step_budget_s: float):
    """(sequences, kv heads, tokens) of a sample whose step takes about ``step_budget_s`` on this host.  The
    reference's recurrence is a Python loop over tokens (src/adkv/train/train_model.py:66-81), so its time is
    tokens x (a fixed cost per token + a cost per channel): two probes give both."""
    T, H = w["T"], w["Hkv"]
    tp = min(T, 256)
    t_small, _ = timed_cpu(lambda s=torch_reference_sample(w, 1, 1, tp): torch_reference_step(s))
    t_wide, _ = timed_cpu(lambda s=torch_reference_sample(w, 1, H, tp): torch_reference_step(s))
    per_tok_head = max((t_wide - t_small) / (tp * max(H - 1, 1)), 1e-9)
    per_tok_fixed = max(t_small / tp - per_tok_head, 1e-9)
    est = lambda heads, toks: toks * (per_tok_fixed + per_tok_head * heads)
    if est(H, T) <= step_budget_s:                      # whole sequences
        n_seq = int(max(1, min(w["B"], step_budget_s // est(H, T))))
        return n_seq, H, T
    heads = int(max(1, min(H, (step_budget_s / T - per_tok_fixed) / per_tok_head)))
    if est(heads, T) <= step_budget_s * 1.5:
        return 1, heads, T
    return 1, 1, int(max(32, min(T, step_budget_s / (per_tok_fixed + per_tok_head))))


def use_all_host_threads(torch) -> int:
    """Let torch use every core this process may run on (launchers export OMP_NUM_THREADS=1 for every rank)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(n)
    return torch.get_num_threads()


def timed_cpu(fn, repeats: int = 1):
    best, res = float("inf"), None
    for _ in range(repeats):
        t0 = time.perf_counter()
        res = fn()
        best = min(best, time.perf_counter() - t0)
    return best, res


def torch_sample_bytes(w, smp) -> float:
    """Algorithmic bytes of the part of the workload the sample stands for (tokens scaled linearly)."""
    return sample_bytes(w, smp["n_seq"] * smp["n_heads"]) * (smp["tokens"] / w["T"])


def describe_torch_sample(w, smp) -> str:
    extra = "" if smp["tokens"] == w["T"] else f", first {smp['tokens']} of {w['T']} tokens (bytes scaled linearly)"
    return (f"{smp['n_seq']} sequence(s) x {smp['n_heads']} of {w['Hkv']} kv heads = {smp['n_seq'] * smp['n_heads']} of "
            f"{w['B'] * w['Hkv']} (batch, kv-head) streams per step{extra}; the reference's _adkv_chunk_forward "
            "(eager) on K and V + torch attention")


def config1_seconds():
    """The reference's CPU-sized configuration (batch 1, 32 heads, 1024 tokens, head_dim 128, 4-bit): seconds for its
    quantise -> dequantise -> single-query attention, best of 3."""
    w1 = dict(B=1, Hq=32, Hkv=32, D=128, T=1023, bits=4)
    smp = torch_reference_sample(w1, 1, 32, 1023)
    return timed_cpu(lambda: torch_reference_step(smp), repeats=3)[0]


def run_reference(args, w, name):
    """The reference's CPU implementation of the path on the host cores, one bounded sample per step: its own torch
    recurrence where oracle/_ref/src holds it, else the C restatement (all threads)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import torch

    from oracle import c_oracle, ref_torch
    w_rank = rank_workload(w, world, 0, args.scaling)
    budget = min(2.0, max(0.05, 120.0 / (args.steps + args.warmup)))
    use_all_host_threads(torch)
    if ref_torch.available():
        smp = torch_reference_sample(w, *pick_torch_sample(w, budget))
        step = lambda: torch_reference_step(smp)
        nbytes, sample = torch_sample_bytes(w, smp), describe_torch_sample(w, smp)
        kind, cores = "reference", torch.get_num_threads()
    else:
        n = pick_sample_streams(w, target_s=budget)
        s = cpu_sample(w, n)
        step = lambda: cpu_step(w, s)
        nbytes = sample_bytes(w, n)
        sample = f"{n} of {w['B'] * w['Hkv']} (batch, kv-head) streams of the workload per step, C restatement with OpenMP"
        kind, cores = "port", c_oracle.num_threads()
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = nbytes * args.steps / dt / 1e9
    res = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(name, w_rank, w, world, args),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if kind == "reference":
        res["cpu_baseline"]["config1_seconds"] = config1_seconds()
    print(json.dumps(res), flush=True)


# --------------------------------------------------------------------------------------- GPU arm

def build_gpu_state(w, seed, device, torch, ckpt_interval=0, half_state=False):
    """Caches prefilled by the encode kernel from on-device synthetic K/V, plus the step's inputs."""
    from adkv_b200 import gemv, synth
    B, Hq, Hkv, D, T, bits = w["B"], w["Hq"], w["Hkv"], w["D"], w["T"], w["bits"]
    ns = gemv.n_super_for(T + 1, bits)
    kp = synth.gen_params(seed + 3, Hkv, D, bits, device=device)
    vp = synth.gen_params(seed + 4, Hkv, D, bits, device=device)
    kc = torch.zeros((B, Hkv, ns, D // 4, 4, 4), dtype=torch.uint8, device=device)
    vc = torch.zeros_like(kc)
    kck = vck = scratch = None
    tk = torch.empty((B, Hkv, 2, D), dtype=torch.float32, device=device)
    tv = torch.empty_like(tk)
    if ckpt_interval:
        kck = gemv.alloc_ckpt(B, Hkv, D, T + 1, ckpt_interval, device)
        vck = gemv.alloc_ckpt(B, Hkv, D, T + 1, ckpt_interval, device)
        scratch = torch.empty(gemv.decode_scratch_bytes(B, Hq, Hkv, T, ckpt_interval), dtype=torch.uint8, device=device)
    chunk = max(1, min(B, (1 << 28) // (Hkv * T * D)))      # keep generator temporaries around 1 GiB
    for b0 in range(0, B, chunk):
        b1 = min(B, b0 + chunk)
        k = synth.gen_kv(seed + 10 * b0, b1 - b0, Hkv, T, D, device=device)
        v = synth.gen_kv(seed + 10 * b0 + 1, b1 - b0, Hkv, T, D, device=device)
        if ckpt_interval:
            gemv.encode_kv_pair(kc[b0:b1], k, kp, vc[b0:b1], v, vp, synth.SCALE_MIN, synth.SCALE_MAX, bits=bits,
                                k_ckpt=kck[b0:b1], v_ckpt=vck[b0:b1], ckpt_interval=ckpt_interval,
                                half_state=half_state, k_tail=tk[b0:b1], v_tail=tv[b0:b1])
        else:
            gemv.encode_kv_pair(kc[b0:b1], k, kp, vc[b0:b1], v, vp, synth.SCALE_MIN, synth.SCALE_MAX, bits=bits,
                                half_state=half_state, k_tail=tk[b0:b1], v_tail=tv[b0:b1])
        del k, v
    q = synth.gen_q(seed + 2, B, Hq, D, device=device)
    kn = synth.gen_kv(seed + 5, B, Hkv, 1, D, device=device, pos0=T)
    vn = synth.gen_kv(seed + 6, B, Hkv, 1, D, device=device, pos0=T)
    torch.cuda.synchronize(device)
    ck = dict(k_ckpt=kck, v_ckpt=vck, ckpt_interval=ckpt_interval, scratch=scratch) if ckpt_interval else {}
    return dict(kc=kc, vc=vc, kp=kp, vp=vp, q=q, kn=kn, vn=vn, ck=ck, tk=tk, tv=tv)


def check_against_oracle(w, st, out, n_streams, torch):
    """Compare the GPU output and appended codes of the first streams with the C restatement; time it."""
    import numpy as np

    from adkv_b200 import synth
    from oracle import c_oracle
    c_oracle.use_all_cores()
    Hq, Hkv, D, T, bits = w["Hq"], w["Hkv"], w["D"], w["T"], w["bits"]
    G = Hq // Hkv
    nb = max(1, min(w["B"], (n_streams + Hkv - 1) // Hkv))
    n_streams = nb * Hkv
    kc_after = st["kc"][:nb].cpu().numpy()
    vc_after = st["vc"][:nb].cpu().numpy()
    kc, vc = kc_after.copy(), vc_after.copy()       # slot T already holds the GPU's append; the CPU rewrites it
    f = lambda ps: tuple(p.float().cpu().numpy() for p in ps)
    args = (st["q"][:nb, :, 0].cpu().numpy(), kc, vc, st["kn"][:nb, :, 0].cpu().numpy(),
            st["vn"][:nb, :, 0].cpu().numpy(), f(st["kp"]), f(st["vp"]), T, D ** -0.5, bits,
            synth.SCALE_MIN, synth.SCALE_MAX)
    c_oracle.decode_attn(*args)                     # warm the threads and page in the sample
    t0 = time.perf_counter()
    want = c_oracle.decode_attn(*args)
    dt = time.perf_counter() - t0
    got = out[:nb].float().cpu().numpy()
    tol = 2e-3 * max(1.0, float(np.abs(want).max()))
    ok = bool(np.allclose(got, want, rtol=2e-3, atol=tol)) and np.array_equal(kc, kc_after) and \
        np.array_equal(vc, vc_after)
    return ok, dt, n_streams, c_oracle.num_threads()


def check_half(w, st, out):
    """fp16-state arithmetic: the first sequence's output and appended codes against the numpy restatement."""
    import numpy as np

    from oracle import adkv_oracle_half as orh
    D, T, bits = w["D"], w["T"], w["bits"]
    kc_after, vc_after = st["kc"][:1].cpu().numpy(), st["vc"][:1].cpu().numpy()
    kc, vc = kc_after.copy(), vc_after.copy()
    f = lambda ps: tuple(p.cpu().numpy() for p in ps)
    want, _ = orh.decode_attn(st["q"][:1, :, 0].cpu().numpy(), kc, vc, st["kn"][:1, :, 0].cpu().numpy(),
                              st["vn"][:1, :, 0].cpu().numpy(), f(st["kp"]), f(st["vp"]), T, D ** -0.5, bits)
    got = out[:1].float().cpu().numpy()
    tol = 2e-2 * max(1.0, float(np.abs(want).max()))    # logits are summed in fp16, as in the reference's kernels
    return bool(np.allclose(got, want, rtol=2e-2, atol=tol)) and np.array_equal(kc, kc_after) and \
        np.array_equal(vc, vc_after)


def time_cuda(fn, torch, device, steps, warmup=3):
    """Average milliseconds per call of ``fn`` (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) / steps


def reference_cuda_module(w):
    """The reference's own CUDA extension (built by oracle/build_ref.py) when it exists and covers the workload:
    4-bit codes, as many query heads as KV heads (src/adkv/hf/llama_adkv.py:235-238)."""
    if w["bits"] != 4 or w["Hq"] != w["Hkv"]:
        return None
    try:
        from oracle import ref_cuda
        return ref_cuda.module()
    except Exception:
        return None


def run_encode(args, w, name):
    """Prefill-quantise workload: a step encodes one layer's K and V (one launch of encode_kernel over both)."""
    import numpy as np
    import torch

    from adkv_b200 import gemv, synth
    from oracle import c_oracle
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == 1, "the prefill workload is a single-GPU measurement"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    B, H, D, T, bits = w["B"], w["Hkv"], w["D"], w["T"], w["bits"]
    kp = synth.gen_params(3, H, D, bits, device=device)
    vp = synth.gen_params(4, H, D, bits, device=device)
    k = torch.cat([synth.gen_kv(10 + b, 1, H, T, D, device=device) for b in range(B)])
    v = torch.cat([synth.gen_kv(110 + b, 1, H, T, D, device=device) for b in range(B)])
    ns = gemv.n_super_for(T + w["appends"], bits)
    kc = torch.zeros((B, H, ns, D // 4, 4, 4), dtype=torch.uint8, device=device)
    vc = torch.zeros_like(kc)
    tk = torch.empty((B, H, 2, D), dtype=torch.float32, device=device)
    tv = torch.empty_like(tk)

    half = args.replay == "half"

    def step(ks=k, vs=v):
        gemv.encode_kv_pair(kc, ks, kp, vc, vs, vp, synth.SCALE_MIN, synth.SCALE_MAX, bits=bits, k_tail=tk, v_tail=tv,
                            half_state=half)

    prop = torch.cuda.get_device_properties(device)
    try:
        bus_id = f"{prop.pci_domain_id:08x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
    except AttributeError:
        bus_id = None
    sampler = ClockSampler(local, bus_id)
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(device)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    t0 = time.perf_counter()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    torch.cuda.synchronize(device)
    t1 = time.perf_counter()
    sampler.stop()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]

    # single-token appends from the persisted tail state (K and V in one launch per appended token)
    kn = synth.gen_kv(5, B, H, w["appends"], D, device=device, pos0=T)
    vn = synth.gen_kv(6, B, H, w["appends"], D, device=device, pos0=T)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for i in range(w["appends"]):
        gemv.append_kv_pair(kc, kn[:, :, i:i + 1], kp, tk, vc, vn[:, :, i:i + 1], vp, tv, T + i,
                            synth.SCALE_MIN, synth.SCALE_MAX, bits=bits, half_state=half)
    a1.record()
    torch.cuda.synchronize(device)
    append_us = a0.elapsed_time(a1) * 1e3 / w["appends"]

    # end to end: fp16 K/V from pinned host memory every step, tail states read back
    hk, hv = k.cpu().pin_memory(), v.cpu().pin_memory()
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    htail = torch.empty_like(tk, device="cpu").pin_memory()
    e2e_steps = max(1, min(args.steps, 5))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(1 + e2e_steps):
        if it == 1:
            e0.record()
        dk.copy_(hk, non_blocking=True)
        dv.copy_(hv, non_blocking=True)
        step(dk, dv)
        htail.copy_(tk, non_blocking=True)
    e1.record()
    torch.cuda.synchronize(device)
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # CPU restatement on a bounded sample of sequences; also checks the GPU's codes for them
    c_oracle.use_all_cores()
    nb = min(B, 4)
    kc_cpu = np.zeros((nb, H, ns, D // 4, 4, 4), np.uint8)
    xk = hk[:nb].numpy()
    f = lambda ps: tuple(p.float().cpu().numpy() for p in ps)
    c_oracle.encode(kc_cpu, xk, f(kp), bits, synth.SCALE_MIN, synth.SCALE_MAX)
    tc0 = time.perf_counter()
    c_oracle.encode(kc_cpu, xk, f(kp), bits, synth.SCALE_MIN, synth.SCALE_MAX)
    cpu_dt = time.perf_counter() - tc0
    step()
    used = gemv.n_super_for(T, bits)
    if half:   # fp16-state arithmetic: the first sequence against its numpy restatement
        from oracle import adkv_oracle_half as orh
        nb_chk = 1
        kc_cpu = np.zeros((nb_chk, H, ns, D // 4, 4, 4), np.uint8)
        orh.encode_kv(kc_cpu, xk[:nb_chk], tuple(p.cpu().numpy() for p in kp), bits)
    else:
        nb_chk = nb
    ok = np.array_equal(kc[:nb_chk, :, :used].cpu().numpy(), kc_cpu[:, :, :used])

    nbytes = algorithmic_bytes(w)
    ref_cuda_leg = None
    ref = None if args.no_cpu else reference_cuda_module(w)     # a baseline leg, like the CPU one
    if ref is not None:
        # the reference's encode kernel (fp16 state), one call per tensor as its caller makes them
        rk, rv = torch.zeros_like(kc), torch.zeros_like(vc)

        def ref_step():
            ref.encode_kv(rk, k, *kp, synth.SCALE_MIN, synth.SCALE_MAX)
            ref.encode_kv(rv, v, *vp, synth.SCALE_MIN, synth.SCALE_MAX)
        ms = time_cuda(ref_step, torch, device, max(1, min(args.steps, 10)), warmup=2)
        ref_cuda_leg = {"ms_per_step": ms, "value": nbytes / (ms * 1e-3) / 1e9, "unit": UNIT,
                        "what": "the reference's encode_kv CUDA kernel (fp16 state) recompiled for sm_100a, K then V, "
                                "same tensors resident in HBM"}
        del rk, rv
    peak, peak_src = measured_peak_gbs()
    avg_ms = sum(per_step) / len(per_step)
    res = {
        "metric": "adkv_prefill_quantize_bandwidth", "value": nbytes * args.steps / (total_ms * 1e-3) / 1e9, "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload=name, per_gpu=w, replay=args.replay, l2="inputs larger than L2; no flush needed"),
        "e2e": {"value": nbytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": 2 * k.numel() * 2,
                "d2h_bytes_per_step": htail.numel() * 4, "ms_per_step": e2e_ms},
        "gpu_launches": args.steps,
        "append_us_per_token_kv": append_us,
        "roofline": {"bound": "hbm", "achieved": nbytes / (avg_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": nbytes / (avg_ms * 1e-3) / 1e9 / peak, "peak_source": peak_src,
                     "traffic": NCU_TRAFFIC_BYTES.get(name), "kernel": "encode_kernel (K and V in one launch per step)",
                     "algorithmic_bytes_per_step": nbytes, "avg_step_ms": avg_ms},
        "clocks": sampler.summary(t0, t1),
        "cpu_baseline": {"value": nb * H * T * D * (2 + bits / 8) / cpu_dt / 1e9, "unit": UNIT,
                         "cores": c_oracle.num_threads(), "kind": "port", "seconds": cpu_dt,
                         "sample": f"K of {nb} of {B} sequences ({nb * H} streams), C restatement with OpenMP"},
        "parity_check": "ok" if ok else "FAILED",
    }
    if ref_cuda_leg:
        res["reference_cuda"] = ref_cuda_leg
    print(json.dumps(res), flush=True)
    if not ok:
        sys.exit(1)


def decode_ms(w, mode, torch, device, steps, seed=2000, ckpt_interval=0):
    """Milliseconds per fused decode step of workload ``w`` on one GPU in replay mode ``mode`` (fresh state)."""
    from adkv_b200 import gemv, synth
    st = build_gpu_state(w, seed=seed, device=device, torch=torch, ckpt_interval=ckpt_interval)
    out = torch.empty((w["B"], w["Hq"], w["D"]), dtype=torch.float16, device=device)
    kw = dict(k_tail=st["tk"], v_tail=st["tv"], tail_keep=True) if mode == "tail" else dict(fast=mode == "fast")
    ms = time_cuda(lambda: gemv.decode_attn(st["q"], st["kc"], st["vc"], st["kn"], st["vn"], st["kp"], st["vp"], w["T"],
                                            w["D"] ** -0.5, synth.SCALE_MIN, synth.SCALE_MAX, bits=w["bits"], out=out,
                                            **kw, **st["ck"]), torch, device, steps)
    assert gemv.device_status(device) == 0, "a kernel gave up on a bounded wait"
    return ms


def encode_ms(w, torch, device, steps):
    """Milliseconds per prefill-quantise step (K and V of one layer, one launch) and microseconds per appended
    K+V token from the tail state, for an encode workload on one GPU."""
    from adkv_b200 import gemv, synth
    B, H, D, T, bits, A = w["B"], w["Hkv"], w["D"], w["T"], w["bits"], min(w["appends"], 32)
    kp, vp = synth.gen_params(3, H, D, bits, device=device), synth.gen_params(4, H, D, bits, device=device)
    k = torch.cat([synth.gen_kv(10 + b, 1, H, T, D, device=device) for b in range(B)])
    v = torch.cat([synth.gen_kv(110 + b, 1, H, T, D, device=device) for b in range(B)])
    ns = gemv.n_super_for(T + A, bits)
    kc = torch.zeros((B, H, ns, D // 4, 4, 4), dtype=torch.uint8, device=device)
    vc = torch.zeros_like(kc)
    tk = torch.empty((B, H, 2, D), dtype=torch.float32, device=device)
    tv = torch.empty_like(tk)
    ms = time_cuda(lambda: gemv.encode_kv_pair(kc, k, kp, vc, v, vp, synth.SCALE_MIN, synth.SCALE_MAX, bits=bits,
                                               k_tail=tk, v_tail=tv), torch, device, steps)
    kn = synth.gen_kv(5, B, H, A, D, device=device, pos0=T)
    vn = synth.gen_kv(6, B, H, A, D, device=device, pos0=T)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for i in range(A):
        gemv.append_kv_pair(kc, kn[:, :, i:i + 1], kp, tk, vc, vn[:, :, i:i + 1], vp, tv, T + i, synth.SCALE_MIN,
                            synth.SCALE_MAX, bits=bits)
    a1.record()
    torch.cuda.synchronize(device)
    append_us = a0.elapsed_time(a1) * 1e3 / A
    # the layered calls: K and V of 8 layers per launch (the same input tensors stand for every layer; each layer
    # has its own caches and tails, so the bytes written and the chains run are those of 8 layers)
    NL = 8
    caches = [(torch.zeros_like(kc), torch.empty_like(tk), torch.zeros_like(vc), torch.empty_like(tv)) for _ in range(NL)]
    ls = gemv.LayerSet([(c[0], kp, c[1], c[2], vp, c[3]) for c in caches], bits=bits)
    ms_layers = time_cuda(lambda: gemv.encode_kv_layers(ls, [k] * NL, [v] * NL, synth.SCALE_MIN, synth.SCALE_MAX),
                          torch, device, max(2, steps // 2), warmup=2) / NL
    kn_l = [kn[:, :, 0:1].contiguous()] * NL
    vn_l = [vn[:, :, 0:1].contiguous()] * NL
    a0.record()
    for i in range(A):
        gemv.append_kv_layers(ls, kn_l, vn_l, T + i, synth.SCALE_MIN, synth.SCALE_MAX)
    a1.record()
    torch.cuda.synchronize(device)
    return ms, append_us, ms_layers, a0.elapsed_time(a1) * 1e3 / A / NL


def other_workload_figures(torch, device, peak):
    """One-GPU figures of the benchmark shapes that are not the headline (a few steps each)."""
    res = {}
    for name in ("config3_prefill_b16_t8192_4bit", "config3_prefill_b16_t8192_2bit"):
        w = WORKLOADS[name]
        ms, app_us, ms_l, app_us_l = encode_ms(w, torch, device, 5)
        gbs, gbs_l = algorithmic_bytes(w) / (ms * 1e-3) / 1e9, algorithmic_bytes(w) / (ms_l * 1e-3) / 1e9
        res[name] = {"ms_per_layer_kv": ms, "value": gbs, "unit": UNIT, "frac_of_measured_peak": gbs / peak,
                     "append_us_per_token_kv": app_us, "layers_in_the_configuration": 32,
                     "eight_layers_per_launch": {"ms_per_layer_kv": ms_l, "value": gbs_l, "unit": UNIT,
                                                 "frac_of_measured_peak": gbs_l / peak,
                                                 "append_us_per_layer_token_kv": app_us_l}}
        torch.cuda.empty_cache()
    name = "config5_llama3_8b_gqa_b32_t32768_2bit"
    w = WORKLOADS[name]
    leg = {}
    for label, mode, iv in (("tail", "tail", 0), ("exact", "exact", 0), ("tail_ckpt2048", "tail", 2048)):
        ms = decode_ms(w, mode, torch, device, 10, ckpt_interval=iv)
        gbs = algorithmic_bytes(w) / (ms * 1e-3) / 1e9
        leg[label] = {"ms_per_step": ms, "value": gbs, "unit": UNIT, "frac_of_measured_peak": gbs / peak}
        torch.cuda.empty_cache()
    res[name] = leg
    return res


def run_ours(args, w, name):
    import torch
    import torch.distributed as dist

    from adkv_b200 import gemv, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    w_global = dict(w)
    w = rank_workload(w_global, world, rank, args.scaling)
    half = args.replay == "half"
    st = build_gpu_state(w, seed=1000 + 7919 * rank, device=device, torch=torch, ckpt_interval=args.ckpt_interval,
                         half_state=half)
    ck = st["ck"]
    B, Hq, Hkv, D, T, bits = w["B"], w["Hq"], w["Hkv"], w["D"], w["T"], w["bits"]
    scaling = D ** -0.5
    out = torch.empty((B, Hq, D), dtype=torch.float16, device=device)

    def mode_kwargs(mode):
        """Keyword arguments of gemv.decode_attn for a replay mode.  "tail": the new token is quantised from the
        persisted tail state (bit-exact codes) and the cache is replayed in the contracted arithmetic; the tails
        are kept as they are so that every timed step is the same step (token T appended at slot T)."""
        if mode == "tail":
            return dict(k_tail=st["tk"], v_tail=st["tv"], tail_keep=True)
        return dict(fast=mode == "fast", half_state=mode == "half")

    headline = mode_kwargs(args.replay)

    def step():
        gemv.decode_attn(st["q"], st["kc"], st["vc"], st["kn"], st["vn"], st["kp"], st["vp"], T, scaling,
                         synth.SCALE_MIN, synth.SCALE_MAX, bits=bits, out=out, **headline, **ck)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident timing
    prop = torch.cuda.get_device_properties(device)
    try:
        bus_id = f"{prop.pci_domain_id:08x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
    except AttributeError:
        bus_id = None
    sampler = ClockSampler(local, bus_id)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    t_wall0 = time.perf_counter()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    t_wall1 = time.perf_counter()
    sampler.stop()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    assert gemv.device_status(device) == 0, "a kernel gave up on a bounded wait"

    # ---- end to end through the public API: host inputs in, host output back, every step
    # the step's q, k_new and v_new sit back to back in one pinned staging buffer and travel in one copy
    srcs = (st["q"], st["kn"], st["vn"])
    n_in = sum(t.numel() for t in srcs)
    h_in = torch.empty(n_in, dtype=torch.float16).pin_memory()
    d_in = torch.empty(n_in, dtype=torch.float16, device=device)
    views, off = [], 0
    for t in srcs:
        h_in[off:off + t.numel()].copy_(t.reshape(-1))
        views.append(d_in[off:off + t.numel()].view(t.shape))
        off += t.numel()
    dq, dk_, dv_ = views
    hq, hk, hv = srcs                       # sizes for the byte count below
    hout = torch.empty((B, Hq, D), dtype=torch.float16).pin_memory()

    def e2e_step():
        d_in.copy_(h_in, non_blocking=True)
        gemv.decode_attn(dq, st["kc"], st["vc"], dk_, dv_, st["kp"], st["vp"], T, scaling,
                         synth.SCALE_MIN, synth.SCALE_MAX, bits=bits, out=out, **headline, **ck)
        hout.copy_(out, non_blocking=True)

    for _ in range(max(3, min(args.warmup, 5))):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    # the other replay arithmetics, same workload and caches, for the record (not the headline)
    others = []
    other_steps = max(1, min(args.steps, 50))
    for mode in ("tail", "exact", "fast", "half"):
        if mode == args.replay or ((mode == "half") != half and args.ckpt_interval) or (mode == "tail" and half):
            continue     # checkpoints and tails hold the states of the arithmetic the caches were written with
        ms = time_cuda(lambda: gemv.decode_attn(st["q"], st["kc"], st["vc"], st["kn"], st["vn"], st["kp"], st["vp"], T,
                                                scaling, synth.SCALE_MIN, synth.SCALE_MAX, bits=bits, out=out,
                                                **mode_kwargs(mode), **ck),
                       torch, device, other_steps)
        others.append([mode, ms])
    # the three-call sequence of the reference's caller (src/adkv/hf/llama_adkv.py:263-276): unscaled logits,
    # torch softmax in fp32, weighted sum -- through this library's kernels and, where it has been built and
    # covers the workload, through the reference's own CUDA kernels recompiled for sm_100a
    trio_legs = {}
    if world == 1 and not args.ckpt_interval:
        def trio(qk, ov, **kw):
            def fn():
                logits = qk(st["q"], kc2, st["kn"], *st["kp"], T, synth.SCALE_MIN, synth.SCALE_MAX, **kw)
                attn = torch.softmax(logits.float() * scaling, dim=-1).to(torch.float16)
                return ov(attn, vc2, st["vn"], *st["vp"], synth.SCALE_MIN, synth.SCALE_MAX, **kw)
            return fn
        kc2, vc2 = st["kc"].clone(), st["vc"].clone()
        n_trio = max(1, min(args.steps, 20))
        ms = time_cuda(trio(gemv.forward_qk, gemv.forward_ov, bits=bits, fast=args.replay == "fast", half_state=half),
                       torch, device, n_trio)
        trio_legs["unfused_trio"] = {"ms_per_step": ms, "value": algorithmic_bytes(w) / (ms * 1e-3) / 1e9, "unit": UNIT,
                                     "what": "forward_qk + torch softmax + forward_ov of this library"}
        ref = None if args.no_cpu else reference_cuda_module(w)     # a baseline leg, like the CPU one
        if ref is not None:
            ms = time_cuda(trio(ref.forward_qk, ref.forward_ov), torch, device, n_trio)
            trio_legs["reference_cuda"] = {
                "ms_per_step": ms, "value": algorithmic_bytes(w) / (ms * 1e-3) / 1e9, "unit": UNIT,
                "what": "the reference's forward_qk + torch softmax + forward_ov, its CUDA kernels (fp16 state and "
                        "accumulation) recompiled for sm_100a, same caches resident in HBM"}
        del kc2, vc2
    step()                      # leave the caches and `out` as the headline arithmetic writes them
    torch.cuda.synchronize(device)

    # the weak-scaling figure next to the strong one: every rank takes the whole workload
    weak_ms = None
    if world > 1 and args.scaling == "strong" and not args.no_weak:
        weak_ms = decode_ms(w_global, args.replay if args.replay in ("tail", "exact", "fast") else "tail", torch, device,
                            max(1, min(args.steps, 30)), seed=3000 + 7919 * rank, ckpt_interval=args.ckpt_interval)

    # and the same strong-scaling shard with state checkpoints (opt-in cache metadata that splits the token axis into
    # independent segments): what a cache owner who knows that a GPU holds few streams would allocate
    ckpt_ms = None
    if world > 1 and args.scaling == "strong" and not args.no_weak and not args.ckpt_interval and args.replay == "tail":
        ckpt_ms = decode_ms(w, "tail", torch, device, max(1, min(args.steps, 50)), seed=1000 + 7919 * rank,
                            ckpt_interval=STRONG_CKPT_INTERVAL)

    bytes_rank = algorithmic_bytes(w)
    bytes_job = bytes_rank
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms, weak_ms or 0.0, ckpt_ms or 0.0] + [ms for _, ms in others],
                         dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms, weak_ms, ckpt_ms = t.tolist()[:4]
        others = [[m, v] for (m, _), v in zip(others, t.tolist()[4:])]
        nb = torch.tensor([bytes_rank, B], dtype=torch.float64, device=device)
        dist.all_reduce(nb, op=dist.ReduceOp.SUM)
        bytes_job, seqs_job = nb.tolist()
    else:
        seqs_job = B
    if args.scaling == "strong":
        seqs_job = w_global["B"]            # kv-head shards of one sequence are not separate sequences

    res = None
    if rank == 0:
        value = bytes_job * args.steps / (total_ms * 1e-3) / 1e9
        e2e_val = bytes_job * args.steps / (e2e_ms * 1e-3) / 1e9
        peak, peak_src = measured_peak_gbs()
        avg_launch_ms = sum(per_launch_ms) / len(per_launch_ms)
        achieved = bytes_rank / (avg_launch_ms * 1e-3) / 1e9
        res = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(name, w, w_global, world, args),
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": world * (hq.numel() + hk.numel() + hv.numel()) * 2,
                    "d2h_bytes_per_step": world * hout.numel() * 2, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps * (2 if args.ckpt_interval else 1),
            "decode_tokens_per_s": {"one_layer": seqs_job * args.steps / (total_ms * 1e-3),
                                    "over_32_layers": seqs_job * args.steps / (total_ms * 1e-3) / 32},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "frac_of_8TBps_nominal": achieved / 8000.0,
                         "traffic": NCU_TRAFFIC_BYTES.get(name) if world == 1 else None, "kernel": "decode_attn_kernel",
                         "algorithmic_bytes_per_launch": bytes_rank, "avg_launch_ms": avg_launch_ms,
                         "median_launch_ms": statistics.median(per_launch_ms)},
            "clocks": sampler.summary(t_wall0, t_wall1),
            "other_replay": [{"replay": m, "ms_per_step": ms, "value": bytes_job / (ms * 1e-3) / 1e9,
                              "unit": UNIT} for m, ms in others],
        }
        if weak_ms:
            wb = algorithmic_bytes(w_global) * world
            res["weak_scaling"] = {"ms_per_step": weak_ms, "value": wb / (weak_ms * 1e-3) / 1e9, "unit": UNIT,
                                   "global_batch": w_global["B"] * world,
                                   "what": "every rank runs the whole workload (per-GPU work fixed)"}
        if ckpt_ms:
            res["strong_with_checkpoints"] = {
                "ms_per_step": ckpt_ms, "value": bytes_job / (ckpt_ms * 1e-3) / 1e9, "unit": UNIT,
                "ckpt_interval": STRONG_CKPT_INTERVAL,
                "what": "the same shards with state checkpoints every %d tokens (adkv_decode_attn_ckpt: segments of a "
                        "stream run on separate warp pairs, one more launch merges them)" % STRONG_CKPT_INTERVAL}
        res.update(trio_legs)
        if world == 1 and not args.no_cpu and half:
            res["parity_check"] = "ok" if check_half(w, st, out) else "FAILED"
        elif world == 1 and not args.no_cpu:
            n = pick_sample_streams(w, target_s=args.cpu_seconds)
            ok, dt, n_used, cores = check_against_oracle(w, st, out, n, torch)
            port = {"value": sample_bytes(w, n_used) / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
                    "seconds": dt, "sample": f"{n_used} of {B * Hkv} (batch, kv-head) streams of the workload, "
                                             "one decode step, C restatement with OpenMP"}
            res["parity_check"] = "ok" if ok else "FAILED"
            from oracle import ref_torch
            if ref_torch.available():
                # the reference's own torch path on the host cores: one sequence of the workload, best of 2
                use_all_host_threads(torch)
                smp = torch_reference_sample(w, *pick_torch_sample(w, 6.0))
                secs, want = timed_cpu(lambda: torch_reference_step(smp), repeats=2)
                res["cpu_baseline"] = {"value": torch_sample_bytes(w, smp) / secs / 1e9, "unit": UNIT,
                                       "cores": torch.get_num_threads(), "kind": "reference", "seconds": secs,
                                       "sample": describe_torch_sample(w, smp), "host_cpus": os.cpu_count(),
                                       "config1_seconds": config1_seconds()}
                res["cpu_baseline_port"] = port
            else:
                res["cpu_baseline"] = port
        if world == 1 and name == DEFAULT_WORKLOAD and not args.no_extra and not args.ckpt_interval:
            del st
            torch.cuda.empty_cache()
            res["other_workloads"] = other_workload_figures(torch, device, peak)
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if res is not None and res.get("parity_check") == "FAILED":
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong",
                    help="strong (default): the workload is fixed and its streams are sharded over the GPUs; "
                         "weak: every GPU runs the whole workload")
    ap.add_argument("--no-weak", action="store_true", help="N > 1, strong scaling: skip the extra weak-scaling figure")
    ap.add_argument("--no-extra", action="store_true", help="skip the figures of the other benchmark shapes")
    ap.add_argument("--replay", choices=["tail", "exact", "fast", "half"], default="tail",
                    help="tail: the fp32 recurrence with a persisted tail state (appended codes bit-exact, contracted "
                         "replay); exact / fast: without tail state, replay in canonical order / contracted; half: the "
                         "fp16-state arithmetic of the reference's CUDA kernels (ADKV_FLAG_HALF_STATE)")
    ap.add_argument("--ckpt-interval", type=int, default=0,
                    help="decode with state checkpoints every N tokens (segment-parallel kernel + merge)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu", action="store_true",
                    help="skip the baseline legs, i.e. everything that executes oracle/: the CPU restatement "
                         "(cpu_baseline, parity_check) and the reference's CUDA kernels (reference_cuda)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]

    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # not launched by torch.distributed.run: do it ourselves, one process per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))

    if args.impl == "reference":
        run_reference(args, w, args.workload)
    elif w.get("kind") == "encode":
        run_encode(args, w, args.workload)
    else:
        run_ours(args, w, args.workload)


if __name__ == "__main__":
    main()
