#!/usr/bin/env python
"""Benchmark of the GGUF quantized-matmul hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  N = 1: the decode GEMV configuration the headline metric is quoted on (Q4_K weight
[11008 x 4096], bf16 activations, M = 1).  A "step" is one pass over R distinct copies of the weight (R chosen so the
copies exceed twice the L2, every launch reads cold weights), replayed as a CUDA graph; `value` is weight GB/s over
exactly K steps timed with CUDA events.  The same line carries the roofline of the GEMV, the prefill GEMM's TFLOP/s
and roofline (Q6_K [4096 x 14336], M = 512), the other configured shapes, the end-to-end number through the artifact /
session API with host buffers, and the reference's CPU kernel timed on this box's host cores.
N > 1 (launched under torchrun, one rank per GPU): the Llama-70B-shaped FFN sharded over N GPUs - gate/up split along N
with an NCCL all-gather, down split along K with an NCCL all-reduce - strong scaling, `value` = total weight bytes of
the three matrices / max-over-ranks step time.
`--impl reference` times the reference's own CPU implementation of the path (its generated gemm_rcr kernel over the
host-dequantized weight) on the host cores instead; rank 0 only."""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG2 = {"qtype": "Q4_K", "n": 11008, "k": 4096}
CFG3 = {"qtype": "Q6_K", "n": 4096, "k": 14336}
NOMINAL_HBM_GBS = 8000.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._thread = index, [], threading.Event(), None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.rows[0][1]) if self.rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(self.rows)}


# ----------------------------------------------------------------------------------------------- GPU helpers
def graph_of(fn, stream):
    import torch
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    return g


def time_steps(step, steps, warmup, stream, barrier=None):
    """W untimed steps, then exactly K steps between two CUDA events on `stream`; returns milliseconds for the K steps."""
    import torch
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            step()
        stream.synchronize()
        if barrier:
            barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        e1.synchronize()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def rotation_copies(nbytes, l2_bytes, cap=24):
    return int(max(2, min(cap, math.ceil(2.0 * l2_bytes / nbytes) + 1)))


def bench_gemm(qtype, n, k, m, steps, warmup, l2, variant="auto", copies=None):
    """Graph-replayed pass over R weight copies; returns per-launch microseconds and the launch count."""
    import torch

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    dev = torch.device("cuda")
    nbytes = encoded_nbytes(qtype, n, k)
    r = copies or rotation_copies(nbytes, l2)
    ws = [synthetic.random_blocks_torch(qtype, n, k, 1000 + i, dev) for i in range(r)]
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    outs = [torch.empty(m, n, device=dev, dtype=torch.bfloat16) for _ in range(r)]

    def one_pass():
        for i in range(r):
            kernels.gemm_rcr(x, ws[i], qtype, variant=variant, out=outs[i])

    stream = torch.cuda.Stream()
    g = graph_of(one_pass, stream)
    ms = time_steps(g.replay, steps, warmup, stream)
    assert kernels.device_status() == 0, "a bounded device-side wait gave up during the benchmark"
    return {"us_per_launch": ms * 1e3 / (steps * r), "launches": steps * r, "copies": r, "weight_bytes": nbytes,
            "variant": kernels.select_variant(qtype, "bfloat16", m, n, k) if variant == "auto" else variant}


def bench_dual(n, k, m, steps, warmup, l2, qtype="Q4_K"):
    """silu(x Wgate^T) * (x Wup^T) in one launch on the row-interleaved pair, next to the two plain launches it replaces."""
    import torch

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    dev = torch.device("cuda")
    nbytes = 2 * encoded_nbytes(qtype, n, k)
    r = rotation_copies(nbytes, l2, cap=6)
    gates = [synthetic.random_blocks_torch(qtype, n, k, 6000 + 2 * i, dev) for i in range(r)]
    ups = [synthetic.random_blocks_torch(qtype, n, k, 6001 + 2 * i, dev) for i in range(r)]
    fused = [kernels.interleave_rows8(g, u) for g, u in zip(gates, ups)]
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    outs = [torch.empty(m, n, device=dev, dtype=torch.bfloat16) for _ in range(2 * r)]

    def one_launch():
        for i in range(r):
            kernels.dual_gemm_rcr(x, fused[i], qtype, "silu", out=outs[i])

    def two_launches():
        for i in range(r):
            kernels.gemm_rcr(x, gates[i], qtype, out=outs[i])
            kernels.gemm_rcr(x, ups[i], qtype, out=outs[r + i])

    stream = torch.cuda.Stream()
    res = {}
    for name, fn in (("dual", one_launch), ("two_gemm_rcr", two_launches)):
        g = graph_of(fn, stream)
        res[name + "_us"] = time_steps(g.replay, steps, warmup, stream) * 1e3 / (steps * r)
    res["weight_gbs"] = nbytes / res["dual_us"] / 1e3
    return res


def bench_dequant(qtype, n, k, dtype, steps, warmup):
    import torch

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    dev = torch.device("cuda")
    r = 3
    ws = [synthetic.random_blocks_torch(qtype, n, k, 2000 + i, dev) for i in range(r)]
    outs = [torch.empty(n, k, device=dev, dtype=getattr(torch, dtype)) for _ in range(r)]

    def one_pass():
        for i in range(r):
            kernels.dequantize_rows(ws[i], qtype, k, dtype, out=outs[i])

    stream = torch.cuda.Stream()
    g = graph_of(one_pass, stream)
    ms = time_steps(g.replay, steps, warmup, stream)
    us = ms * 1e3 / (steps * r)
    total = encoded_nbytes(qtype, n, k) + n * k * outs[0].element_size()
    return {"us_per_launch": us, "gbs": total / us / 1e3, "bytes": total}


LLAMA8B_LAYER = [("q", "Q4_K", 4096, 4096), ("k", "Q4_K", 1024, 4096), ("v", "Q6_K", 1024, 4096), ("o", "Q4_K", 4096, 4096),
                 ("gate", "Q4_K", 14336, 4096), ("up", "Q4_K", 14336, 4096), ("down", "Q6_K", 4096, 14336)]


def bench_decode_step(steps, warmup):
    """Llama-3-8B-shaped decode step, quantized linears only, batch 1: 32 layers x 7 linears + lm_head = 225 launches
    captured in one CUDA graph (weights total 4.88 GB, far beyond L2)."""
    import torch

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    dev = torch.device("cuda")
    layers, total = [], 0
    for layer in range(32):
        for j, (name, qtype, n, k) in enumerate(LLAMA8B_LAYER):
            layers.append((qtype, synthetic.random_blocks_torch(qtype, n, k, 3000 + layer * 8 + j, dev), n, k))
            total += encoded_nbytes(qtype, n, k)
    layers.append(("Q6_K", synthetic.random_blocks_torch("Q6_K", 128256, 4096, 3999, dev), 128256, 4096))
    total += encoded_nbytes("Q6_K", 128256, 4096)
    xs = {k: torch.randn(1, k, device=dev).to(torch.bfloat16) for k in (4096, 14336)}
    outs = [torch.empty(1, n, device=dev, dtype=torch.bfloat16) for (_, _, n, _) in layers]

    def one_step():
        for (qtype, w, n, k), out in zip(layers, outs):
            kernels.gemm_rcr(xs[k], w, qtype, out=out)

    stream = torch.cuda.Stream()
    g = graph_of(one_step, stream)
    ms = time_steps(g.replay, steps, warmup, stream) / steps
    return {"ms_per_step": ms, "weight_bytes": total, "gbs": total / ms / 1e6, "launches_per_step": len(layers)}


# ----------------------------------------------------------------------------------------------- end to end
def bench_e2e(steps, warmup, copies, tmp_dir):
    """The headline metric through the public artifact / session API with HOST buffers: per step, R activations go
    pinned-host -> device, R quantized linears run, R outputs come back to the host; all inside the timed region."""
    import dinoml_v2_b200 as dml
    from dinoml_v2_b200 import synthetic
    from dinoml_v2_b200.constant_sources import GGUFConstant
    n, k, qtype = CFG2["n"], CFG2["k"], CFG2["qtype"]

    class Bank(dml.Module):
        def __init__(self):
            for i in range(copies):
                setattr(self, f"w{i}", dml.Parameter([n, k], dtype="bfloat16"))

        def forward(self, **xs):
            return [dml.ops.gemm_rcr(xs[f"x{i}"], getattr(self, f"w{i}")) for i in range(copies)]

    blocks = [synthetic.random_blocks(qtype, n, k, 4000 + i) for i in range(copies)]
    spec = dml.trace(Bank(), inputs={f"x{i}": dml.TensorSpec([1, k], "bfloat16") for i in range(copies)},
                     constants={f"w{i}": GGUFConstant.from_blocks(blocks[i], qtype, (n, k), tensor=f"w{i}") for i in range(copies)})
    art = dml.compile(spec, dml.Target("cuda"), tmp_dir)
    mod = dml.runtime.load(art.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    inputs = {f"x{i}": synthetic.random_activations(1, k, 5000 + i, "bfloat16") for i in range(copies)}
    for _ in range(warmup):
        out = sess.run_numpy(inputs)
    import torch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = sess.run_numpy(inputs)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    assert all(np.isfinite(v).all() for v in out.values())
    mod.close()
    wbytes = copies * blocks[0].nbytes
    return {"value": wbytes / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": copies * k * 2, "d2h_bytes_per_step": copies * n * 2,
            "ms_per_step": dt * 1e3, "api": "dml.compile -> runtime.load -> Session.run_numpy", "linears_per_step": copies}


# ----------------------------------------------------------------------------------------------- CPU reference arm
def _ref_library():
    """The reference's CPU gemm kernel built into oracle/_ref (kind "reference"), else None."""
    ref = ROOT / "oracle" / "_ref"
    info = ref / "BUILD_INFO.json"
    if not info.exists():
        return None
    flags = set()
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                flags = set(line.split(":", 1)[1].split())
                break
    except OSError:
        pass
    built = set(json.loads(info.read_text()).get("build_host_cpu_flags", []))
    tag = "native" if built and built <= flags else "v3"
    path = ref / f"libref_gemm_cpu_{tag}.so"
    return (ctypes.CDLL(str(path)), tag) if path.exists() else None


def cpu_reference_timing(budget_s, min_iters=3):
    """Times the reference CPU path on the headline configuration (M = 1, bf16, dense weights = host-dequantized GGUF
    blocks rounded to bf16, as GGUFConstant.materialize produces on the CPU target).  Bounded: runs until `budget_s`."""
    import oracle
    from dinoml_v2_b200 import synthetic
    n, k, qtype = CFG2["n"], CFG2["k"], CFG2["qtype"]
    blocks = synthetic.random_blocks(qtype, n, k, 1000)
    wb = oracle.dequantize(blocks, qtype, k, "bfloat16")
    x = synthetic.random_activations(1, k, 7, "bfloat16")
    y = np.empty((1, n), dtype=np.uint16)
    lib = _ref_library()
    if lib is not None:
        fn = lib[0].ref_gemm_rcr_bfloat16
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 3
        call = lambda: fn(x.ctypes.data, wb.ctypes.data, y.ctypes.data, 1, n, k)
        kind, detail = "reference", f"gemm_cpu.cpp.j2 kernel built -O3 -ffast-math -fopenmp ({lib[1]})"
    else:
        call = lambda: oracle.gemm_rcr_dense(x, wb, "bfloat16")
        kind, detail = "port", "C restatement of gemm_cpu.cpp.j2 (strict k order)"
    call()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_iters or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        call()
        times.append(time.perf_counter() - t0)
    med = sorted(times)[len(times) // 2]
    # the reference's OpenMP loop runs over the M activation rows (gemm_cpu.cpp.j2:35-38): one row => one core
    return {"value": blocks.nbytes / med / 1e9, "unit": "GB/s", "cores": 1, "kind": kind, "ms_per_call": med * 1e3,
            "sample": f"{len(times)} calls of one {qtype} [{n}x{k}] M=1 bf16 gemm_rcr over host-dequantized dense weights "
                      f"({detail}); weight bytes counted GGUF-encoded; host has {os.cpu_count()} logical cores, the kernel's "
                      "OpenMP loop is over M rows so M=1 uses one"}, times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, times = cpu_reference_timing(budget_s=0.0, min_iters=args.warmup + args.steps)
    timed = times[args.warmup:args.warmup + args.steps]
    total = sum(timed)
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    nbytes = encoded_nbytes(CFG2["qtype"], CFG2["n"], CFG2["k"])
    value = nbytes * len(timed) / total / 1e9
    base["value"] = value
    print(json.dumps({
        "impl": "reference", "metric": "GGUF qmatmul weight GB/s at M=1 (Q4_K 11008x4096)", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / len(timed) * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "cfg2 Q4_K [11008x4096] GEMV, M=1, bf16 - reference CPU path (host dequantize once, dense "
                               "gemm_rcr per step); each step is ONE matmul (bounded sample of the R-copy GPU step)"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ----------------------------------------------------------------------------------------------- single GPU
def run_single(args):
    import torch

    from dinoml_v2_b200 import _native
    _native.lib()                                     # fail loudly if the sm_100a library is missing
    torch.cuda.set_device(0)
    props = torch.cuda.get_device_properties(0)
    l2 = props.L2_cache_size
    peaks, peak_kind = measured_peaks()
    K, W = args.steps, args.warmup

    # ---- headline: cfg2 M=1, timed exactly K steps with clocks sampled
    import tempfile

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    dev = torch.device("cuda")
    qtype, n, k = CFG2["qtype"], CFG2["n"], CFG2["k"]
    nbytes = encoded_nbytes(qtype, n, k)
    r = rotation_copies(nbytes, l2)
    ws = [synthetic.random_blocks_torch(qtype, n, k, 1000 + i, dev) for i in range(r)]
    x = torch.randn(1, k, device=dev).to(torch.bfloat16)
    outs = [torch.empty(1, n, device=dev, dtype=torch.bfloat16) for _ in range(r)]

    def one_pass():
        for i in range(r):
            kernels.gemm_rcr(x, ws[i], qtype, out=outs[i])

    stream = torch.cuda.Stream()
    g = graph_of(one_pass, stream)
    with ClockSampler(0) as clocks:
        ms_total = time_steps(g.replay, K, W, stream)
    ms_step = ms_total / K
    us_launch = ms_step * 1e3 / r
    value = r * nbytes / ms_step / 1e6
    del ws, outs

    extra_steps, extra_warm = max(3, min(K, 10)), 3
    extras = {}
    for m in (4, 16):
        b = bench_gemm(qtype, n, k, m, extra_steps, extra_warm, l2)
        extras[f"cfg2_q4k_m{m}"] = {"us_per_launch": b["us_per_launch"], "weight_gbs": nbytes / b["us_per_launch"] / 1e3,
                                    "tflops": 2.0 * m * n * k / b["us_per_launch"] / 1e6, "variant": b["variant"]}
    for m in (1, 16):
        b = bench_gemm(CFG3["qtype"], CFG3["n"], CFG3["k"], m, extra_steps, extra_warm, l2, copies=4)
        extras[f"cfg3_q6k_m{m}"] = {"us_per_launch": b["us_per_launch"], "weight_gbs": b["weight_bytes"] / b["us_per_launch"] / 1e3,
                                    "variant": b["variant"]}
    prefill = {}
    for m in (64, 512, 2048):
        b = bench_gemm(CFG3["qtype"], CFG3["n"], CFG3["k"], m, extra_steps, extra_warm, l2, copies=3)
        tf = 2.0 * m * CFG3["n"] * CFG3["k"] / b["us_per_launch"] / 1e6
        prefill[f"m{m}"] = {"us_per_launch": b["us_per_launch"], "tflops": tf, "variant": b["variant"],
                            "frac_of_measured_burst": tf / peaks["bf16_tflops"],
                            "frac_of_measured_sustained": tf / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]),
                            "frac_of_nominal_2250": tf / 2250.0}
    extras["cfg3_q6k_prefill"] = prefill
    extras["cfg1_q8_0_m1_gpu"] = (lambda b: {"us_per_launch": b["us_per_launch"], "weight_gbs": b["weight_bytes"] / b["us_per_launch"] / 1e3,
                                             "variant": b["variant"]})(bench_gemm("Q8_0", 4096, 4096, 1, extra_steps, extra_warm, l2))
    extras["cfg1_q8_0_prefill"] = {}
    for (nn, kk, m) in ((4096, 4096, 512), (4096, 14336, 512)):
        b = bench_gemm("Q8_0", nn, kk, m, extra_steps, extra_warm, l2, copies=3)
        extras["cfg1_q8_0_prefill"][f"{nn}x{kk}_m{m}"] = {"us_per_launch": b["us_per_launch"], "variant": b["variant"],
                                                          "tflops": 2.0 * m * nn * kk / b["us_per_launch"] / 1e6}
    extras["dequant"] = {f"{q}_{dt}": bench_dequant(q, nn, kk, dt, extra_steps, extra_warm)
                         for (q, nn, kk) in (("Q4_K", 11008, 4096), ("Q6_K", 4096, 14336), ("Q8_0", 4096, 4096)) for dt in ("float16", "float32")}
    extras["dual_gate_up_q4k_14336x4096"] = {f"m{m}": bench_dual(14336, 4096, m, extra_steps, extra_warm, l2) for m in (1, 16)}
    try:
        extras["cfg4_llama8b_decode_step"] = bench_decode_step(extra_steps, extra_warm)
    except torch.cuda.OutOfMemoryError as exc:       # pragma: no cover - 4.9 GB of weights, not expected on a B200
        extras["cfg4_llama8b_decode_step"] = {"error": str(exc)[:120]}
    torch.cuda.empty_cache()

    with tempfile.TemporaryDirectory() as tmp:
        e2e = bench_e2e(max(3, min(K, 20)), 3, r, Path(tmp) / "artifact")
    cpu, _ = cpu_reference_timing(budget_s=args.cpu_budget)

    m512 = prefill["m512"]
    line = {
        "metric": "GGUF qmatmul weight GB/s at M=1 (Q4_K 11008x4096) [TFLOP/s at M=512 in roofline_prefill]",
        "value": value, "unit": "GB/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg2 Q4_K [11008x4096] decode GEMV, M=1, bf16 activations/outputs", "launches_per_step": r,
                   "l2_policy": f"each step walks {r} distinct weight copies ({r * nbytes / 1e6:.0f} MB > 2 x L2 {l2 / 1e6:.0f} MB), so every launch reads cold weights",
                   "timing": "CUDA graph replay, CUDA events on the launching stream", "variant": kernels.select_variant(qtype, "bfloat16", 1, n, k)},
        "roofline": {"kernel": "gemv_q4k_mma_kernel (Q4_K M=1)", "bound": "hbm", "achieved": nbytes / us_launch / 1e3, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": nbytes / us_launch / 1e3 / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind} copy bandwidth",
                     "frac_of_nominal_8tbs": nbytes / us_launch / 1e3 / NOMINAL_HBM_GBS, "us_per_launch": us_launch,
                     "algorithmic_bytes_per_launch": nbytes, "traffic": 25_387_776,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture (profiles/)"},
        "roofline_prefill": {"kernel": "gemm_umma_kernel (Q6_K 4096x14336, M=512)", "bound": "tensor", "achieved": m512["tflops"],
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": m512["frac_of_measured_burst"],
                             "peak_kind": f"of {peak_kind} cuBLAS bf16 burst", "us_per_launch": m512["us_per_launch"],
                             "frac_of_sustained": m512["frac_of_measured_sustained"], "traffic": 68_747_520,
                             "traffic_source": "dram bytes read + written of one ncu capture (profiles/): weights 48.2 MB + activations 14.7 MB + output 4.2 MB + spilled partial tiles"},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": K * r, "clocks": clocks.summary(), "extras": extras,
        "device": {"name": props.name, "sms": props.multi_processor_count, "l2_bytes": l2},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------- profiling cases
PROFILE_CASES = {  # name -> (qtype, n, k, m, variant, weight copies): small, eager, few launches; inputs exceed the L2
    "gemv_q4k_m1": ("Q4_K", 11008, 4096, 1, "mma", 6),
    "gemv_q6k_m1": ("Q6_K", 4096, 14336, 1, "mma", 3),
    "gemm_umma_q6k_m512": ("Q6_K", 4096, 14336, 512, "umma", 3),
    "gemm_umma_q4k_m256": ("Q4_K", 11008, 4096, 256, "umma", 6),
    "gemm_umma_q8_0_m512": ("Q8_0", 4096, 14336, 512, "umma", 3),
    "gemv_q8_0_m1": ("Q8_0", 4096, 4096, 1, "mma", 12),
    "dequant_q4k_f16": ("Q4_K", 11008, 4096, 0, "dequant", 3),
}


def run_profile_case(args):
    """One warm-up pass and one measured pass of a single kernel over distinct weight copies, launched eagerly: the
    command an `ncu -k <kernel> -c <n>` capture wraps.  Prints a short JSON line of its own (not the benchmark line)."""
    import torch

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    qtype, n, k, m, variant, copies = PROFILE_CASES[args.only]
    dev = torch.device("cuda")
    ws = [synthetic.random_blocks_torch(qtype, n, k, 1000 + i, dev) for i in range(copies)]
    if variant == "dequant":
        outs = [torch.empty(n, k, device=dev, dtype=torch.float16) for _ in range(copies)]
        launch = lambda i: kernels.dequantize_rows(ws[i], qtype, k, "float16", out=outs[i])
    else:
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        outs = [torch.empty(m, n, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
        launch = lambda i: kernels.gemm_rcr(x, ws[i], qtype, variant=variant, out=outs[i])
    for i in range(copies):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(copies):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    assert kernels.device_status() == 0
    print(json.dumps({"case": args.only, "launches": 2 * copies, "us_per_launch_eager": e0.elapsed_time(e1) * 1e3 / copies,
                      "weight_bytes": encoded_nbytes(qtype, n, k), "device_bytes": copies * encoded_nbytes(qtype, n, k)}))


# ----------------------------------------------------------------------------------------------- multi GPU
def run_multi(args):
    import torch
    import torch.distributed as dist

    from dinoml_v2_b200 import _native, kernels, sharding, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    _native.lib()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    l2 = torch.cuda.get_device_properties(local).L2_cache_size
    hidden, ffn, qtype = 8192, 28672, "Q4_K"
    n_shard, k_shard = ffn // world, ffn // world
    shard_bytes = 2 * encoded_nbytes(qtype, n_shard, hidden) + encoded_nbytes(qtype, hidden, k_shard)
    total_bytes = 3 * encoded_nbytes(qtype, ffn, hidden)
    r = rotation_copies(shard_bytes, l2, cap=8)
    K, W = args.steps, args.warmup
    results = {}
    for m in (1, 16, 256):
        ffns = []
        for i in range(r):
            # random shard contents: the distributions are per block, so a shard of a random matrix is a random matrix
            gate = synthetic.random_blocks_torch(qtype, n_shard, hidden, 7000 + 10 * i + rank * 100, dev)
            up = synthetic.random_blocks_torch(qtype, n_shard, hidden, 7001 + 10 * i + rank * 100, dev)
            down = synthetic.random_blocks_torch(qtype, hidden, k_shard, 7002 + 10 * i + rank * 100, dev)
            ffns.append(sharding.ShardedFFN(gate, up, down, qtype, hidden, ffn))
        gx = torch.Generator(device=dev)
        gx.manual_seed(99)                                  # activations are replicated: same seed on every rank
        x = torch.randn(m, hidden, device=dev, generator=gx).to(torch.bfloat16)
        h = torch.randn(m, ffn, device=dev, generator=gx).to(torch.bfloat16)
        h_slice = h[:, rank * k_shard:(rank + 1) * k_shard].contiguous()
        og, ou = (torch.empty(m, n_shard, device=dev, dtype=torch.bfloat16) for _ in range(2))
        gg, gu = (torch.empty(world, m, n_shard, device=dev, dtype=torch.bfloat16) for _ in range(2))
        od = torch.empty(m, hidden, device=dev, dtype=torch.bfloat16)

        def step_nccl():
            for f in ffns:
                f.gate_up(x, og, ou, gg, gu)
                f.down_proj(h_slice, od)

        def step_peer():
            for f in ffns:
                f.gate_up_peer(x)
                f.down_proj_peer(h_slice, od)

        stream = torch.cuda.current_stream()
        # Decode sizes go over peer memory (the GEMV kernel stores into every GPU's gather buffer, one small kernel
        # finishes each collective); NCCL is the fallback and is timed beside it.
        step, mode, nccl_ms, swiglu_ms = step_nccl, "nccl", None, None
        if m <= 64 and os.environ.get("DINOML_B200_PEER_PATH", "1") != "0":   # decode and small-batch sizes: mma GEMV or tcgen05 kernel, both with a scatter epilogue
            try:
                for f in ffns:
                    f.enable_peer_path(m, torch.bfloat16, share_with=ffns[0] if f is not ffns[0] else None)
                step_nccl(); step_peer()
                torch.cuda.synchronize()
                assert kernels.device_status() == 0, "a bounded device-side wait gave up on the peer path"
                ref = od.clone()
                ffns[-1].down_proj(h_slice, od)
                torch.cuda.synchronize()
                # fp32 accumulation in rank order here, NCCL's own order and precision there: equal up to bf16 rounding
                assert float((ref.float() - od.float()).abs().max()) <= 2e-2 * float(od.float().abs().max()), "peer all-reduce differs from NCCL"
                nccl_ms = time_steps(step_nccl, max(3, K // 2), W, stream, barrier=dist.barrier)
                step, mode = step_peer, "peer"

                def step_swiglu():                          # extra: the gated MLP with no all-gather at all
                    for f in ffns:
                        f.swiglu_mlp_peer(x, od)
                swiglu_ms = time_steps(step_swiglu, max(3, K // 2), W, stream, barrier=dist.barrier)
            except Exception as exc:                        # pragma: no cover - no symmetric memory on this box
                if rank == 0:
                    print(f"peer path unavailable ({type(exc).__name__}: {str(exc)[:200]}); using NCCL", file=sys.stderr)
                step, mode = step_nccl, "nccl"
        clock_ctx = ClockSampler(local) if (m == 1 and rank == 0) else None
        if clock_ctx:
            clock_ctx.__enter__()
        ms = time_steps(step, K, W, stream, barrier=dist.barrier)
        if clock_ctx:
            clock_ctx.__exit__(None, None, None)
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)            # max over ranks
        ms_step = float(t.item()) / K
        results[m] = {"ms_per_step": ms_step, "ms_per_ffn": ms_step / r, "weight_gbs": r * total_bytes / ms_step / 1e6,
                      "tflops": r * 6.0 * m * hidden * ffn / ms_step / 1e9, "collectives": mode}
        if nccl_ms is not None:
            tn = torch.tensor([nccl_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tn, op=dist.ReduceOp.MAX)
            results[m]["nccl_ms_per_ffn"] = float(tn.item()) / max(3, K // 2) / r
        if swiglu_ms is not None:
            ts = torch.tensor([swiglu_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(ts, op=dist.ReduceOp.MAX)
            results[m]["fused_swiglu_mlp_ms_per_ffn"] = float(ts.item()) / max(3, K // 2) / r
        if m == 1:
            clocks = clock_ctx.summary() if clock_ctx else None
        del ffns
        torch.cuda.empty_cache()
    assert kernels.device_status() == 0
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        r1 = results[1]
        per_gpu = r1["weight_gbs"] / world
        print(json.dumps({
            "metric": "GGUF qmatmul weight GB/s at M=1 (Llama-70B FFN sharded, Q4_K gate/up/down)", "value": r1["weight_gbs"], "unit": "GB/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": r1["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "cfg5 Llama-3-70B FFN: Q4_K gate,up [28672x8192] N-split + all-gather; down [8192x28672] K-split + "
                                   "all-reduce (bf16); M=1; collectives: " + ("GEMV epilogue stores into peer GPUs' buffers + one "
                                   "barrier / barrier-and-sum kernel each" if r1["collectives"] == "peer" else "NCCL"),
                       "parallelism": f"tp{world}", "ffns_per_step": r,
                       "l2_policy": f"each step walks {r} distinct shard sets ({r * shard_bytes / 1e6:.0f} MB per GPU > 2 x L2)",
                       "timing": "eager launches on one stream, CUDA events, max over ranks"},
            "roofline": {"kernel": "gemv_q4k_mma_kernel (scatter) + peer_exchange_kernel" if r1["collectives"] == "peer" else "gemv_q4k_mma_kernel + NCCL", "bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu / peaks["hbm_gbs"], "peak_kind": f"per GPU, of {peak_kind} copy bandwidth", "traffic": None},
            "cpu_baseline": None,
            "e2e": {"value": None, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "the artifact / session API is single-GPU; the sharded FFN is measured at the kernel + collective level"},
            "gpu_launches": K * r * (4 if r1["collectives"] == "peer" else 3), "clocks": clocks, "extras": {f"m{m}": v for m, v in results.items()}}))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=10.0, help="seconds of CPU work for the cpu_baseline leg")
    ap.add_argument("--only", choices=sorted(PROFILE_CASES), help="run one small single-kernel case (for profiler captures) and exit")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.only:
        return run_profile_case(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus > 1:
        if "RANK" not in os.environ:
            raise SystemExit("--gpus > 1 must be launched with torchrun (one rank per GPU)")
        return run_multi(args)
    return run_single(args)


if __name__ == "__main__":
    main()
