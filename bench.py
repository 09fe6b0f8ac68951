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
# One metric string for every line of both arms (the path's headline metric); what a line measures is in `config`.
METRIC = "GGUF qmatmul weight GB/s at M=1 and TFLOP/s at M=512, % of roofline"
WORKLOAD_N1 = "cfg2 Q4_K [11008x4096] decode GEMV, M=1, bf16 activations/outputs"
WORKLOAD_MULTI = ("cfg5 Llama-3-70B FFN, M=1, bf16: Q4_K gate,up [28672x8192] split along N + all-gather; "
                  "down [8192x28672] split along K + all-reduce")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML about every millisecond when the
    binding works (a timed region of a few milliseconds still gets samples; the context waits for the first sample before
    the region starts and takes a last one when it ends), else through nvidia-smi every 50 ms."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    # The same NVML loop as a child process: it shares no interpreter lock with a timed region whose launches are issued
    # from Python (the multi-GPU step), where a sampling thread would slow down what it observes.
    _CHILD = (
        "import sys, time\n"
        "import pynvml as nv\n"
        "nv.nvmlInit()\n"
        "spec, path = sys.argv[1], sys.argv[2]\n"
        "h = nv.nvmlDeviceGetHandleByUUID(spec) if spec.startswith('GPU-') else nv.nvmlDeviceGetHandleByIndex(int(spec))\n"
        "fn = getattr(nv, 'nvmlDeviceGetCurrentClocksEventReasons', None) or getattr(nv, 'nvmlDeviceGetCurrentClocksThrottleReasons')\n"
        "f = open(path, 'w')\n"
        "while True:\n"
        "    mask = int(fn(h))\n"
        "    row = [str(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))), str(float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))]\n"
        "    row += ['Active' if mask & b else 'Not Active' for b in (0x8, 0x40, 0x20, 0x4)]\n"
        "    f.write(','.join(row) + '\\n'); f.flush()\n"
        "    time.sleep(0.001)\n")

    def __init__(self, index: int, isolated: bool = False):
        self.index, self.rows, self._stop, self._thread = index, [], threading.Event(), None
        self._isolated, self._child, self._child_path, self._spec = isolated, None, None, str(index)
        self._first = threading.Event()
        self.source, self.error = "nvidia-smi", None
        self._nvml = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = visible.split(",") if visible else []
            if index < len(ids) and ids[index].strip().isdigit():
                self._spec = ids[index].strip()
                handle = nv.nvmlDeviceGetHandleByIndex(int(ids[index]))
            elif index < len(ids) and ids[index].strip().startswith("GPU-"):
                self._spec = ids[index].strip()
                handle = nv.nvmlDeviceGetHandleByUUID(ids[index].strip())
            else:
                handle = nv.nvmlDeviceGetHandleByIndex(index)
            self._nvml, self.source = (nv, handle), "nvml"
        except Exception as exc:                          # no binding / no NVML: fall back to nvidia-smi
            self.error = f"{type(exc).__name__}: {exc}"[:120]

    def _nvml_sample(self):
        nv, h = self._nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        bits = [0x8, 0x40, 0x20, 0x4]                     # hw slowdown, hw thermal slowdown, sw thermal slowdown, sw power cap
        sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
        top = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        mask = int(reasons_fn(h))
        self.rows.append([str(sm), str(top)] + ["Active" if mask & bit else "Not Active" for bit in bits])

    def _smi_sample(self):
        out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        if out:
            self.rows.append([c.strip() for c in out.splitlines()[0].split(",")])

    def _sample(self):
        try:
            if self._nvml is not None:
                self._nvml_sample()
            else:
                self._smi_sample()
        except Exception as exc:
            self.error = f"{type(exc).__name__}: {exc}"[:120]
            if self._nvml is not None:                    # NVML answered with an error: use nvidia-smi from here on
                self._nvml, self.source = None, "nvidia-smi"

    def _loop(self):
        while not self._stop.is_set():
            self._sample()
            self._first.set()
            self._stop.wait(0.001 if self._nvml is not None else 0.05)

    def _start_child(self) -> bool:
        import tempfile
        fd, self._child_path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
        os.close(fd)
        try:
            self._child = subprocess.Popen([sys.executable, "-c", self._CHILD, self._spec, self._child_path],
                                           stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self._child = None
            return False
        deadline = time.time() + 10
        while time.time() < deadline and self._child.poll() is None and os.path.getsize(self._child_path) == 0:
            time.sleep(0.01)
        if os.path.getsize(self._child_path) == 0:          # the child never sampled: stop it, use the thread
            self._stop_child()
            return False
        self.source = "nvml (child process)"
        return True

    def _stop_child(self):
        if self._child is not None:
            self._child.terminate()
            try:
                self._child.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._child.kill()
            self._child = None
        if self._child_path and os.path.exists(self._child_path):
            with open(self._child_path) as f:
                self.rows += [line.strip().split(",") for line in f if line.count(",") >= 5]
            os.unlink(self._child_path)
        self._child_path = None

    def __enter__(self):
        if self._isolated and self._nvml is not None and self._start_child():
            return self
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        self._first.wait(timeout=6)                       # the timed region starts with one sample on record
        return self

    def __exit__(self, *exc):
        if self._thread is None:                          # child-process mode
            self._stop_child()
            self._sample()
            return
        self._stop.set()
        self._thread.join(timeout=6)
        self._sample()                                    # and ends with one

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": self.source, "error": self.error}
        sm = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        reasons = [n for i, n in enumerate(self.NAMES) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": float(self.rows[0][1]) if self.rows[0][1].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(self.rows), "source": self.source}


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


def profile_traffic(profile_name):
    """DRAM bytes per launch recorded in a committed ncu summary (a line `dram_bytes_per_launch: N` in profiles/<name>), or
    None.  The benchmark reports what the summary on file says; it never carries a typed-in copy of it."""
    import re
    path = ROOT / "profiles" / profile_name
    if not path.exists():
        return None, None
    m = re.search(r"^dram_bytes_per_launch:\s*([0-9_,]+)", path.read_text(), flags=re.M)
    return (int(m.group(1).replace(",", "").replace("_", "")) if m else None), f"profiles/{profile_name}"


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


FFN70B = {"hidden": 8192, "ffn": 28672, "qtype": "Q4_K"}


def bench_ffn_1gpu(ms, steps, warmup, l2, device=None):
    """Config 5's FFN on ONE GPU, unsharded: gate and up [28672 x 8192], down [8192 x 28672], three launches per FFN
    (the baseline the sharded runs are compared with).  Returns {m: {...}}."""
    import torch

    from dinoml_v2_b200 import kernels, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    dev = device or torch.device("cuda")
    hidden, ffn, qtype = FFN70B["hidden"], FFN70B["ffn"], FFN70B["qtype"]
    total = 3 * encoded_nbytes(qtype, ffn, hidden)
    r = rotation_copies(total, l2, cap=3)
    sets = [(synthetic.random_blocks_torch(qtype, ffn, hidden, 8000 + 3 * i, dev), synthetic.random_blocks_torch(qtype, ffn, hidden, 8001 + 3 * i, dev),
             synthetic.random_blocks_torch(qtype, hidden, ffn, 8002 + 3 * i, dev)) for i in range(r)]
    out = {}
    stream = torch.cuda.Stream(device=dev)
    for m in ms:
        x = torch.randn(m, hidden, device=dev).to(torch.bfloat16)
        h = torch.randn(m, ffn, device=dev).to(torch.bfloat16)
        og, ou = (torch.empty(m, ffn, device=dev, dtype=torch.bfloat16) for _ in range(2))
        od = torch.empty(m, hidden, device=dev, dtype=torch.bfloat16)

        def one_pass():
            for (gate, up, down) in sets:
                kernels.gemm_rcr(x, gate, qtype, out=og)
                kernels.gemm_rcr(x, up, qtype, out=ou)
                kernels.gemm_rcr(h, down, qtype, out=od)

        g = graph_of(one_pass, stream)
        ms_ffn = time_steps(g.replay, steps, warmup, stream) / (steps * r)
        out[m] = {"ms_per_ffn": ms_ffn, "weight_gbs": total / ms_ffn / 1e6, "tflops": 6.0 * m * hidden * ffn / ms_ffn / 1e9,
                  "launches_per_ffn": 3, "weight_sets": r}
    assert kernels.device_status() == 0
    del sets
    torch.cuda.empty_cache()
    return out


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
            "ms_per_step": dt * 1e3, "steps": steps, "api": "dml.compile -> runtime.load -> Session.run_numpy", "linears_per_step": copies}


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


def _cpu_gemm_call(lib):
    """call(x, w, y, m, n, k) running the reference CPU kernel (bf16), or the oracle's restatement when it is not built."""
    import oracle
    if lib is not None:
        fn = lib[0].ref_gemm_rcr_bfloat16
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 3
        return (lambda x, w, y, m, n, k: fn(x.ctypes.data, w.ctypes.data, y.ctypes.data, m, n, k)), "reference", \
            f"gemm_cpu.cpp.j2 kernel built -O3 -ffast-math -fopenmp ({lib[1]})"

    def call(x, w, y, m, n, k):
        y[...] = oracle.gemm_rcr_dense(x, w, "bfloat16")
    return call, "port", "C restatement of gemm_cpu.cpp.j2 (strict k order)"


def cpu_reference_timing(budget_s, min_iters=3, workload="cfg2"):
    """Times the reference CPU path (M = 1, bf16, dense weights = host-dequantized GGUF blocks rounded to bf16, as
    GGUFConstant.materialize produces on the CPU target) on `workload`: "cfg2" = one [11008 x 4096] linear per call,
    "cfg5" = the three linears of one 70B FFN per call.  Bounded: runs until `budget_s` and at least `min_iters` calls."""
    import oracle
    from dinoml_v2_b200 import synthetic
    if workload == "cfg2":
        shapes = [(CFG2["qtype"], CFG2["n"], CFG2["k"])]
    else:
        shapes = [(FFN70B["qtype"], FFN70B["ffn"], FFN70B["hidden"])] * 2 + [(FFN70B["qtype"], FFN70B["hidden"], FFN70B["ffn"])]
    oracle.set_threads(os.cpu_count() or 1)           # the one-off host dequantization may use every core; the matmul below cannot
    mats, nbytes = [], 0
    for i, (qtype, n, k) in enumerate(shapes):
        blocks = synthetic.random_blocks(qtype, n, k, 1000 + i)
        nbytes += blocks.nbytes
        mats.append((oracle.dequantize(blocks, qtype, k, "bfloat16"), synthetic.random_activations(1, k, 7 + i, "bfloat16"),
                     np.empty((1, n), dtype=np.uint16), n, k))
        del blocks
    call, kind, detail = _cpu_gemm_call(_ref_library())

    def one():
        for (w, x, y, n, k) in mats:
            call(x, w, y, 1, n, k)
    one()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_iters or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
    med = sorted(times)[len(times) // 2]
    what = "one Q4_K [11008x4096]" if workload == "cfg2" else "the three Q4_K linears of one 70B FFN (2 x [28672x8192], [8192x28672])"
    # the reference's OpenMP loop runs over the M activation rows (gemm_cpu.cpp.j2:35-38): one row => one core
    return {"value": nbytes / med / 1e9, "unit": "GB/s", "cores": 1, "kind": kind, "ms_per_call": med * 1e3,
            "sample": f"{len(times)} calls of {what} M=1 bf16 gemm_rcr over host-dequantized dense weights "
                      f"({detail}); weight bytes counted GGUF-encoded; host has {os.cpu_count()} logical cores, the kernel's "
                      "OpenMP loop is over M rows so M=1 uses one"}, times, nbytes


def run_reference_arm(args):
    """The reference's own CPU implementation of the path on this box's host cores, on the workload the b200 arm runs at
    the same --gpus: config 2 at one GPU, the config-5 FFN (unsharded: the reference has no distributed code) above."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    multi = args.gpus > 1
    base, times, nbytes = cpu_reference_timing(budget_s=0.0, min_iters=args.warmup + args.steps, workload="cfg5" if multi else "cfg2")
    timed = times[args.warmup:args.warmup + args.steps]
    total = sum(timed)
    value = nbytes * len(timed) / total / 1e9
    base["value"] = value
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / len(timed) * 1e3,
        "higher_is_better": True, "scaling": "strong" if multi else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_MULTI if multi else WORKLOAD_N1,
                   "arm": "reference CPU path: host dequantize once, dense gemm_rcr per step; each step is ONE "
                          + ("FFN (three matmuls, unsharded)" if multi else "matmul") + ", a bounded sample of the GPU arm's step"},
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
    # the six further types of the reference prototype: dequantizer, decode GEMV and (where built) prefill GEMM on a [4096 x 4096] weight
    extras["further_qtypes_4096x4096"] = {}
    for q in ("Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4"):
        dq = bench_dequant(q, 4096, 4096, "float16", extra_steps, extra_warm)
        gv = bench_gemm(q, 4096, 4096, 1, extra_steps, extra_warm, l2)
        extras["further_qtypes_4096x4096"][q] = {"dequant_f16_gbs": dq["gbs"], "dequant_f16_frac_of_measured_hbm": dq["gbs"] / peaks["hbm_gbs"],
                                                 "gemv_m1_us": gv["us_per_launch"], "gemv_m1_weight_gbs": gv["weight_bytes"] / gv["us_per_launch"] / 1e3,
                                                 "gemv_m1_frac_of_measured_hbm": gv["weight_bytes"] / gv["us_per_launch"] / 1e3 / peaks["hbm_gbs"],
                                                 "variant": gv["variant"]}
        pf = bench_gemm(q, 4096, 4096, 512, extra_steps, extra_warm, l2)      # prefill on the same weight (tcgen05 GEMM)
        extras["further_qtypes_4096x4096"][q].update({"gemm_m512_us": pf["us_per_launch"], "gemm_m512_variant": pf["variant"],
                                                      "gemm_m512_tflops": 2.0 * 512 * 4096 * 4096 / pf["us_per_launch"] / 1e6})
    extras["dual_gate_up_q4k_14336x4096"] = {f"m{m}": bench_dual(14336, 4096, m, extra_steps, extra_warm, l2) for m in (1, 16)}
    extras["cfg5_ffn_1gpu"] = {f"m{m}": v for m, v in bench_ffn_1gpu((1, 16, 256), extra_steps, extra_warm, l2).items()}
    try:
        extras["cfg4_llama8b_decode_step"] = bench_decode_step(extra_steps, extra_warm)
    except torch.cuda.OutOfMemoryError as exc:       # pragma: no cover - 4.9 GB of weights, not expected on a B200
        extras["cfg4_llama8b_decode_step"] = {"error": str(exc)[:120]}
    torch.cuda.empty_cache()

    with tempfile.TemporaryDirectory() as tmp:
        # a step is ~0.2 ms of host + device work: enough of them that scheduler noise on the host averages out
        e2e = bench_e2e(max(20, min(8 * K, 400)), 10, r, Path(tmp) / "artifact")
    cpu, _, _ = cpu_reference_timing(budget_s=args.cpu_budget)

    m512 = prefill["m512"]
    variant = kernels.select_variant(qtype, "bfloat16", 1, n, k)
    gemv_profile = {"stream": "gemv_q4k_stream_m1_q4k_11008x4096.md", "mma": "gemv_q4k_mma_m1_q4k_11008x4096.md"}.get(variant, "")
    gemv_traffic, gemv_traffic_src = profile_traffic(gemv_profile)
    gemm_traffic, gemm_traffic_src = profile_traffic("gemm_umma_q6k_4096x14336_m512.md")
    line = {
        "metric": METRIC,
        "value": value, "unit": "GB/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD_N1, "launches_per_step": r,
                   "value_is": "weight GB/s at M=1 (the TFLOP/s at M=512 half of the metric is in roofline_prefill)",
                   "l2_policy": f"each step walks {r} distinct weight copies ({r * nbytes / 1e6:.0f} MB > 2 x L2 {l2 / 1e6:.0f} MB), so every launch reads cold weights",
                   "timing": "CUDA graph replay, CUDA events on the launching stream", "variant": variant},
        "roofline": {"kernel": f"gemv_q4k_{variant}_kernel (Q4_K M=1)", "bound": "hbm", "achieved": nbytes / us_launch / 1e3, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": nbytes / us_launch / 1e3 / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind} copy bandwidth",
                     "frac_of_nominal_8tbs": nbytes / us_launch / 1e3 / NOMINAL_HBM_GBS, "us_per_launch": us_launch,
                     "algorithmic_bytes_per_launch": nbytes, "traffic": gemv_traffic,
                     "traffic_source": f"dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, read from {gemv_traffic_src}"},
        "roofline_prefill": {"kernel": "gemm_umma_kernel (Q6_K 4096x14336, M=512)", "bound": "tensor", "achieved": m512["tflops"],
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": m512["frac_of_measured_burst"],
                             "peak_kind": f"of {peak_kind} cuBLAS bf16 burst", "us_per_launch": m512["us_per_launch"],
                             "frac_of_sustained": m512["frac_of_measured_sustained"], "traffic": gemm_traffic,
                             "traffic_source": f"dram bytes read + written of one ncu capture, read from {gemm_traffic_src}: weights 48.2 MB + activations 14.7 MB + output 4.2 MB + spilled partial tiles"},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": K * r, "clocks": clocks.summary(), "extras": extras,
        "device": {"name": props.name, "sms": props.multi_processor_count, "l2_bytes": l2},
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------- profiling cases
PROFILE_CASES = {  # name -> (qtype, n, k, m, variant, weight copies): small, eager, few launches; inputs exceed the L2
    "gemv_q4k_m1": ("Q4_K", 11008, 4096, 1, "mma", 6),
    "gemv_stream_q4k_m1_c1": ("Q4_K", 11008, 4096, 1, "stream:1", 6),
    "gemv_stream_q4k_m1_c4": ("Q4_K", 11008, 4096, 1, "stream:4", 6),
    "gemv_stream_q4k_m4": ("Q4_K", 11008, 4096, 4, "stream", 6),
    "gemv_stream_q6k_m1": ("Q6_K", 4096, 14336, 1, "stream", 3),
    "gemv_stream_probe_q4k_c4": ("Q4_K", 11008, 4096, 1, "stream:132", 6),
    "gemv_q4k_m4": ("Q4_K", 11008, 4096, 4, "mma", 6),
    "gemm_umma_q4k_m16": ("Q4_K", 11008, 4096, 16, "umma", 6),
    "gemm_umma_q6k_m64": ("Q6_K", 4096, 14336, 64, "umma", 3),
    "gemv_q6k_m1": ("Q6_K", 4096, 14336, 1, "mma", 3),
    "gemm_umma_q6k_m512": ("Q6_K", 4096, 14336, 512, "umma", 3),
    "gemm_umma_q4k_m256": ("Q4_K", 11008, 4096, 256, "umma", 6),
    "gemm_umma_q8_0_m512": ("Q8_0", 4096, 14336, 512, "umma", 3),
    "gemv_q8_0_m1": ("Q8_0", 4096, 4096, 1, "mma", 12),
    "gemm_umma_mxfp4_m512": ("MXFP4", 4096, 14336, 512, "umma", 4),
    "gemv_stream_mxfp4_m1": ("MXFP4", 11008, 4096, 1, "stream", 6),
    "gemv_stream_nvfp4_m1": ("NVFP4", 11008, 4096, 1, "stream", 6),
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
def _max_over_ranks(ms, dev):
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _all_ranks_agree(flag: bool, dev) -> bool:
    """True only if `flag` is true on every rank: the ranks must take the same code path (peer kernels or NCCL)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([1 if flag else 0], device=dev, dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def run_multi(args):
    import torch
    import torch.distributed as dist

    from dinoml_v2_b200 import _native, kernels, sharding, synthetic
    from dinoml_v2_b200.gguf_blocks import encoded_nbytes
    _native.lib()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"                   # keep NCCL's version banner off stdout: rank 0 prints one JSON line
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    l2 = torch.cuda.get_device_properties(local).L2_cache_size
    hidden, ffn, qtype = FFN70B["hidden"], FFN70B["ffn"], FFN70B["qtype"]
    n_shard, k_shard = ffn // world, ffn // world
    shard_bytes = 2 * encoded_nbytes(qtype, n_shard, hidden) + encoded_nbytes(qtype, hidden, k_shard)
    total_bytes = 3 * encoded_nbytes(qtype, ffn, hidden)
    r = rotation_copies(shard_bytes, l2, cap=8)
    K, W = args.steps, args.warmup
    half = max(3, K // 2)
    use_peer_env = os.environ.get("DINOML_B200_PEER_PATH", "1") != "0"
    results, clocks, e2e = {}, None, None
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

        def step_pull():                                    # peer memory, pulled: GEMMs store locally, one kernel per gather / two per reduce
            for f in ffns:
                f.gate_up_pull(x)
                f.down_proj_pull(h_slice, od)

        def comm_pull():
            for f in ffns:
                f.xchg_gate_up.pull_gather()
                f.xchg_down.pull_all_reduce(od)

        def comm_nccl():                                    # the collectives of step_nccl alone
            for _ in ffns:
                dist.all_gather_into_tensor(gg.view(-1, n_shard), og)
                dist.all_gather_into_tensor(gu.view(-1, n_shard), ou)
                dist.all_reduce(od)

        def comm_peer():                                    # the exchange kernels of step_peer alone (they sum whatever the slots hold)
            for f in ffns:
                f.xchg_gate_up.finish_gather()
                f.xchg_down.finish_reduce(od)

        stream = torch.cuda.current_stream()
        # Decode sizes go over peer memory (the GEMV kernel stores into every GPU's gather buffer, one small kernel
        # finishes each collective); NCCL is the fallback and is timed beside it.  Only a failure to SET UP the peer
        # buffers falls back; a wrong result or a device-side give-up is an error, and the ranks agree on the mode first.
        want_peer = use_peer_env
        peer_ok = False
        if want_peer:
            try:
                for f in ffns:
                    f.enable_peer_path(m, torch.bfloat16, share_with=ffns[0] if f is not ffns[0] else None, device_epoch=True)
                peer_ok = True
            except (RuntimeError, ImportError, AttributeError, OSError) as exc:   # no symmetric memory on this box / torch build
                if rank == 0:
                    print(f"peer buffers unavailable ({type(exc).__name__}: {str(exc)[:200]}); using NCCL", file=sys.stderr)
        mode = "peer" if (want_peer and _all_ranks_agree(peer_ok, dev)) else "nccl"
        nccl_ms = peer_ms = pull_ms = swiglu_ms = None
        if mode == "peer":
            # correctness before timing: the peer all-reduce against NCCL's, several back-to-back calls on one exchange
            step_nccl()
            ref = od.clone()
            for _ in range(3):
                step_peer()
            torch.cuda.synchronize()
            assert kernels.device_status() == 0, "a bounded device-side wait gave up on the peer path"
            # fp32 accumulation in rank order here, NCCL's own order and precision there: equal up to bf16 rounding
            assert float((ref.float() - od.float()).abs().max()) <= 2e-2 * float(ref.float().abs().max()), "peer all-reduce differs from NCCL"
            # the fused gated MLP against the same thing built from the dual GEMM and NCCL, three consecutive calls
            f0 = ffns[0]
            hloc = kernels.dual_gemm_rcr(x, kernels.interleave_rows8(f0.gate, f0.up), qtype, "silu")
            want = torch.empty(m, hidden, device=dev, dtype=torch.bfloat16)
            f0.down_proj(hloc, want)
            for _ in range(3):
                got = torch.empty(m, hidden, device=dev, dtype=torch.bfloat16)
                f0.swiglu_mlp_peer(x, got)
                torch.cuda.synchronize()
                assert float((want.float() - got.float()).abs().max()) <= 2e-2 * float(want.float().abs().max()), "fused gated MLP differs from NCCL"
            # the pull path against the same reference, two consecutive calls
            for _ in range(2):
                step_pull()
            torch.cuda.synchronize()
            assert kernels.device_status() == 0, "a bounded device-side wait gave up on the pull path"
            assert float((ref.float() - od.float()).abs().max()) <= 2e-2 * float(ref.float().abs().max()), "pull all-reduce differs from NCCL"
            nccl_ms = _max_over_ranks(time_steps(step_nccl, half, W, stream, barrier=dist.barrier), dev)
            peer_ms = _max_over_ranks(time_steps(step_peer, half, W, stream, barrier=dist.barrier), dev)
            pull_ms = _max_over_ranks(time_steps(step_pull, half, W, stream, barrier=dist.barrier), dev)
            mode = min((peer_ms, "peer"), (pull_ms, "pull"), (nccl_ms, "nccl"))[1]      # every rank sees the same three maxima

            def step_swiglu():                              # extra: the gated MLP with no all-gather at all
                for f in ffns:
                    f.swiglu_mlp_peer(x, od)
            swiglu_ms = time_steps(step_swiglu, half, W, stream, barrier=dist.barrier)
        step, comm = {"peer": (step_peer, comm_peer), "pull": (step_pull, comm_pull), "nccl": (step_nccl, comm_nccl)}[mode]
        clock_ctx = ClockSampler(local, isolated=True) if (m == 1 and rank == 0) else None
        if clock_ctx:
            clock_ctx.__enter__()
        ms = time_steps(step, K, W, stream, barrier=dist.barrier)
        ms_step = _max_over_ranks(ms, dev) / K
        timing = "eager launches on one stream"
        graph_ms_step = None
        if mode != "nccl" and K % 2 == 0:
            # The same step replayed from a CUDA graph: no library collective inside (only this repository's kernels; their
            # epochs live on the device), so the capture is per rank and the replays meet in the exchange kernels.  A graph
            # holds TWO steps: the exchange buffers alternate per collective, and an even count per replay keeps that in phase.
            graph, ok = None, True
            try:
                torch.cuda.synchronize()
                graph = graph_of(lambda: (step(), step()), torch.cuda.Stream(device=dev))     # capture needs a non-default stream
                torch.cuda.synchronize()
            except RuntimeError as exc:
                ok = False
                if rank == 0:
                    print(f"graph capture of the {mode} step failed ({str(exc)[:160]}); eager timing stands", file=sys.stderr)
            if _all_ranks_agree(ok, dev):
                gms = time_steps(graph.replay, K // 2, W, stream, barrier=dist.barrier)
                torch.cuda.synchronize()
                assert kernels.device_status() == 0, "a bounded device-side wait gave up during graph replay"
                assert float((ref.float() - od.float()).abs().max()) <= 2e-2 * float(ref.float().abs().max()), "graph-replayed step differs from NCCL"
                graph_ms_step = _max_over_ranks(gms, dev) / K
                if graph_ms_step < ms_step:
                    ms_step, timing = graph_ms_step, "CUDA graph replay (two steps per graph)"
        if clock_ctx:
            clock_ctx.__exit__(None, None, None)
            clocks = clock_ctx.summary()
        comm_ms = _max_over_ranks(time_steps(comm, half, W, stream, barrier=dist.barrier), dev) / half
        results[m] = {"ms_per_step": ms_step, "ms_per_ffn": ms_step / r, "weight_gbs": r * total_bytes / ms_step / 1e6,
                      "tflops": r * 6.0 * m * hidden * ffn / ms_step / 1e9, "collectives": mode,
                      "comm_us_per_ffn": comm_ms * 1e3 / r,
                      "comm_is": {"peer": "peer_exchange_kernel x 2 alone", "pull": "peer_pull_kernel x 3 alone (gather, reduce slice, gather)",
                                  "nccl": "ncclAllGather x 2 + ncclAllReduce alone"}[mode],
                      "bound_by": None, "timing": timing,
                      "eager_ms_per_ffn": _max_over_ranks(ms, dev) / K / r, "graph_ms_per_ffn": graph_ms_step / r if graph_ms_step else None}
        if nccl_ms is not None:
            results[m]["nccl_ms_per_ffn"] = nccl_ms / half / r
            results[m]["peer_ms_per_ffn"] = peer_ms / half / r
            results[m]["pull_ms_per_ffn"] = pull_ms / half / r
        if swiglu_ms is not None:
            results[m]["fused_swiglu_mlp_ms_per_ffn"] = _max_over_ranks(swiglu_ms, dev) / half / r
        if m == 1:
            # end to end: activations start in pinned host memory and the result ends in host memory, every step
            x_host = x.cpu().pin_memory()
            h_host = h_slice.cpu().pin_memory()
            y_host = torch.empty(m, hidden, dtype=torch.bfloat16).pin_memory()

            def step_e2e():
                x.copy_(x_host, non_blocking=True)
                h_slice.copy_(h_host, non_blocking=True)
                step()
                y_host.copy_(od, non_blocking=True)
                stream.synchronize()
            for _ in range(W):
                step_e2e()
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(K):
                step_e2e()
            torch.cuda.synchronize()
            wall_ms = _max_over_ranks((time.perf_counter() - t0) * 1e3, dev) / K
            e2e = {"value": r * total_bytes / wall_ms / 1e6, "unit": "GB/s", "h2d_bytes_per_step": (m * hidden + m * k_shard) * 2,
                   "d2h_bytes_per_step": m * hidden * 2, "ms_per_step": wall_ms,
                   "api": "ShardedFFN.gate_up[_peer] + down_proj[_peer] per FFN, host activations in, host result out, wall clock, max over ranks"}
        del ffns
        torch.cuda.empty_cache()
    assert kernels.device_status() == 0
    # the same FFN on one GPU, unsharded, measured by rank 0 in this run: the baseline of the speed-ups below
    base = bench_ffn_1gpu((1, 16, 256), max(3, min(K, 10)), 3, l2, dev) if rank == 0 else None
    dist.barrier()
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        for m, v in results.items():
            v["one_gpu_ms_per_ffn"] = base[m]["ms_per_ffn"]
            v["speedup_vs_1gpu"] = base[m]["ms_per_ffn"] / v["ms_per_ffn"]
            compute_us = v["ms_per_ffn"] * 1e3 - v["comm_us_per_ffn"]
            v["bound_by"] = ("the collective step (" + v["comm_is"] + ")") if v["comm_us_per_ffn"] > compute_us else \
                "the quantized matmul kernels (HBM at small M, tensor cores at M=256)"
        r1 = results[1]
        per_gpu = r1["weight_gbs"] / world
        cpu, _, _ = cpu_reference_timing(budget_s=min(args.cpu_budget, 5.0), workload="cfg5")
        print(json.dumps({
            "metric": METRIC, "value": r1["weight_gbs"], "unit": "GB/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": r1["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD_MULTI,
                       "value_is": "total GGUF-encoded weight bytes of the three matrices / max-over-ranks step time, M=1",
                       "collectives": {"peer": "GEMV epilogue stores into peer GPUs' buffers + one barrier / barrier-and-sum kernel each",
                                       "pull": "GEMV stores locally + one pull kernel per gather, two per all-reduce (16-byte peer loads)",
                                       "nccl": "NCCL all-gather x 2 + all-reduce"}[r1["collectives"]],
                       "parallelism": f"tp{world}", "ffns_per_step": r,
                       "l2_policy": f"each step walks {r} distinct shard sets ({r * shard_bytes / 1e6:.0f} MB per GPU > 2 x L2)",
                       "timing": r1["timing"] + ", CUDA events, max over ranks"},
            "roofline": {"kernel": {"peer": "gemv_q4k kernel (scatter epilogue) + peer_exchange_kernel", "pull": "gemv_q4k kernel + peer_pull_kernel",
                                    "nccl": "gemv_q4k kernel + NCCL"}[r1["collectives"]],
                         "bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu / peaks["hbm_gbs"], "peak_kind": f"per GPU, of {peak_kind} copy bandwidth", "traffic": None},
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": K * r * {"peer": 4, "pull": 5, "nccl": 3}[r1["collectives"]], "clocks": clocks,
            "extras": {**{f"m{m}": v for m, v in results.items()}, "one_gpu_unsharded": {f"m{m}": v for m, v in base.items()}}}))
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
