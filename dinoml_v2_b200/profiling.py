"""Profiling-based candidate selection for GGUF quantized linears.

The reference profiles only the dense GEMM that follows its dequantize step (src/dinoml/kernels/profiling.py:
1691-, 4896-4942; native timer tools/cutlass_gemm_profiler_core.cuh:254-343) and picks the lowest median per
(node, shape) with a confidence rule (:4462-4524, 4647-4714).  Here the fused kernels themselves are timed, on the
node's real encoded weights with N(0, 0.125^2) activations (the reference timer's distribution, core.cuh:66-88),
through the library's `dinoml_profile_*` symbols; report, plan and confidence fields keep the reference's names.
The quantization type is part of the problem identity in every cache key (the reference's key has no such field
because it never times a quantized kernel, :4111-4165, 4219-4315)."""
from __future__ import annotations

import itertools
import json
import math
import sqlite3
import statistics
import subprocess
from pathlib import Path
from typing import Any, Mapping, Sequence

import numpy as np

from . import manifest as mf

PROFILE_REPORT_SCHEMA_VERSION = 1
SELECTION_POLICY = "lowest_median_elapsed_ms_per_node_shape"
# src/dinoml/kernels/profiling.py:62-72, 4686-4697
CONFIDENCE = {"min_repeats": 3, "min_margin_ms": 0.002, "min_margin_fraction": 0.02, "z": 1.96}


def shape_scenarios(graph: Mapping[str, Any], overrides: Mapping[str, Sequence[int]] | None = None) -> list[dict[str, int]]:
    """Cartesian product of each dynamic dim's buckets (+ max), as src/dinoml/kernels/profiling.py:2485-2535."""
    dims: dict[str, list[int]] = {}
    for t in graph["inputs"]:
        for d in t["shape_spec"]:
            if d["kind"] == "dynamic":
                vals = list((overrides or {}).get(d["name"], [])) or sorted(set(list(d["buckets"]) + [d["max"]]))
                dims[d["name"]] = vals
    names = sorted(dims)
    return [dict(zip(names, combo)) for combo in itertools.product(*[dims[n] for n in names])] or [{}]


def _resolve(shape_spec, scenario) -> tuple[int, ...]:
    return tuple(scenario[d["name"]] if d["kind"] == "dynamic" else d["value"] for d in shape_spec)


def hardware_fingerprint() -> dict[str, Any]:
    """nvidia-smi device identity + nvcc version (src/dinoml/kernels/profiling.py:3828-3838)."""
    def run(cmd):
        try:
            return subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout.strip()
        except Exception:
            return ""
    return {"gpu": run(["nvidia-smi", "--query-gpu=name,driver_version,memory.total", "--format=csv,noheader"]).splitlines()[:1],
            "nvcc": run(["nvcc", "--version"]).splitlines()[-1:] }


def profile_key(target, fingerprint_key, item, cand, shape) -> str:
    return mf.sha256_of({
        "schema_version": mf.PROFILE_CACHE_SCHEMA_VERSION, "target": target, "hardware_fingerprint_key": fingerprint_key,
        "provider_problem": {"provider": {"kernel_library": mf.KERNEL_LIBRARY, "op_family": "gemm", "op": item["op"], "dtype": item["dtype"]},
                             "semantics": {"layouts": cand["layouts"], "epilogue": cand["epilogue"], "qtype": item["qtype"],
                                           "activation_dtype": item["dtype"], "output_dtype": item["dtype"]},
                             "problem": dict(shape)},
        "candidate": {"candidate_set_key": item["candidate_set_key"], "candidate_id": cand["candidate_id"],
                      "candidate_config_key": cand["candidate_config_key"]},
        "profile_variant": {"split_k": 1}})


class ProfileCache:
    """SQLite cache of timings, shared per directory (src/dinoml/kernels/profile_cache.py:39-48)."""
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.db = sqlite3.connect(str(self.path))
        self.db.execute("CREATE TABLE IF NOT EXISTS profiles (profile_key TEXT PRIMARY KEY, iterations INTEGER, repeats INTEGER, payload TEXT)")

    def get(self, key: str, iterations: int, repeats: int) -> dict[str, Any] | None:
        row = self.db.execute("SELECT iterations, repeats, payload FROM profiles WHERE profile_key=?", (key,)).fetchone()
        if row and row[0] >= iterations and row[1] >= repeats:       # reused only if at least as thorough (:4322-4352)
            return json.loads(row[2])
        return None

    def put(self, key: str, iterations: int, repeats: int, payload: Mapping[str, Any]) -> None:
        self.db.execute("INSERT OR REPLACE INTO profiles VALUES (?,?,?,?)", (key, iterations, repeats, json.dumps(payload)))
        self.db.commit()


def profile_timing(samples_ms: Sequence[float]) -> dict[str, float]:
    """median / mean / stderr / 95% CI, as _profile_timing (src/dinoml/kernels/profiling.py:4430-4459)."""
    n = len(samples_ms)
    mean = statistics.fmean(samples_ms)
    sd = statistics.stdev(samples_ms) if n > 1 else 0.0
    se = sd / math.sqrt(n) if n > 0 else 0.0
    return {"median_ms": statistics.median(samples_ms), "mean_ms": mean, "stderr_ms": se, "ci95_ms": 1.96 * se, "repeats": n,
            "samples_ms": list(samples_ms)}


def profile_artifact(artifact_dir: str | Path, *, shapes: Mapping[str, Sequence[int]] | None = None, iterations: int = 20,
                     repeats: int = 5, cache: ProfileCache | None = None, rotate_copies: int | None = None) -> dict[str, Any]:
    """Times every applicable candidate of every node on every shape scenario.  Weight copies are rotated between
    launches so each launch reads cold weights when the tensor fits in L2."""
    import torch

    from . import kernels
    artifact_dir = Path(artifact_dir)
    graph = json.loads((artifact_dir / "graph.dinoir.json").read_text())
    manifest = json.loads((artifact_dir / "kernel_manifest.json").read_text())
    consts = {c["name"]: c for c in graph["constants"]}
    fp = hardware_fingerprint()
    fp_key = mf.sha256_of(fp)
    dev = torch.device("cuda")
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    results = []
    for item, node in zip(manifest["required_kernels"], graph["nodes"]):
        if not item.get("has_profiler", True):      # dual GEMM nodes: no candidate timer, the built-in shape guard selects
            continue
        w = consts[node["inputs"][1]]
        raw = np.fromfile(artifact_dir / "constants.bin", dtype=np.uint8, count=w["nbytes"], offset=w["offset"])
        n, k = w["shape"]
        copies = rotate_copies or max(1, min(16, math.ceil(2 * l2 / max(1, raw.nbytes))))
        wdev = [torch.from_numpy(raw.reshape(n, -1)).to(dev) for _ in range(copies)]
        a_spec = next(t for t in graph["inputs"] + graph["tensors"] if t["name"] == node["inputs"][0])
        for scenario in shape_scenarios(graph, shapes):
            a_shape = _resolve(a_spec["shape_spec"], scenario)
            m = int(np.prod(a_shape[:-1], dtype=np.int64))
            shape = {"m": m, "n": n, "k": k}
            x = (torch.randn(m, k, device=dev) * 0.125).to(getattr(torch, item["dtype"]))
            out = torch.empty(m, n, device=dev, dtype=x.dtype)
            for cand in item["candidates"]:
                # the library's own predicate for the whole problem (M range, K multiples, row alignment), not M alone
                if not mf.variant_supports(cand["variant"], m, qtype=item["qtype"], dtype=item["dtype"], n=n, k=k):
                    continue
                key = profile_key(manifest["target"], fp_key, item, cand, shape)
                cached = cache.get(key, iterations, repeats) if cache else None
                if cached is None:
                    samples = []
                    for r in range(repeats):
                        ms = kernels.profile_gemm_rcr(x, wdev[r % copies], item["qtype"], out, variant=cand["variant"], iterations=iterations)
                        if ms < 0:
                            samples = []
                            break
                        samples.append(ms)
                    if not samples:
                        continue
                    cached = profile_timing(samples)
                    if cache:
                        cache.put(key, iterations, repeats, cached)
                results.append({"node_id": item["node_id"], "op": item["op"], "dtype": item["dtype"], "qtype": item["qtype"],
                                "candidate_set_id": item["candidate_set_id"], "candidate_set_key": item["candidate_set_key"],
                                "candidate_id": cand["candidate_id"], "candidate_config_key": cand["candidate_config_key"],
                                "kernel_symbol": cand["kernel_symbol"], "profiler_symbol": cand["profiler_symbol"],
                                "kernel_library": mf.KERNEL_LIBRARY, "shape": shape, "scenario": scenario, "iterations": iterations,
                                "profile_key": key, "gflops": 2.0 * m * n * k / (cached["median_ms"] * 1e6), **cached})
    return {"schema_version": PROFILE_REPORT_SCHEMA_VERSION, "kind": "dinoml.profile_report", "target": manifest["target"],
            "kernel_manifest_cache_key": manifest["cache_key"], "fingerprint": fp, "hardware_cache_key": fp_key, "results": results}


def selection_confidence(best: Mapping[str, Any], runner_up: Mapping[str, Any] | None) -> dict[str, Any]:
    """confident iff margin >= max(0.002 ms, 2 % of best, 1.96 * combined stderr) and >= 3 repeats
    (src/dinoml/kernels/profiling.py:4686-4697)."""
    if runner_up is None:
        return {"confident": best["repeats"] >= CONFIDENCE["min_repeats"], "reason": "single_candidate", "margin_ms": None}
    margin = runner_up["median_ms"] - best["median_ms"]
    need = max(CONFIDENCE["min_margin_ms"], CONFIDENCE["min_margin_fraction"] * best["median_ms"],
               CONFIDENCE["z"] * math.hypot(best["stderr_ms"], runner_up["stderr_ms"]))
    ok = margin >= need and min(best["repeats"], runner_up["repeats"]) >= CONFIDENCE["min_repeats"]
    return {"confident": bool(ok), "margin_ms": margin, "required_margin_ms": need, "runner_up_candidate_id": runner_up["candidate_id"],
            "reason": "margin" if ok else "margin_below_threshold"}


def build_execution_plan(report: Mapping[str, Any]) -> dict[str, Any]:
    groups: dict[tuple, list[dict[str, Any]]] = {}
    for r in report["results"]:
        groups.setdefault((r["node_id"], r["shape"]["m"], r["shape"]["n"], r["shape"]["k"]), []).append(r)
    selections, low = [], []
    for key in sorted(groups):
        ranked = sorted(groups[key], key=lambda r: r["median_ms"])
        best, runner = ranked[0], ranked[1] if len(ranked) > 1 else None
        conf = selection_confidence(best, runner)
        sel = {"selection_key": mf.sha256_of({"node": key[0], "shape": key[1:], "candidate": best["candidate_id"]}),
               "node_id": best["node_id"], "op": best["op"], "dtype": best["dtype"], "qtype": best["qtype"],
               "candidate_set_id": best["candidate_set_id"], "candidate_set_key": best["candidate_set_key"],
               "selected_candidate_id": best["candidate_id"], "candidate_config_key": best["candidate_config_key"],
               "kernel_symbol": best["kernel_symbol"], "profiler_symbol": best["profiler_symbol"], "shape": best["shape"],
               "workspace_nbytes": 0, "split_k": 1, "kernel_library": best["kernel_library"], "avg_ms": best["mean_ms"],
               "median_ms": best["median_ms"], "gflops": best["gflops"], "iterations": best["iterations"],
               "profile_key": best["profile_key"], "status": "selected", "confidence": conf}
        selections.append(sel)
        if not conf["confident"]:
            low.append(sel["selection_key"])
    static, conflicts = [], []
    by_set: dict[tuple, set] = {}
    for s in selections:
        by_set.setdefault((s["op"], s["dtype"], s["candidate_set_key"]), set()).add(s["selected_candidate_id"])
    for (op, dtype, set_key), chosen in sorted(by_set.items()):
        if len(chosen) == 1:
            static.append({"op": op, "dtype": dtype, "candidate_set_key": set_key, "selected_candidate_id": next(iter(chosen))})
        else:
            conflicts.append({"op": op, "dtype": dtype, "candidate_set_key": set_key, "candidates": sorted(chosen)})
    plan = {"schema_version": 1, "kind": "dinoml.execution_plan", "profile_report_schema_version": PROFILE_REPORT_SCHEMA_VERSION,
            "profile_cache_schema_version": mf.PROFILE_CACHE_SCHEMA_VERSION, "target": report["target"],
            "kernel_manifest_cache_key": report["kernel_manifest_cache_key"], "fingerprint": report["fingerprint"],
            "hardware_cache_key": report["hardware_cache_key"], "selection_policy": SELECTION_POLICY,
            "selection_confidence_policy": dict(CONFIDENCE),
            "static_selection_policy": "unique_selected_candidate_per_op_dtype_candidate_set",
            "selections": selections, "low_confidence_selections": low, "static_selections": static, "conflicts": conflicts,
            "summary": {"selection_count": len(selections), "low_confidence_count": len(low),
                        "static_selection_count": len(static), "conflict_count": len(conflicts)}}
    plan["execution_plan_key"] = mf.sha256_of(plan)
    return plan


def validate_execution_plan(plan: Mapping[str, Any]) -> None:
    """Key check on load (src/dinoml/compiler.py:599-611)."""
    body = {k: v for k, v in plan.items() if k != "execution_plan_key"}
    if mf.sha256_of(body) != plan.get("execution_plan_key"):
        raise ValueError("execution plan key does not match its contents")
