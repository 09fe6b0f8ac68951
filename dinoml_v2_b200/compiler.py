"""`dml.compile` for the quantized-linear path: graph -> artifact directory.

Mirrors the steps of the reference compiler (src/dinoml/compiler.py:50-93, 348-452): write constants.bin
(GGUF constants go in as their encoded bytes, :659-661), build the kernel manifest, optionally profile and
overlay an execution plan (:96-179), write `encoded_constants.json` (:847-900) and the metadata the Python
loader reads.  Instead of generating and compiling a per-model module.cu, it writes `module_plan.txt`, which
the prebuilt runtime library interprets, and links `module.so` to that library."""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from . import _native, manifest as mf
from .frontend import DTYPE_ENUM, RUNTIME_ABI_VERSION, ModelSpec


@dataclass(frozen=True)
class Target:
    """src/dinoml/backends/target.py:9-29.  Only the CUDA target exists here; arch is fixed to sm_100a."""
    name: str = "cuda"
    arch: str = "sm_100a"

    def __post_init__(self):
        if self.name != "cuda":
            raise NotImplementedError(f"target {self.name!r} is not built by this runtime (B200 / CUDA only)")
        if self.arch != "sm_100a":
            raise NotImplementedError("the kernels are written for sm_100a only")

    def as_dict(self) -> dict[str, Any]:
        return {"name": self.name, "arch": self.arch}


@dataclass(frozen=True)
class Artifact:
    path: Path


def _dim_token(spec: Mapping[str, Any]) -> str:
    return f"?{spec['min']}:{spec['max']}" if spec["kind"] == "dynamic" else str(spec["value"])


def render_module_plan(graph: Mapping[str, Any], manifest: Mapping[str, Any]) -> str:
    """The launch plan the native runtime walks - the counterpart of the generated launch text
    (src/dinoml/lowering/ops/gemm.py:36-210): one fused launch per node, shape-guarded dispatch records from the
    execution plan (:656-698), no scratch rebinding."""
    lines = ["dinoml_b200_module_plan 1"]
    outputs = {o["name"] for o in graph["outputs"]}
    for t in graph["inputs"]:
        lines.append(f"tensor {t['name']} input {DTYPE_ENUM[t['dtype']]} {len(t['shape_spec'])} " + " ".join(map(_dim_token, t["shape_spec"])))
    for t in graph["tensors"]:
        role = "output" if t["name"] in outputs else "temp"
        lines.append(f"tensor {t['name']} {role} {DTYPE_ENUM[t['dtype']]} {len(t['shape_spec'])} " + " ".join(map(_dim_token, t["shape_spec"])))
    for c in graph["constants"]:
        st = c.get("storage")
        if st and st.get("kind") == "gguf":
            lines.append(f"constant {c['name']} gguf {st['qtype_value']} {c['offset']} {c['nbytes']} {c['shape'][0]} {st['n_per_row']} {st['residency']}")
        else:
            lines.append(f"constant {c['name']} dense {DTYPE_ENUM[c['dtype']]} {c['offset']} {c['nbytes']} {len(c['shape'])} " + " ".join(map(str, c["shape"])))
    items = {i["node_id"]: i for i in manifest["required_kernels"]}
    for idx, node in enumerate(graph["nodes"]):
        item = items[node["id"]]
        bias = node["inputs"][2] if len(node["inputs"]) > 2 else "-"
        variant = 0
        if item.get("selected_candidate_id"):
            variant = next(c["variant_code"] for c in item["candidates"] if c["candidate_id"] == item["selected_candidate_id"])
            if item.get("execution_plan_dispatch"):
                variant = 0        # static choice only holds on the profiled shapes; others use the built-in guard
        lines.append(f"node {node['op']} {node['inputs'][0]} {node['inputs'][1]} {bias} {node['outputs'][0]} {variant}")
        for d in item.get("execution_plan_dispatch", []):
            lines.append(f"dispatch {idx} {d['m']} {d['n']} {d['k']} {d['variant_code']}")
    return "\n".join(lines) + "\n"


def encoded_constants_manifest(graph: Mapping[str, Any]) -> dict[str, Any]:
    """`encoded_constants.json` with the reference's summary block (src/dinoml/compiler.py:847-900)."""
    entries, logical, encoded = [], 0, 0
    for c in graph["constants"]:
        st = c.get("storage")
        if not st or st.get("kind") != "gguf":
            continue
        numel = 1
        for d in c["shape"]:
            numel *= d
        lb = numel * {"float16": 2, "bfloat16": 2, "float32": 4}[c["dtype"]]
        logical += lb
        encoded += c["nbytes"]
        entries.append({"name": c["name"], "dtype": c["dtype"], "shape": c["shape"], "offset": c["offset"], "nbytes": c["nbytes"],
                        "logical_nbytes": lb, "storage": st, "runtime_status": "runtime_supported"})
    return {"schema_version": 1, "constants": entries,
            "summary": {"constant_count": len(entries), "logical_nbytes": logical, "encoded_nbytes": encoded,
                        "runtime_supported_count": len(entries)}}


def compile(spec: ModelSpec, target: Target | None = None, out: str | os.PathLike = "artifact", *, profile: bool = False,
            execution_plan: Mapping[str, Any] | str | os.PathLike | None = None, constant_load_policy: str = "eager",
            profile_options: Mapping[str, Any] | None = None) -> Artifact:
    target = target or Target()
    if constant_load_policy not in ("eager", "deferred"):
        raise ValueError("constant_load_policy must be 'eager' or 'deferred'")
    out = Path(out)
    out.mkdir(parents=True, exist_ok=True)
    graph = spec.graph
    manifest = mf.build_kernel_manifest(graph, target.as_dict())

    size = max((c["offset"] + c["nbytes"] for c in graph["constants"]), default=0)
    with open(out / "constants.bin", "wb") as f:
        f.truncate(size)
        for c in graph["constants"]:
            f.seek(c["offset"])
            f.write(spec.constant_arrays[c["name"]].tobytes())

    if isinstance(execution_plan, (str, os.PathLike)):
        execution_plan = json.loads(Path(execution_plan).read_text())

    def write_all(man):
        (out / "graph.dinoir.json").write_text(json.dumps(graph, indent=1))
        (out / "kernel_manifest.json").write_text(json.dumps(man, indent=1))
        (out / "kernel_codegen_plan.json").write_text(json.dumps({
            "schema_version": 1, "strategy": man["codegen_strategy"],
            "support_libraries": [{"name": "b200_gguf_native", "library": "libdinoml_b200_gguf.so", "kind": "shared",
                                   "arch": target.arch, "kernel_abi_version": mf.KERNEL_ABI_VERSION}]}, indent=1))
        (out / "encoded_constants.json").write_text(json.dumps(encoded_constants_manifest(graph), indent=1))
        (out / "module_plan.txt").write_text(render_module_plan(graph, man))
        meta = {"name": graph["name"], "runtime_abi_version": RUNTIME_ABI_VERSION, "target": target.as_dict(),
                "inputs": graph["inputs"], "outputs": graph["outputs"], "constants": graph["constants"],
                "constant_load_policy": constant_load_policy, "kernel_manifest_cache_key": man["cache_key"]}
        (out / "metadata.json").write_text(json.dumps(meta, indent=1))
        (out / "manifest.json").write_text(json.dumps({"schema_version": 1, "runtime_abi_version": RUNTIME_ABI_VERSION,
                                                       "target": target.as_dict(), "module": "module.so",
                                                       "constants": "constants.bin", "metadata": "metadata.json"}, indent=1))

    write_all(manifest)
    module = out / "module.so"
    if module.exists() or module.is_symlink():
        module.unlink()
    try:
        os.symlink(os.path.relpath(_native.LIB_PATH, out), module)
    except OSError:
        shutil.copy2(_native.LIB_PATH, module)

    if profile and execution_plan is None:
        from . import profiling
        report = profiling.profile_artifact(out, **dict(profile_options or {}))
        execution_plan = profiling.build_execution_plan(report)
        (out / "debug").mkdir(exist_ok=True)
        (out / "debug" / "profile_report.json").write_text(json.dumps(report, indent=1))
    if execution_plan is not None:
        manifest = mf.apply_execution_plan(manifest, execution_plan)
        (out / "debug").mkdir(exist_ok=True)
        (out / "debug" / "execution_plan.json").write_text(json.dumps(execution_plan, indent=1))
        write_all(manifest)
    return Artifact(out)
