"""Kernel manifest for GGUF quantized linears: provider `b200_gguf_gemm`, its candidate catalogue, the
per-node `gguf_direct` plan and the execution-plan overlay.

Schema follows the reference so its tooling reads the same keys: a required-kernel item like
src/dinoml/kernels/manifest.py:265-321, candidates like src/dinoml/kernels/providers/cutlass/gemm.py:
517-554 (the `cutlass{...}` tuning block is replaced by a `b200{...}` block), the plan object like
`_gguf_runtime_dequant_gemm_rhs_plan` (src/dinoml/kernels/manifest.py:754-817) and `apply_execution_plan`
like src/dinoml/kernels/manifest.py:1034-1131.  What changes: kind is `gguf_direct_dequantize_in_kernel`,
there is no dequantization scratch and so no `session_resources` entry of that kind, bfloat16 is
admitted, and the quantization type is part of every cache key."""
from __future__ import annotations

import hashlib
import json
from typing import Any, Mapping

from .constant_sources import GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL, validate_gguf_constant_policy
from .gguf_blocks import qtype_of

KERNEL_LIBRARY = "b200_gguf_gemm"
KERNEL_MANIFEST_SCHEMA_VERSION = 4
KERNEL_ABI_VERSION = 1
PROFILE_CACHE_SCHEMA_VERSION = 9
EXECUTION_PLAN_KERNEL_LIBRARIES = (KERNEL_LIBRARY,)          # src/dinoml/kernels/manifest.py:98-105
DUAL_OPS = ("dual_gemm_rcr_silu", "dual_gemm_rcr_fast_gelu", "dual_gemm_rcr_bias_silu", "dual_gemm_rcr_bias_fast_gelu")
SUPPORTED_OPS = ("gemm_rcr", "gemm_rcr_bias") + DUAL_OPS
VARIANT_CODES = {"simt": 1, "mma": 2, "umma": 3, "stream": 4}
# Tuning configurations of the persistent GEMV (csrc/gemv_stream.cu): each is a candidate of its own, as the tile / stage /
# warp entries of the reference's CUTLASS catalogue are (src/dinoml/kernels/providers/cutlass/gemm.py:19-127).
STREAM_CONFIGS = {1: {"consumer_warps": 8, "ring_slots": {"Q4_K": 5, "Q6_K": 4, "Q5_K": 4, "Q4_0": 5, "MXFP4": 5, "NVFP4": 5, "Q2_K": 5, "Q3_K": 5}, "ctas_per_sm": 1},
                  2: {"consumer_warps": 16, "ring_slots": {"Q4_K": 6, "Q6_K": 4, "Q5_K": 4, "Q4_0": 6, "MXFP4": 6, "NVFP4": 6, "Q2_K": 6, "Q3_K": 6}, "ctas_per_sm": 1},
                  3: {"consumer_warps": 16, "ring_slots": {"Q4_K": 8, "Q6_K": 6, "Q5_K": 6, "Q4_0": 8, "MXFP4": 8, "NVFP4": 8, "Q2_K": 8, "Q3_K": 8}, "ctas_per_sm": 1},
                  4: {"consumer_warps": 8, "ring_slots": {"Q4_K": 4, "Q6_K": 3, "Q5_K": 3, "Q4_0": 4, "MXFP4": 4, "NVFP4": 4, "Q2_K": 4, "Q3_K": 4}, "ctas_per_sm": 2}}
STREAM_QTYPES = ("Q4_K", "Q6_K", "Q5_K", "Q4_0", "MXFP4", "NVFP4", "Q2_K", "Q3_K")
# further types the tcgen05 GEMM unpacks (besides Q4_K, Q6_K, Q8_0); MXFP4 and NVFP4 become exact 16-bit operands
UMMA_MORE_QTYPES = ("Q5_K", "Q4_0", "MXFP4", "NVFP4", "Q2_K", "Q3_K")

_B200_TUNING = {
    "simt": {"kind": "gemv_simt", "rows_per_warp": 1, "activation_rows_per_pass": 4, "staging": "ldg", "tensor_cores": "none"},
    "mma": {"kind": "gemv", "rows_per_cta": 16, "stage_super_blocks": 4, "stages": [3, 4, 6], "staging": "cp_async16",
            "k_slices": "cluster_dsmem for m > 2", "tensor_cores": "mma.sync.m16n8k16", "max_m": 16},
    "stream": {"kind": "gemv_persistent", "rows_per_tile": 16, "stage_super_blocks": 8, "staging": "cp.async.bulk + mbarrier ring",
               "work_split": "contiguous 16-row tiles per CTA", "tensor_cores": "mma.sync.m16n8k16", "max_m": 8},
    "umma": {"kind": "umma_gemm", "tile_n": 128, "tile_m": [64, 128, 256], "tile_k": 64, "stages": 4, "staging": "tma",
             "tensor_cores": "tcgen05.mma.cta_group::1.kind::f16", "weight_operand": "tmem", "accumulator": "tmem",
             "work_split": "stream_k", "min_m": 9},
}


def canonical_json(obj: Any) -> str:
    return json.dumps(obj, sort_keys=True, separators=(",", ":"))


def sha256_of(obj: Any) -> str:
    return hashlib.sha256(canonical_json(obj).encode("utf-8")).hexdigest()


def candidate_variants(qtype: str, dtype: str) -> list[str]:
    """Which kernel variants exist for a (qtype, dtype)."""
    variants = ["simt"]
    if dtype in ("float16", "bfloat16"):
        if qtype in ("Q4_K", "Q6_K", "Q8_0"):
            variants.append("mma")
            variants.append("umma")
        elif qtype in UMMA_MORE_QTYPES:             # the further types: tcgen05 GEMM and persistent GEMV, no tile GEMV
            variants.append("umma")
        if qtype in STREAM_QTYPES:
            variants += [f"stream:{c}" for c in sorted(STREAM_CONFIGS)]
    return variants


def variant_code(variant: str) -> int:
    """"stream:4" -> family code | configuration << 8 (the C ABI's variant argument)."""
    family, _, config = variant.partition(":")
    return VARIANT_CODES[family] | (int(config) << 8 if config else 0)


def variant_supports(variant: str, m: int, *, qtype: str | None = None, dtype: str | None = None, n: int | None = None,
                     k: int | None = None) -> bool:
    """Does the variant serve the problem?  With the full problem given this is the library's own predicate
    (dinoml_b200_gguf_variant_supports: M range, K multiples, row-pitch alignment per qtype); with M alone, the M range."""
    family = variant.partition(":")[0]
    if None not in (qtype, dtype, n, k):
        from . import _native
        return bool(_native.lib().dinoml_b200_gguf_variant_supports(VARIANT_CODES[family], qtype_of(qtype).value, _native.DINO_DTYPE[dtype],
                                                                    int(m), int(n), int(k)))
    return {"simt": True, "mma": 1 <= m <= 16, "umma": m >= 9, "stream": 1 <= m <= 8}[family]


def kernel_symbol(qtype: str, op: str, dtype: str, variant: str, *, profile: bool = False) -> str:
    q = qtype_of(qtype)
    return f"dinoml_{'profile_' if profile else ''}b200_gguf_{q.symbol}_{op}_{dtype}_{variant}_v1"


def gguf_candidate(qtype: str, op: str, dtype: str, variant: str) -> dict[str, Any]:
    q = qtype_of(qtype)
    has_bias = op.endswith("_bias")
    dual_act = op[len("dual_gemm_rcr_"):] if op.startswith("dual_gemm_rcr_") else None
    dual_bias = bool(dual_act) and dual_act.startswith("bias_")
    if dual_bias:
        dual_act = dual_act[len("bias_"):]
    family, _, config = variant.partition(":")
    tag = family + (f"_c{config}" if config else "")
    tuning = dict(_B200_TUNING[family])
    if config:
        tuning.update(STREAM_CONFIGS[int(config)], config=int(config))
        tuning["ring_slots"] = tuning["ring_slots"][q.name]
    cand = {
        "candidate_id": f"b200_gguf_{q.symbol}_{dtype}_{tag}_v1",
        "symbol_id": f"{q.symbol}_{tag}_v1",
        "provider": KERNEL_LIBRARY, "family": "gemm", "op": op, "dtype": dtype, "qtype": q.name,
        "layouts": {"a": "row", "b": "column", "c": "row"},
        "epilogue": "linear_combination_bias" if has_bias else "linear_combination",
        "epilogue_config": {"name": "bias" if has_bias else "identity", "inputs": ["bias"] if has_bias else [], "activation": None,
                            "bias_axis": "n" if has_bias else None, "accumulator_dtype": "float32", "output_dtype": dtype,
                            "launch_abi": "gguf_gemm_rcr_bias_v1" if has_bias else "gguf_gemm_rcr_v1"},
        "accumulator_dtype": "float32", "optional": variant != "simt",
        "launch_abi": "gguf_gemm_rcr_bias_v1" if has_bias else "gguf_gemm_rcr_v1",
        "split_k_values": [1], "split_k_default": 1, "supports_split_k": False, "workspace_nbytes": 0,
        "b200": tuning,
        # a tuning configuration has no symbol of its own: it is the generic entry point with its variant code
        "kernel_symbol": "dinoml_b200_gguf_gemm_rcr" if config else kernel_symbol(q.name, op, dtype, family),
        "profiler_symbol": "dinoml_profile_b200_gguf_gemm_rcr" if config else kernel_symbol(q.name, "gemm_rcr", dtype, family, profile=True),
        "variant": variant, "variant_code": variant_code(variant),
    }
    if dual_act:      # one generic entry point (activation and variant are arguments); epilogue named as in the reference
        # names of the reference's epilogues: left_<act>_and_mul / left_bias_<act>_and_mul (kernels/families/dual_gemm.py:93-135)
        epi = f"left_{'bias_' if dual_bias else ''}{dual_act}_and_mul"
        abi = "gguf_dual_gemm_rcr_bias_v1" if dual_bias else "gguf_dual_gemm_rcr_v1"
        cand.update({"family": "dual_gemm", "layouts": {"a": "row", "b0": "column", "b1": "column", "c": "row"},
                     "epilogue": epi, "launch_abi": abi,
                     "kernel_symbol": "dinoml_b200_gguf_dual_gemm_rcr_bias" if dual_bias else "dinoml_b200_gguf_dual_gemm_rcr",
                     "profiler_symbol": None})
        cand["epilogue_config"] = {"name": epi, "inputs": ["bias0", "bias1"] if dual_bias else [], "activation": dual_act,
                                   "bias_axis": "n" if dual_bias else None,
                                   "accumulator_dtype": "float32", "output_dtype": dtype, "launch_abi": abi,
                                   "weight_rows": "interleave_rows8"}
    cand["candidate_config_key"] = sha256_of({k: cand[k] for k in ("provider", "op", "dtype", "qtype", "variant", "b200", "launch_abi")})
    return cand


def gguf_candidate_set(qtype: str, op: str, dtype: str) -> dict[str, Any]:
    cands = [gguf_candidate(qtype, op, dtype, v) for v in candidate_variants(qtype, dtype)]
    set_id = f"{KERNEL_LIBRARY}_{qtype_of(qtype).symbol}_{op}_{dtype}_v1"
    return {"candidate_set_id": set_id, "candidates": cands,
            "candidate_set_key": sha256_of({"id": set_id, "configs": [c["candidate_config_key"] for c in cands]})}


def validate_gguf_direct_admission(node: Mapping[str, Any], const: Mapping[str, Any], target: str) -> None:
    """Counterpart of _validate_gguf_runtime_dequant_admission (src/dinoml/compiler.py:903-972)."""
    storage = const.get("storage") or {}
    if target != "cuda":
        raise NotImplementedError(f"GGUF-encoded constants are only lowered for the cuda target, got {target!r}")
    if node["op"] not in SUPPORTED_OPS:
        raise NotImplementedError(f"GGUF-encoded weights are supported for {SUPPORTED_OPS}, got {node['op']!r}")
    if node["inputs"].index(const["name"]) != 1:
        raise NotImplementedError("a GGUF-encoded constant must be the B (weight) operand of gemm_rcr")
    if const["dtype"] not in ("float16", "float32", "bfloat16"):
        raise NotImplementedError(f"unsupported logical dtype {const['dtype']!r}")
    if storage.get("materialization") != GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL:
        raise NotImplementedError(f"materialization {storage.get('materialization')!r} is not lowered; use "
                                  f"{GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL!r}")
    validate_gguf_constant_policy(storage["materialization"], storage["residency"], require_runtime_supported=True)


def gguf_direct_plan(node: Mapping[str, Any], const: Mapping[str, Any]) -> dict[str, Any]:
    st = const["storage"]
    return {
        "schema_version": 1, "kind": "gguf_direct_dequantize_in_kernel", "status": "lowered_fused_kernel",
        "node_id": node["id"], "op": node["op"], "operand": "b", "constant": const["name"], "storage_kind": "gguf",
        "materialization": st["materialization"], "residency": st["residency"], "qtype": st["qtype"], "qtype_value": st["qtype_value"],
        "encoded_nbytes": st["encoded_nbytes"], "n_per_row": st["n_per_row"], "logical_dtype": const["dtype"],
        "logical_shape": list(const["shape"]), "scratch_nbytes": 0, "dequant_scratch": None, "dense_launcher": None,
    }


def build_kernel_manifest(graph: Mapping[str, Any], target: Mapping[str, Any]) -> dict[str, Any]:
    consts = {c["name"]: c for c in graph["constants"]}
    required = []
    for node in graph["nodes"]:
        if node["op"] not in SUPPORTED_OPS:
            raise NotImplementedError(f"op {node['op']!r} is outside the quantized-linear path")
        weight = consts.get(node["inputs"][1])
        if weight is None or (weight.get("storage") or {}).get("kind") != "gguf":
            raise NotImplementedError(f"node {node['id']}: the weight of {node['op']} must be a GGUF-encoded constant "
                                      "(dense GEMMs are outside this runtime)")
        validate_gguf_direct_admission(node, weight, target["name"])
        qtype, dtype = weight["storage"]["qtype"], weight["dtype"]
        cset = gguf_candidate_set(qtype, node["op"], dtype)
        dual = node["op"] in DUAL_OPS
        if dual:      # only the tensor-core variants have the gated epilogue; selection is the built-in shape guard
            cset = dict(cset, candidates=[c for c in cset["candidates"] if c["variant"] != "simt"])
            if not cset["candidates"]:
                raise NotImplementedError(f"{node['op']} needs a tensor-core variant: {qtype} / {dtype} has none")
        required.append({
            "node_id": node["id"], "op": node["op"], "dtype": dtype, "qtype": qtype,
            "kernel_symbol": ("dinoml_b200_gguf_dual_gemm_rcr_bias" if "_bias_" in node["op"] else "dinoml_b200_gguf_dual_gemm_rcr") if dual
                             else "dinoml_b200_gguf_gemm_rcr", "kernel_library": KERNEL_LIBRARY,
            "profiler_symbol": None if dual else "dinoml_profile_b200_gguf_gemm_rcr", "has_profiler": not dual,
            "support_archive": "libdinoml_b200_gguf.so",
            "selected_candidate_id": None, "selection": "shape_guarded_auto",
            "candidates": cset["candidates"], "candidate_set_id": cset["candidate_set_id"], "candidate_set_key": cset["candidate_set_key"],
            "gguf_direct": gguf_direct_plan(node, weight), "execution_plan_dispatch": [],
        })
    manifest = {"schema_version": KERNEL_MANIFEST_SCHEMA_VERSION, "kernel_abi_version": KERNEL_ABI_VERSION,
                "profile_cache_schema_version": PROFILE_CACHE_SCHEMA_VERSION, "target": dict(target), "required_kernels": required,
                "codegen_strategy": "interpreted_launch_plan", "profiler_strategy": "native_candidate_timer", "session_resources": []}
    manifest["cache_key"] = sha256_of(manifest)
    return manifest


def apply_execution_plan(manifest: Mapping[str, Any], plan: Mapping[str, Any]) -> dict[str, Any]:
    """Overlays profiled selections: one static candidate per node when every profiled shape agreed, else a guarded
    per-shape dispatch list (src/dinoml/kernels/manifest.py:1086-1116)."""
    out = json.loads(json.dumps(manifest))
    if plan.get("kind") != "dinoml.execution_plan":
        raise ValueError("not an execution plan")
    by_node: dict[str, list[dict[str, Any]]] = {}
    for sel in plan.get("selections", []):
        if sel.get("kernel_library") in EXECUTION_PLAN_KERNEL_LIBRARIES:
            by_node.setdefault(sel["node_id"], []).append(sel)
    for item in out["required_kernels"]:
        sels = by_node.get(item["node_id"], [])
        valid = {c["candidate_id"]: c for c in item["candidates"]}
        sels = [s for s in sels if s["selected_candidate_id"] in valid and s["candidate_set_key"] == item["candidate_set_key"]]
        if not sels:
            continue
        chosen = {s["selected_candidate_id"] for s in sels}
        if len(chosen) == 1:
            item["selected_candidate_id"] = next(iter(chosen))
            item["execution_plan_selection"] = "static"
        item["execution_plan_dispatch"] = [
            {"m": s["shape"]["m"], "n": s["shape"]["n"], "k": s["shape"]["k"], "candidate_id": s["selected_candidate_id"],
             "variant": valid[s["selected_candidate_id"]]["variant"], "variant_code": valid[s["selected_candidate_id"]]["variant_code"],
             "confident": bool(s.get("confidence", {}).get("confident", False))} for s in sels]
    out["execution_plan_key"] = plan.get("execution_plan_key")
    out.pop("cache_key", None)
    out["cache_key"] = sha256_of(out)
    return out
