"""CPU tests of the host-side mirror of the reference API: descriptors and policies, GGUF container reader,
tracing, kernel manifest, launch-plan text, execution-plan logic, and the native module loader's parsing /
error paths (no kernel is launched)."""
import ctypes
import json

import numpy as np
import pytest

import dinoml_v2_b200 as dml
from dinoml_v2_b200 import constant_sources as cs
from dinoml_v2_b200 import gguf_file, manifest as mf, profiling, synthetic as S
from dinoml_v2_b200.compiler import render_module_plan


def _linear_spec(tmp_path, qtype="Q4_K", n=64, k=512, dtype="bfloat16", bias=True, dynamic=True, residency=cs.GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD):
    blocks = S.random_blocks(qtype, n, k, 1)
    path = tmp_path / "w.gguf"
    gguf_file.write_gguf(path, {"blk.0.w": (qtype, (n, k), blocks)})
    lin = dml.nn.Linear(k, n, bias=bias, dtype=dtype)
    m = dml.Dim("m", 1, 2048, buckets=(1, 16, 512)) if dynamic else 4
    consts = {"weight": dml.gguf_constant(path, "blk.0.w", residency=residency)}
    if bias:
        consts["bias"] = np.arange(n, dtype=np.float32)
    return dml.trace(lin, inputs={"x": dml.TensorSpec([m, k], dtype)}, constants=consts), blocks


def test_policy_tables_and_descriptor():
    assert cs.GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL == "direct_dequantize_in_kernel"   # reference name, constant_sources.py:15
    assert cs.GGUF_MATERIALIZATION_POLICIES["direct_dequantize_in_kernel"] == "runtime_supported"
    with pytest.raises(ValueError):
        dml.gguf_constant("x.gguf", "t", materialization="nope")
    with pytest.raises(ValueError):
        dml.gguf_constant("x.gguf", "t", residency="nope")
    c = dml.gguf_constant("x.gguf", "t", qtype="Q4_K", n_per_row=256)
    assert (c.path, c.tensor, c.qtype, c.n_per_row) == ("x.gguf", "t", "Q4_K", 256)
    with pytest.raises(NotImplementedError):
        c.materialize("float16", (1, 256))            # no host dequantizer: refuses instead of falling back
    with pytest.raises(NotImplementedError):
        cs.validate_gguf_constant_policy("dequantize_full_before_launch", "eager_dense_device", require_runtime_supported=True)
    # the host-residency policies the reference only declares (src/dinoml/constant_sources.py:29-33) are implemented here
    for residency in ("cpu_until_first_use", "sequential_offload", "grouped_offload", "manual_runtime_load", "eager_encoded_device"):
        cs.validate_gguf_constant_policy("direct_dequantize_in_kernel", residency, require_runtime_supported=True)
    g = dml.gguf_constant("x.gguf", "t", residency="grouped_offload", offload_group=3)
    assert g.offload_group == 3
    with pytest.raises(ValueError):
        dml.gguf_constant("x.gguf", "t", residency="sequential_offload", offload_group=1)   # group numbers belong to grouped_offload


def test_gguf_file_round_trip_and_hint_validation(tmp_path):
    blocks = {q: S.random_blocks(q, 8, 512, 3) for q in ("Q8_0", "Q4_K", "Q6_K")}
    gguf_file.write_gguf(tmp_path / "m.gguf", {f"t.{q}": (q, (8, 512), b) for q, b in blocks.items()}, {"general.name": "x"})
    with gguf_file.open_gguf(tmp_path / "m.gguf") as f:
        assert f.metadata["general.name"] == "x"
        for q, b in blocks.items():
            info = f.get_tensor(f"t.{q}")
            assert info.shape == (512, 8) and info.qtype == q          # GGUF order is innermost-first
            assert np.array_equal(np.frombuffer(f.read_tensor_bytes(info), np.uint8), b.reshape(-1))
            assert info.data_offset % 32 == 0
        assert f.get_tensor("missing") is None
    mat = cs.materialize_gguf_encoded_constant(dml.gguf_constant(tmp_path / "m.gguf", "t.Q6_K"), "float16", (8, 512))
    assert mat.array.dtype == np.uint8 and mat.array.nbytes == 8 * 2 * 210
    st = mat.storage
    assert (st["kind"], st["qtype"], st["qtype_value"], st["n_per_row"], st["gguf_shape"]) == ("gguf", "Q6_K", 14, 512, [512, 8])
    with pytest.raises(ValueError, match="logical shape"):
        cs.materialize_gguf_encoded_constant(dml.gguf_constant(tmp_path / "m.gguf", "t.Q6_K"), "float16", (512, 8))
    with pytest.raises(ValueError, match="expected qtype"):
        cs.materialize_gguf_encoded_constant(dml.gguf_constant(tmp_path / "m.gguf", "t.Q6_K", qtype="Q4_K"), "float16", (8, 512))
    with pytest.raises(ValueError, match="not found"):
        cs.materialize_gguf_encoded_constant(dml.gguf_constant(tmp_path / "m.gguf", "nope"), "float16", (8, 512))
    # an independent reader (the `gguf` package) sees the same file: names, ggml types, shapes, data offsets and every byte
    gguf = pytest.importorskip("gguf")
    r = gguf.GGUFReader(str(tmp_path / "m.gguf"))
    assert {t.name for t in r.tensors} == {"t.Q8_0", "t.Q4_K", "t.Q6_K"}
    with gguf_file.open_gguf(tmp_path / "m.gguf") as f:
        for t in r.tensors:
            info = f.get_tensor(t.name)
            assert int(t.tensor_type) == info.qtype_value and t.tensor_type.name == info.qtype
            assert tuple(int(d) for d in t.shape) == info.shape                     # both innermost-first
            assert int(t.data_offset) == info.data_offset and int(t.n_bytes) == info.nbytes
            assert np.array_equal(np.asarray(t.data).reshape(-1).view(np.uint8), np.frombuffer(f.read_tensor_bytes(info), np.uint8))


def test_trace_produces_reference_shaped_ir(tmp_path):
    spec, blocks = _linear_spec(tmp_path)
    g = spec.graph
    assert g["nodes"] == [{"id": "n0", "op": "gemm_rcr_bias", "inputs": ["x", "weight", "bias"], "outputs": ["t0"], "attrs": {}}]
    w = spec.constant("weight")
    assert w["shape"] == [64, 512] and w["nbytes"] == blocks.nbytes and w["layout"]["strides"] == [512, 1]
    assert w["storage"]["materialization"] == "direct_dequantize_in_kernel"
    assert np.array_equal(spec.constant_arrays["weight"], blocks.reshape(-1))
    assert spec.constant("bias")["dtype"] == "bfloat16" and spec.constant_arrays["bias"].dtype == np.uint16
    assert g["outputs"][0]["shape_spec"][0]["kind"] == "dynamic" and g["outputs"][0]["shape_spec"][1] == {"kind": "static", "value": 64}


def test_op_shape_and_dtype_checks():
    from dinoml_v2_b200.frontend import GraphBuilder, Tensor
    GraphBuilder._active = GraphBuilder()
    try:
        a, b = Tensor("a", (2, 3, 256), "float16"), Tensor("b", (8, 256), "float16")
        assert dml.ops.gemm_rcr(a, b).shape == (2, 3, 8)
        with pytest.raises(ValueError):
            dml.ops.gemm_rcr(a, Tensor("b", (8, 128), "float16"))
        with pytest.raises(ValueError):
            dml.ops.gemm_rcr(a, Tensor("b", (8, 256), "float32"))
        with pytest.raises(ValueError):
            dml.ops.gemm_rcr_bias(a, b, Tensor("c", (7,), "float16"))
        assert dml.ops.gemm_rcr_bias(a, b, Tensor("c", (1, 8), "float16")).shape == (2, 3, 8)
    finally:
        GraphBuilder._active = None
    with pytest.raises(RuntimeError):
        dml.ops.gemm_rcr(a, b)


def test_kernel_manifest_and_plan_text(tmp_path):
    spec, _ = _linear_spec(tmp_path)
    man = mf.build_kernel_manifest(spec.graph, dml.Target().as_dict())
    item = man["required_kernels"][0]
    assert item["kernel_library"] == "b200_gguf_gemm" and item["qtype"] == "Q4_K" and man["session_resources"] == []
    assert [c["variant"] for c in item["candidates"]] == ["simt", "mma", "umma", "stream:1", "stream:2", "stream:3", "stream:4"]
    tuned = item["candidates"][-1]          # a tuning configuration is a candidate of its own: generic entry + variant code
    assert tuned["variant_code"] == 4 | (4 << 8) and tuned["kernel_symbol"] == "dinoml_b200_gguf_gemm_rcr"
    assert tuned["b200"]["ctas_per_sm"] == 2 and tuned["candidate_id"].endswith("stream_c4_v1")
    assert len({c["candidate_config_key"] for c in item["candidates"]}) == len(item["candidates"])
    for key in ("candidate_id", "symbol_id", "provider", "family", "op", "dtype", "layouts", "epilogue", "accumulator_dtype",
                "launch_abi", "kernel_symbol", "profiler_symbol", "candidate_config_key"):       # providers/cutlass/gemm.py:526-553
        assert key in item["candidates"][0]
    assert item["candidates"][1]["kernel_symbol"] == "dinoml_b200_gguf_q4_k_gemm_rcr_bias_bfloat16_mma_v1"
    plan = item["gguf_direct"]
    assert plan["kind"] == "gguf_direct_dequantize_in_kernel" and plan["scratch_nbytes"] == 0 and plan["n_per_row"] == 512
    # every advertised symbol exists in the library
    from dinoml_v2_b200 import _native
    lib = ctypes.CDLL(str(_native.LIB_PATH))
    for c in item["candidates"]:
        assert hasattr(lib, c["kernel_symbol"]) and hasattr(lib, c["profiler_symbol"])
    text = render_module_plan(spec.graph, man)
    assert "tensor x input 6 2 ?1:2048 512" in text and "constant weight gguf 12 0 18432 64 512 manual_runtime_load" in text
    assert "node gemm_rcr_bias x weight bias t0 0" in text
    # the quantization type separates cache keys of equal (m, n, k)
    k4 = profiling.profile_key(man["target"], "hw", item, item["candidates"][0], {"m": 1, "n": 64, "k": 512})
    item6 = dict(item, qtype="Q6_K")
    assert k4 != profiling.profile_key(man["target"], "hw", item6, item["candidates"][0], {"m": 1, "n": 64, "k": 512})


def test_candidates_of_the_further_types():
    """Every further type of the reference prototype: the CUDA-core kernel, the tcgen05 GEMM and the four configurations of the
    persistent GEMV - no tile GEMV; float32 activations keep the CUDA-core kernel only.  The symbols the candidates name exist."""
    import ctypes

    from dinoml_v2_b200 import _native
    lib = ctypes.CDLL(str(_native.LIB_PATH)) if _native.LIB_PATH.exists() else None
    for q in ("Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4"):
        assert mf.candidate_variants(q, "bfloat16") == ["simt", "umma", "stream:1", "stream:2", "stream:3", "stream:4"]
        assert mf.candidate_variants(q, "float32") == ["simt"]
        for variant in ("simt", "umma", "stream"):
            cand = mf.gguf_candidate(q, "gemm_rcr_bias", "float16", variant)
            assert cand["qtype"] == q and cand["kernel_symbol"].endswith(f"_gemm_rcr_bias_float16_{variant}_v1")
            if lib is not None:
                assert hasattr(lib, cand["kernel_symbol"]), cand["kernel_symbol"]
        tuned = mf.gguf_candidate(q, "gemm_rcr", "bfloat16", "stream:3")
        assert tuned["b200"]["ring_slots"] == (6 if q == "Q5_K" else 8) and tuned["b200"]["consumer_warps"] == 16   # Q5_K stages are 23 KB


def test_admission_rules(tmp_path):
    spec, _ = _linear_spec(tmp_path)
    with pytest.raises(NotImplementedError):
        dml.Target("cpu")
    g = json.loads(json.dumps(spec.graph))
    g["constants"][0]["storage"]["materialization"] = "dequantize_on_gpu_before_launch"
    with pytest.raises(NotImplementedError, match="not lowered"):
        mf.build_kernel_manifest(g, dml.Target().as_dict())
    g = json.loads(json.dumps(spec.graph))
    g["constants"][0]["storage"] = None
    with pytest.raises(NotImplementedError, match="GGUF-encoded"):
        mf.build_kernel_manifest(g, dml.Target().as_dict())


def _fake_report(man, timings):
    item = man["required_kernels"][0]
    results = []
    for (m, variant), (median, stderr) in timings.items():
        cand = next(c for c in item["candidates"] if c["variant"] == variant)
        results.append({"node_id": item["node_id"], "op": item["op"], "dtype": item["dtype"], "qtype": item["qtype"],
                        "candidate_set_id": item["candidate_set_id"], "candidate_set_key": item["candidate_set_key"],
                        "candidate_id": cand["candidate_id"], "candidate_config_key": cand["candidate_config_key"],
                        "kernel_symbol": cand["kernel_symbol"], "profiler_symbol": cand["profiler_symbol"],
                        "kernel_library": mf.KERNEL_LIBRARY, "shape": {"m": m, "n": 64, "k": 512}, "scenario": {"m": m},
                        "iterations": 20, "profile_key": f"k{m}{variant}", "gflops": 1.0, "median_ms": median, "mean_ms": median,
                        "stderr_ms": stderr, "ci95_ms": 1.96 * stderr, "repeats": 5, "samples_ms": [median] * 5})
    return {"schema_version": 1, "kind": "dinoml.profile_report", "target": man["target"],
            "kernel_manifest_cache_key": man["cache_key"], "fingerprint": {}, "hardware_cache_key": "hw", "results": results}


def test_execution_plan_selection_confidence_and_overlay(tmp_path):
    spec, _ = _linear_spec(tmp_path)
    man = mf.build_kernel_manifest(spec.graph, dml.Target().as_dict())
    report = _fake_report(man, {(1, "simt"): (0.030, 1e-4), (1, "mma"): (0.010, 1e-4),
                                (16, "simt"): (0.0400, 1e-4), (16, "mma"): (0.0395, 1e-4),      # inside the 2 % margin
                                (512, "simt"): (5.0, 1e-3), (512, "umma"): (0.05, 1e-3)})
    plan = profiling.build_execution_plan(report)
    profiling.validate_execution_plan(plan)
    sel = {s["shape"]["m"]: s for s in plan["selections"]}
    assert sel[1]["selected_candidate_id"].endswith("mma_v1") and sel[1]["confidence"]["confident"]
    assert sel[16]["selected_candidate_id"].endswith("mma_v1") and not sel[16]["confidence"]["confident"]
    assert sel[512]["selected_candidate_id"].endswith("umma_v1")
    assert plan["summary"] == {"selection_count": 3, "low_confidence_count": 1, "static_selection_count": 0, "conflict_count": 1}
    assert plan["selection_policy"] == "lowest_median_elapsed_ms_per_node_shape"
    bad = dict(plan, selections=[])
    with pytest.raises(ValueError):
        profiling.validate_execution_plan(bad)
    man2 = mf.apply_execution_plan(man, plan)
    disp = man2["required_kernels"][0]["execution_plan_dispatch"]
    assert [(d["m"], d["variant"]) for d in disp] == [(1, "mma"), (16, "mma"), (512, "umma")]
    text = render_module_plan(spec.graph, man2)
    assert "dispatch 0 1 64 512 2" in text and "dispatch 0 512 64 512 3" in text
    t = profiling.profile_timing([1.0, 2.0, 3.0])
    assert t["median_ms"] == 2.0 and abs(t["stderr_ms"] - 1.0 / np.sqrt(3)) < 1e-12
    assert profiling.shape_scenarios(spec.graph) == [{"m": 1}, {"m": 16}, {"m": 512}, {"m": 2048}]


def test_profile_cache_round_trip(tmp_path):
    cache = profiling.ProfileCache(tmp_path / "c" / "profiles.sqlite")
    assert cache.get("k", 10, 3) is None
    cache.put("k", 10, 3, {"median_ms": 1.5})
    assert cache.get("k", 10, 3) == {"median_ms": 1.5}
    assert cache.get("k", 20, 3) is None          # a cached entry is reused only if at least as thorough


def test_compile_writes_artifact_and_native_loader_parses_it(tmp_path):
    spec, blocks = _linear_spec(tmp_path)
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / "art")
    names = {p.name for p in art.path.iterdir()}
    assert {"manifest.json", "metadata.json", "graph.dinoir.json", "kernel_manifest.json", "kernel_codegen_plan.json",
            "encoded_constants.json", "constants.bin", "module_plan.txt", "module.so"} <= names
    assert json.loads((art.path / "manifest.json").read_text())["runtime_abi_version"] == 7
    enc = json.loads((art.path / "encoded_constants.json").read_text())
    assert enc["summary"] == {"constant_count": 1, "logical_nbytes": 64 * 512 * 2, "encoded_nbytes": 18432, "runtime_supported_count": 1}
    raw = np.fromfile(art.path / "constants.bin", dtype=np.uint8, count=blocks.nbytes)
    assert np.array_equal(raw, blocks.reshape(-1))
    # deferred load parses the plan without touching the GPU
    lib = ctypes.CDLL(str(art.path / "module.so"))
    lib.dino_module_load_deferred.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.dino_module_get_metadata_json.restype = ctypes.c_char_p
    lib.dino_module_get_metadata_json.argtypes = [ctypes.c_void_p]
    lib.dino_get_last_error.restype = ctypes.c_char_p
    lib.dino_module_free.argtypes = [ctypes.c_void_p]
    h = ctypes.c_void_p()
    assert lib.dino_module_load_deferred(str(art.path).encode(), ctypes.byref(h)) == 0
    assert json.loads(lib.dino_module_get_metadata_json(h))["name"] == "model"
    lib.dino_module_free(h)
    # error paths: missing directory, corrupt plan
    assert lib.dino_module_load_deferred(str(tmp_path / "nope").encode(), ctypes.byref(h)) != 0
    assert b"cannot open" in lib.dino_get_last_error()
    (art.path / "module_plan.txt").write_text("dinoml_b200_module_plan 1\nconstant w gguf 12 0 100 64 512 manual_runtime_load\n")
    assert lib.dino_module_load_deferred(str(art.path).encode(), ctypes.byref(h)) != 0
    assert b"encoded_nbytes does not match" in lib.dino_get_last_error()


def test_dual_gemm_trace_fuses_the_two_weights_and_compiles(tmp_path):
    """dml.ops.dual_gemm_rcr_silu on two GGUF weights: the traced node reads ONE constant with the rows interleaved in
    groups of 8, the sources leave the artifact, manifest and launch plan name the gated kernel entry."""
    n, k = 16, 256
    b0, b1 = S.random_blocks("Q4_K", n, k, 1), S.random_blocks("Q4_K", n, k, 2)

    class Gate(dml.Module):
        def __init__(self):
            self.w_gate = dml.Parameter([n, k], dtype="bfloat16")
            self.w_up = dml.Parameter([n, k], dtype="bfloat16")

        def forward(self, x):
            return dml.ops.dual_gemm_rcr_silu(x, self.w_gate, self.w_up)

    consts = {"w_gate": cs.GGUFConstant.from_blocks(b0, "Q4_K", (n, k), tensor="gate"),
              "w_up": cs.GGUFConstant.from_blocks(b1, "Q4_K", (n, k), tensor="up")}
    spec = dml.trace(Gate(), inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 8), k], "bfloat16")}, constants=consts)
    node = spec.graph["nodes"][0]
    assert node["op"] == "dual_gemm_rcr_silu" and node["inputs"] == ["x", "w_gate+w_up.rows8"] and node["attrs"]["sources"] == ["w_gate", "w_up"]
    assert [c["name"] for c in spec.graph["constants"]] == ["w_gate+w_up.rows8"]
    fused = spec.constant_arrays["w_gate+w_up.rows8"].reshape(2 * n, -1)
    assert np.array_equal(fused[0:8], b0[0:8]) and np.array_equal(fused[8:16], b1[0:8]) and np.array_equal(fused[16:24], b0[8:16])
    c = spec.graph["constants"][0]
    assert c["shape"] == [2 * n, k] and c["storage"]["derived"]["kind"] == "interleave_rows8" and c["nbytes"] == 2 * b0.nbytes
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / "art")
    item = json.loads((art.path / "kernel_manifest.json").read_text())["required_kernels"][0]
    assert item["kernel_symbol"] == "dinoml_b200_gguf_dual_gemm_rcr" and not item["has_profiler"]
    assert [cand["variant"] for cand in item["candidates"]] == ["mma", "umma", "stream:1", "stream:2", "stream:3", "stream:4"]
    assert item["candidates"][0]["epilogue"] == "left_silu_and_mul"
    plan = (art.path / "module_plan.txt").read_text()
    assert "node dual_gemm_rcr_silu x w_gate+w_up.rows8 - t0 0" in plan
    # mismatched weights are refused at trace time
    consts["w_up"] = cs.GGUFConstant.from_blocks(S.random_blocks("Q6_K", n, k, 3), "Q6_K", (n, k), tensor="up")
    with pytest.raises(NotImplementedError):
        dml.trace(Gate(), inputs={"x": dml.TensorSpec([1, k], "bfloat16")}, constants=consts)


def test_dual_gemm_bias_and_b1_broadcast_trace(tmp_path):
    """dual_gemm_rcr_bias_fast_gelu with B1 [1, K] and bias1 [1] (the reference's broadcast form): the one row and the one bias
    value are repeated when the interleaved constants are built; the plan names the fused bias."""
    n, k = 16, 256
    b0, b1 = S.random_blocks("Q4_K", n, k, 1), S.random_blocks("Q4_K", 1, k, 2)
    bias0, bias1 = np.arange(n, dtype=np.float32), np.array([5.0], dtype=np.float32)

    class Gate(dml.Module):
        def __init__(self):
            self.w_gate = dml.Parameter([n, k], dtype="bfloat16")
            self.w_up = dml.Parameter([1, k], dtype="bfloat16")
            self.b_gate = dml.Parameter([n], dtype="bfloat16")
            self.b_up = dml.Parameter([1], dtype="bfloat16")

        def forward(self, x):
            return dml.ops.dual_gemm_rcr_bias_fast_gelu(x, self.w_gate, self.w_up, self.b_gate, self.b_up)

    consts = {"w_gate": cs.GGUFConstant.from_blocks(b0, "Q4_K", (n, k), tensor="gate"),
              "w_up": cs.GGUFConstant.from_blocks(b1, "Q4_K", (1, k), tensor="up"), "b_gate": bias0, "b_up": bias1}
    spec = dml.trace(Gate(), inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 8), k], "bfloat16")}, constants=consts)
    node = spec.graph["nodes"][0]
    assert node["op"] == "dual_gemm_rcr_bias_fast_gelu" and node["inputs"] == ["x", "w_gate+w_up.rows8", "b_gate+b_up.rows8"]
    fused = spec.constant_arrays["w_gate+w_up.rows8"].reshape(2 * n, -1)
    assert np.array_equal(fused[0:8], b0[0:8]) and all(np.array_equal(fused[8 + i], b1[0]) for i in range(8)) and np.array_equal(fused[16:24], b0[8:16])
    fb = S.bf16_bits_to_float32(np.asarray(spec.constant_arrays["b_gate+b_up.rows8"]).reshape(-1))
    assert fb.tolist() == [0, 1, 2, 3, 4, 5, 6, 7] + [5.0] * 8 + [8, 9, 10, 11, 12, 13, 14, 15] + [5.0] * 8
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / "art")
    item = json.loads((art.path / "kernel_manifest.json").read_text())["required_kernels"][0]
    assert item["kernel_symbol"] == "dinoml_b200_gguf_dual_gemm_rcr_bias"
    assert item["candidates"][0]["epilogue"] == "left_bias_fast_gelu_and_mul" and item["candidates"][0]["epilogue_config"]["inputs"] == ["bias0", "bias1"]
    assert "node dual_gemm_rcr_bias_fast_gelu x w_gate+w_up.rows8 b_gate+b_up.rows8 t0 0" in (art.path / "module_plan.txt").read_text()
    with pytest.raises(ValueError):
        dml.trace(Gate(), inputs={"x": dml.TensorSpec([1, k], "bfloat16")}, constants=dict(consts, b_up=np.zeros(3, dtype=np.float32)))


def test_variant_predicate_is_the_librarys_own():
    """Candidates are filtered with the native predicate for the whole problem, not by M alone (a Q8_0 weight whose K is a
    multiple of 32 but not of 256 has no tensor-core variant; Q6_K rows must be 16-byte multiples for the tcgen05 kernel)."""
    assert mf.variant_supports("umma", 32)                                             # M range only
    assert not mf.variant_supports("umma", 32, qtype="Q8_0", dtype="bfloat16", n=64, k=288)
    assert mf.variant_supports("umma", 32, qtype="Q8_0", dtype="bfloat16", n=64, k=512)
    assert not mf.variant_supports("umma", 32, qtype="Q6_K", dtype="bfloat16", n=64, k=1024)
    assert mf.variant_supports("stream:4", 8, qtype="Q4_K", dtype="float16", n=64, k=512)
    assert not mf.variant_supports("stream:4", 9, qtype="Q4_K", dtype="float16", n=64, k=512)
    assert not mf.variant_supports("mma", 4, qtype="Q4_K", dtype="float32", n=64, k=512)
    assert mf.variant_code("stream:3") == 4 | (3 << 8) and mf.variant_code("umma") == 3
