"""GPU tests of the artifact / session path: compile -> load -> upload encoded constants -> run, against the oracle."""
import json
import os
from pathlib import Path

import numpy as np
import pytest
import torch

import dinoml_v2_b200 as dml
import oracle
from dinoml_v2_b200 import gguf_file, profiling, synthetic as S

pytestmark = pytest.mark.gpu


def _artifact(tmp_path, qtype, n, k, dtype="bfloat16", bias=False, buckets=(1, 16, 64), max_m=64):
    blocks = S.random_blocks(qtype, n, k, 7)
    gguf_file.write_gguf(tmp_path / "w.gguf", {"w": (qtype, (n, k), blocks)})
    lin = dml.nn.Linear(k, n, bias=bias, dtype=dtype)
    consts = {"weight": dml.gguf_constant(tmp_path / "w.gguf", "w")}
    bias_v = None
    if bias:
        bias_v = np.random.default_rng(3).standard_normal(n).astype(np.float32)
        consts["bias"] = bias_v
    spec = dml.trace(lin, inputs={"x": dml.TensorSpec([dml.Dim("m", 1, max_m, buckets=buckets), k], dtype)}, constants=consts)
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / "art")
    return art, blocks, bias_v


@pytest.mark.parametrize("qtype", ["Q4_K", "Q6_K", "Q8_0", "Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4"])
def test_session_run_numpy_matches_oracle(tmp_path, qtype):
    n, k = 96, 1024
    art, blocks, bias = _artifact(tmp_path, qtype, n, k, bias=True)
    mod = dml.runtime.load(art.path)
    sess = mod.create_session()
    x = S.random_activations(3, k, 11, "float32")
    with pytest.raises(RuntimeError, match="not loaded"):
        sess.run_numpy({"x": x})                       # manual_runtime_load: encoded bytes must be uploaded first
    plan = mod.load_encoded_constants()
    assert [p["name"] for p in plan] == ["weight"] and plan[0]["action"] == "upload_encoded"
    for m in (1, 3, 40):
        x = S.random_activations(m, k, 11 + m, "float32")
        xb = S.bf16_bits_to_float32(S.float32_to_bf16_bits(x))
        y = sess.run_numpy({"x": x})["t0"]
        bias_b = S.bf16_bits_to_float32(S.float32_to_bf16_bits(bias))
        ref = oracle.gemm_quant(xb, blocks, qtype, n, k) + bias_b
        _, _, norm = oracle.max_errors(ref, y)
        assert y.shape == (m, n) and norm <= 2e-2, (qtype, m, norm)
    with pytest.raises(RuntimeError, match="outside"):
        sess.run_numpy({"x": S.random_activations(65, k, 1, "float32")})      # beyond Dim max
    with pytest.raises(RuntimeError, match="exactly"):
        mod.set_encoded_constant_host_bytes("weight", np.zeros(10, np.uint8))
    sess.close()
    mod.close()


@pytest.mark.parametrize("dtype", ["float16", "float32"])
def test_session_run_numpy_other_dtypes_and_shape_changes(tmp_path, dtype):
    """float16 / float32 modules keep their numpy dtypes; a new input shape gets its own cached arenas; a stream the
    caller set stays in place after run_numpy."""
    n, k = 80, 512
    art, blocks, _ = _artifact(tmp_path, "Q4_K", n, k, dtype=dtype)
    mod = dml.runtime.load(art.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    stream = torch.cuda.Stream()
    sess.set_stream(stream.cuda_stream)
    for m in (1, 5, 1, 33):
        x = S.random_activations(m, k, 40 + m, dtype)
        y = sess.run_numpy({"x": x})["t0"]
        assert y.dtype == np.dtype(dtype) and y.shape == (m, n)
        ref = oracle.gemm_quant(x.astype(np.float32), blocks, "Q4_K", n, k)
        _, _, norm = oracle.max_errors(ref, y.astype(np.float32))
        assert norm <= (2e-2 if dtype == "float16" else 1e-4), (dtype, m, norm)
    assert len(sess._numpy_plans) == 3 and sess._user_stream == stream.cuda_stream
    # the result does not alias the pinned arena: a second call must not change the first result
    a = sess.run_numpy({"x": S.random_activations(1, k, 1, dtype)})["t0"]
    keep = a.copy()
    sess.run_numpy({"x": S.random_activations(1, k, 2, dtype)})
    assert np.array_equal(a, keep)
    mod.close()


@pytest.mark.parametrize("activation", ["silu", "fast_gelu"])
def test_session_dual_gemm_matches_oracle(tmp_path, activation):
    """dual_gemm_rcr_<act> on two GGUF weights through compile -> load -> run, decode and prefill sizes."""
    from dinoml_v2_b200.constant_sources import GGUFConstant
    n, k = 136, 2048
    b0, b1 = S.random_blocks("Q6_K", n, k, 21), S.random_blocks("Q6_K", n, k, 22)
    op = getattr(dml.ops, f"dual_gemm_rcr_{activation}")

    class Gate(dml.Module):
        def __init__(self):
            self.w_gate = dml.Parameter([n, k], dtype="bfloat16")
            self.w_up = dml.Parameter([n, k], dtype="bfloat16")

        def forward(self, x):
            return op(x, self.w_gate, self.w_up)

    spec = dml.trace(Gate(), inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 64), k], "bfloat16")},
                     constants={"w_gate": GGUFConstant.from_blocks(b0, "Q6_K", (n, k), tensor="gate"),
                                "w_up": GGUFConstant.from_blocks(b1, "Q6_K", (n, k), tensor="up")})
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / "art")
    mod = dml.runtime.load(art.path)
    plan = mod.load_encoded_constants()
    assert [p["name"] for p in plan] == ["w_gate+w_up.rows8"]
    sess = mod.create_session()
    for m in (1, 7, 48):
        x = S.random_activations(m, k, 30 + m, "float32")
        xb = S.bf16_bits_to_float32(S.float32_to_bf16_bits(x))
        y = sess.run_numpy({"x": x})["t0"]
        ref = oracle.dual_gemm_quant(xb, b0, b1, "Q6_K", n, k, activation)
        _, _, norm = oracle.max_errors(ref, y)
        assert y.shape == (m, n) and norm <= 2e-2, (activation, m, norm)
    mod.close()


def test_session_dual_gemm_bias_broadcast_matches_oracle(tmp_path):
    """dual_gemm_rcr_bias_silu with B1 [1, K] / bias1 [1] through compile -> load -> run."""
    from dinoml_v2_b200.constant_sources import GGUFConstant
    n, k = 72, 1024
    b0, b1 = S.random_blocks("Q4_K", n, k, 41), S.random_blocks("Q4_K", 1, k, 42)
    bias0 = np.linspace(-2, 2, n).astype(np.float32)
    bias1 = np.array([0.5], dtype=np.float32)

    class Gate(dml.Module):
        def __init__(self):
            self.w_gate = dml.Parameter([n, k], dtype="bfloat16")
            self.w_up = dml.Parameter([1, k], dtype="bfloat16")
            self.b_gate = dml.Parameter([n], dtype="bfloat16")
            self.b_up = dml.Parameter([1], dtype="bfloat16")

        def forward(self, x):
            return dml.ops.dual_gemm_rcr_bias_silu(x, self.w_gate, self.w_up, self.b_gate, self.b_up)

    spec = dml.trace(Gate(), inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 64), k], "bfloat16")},
                     constants={"w_gate": GGUFConstant.from_blocks(b0, "Q4_K", (n, k), tensor="gate"),
                                "w_up": GGUFConstant.from_blocks(b1, "Q4_K", (1, k), tensor="up"), "b_gate": bias0, "b_up": bias1})
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / "art")
    mod = dml.runtime.load(art.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    rb = lambda v: S.bf16_bits_to_float32(S.float32_to_bf16_bits(v))
    for m in (1, 5, 33):
        x = S.random_activations(m, k, 50 + m, "float32")
        y = sess.run_numpy({"x": x})["t0"]
        ref = oracle.dual_gemm_quant(rb(x), b0, b1, "Q4_K", n, k, "silu", rb(bias0), rb(bias1))
        _, _, norm = oracle.max_errors(ref, y)
        assert y.shape == (m, n) and norm <= 2e-2, (m, norm)
    mod.close()


def test_session_benchmark_and_external_stream(tmp_path):
    n, k = 256, 1024
    art, blocks, _ = _artifact(tmp_path, "Q4_K", n, k)
    mod = dml.runtime.load(art.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    x = torch.randn(1, k, device="cuda", dtype=torch.bfloat16)
    summary = sess.benchmark_torch({"x": x}, warmup=3, iterations=5)
    assert summary["iterations"] == 5 and summary["min_ms"] > 0 and summary["graph_replay"]
    stream = torch.cuda.Stream()
    sess.set_stream(stream.cuda_stream)
    y = sess.run_torch({"x": x})["t0"]
    stream.synchronize()
    ref = oracle.gemm_quant(x.float().cpu().numpy(), blocks, "Q4_K", n, k)
    _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
    assert norm <= 2e-2
    sess.set_stream(None)
    mod.close()


def test_profile_then_execution_plan_dispatch(tmp_path):
    n, k = 512, 1024
    art, blocks, _ = _artifact(tmp_path, "Q4_K", n, k, buckets=(1, 32))
    cache = profiling.ProfileCache(tmp_path / "cache" / "p.sqlite")
    report = profiling.profile_artifact(art.path, iterations=5, repeats=3, cache=cache)
    assert {r["shape"]["m"] for r in report["results"]} == {1, 32, 64}
    plan = profiling.build_execution_plan(report)
    sel = {s["shape"]["m"]: s["selected_candidate_id"] for s in plan["selections"]}
    assert ("_stream_c" in sel[1] or sel[1].endswith(("mma_v1", "simt_v1"))) and sel[64].endswith(("umma_v1", "simt_v1"))
    again = profiling.profile_artifact(art.path, iterations=5, repeats=3, cache=cache)      # served from the SQLite cache
    assert [r["median_ms"] for r in again["results"]] == [r["median_ms"] for r in report["results"]]
    # re-compile with the plan: dispatch records reach the native module and results stay correct
    gguf_path = tmp_path / "w.gguf"
    lin = dml.nn.Linear(k, n, bias=False, dtype="bfloat16")
    spec = dml.trace(lin, inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 64, buckets=(1, 32)), k], "bfloat16")},
                     constants={"weight": dml.gguf_constant(gguf_path, "w")})
    art2 = dml.compile(spec, dml.Target("cuda"), tmp_path / "art2", execution_plan=plan)
    assert "dispatch 0 1 512 1024" in (art2.path / "module_plan.txt").read_text()
    mod = dml.runtime.load(art2.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    for m in (1, 32, 64, 5):
        x = S.random_activations(m, k, 20 + m, "float32")
        y = sess.run_numpy({"x": x})["t0"]
        ref = oracle.gemm_quant(S.bf16_bits_to_float32(S.float32_to_bf16_bits(x)), blocks, "Q4_K", n, k)
        _, _, norm = oracle.max_errors(ref, y)
        assert norm <= 2e-2, (m, norm)
    mod.close()


def test_profiled_plan_dispatches_several_tuning_configurations(tmp_path):
    """The benchmark's decode weight (Q4_K [11008 x 4096]) profiled over M buckets 1 .. 2048: the plan ranks the tuning
    configurations of the persistent GEMV next to the other variants per shape, the chosen variant codes (family | config
    << 8) reach the native module as dispatch records, and the dispatched kernels give the oracle's results."""
    n, k = 11008, 4096
    art, blocks, _ = _artifact(tmp_path, "Q4_K", n, k, buckets=(1, 4, 16, 64, 512), max_m=2048)
    report = profiling.profile_artifact(art.path, iterations=10, repeats=3)
    timed = {(r["shape"]["m"], r["candidate_id"]) for r in report["results"]}
    assert any("_stream_c" in cid for (m, cid) in timed if m == 4) and not any("_stream_c" in cid for (m, cid) in timed if m == 16)
    plan = profiling.build_execution_plan(report)
    chosen = {s["shape"]["m"]: s["selected_candidate_id"] for s in plan["selections"]}
    assert set(chosen) == {1, 4, 16, 64, 512, 2048}
    assert len(set(chosen.values())) >= 2 and chosen[2048].endswith("umma_v1")
    gguf_path = tmp_path / "w.gguf"
    lin = dml.nn.Linear(k, n, bias=False, dtype="bfloat16")
    spec = dml.trace(lin, inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 2048, buckets=(1, 4, 16, 64, 512)), k], "bfloat16")},
                     constants={"weight": dml.gguf_constant(gguf_path, "w")})
    art2 = dml.compile(spec, dml.Target("cuda"), tmp_path / "art2", execution_plan=plan)
    text = (art2.path / "module_plan.txt").read_text()
    codes = {int(line.split()[-1]) for line in text.splitlines() if line.startswith("dispatch ")}
    assert len(codes) >= 2 and all((c & 0xff) in (1, 2, 3, 4) for c in codes)
    mod = dml.runtime.load(art2.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    rows = np.r_[0:32, n - 32:n]
    for m in (1, 4, 16):
        x = S.random_activations(m, k, 50 + m, "float32")
        y = sess.run_numpy({"x": x})["t0"]
        ref = oracle.gemm_quant(S.bf16_bits_to_float32(S.float32_to_bf16_bits(x)), blocks[rows], "Q4_K", len(rows), k)
        _, _, norm = oracle.max_errors(ref, y[:, rows])
        assert norm <= 2e-2, (m, norm)
    mod.close()
    out = os.environ.get("DINOML_TEST_REPORT_DIR")
    if out and Path(out).is_dir():                      # keep the selection for whoever asked for reports
        (Path(out) / "plan_cfg2.json").write_text(json.dumps(chosen, indent=1))


def _bank_artifact(tmp_path, residency, count=4, n=192, k=1024, groups=None):
    """`count` independent quantized linears on one input (mixed qtypes), all weights with the given residency."""
    qtypes = ["Q4_K", "Q6_K", "Q8_0", "Q4_K", "Q5_K", "Q4_K"][:count]
    blocks = [S.random_blocks(q, n, k, 70 + i) for i, q in enumerate(qtypes)]

    class Bank(dml.Module):
        def __init__(self):
            for i in range(count):
                setattr(self, f"w{i}", dml.Parameter([n, k], dtype="bfloat16"))

        def forward(self, x):
            return [dml.ops.gemm_rcr(x, getattr(self, f"w{i}")) for i in range(count)]

    consts = {f"w{i}": dml.GGUFConstant.from_blocks(blocks[i], qtypes[i], (n, k), tensor=f"w{i}", residency=residency,
                                                   offload_group=None if groups is None else groups[i]) for i in range(count)}
    spec = dml.trace(Bank(), inputs={"x": dml.TensorSpec([dml.Dim("m", 1, 8), k], "bfloat16")}, constants=consts)
    art = dml.compile(spec, dml.Target("cuda"), tmp_path / f"art_{residency}")
    return art, qtypes, blocks


def _check_bank(sess, qtypes, blocks, m, seed):
    n, k = blocks[0].shape[0], 1024
    x = S.random_activations(m, k, seed, "float32")
    xb = S.bf16_bits_to_float32(S.float32_to_bf16_bits(x))
    out = sess.run_numpy({"x": x})
    names = sorted(out, key=lambda s: int("".join(ch for ch in s if ch.isdigit()) or 0))
    assert len(names) == len(qtypes)
    for name, q, b in zip(names, qtypes, blocks):
        _, _, norm = oracle.max_errors(oracle.gemm_quant(xb, b, q, n, k), out[name])
        assert norm <= 2e-2, (name, q, m, norm)


def test_residency_cpu_until_first_use(tmp_path):
    art, qtypes, blocks = _bank_artifact(tmp_path, "cpu_until_first_use")
    mod = dml.runtime.load(art.path)
    plan = mod.load_encoded_constants()
    assert [p["action"] for p in plan] == ["register_host_resident"] * 4
    total = sum(b.nbytes for b in blocks)
    st = mod.residency_stats()
    assert st["device_resident_bytes"] == 0 and st["pinned_host_bytes"] == total        # nothing on the device before the first run
    sess = mod.create_session()
    _check_bank(sess, qtypes, blocks, 1, 81)
    assert mod.residency_stats()["device_resident_bytes"] == total                      # uploaded on first use, resident from then on
    _check_bank(sess, qtypes, blocks, 5, 82)
    assert mod.residency_stats()["device_resident_bytes"] == total
    mod.close()


def test_residency_sequential_offload(tmp_path):
    art, qtypes, blocks = _bank_artifact(tmp_path, "sequential_offload")
    mod = dml.runtime.load(art.path)
    assert [p["offload_group"] for p in mod.load_encoded_constants()] == [0, 1, 2, 3]
    sess = mod.create_session()
    for run, m in enumerate((1, 3, 8)):
        _check_bank(sess, qtypes, blocks, m, 90 + m)
        st = mod.residency_stats()
        # never resident: two slots of the largest weight hold whatever is in flight; every run streams all four weights
        assert st["device_resident_bytes"] == 0 and st["device_slot_bytes"] >= 2 * max(b.nbytes for b in blocks)
        assert st["device_slot_bytes"] < sum(b.nbytes for b in blocks)
        assert st["uploads"] in (4 * (run + 1), 4 * (run + 1) - 1)      # the weight left in a slot by the last run may be reused
    mod.close()


def test_residency_grouped_offload(tmp_path):
    # explicit groups: {w0, w1} {w2} {w3, w4, w5}; three groups through two slots
    art, qtypes, blocks = _bank_artifact(tmp_path, "grouped_offload", count=6, groups=[0, 0, 1, 2, 2, 2])
    mod = dml.runtime.load(art.path)
    plan = mod.load_encoded_constants()
    assert [p["offload_group"] - (1 << 20) for p in plan] == [0, 0, 1, 2, 2, 2]
    sess = mod.create_session()
    for m in (2, 7):
        _check_bank(sess, qtypes, blocks, m, 100 + m)
    st = mod.residency_stats()
    assert st["device_resident_bytes"] == 0 and st["uploads"] >= 6
    largest = max(sum(-(-b.nbytes // 256) * 256 for b, g in zip(blocks, [0, 0, 1, 2, 2, 2]) if g == gid) for gid in (0, 1, 2))
    assert st["device_slot_bytes"] == 2 * largest
    mod.close()
    # two groups fit the two slots: after the first run nothing is uploaded again
    art2, qtypes2, blocks2 = _bank_artifact(tmp_path / "b", "grouped_offload", count=4)
    mod2 = dml.runtime.load(art2.path)
    mod2.load_encoded_constants()                    # default grouping: two consecutive constants per group
    sess2 = mod2.create_session()
    _check_bank(sess2, qtypes2, blocks2, 1, 111)
    first = mod2.residency_stats()["uploads"]
    _check_bank(sess2, qtypes2, blocks2, 4, 112)
    assert first == 4 and mod2.residency_stats()["uploads"] == 4
    mod2.close()


def test_run_numpy_replays_a_graph_in_steady_state(tmp_path):
    n, k = 256, 1024
    art, blocks, _ = _artifact(tmp_path, "Q4_K", n, k)
    mod = dml.runtime.load(art.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    x = S.random_activations(4, k, 5, "float32")
    outs = [sess.run_numpy({"x": x})["t0"] for _ in range(5)]
    st = sess.graph_stats()
    assert st["cached_graphs"] == 1 and st["graph_launches"] == 4            # first call eager, captured on the second, replayed after
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    ref = oracle.gemm_quant(S.bf16_bits_to_float32(S.float32_to_bf16_bits(x)), blocks, "Q4_K", n, k)
    assert oracle.max_errors(ref, outs[-1])[2] <= 2e-2
    y2 = sess.run_numpy({"x": S.random_activations(9, k, 6, "float32")})["t0"]      # another shape: its own plan and graph
    assert y2.shape == (9, n) and sess.graph_stats()["cached_graphs"] == 1
    sess.numpy_graph_replay = False
    assert np.array_equal(sess.run_numpy({"x": x})["t0"], outs[0]) and sess.graph_stats()["graph_launches"] == 4
    # the benchmark helpers of the reference loader
    s1 = sess.benchmark_numpy({"x": x}, warmup=2, iterations=4)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    yt = torch.empty(4, n, device="cuda", dtype=torch.bfloat16)
    s2 = sess.benchmark_device_pointers({"x": (xt.data_ptr(), (4, k), "bfloat16")}, {"t0": (yt.data_ptr(), (4, n), "bfloat16")}, warmup=2, iterations=4)
    assert s1["iterations"] == 4 and s2["iterations"] == 4 and s1["min_ms"] > 0 and s2["min_ms"] > 0
    mod.close()


def test_profile_run_environment_contract(tmp_path, capfd, monkeypatch):
    art, qtypes, blocks = _bank_artifact(tmp_path, "manual_runtime_load", count=3)
    mod = dml.runtime.load(art.path)
    mod.load_encoded_constants()
    sess = mod.create_session()
    monkeypatch.setenv("DINOML_PROFILE_RUN", "1")
    monkeypatch.setenv("DINOML_PROFILE_RUN_VERBOSE", "1")
    monkeypatch.setenv("DINOML_PROFILE_RUN_SECTIONS", "first_two:0:1,last:2:2")
    _check_bank(sess, qtypes, blocks, 2, 120)
    err = capfd.readouterr().err
    assert "[dinoml_profile] total_gpu_ms=" in err and "[dinoml_profile] op=gemm_rcr count=3" in err
    assert err.count("[dinoml_profile_launch] label=node") == 3
    assert "[dinoml_profile_section] name=first_two start=0 end=1 ms=" in err and "[dinoml_profile_section] name=last start=2 end=2" in err
    monkeypatch.setenv("DINOML_PROFILE_RUN_SECTIONS", "bad:5:9")
    with pytest.raises(RuntimeError, match="did not match"):
        sess.run_numpy({"x": S.random_activations(2, 1024, 1, "float32")})
    mod.close()
