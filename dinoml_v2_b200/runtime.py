"""Python runtime loader: `runtime.load(artifact)` -> RuntimeModule -> Session, over the `dino_*` C ABI with ctypes.

Same surface as the reference loader for this path (src/dinoml/runtime.py): ABI check (:141,160), deferred module
load (:165), `load_constants` (:213-232), `load_encoded_constants` with its load plan (:249-346), H2D staging +
`dino_module_set_encoded_constant` (:660-703), sessions (:209-211, 888-909), `run_numpy` / `run_torch` /
`run_device_pointers` (:942, :1371-1431, :1172-1192) and the native benchmark with its summary
(:966-977, 1311-1369, 1854-1866).  torch is used only to own device buffers and streams."""
from __future__ import annotations

import ctypes
import json
import statistics
import weakref
from pathlib import Path
from typing import Any, Mapping

import numpy as np

from .frontend import DTYPE_ENUM, DTYPE_NBYTES, RUNTIME_ABI_VERSION

DEVICE_CUDA = 1
FLAG_CONTIGUOUS = 1


class _DinoTensor(ctypes.Structure):      # runtime/include/dinoml/abi.h:36-57
    _fields_ = [("data", ctypes.c_void_p), ("shape", ctypes.POINTER(ctypes.c_int64)), ("ndim", ctypes.c_size_t),
                ("dtype", ctypes.c_int), ("strides", ctypes.POINTER(ctypes.c_int64)), ("byte_offset", ctypes.c_size_t),
                ("nbytes", ctypes.c_size_t), ("device_type", ctypes.c_int), ("flags", ctypes.c_uint32),
                ("alignment", ctypes.c_size_t)]


def _configure(lib: ctypes.CDLL) -> None:
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    T = ctypes.POINTER(_DinoTensor)
    lib.dino_abi_version.restype = ci
    lib.dino_get_last_error.restype = ctypes.c_char_p
    for name, args in {
        "dino_module_load": [ctypes.c_char_p, ctypes.POINTER(vp)], "dino_module_load_deferred": [ctypes.c_char_p, ctypes.POINTER(vp)],
        "dino_module_load_constants": [vp, ctypes.c_char_p], "dino_module_unload_constants": [vp],
        "dino_module_set_constant": [vp, ctypes.c_char_p, T], "dino_module_set_encoded_constant": [vp, ctypes.c_char_p, vp, sz],
        "dino_module_free": [vp], "dino_session_create": [vp, ctypes.POINTER(vp)], "dino_session_destroy": [vp],
        "dino_session_set_stream": [vp, vp],
        "dino_session_get_output_shape": [vp, sz, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(sz)],
        "dino_session_run": [vp, T, sz, T, sz],
        "dino_session_benchmark": [vp, T, sz, T, sz, sz, sz, ctypes.POINTER(ctypes.c_double), sz],
        "dino_device_malloc": [ctypes.POINTER(vp), sz], "dino_device_free": [vp], "dino_copy_host_to_device": [vp, vp, sz],
        "dino_module_set_offloaded_encoded_constant": [vp, ctypes.c_char_p, vp, sz, ci],
        "dino_module_get_residency_stats": [vp] + [ctypes.POINTER(sz)] * 5,
        "dino_session_run_staged": [vp, vp, vp, sz, T, sz, T, sz, vp, vp, sz],
        "dino_session_run_staged_on": [vp, vp, ci, vp, vp, sz, T, sz, T, sz, vp, vp, sz],
        "dino_session_set_graph_replay": [vp, ci], "dino_session_get_graph_stats": [vp, ctypes.POINTER(sz), ctypes.POINTER(sz)],
    }.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, ci
    for name in ("dino_convert_f32_to_bf16", "dino_convert_bf16_to_f32"):
        getattr(lib, name).argtypes, getattr(lib, name).restype = [vp, vp, sz], None
    lib.dino_module_get_metadata_json.argtypes = [vp]
    lib.dino_module_get_metadata_json.restype = ctypes.c_char_p


def _tensor_struct(ptr: int, shape, dtype: str, keep: list) -> _DinoTensor:
    arr = (ctypes.c_int64 * len(shape))(*[int(d) for d in shape])
    keep.append(arr)
    numel = 1
    for d in shape:
        numel *= int(d)
    return _DinoTensor(ptr, arr, len(shape), DTYPE_ENUM[dtype], None, 0, numel * DTYPE_NBYTES[dtype], DEVICE_CUDA, FLAG_CONTIGUOUS, 0)


def load(path: str | Path, *, load_constants: bool | None = None) -> "RuntimeModule":
    return RuntimeModule(Path(path), load_constants=load_constants)


class RuntimeModule:
    def __init__(self, path: Path, load_constants: bool | None = None):
        self.path = Path(path)
        manifest = json.loads((self.path / "manifest.json").read_text())
        if manifest.get("runtime_abi_version") != RUNTIME_ABI_VERSION:
            raise RuntimeError(f"artifact ABI {manifest.get('runtime_abi_version')} != runtime ABI {RUNTIME_ABI_VERSION}")
        module_path = self.path / manifest.get("module", "module.so")
        if not module_path.exists():
            raise RuntimeError(f"{module_path} is missing: the CUDA library was not built (there is no CPU fallback)")
        self._lib = ctypes.CDLL(str(module_path))
        _configure(self._lib)
        if self._lib.dino_abi_version() != RUNTIME_ABI_VERSION:
            raise RuntimeError(f"module.so reports ABI {self._lib.dino_abi_version()}, expected {RUNTIME_ABI_VERSION}")
        self._handle = ctypes.c_void_p()
        self._sessions: "weakref.WeakSet[Session]" = weakref.WeakSet()
        self.offload_group_size = 2           # grouped_offload constants that name no group: this many consecutive ones per group
        self._check(self._lib.dino_module_load_deferred(str(self.path).encode(), ctypes.byref(self._handle)))
        try:
            self.metadata = json.loads(self._lib.dino_module_get_metadata_json(self._handle).decode())
            policy = self.metadata.get("constant_load_policy", "eager")
            if load_constants if load_constants is not None else policy == "eager":
                self.load_constants()
        except Exception:
            self.close()
            raise

    # -- errors
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError((self._lib.dino_get_last_error() or b"unknown error").decode("utf-8", "replace"))

    # -- constants
    def load_constants(self, path: str | Path | None = None) -> None:
        """Dense constants and eagerly-resident encoded ones; `manual_runtime_load` GGUF constants are skipped."""
        self._check(self._lib.dino_module_load_constants(self._handle, str(path or self.path / "constants.bin").encode()))

    def unload_constants(self) -> None:
        self._check(self._lib.dino_module_unload_constants(self._handle))

    def encoded_constant_load_plan(self) -> list[dict[str, Any]]:
        plan = []
        for c in self.metadata["constants"]:
            st = c.get("storage") or {}
            if st.get("kind") != "gguf":
                continue
            host = st["residency"] in ("cpu_until_first_use", "sequential_offload", "grouped_offload")
            entry = {"name": c["name"], "qtype": st["qtype"], "encoded_nbytes": c["nbytes"], "offset": c["offset"],
                     "residency": st["residency"], "materialization": st["materialization"],
                     "action": "register_host_resident" if host else "upload_encoded" if st["residency"] == "manual_runtime_load"
                     else "loaded_with_constants", "status": "runtime_supported"}
            if st["residency"] == "sequential_offload":
                entry["offload_group"] = sum(1 for p in plan if p["residency"] == "sequential_offload")      # one constant per group
            elif st["residency"] == "grouped_offload":
                # group numbers of the two policies are kept apart (grouped ones start at 2^20)
                entry["offload_group"] = (1 << 20) + (int(st["offload_group"]) if "offload_group" in st else
                                                      sum(1 for p in plan if p["residency"] == "grouped_offload") // self.offload_group_size)
            plan.append(entry)
        return plan

    def load_encoded_constants(self, sources: Mapping[str, np.ndarray] | None = None) -> list[dict[str, Any]]:
        """Uploads the raw GGUF bytes of every `manual_runtime_load` constant (from `sources`, else from the artifact's
        constants.bin): device malloc, H2D, `dino_module_set_encoded_constant` (device-to-device copy into the module's own
        buffer), free the staging buffer."""
        done = []
        for entry in self.encoded_constant_load_plan():
            if entry["action"] not in ("upload_encoded", "register_host_resident"):
                continue
            if sources is not None and entry["name"] in sources:
                raw = np.ascontiguousarray(sources[entry["name"]], dtype=np.uint8).reshape(-1)
            else:
                raw = np.fromfile(self.path / "constants.bin", dtype=np.uint8, count=entry["encoded_nbytes"], offset=entry["offset"])
            if entry["action"] == "upload_encoded":
                self.set_encoded_constant_host_bytes(entry["name"], raw)
            else:       # host-resident policies: the module keeps a pinned copy and moves the bytes itself at run time
                self._check(self._lib.dino_module_set_offloaded_encoded_constant(self._handle, entry["name"].encode(), raw.ctypes.data,
                                                                                 raw.nbytes, int(entry.get("offload_group", 0))))
            done.append(entry)
        return done

    def residency_stats(self) -> dict[str, int]:
        """Where the encoded constants are right now and how much a run has streamed: bytes resident on the device, bytes
        of the two offload slots, pinned host bytes, host-to-device uploads and their bytes since load."""
        vals = [ctypes.c_size_t() for _ in range(5)]
        self._check(self._lib.dino_module_get_residency_stats(self._handle, *[ctypes.byref(v) for v in vals]))
        keys = ("device_resident_bytes", "device_slot_bytes", "pinned_host_bytes", "uploads", "upload_bytes")
        return {k: int(v.value) for k, v in zip(keys, vals)}

    def set_encoded_constant_host_bytes(self, name: str, raw: np.ndarray) -> None:
        staging = ctypes.c_void_p()
        self._check(self._lib.dino_device_malloc(ctypes.byref(staging), raw.nbytes))
        try:
            self._check(self._lib.dino_copy_host_to_device(staging, raw.ctypes.data, raw.nbytes))
            self._check(self._lib.dino_module_set_encoded_constant(self._handle, name.encode(), staging, raw.nbytes))
        finally:
            self._lib.dino_device_free(staging)

    def set_encoded_constant_device(self, name: str, device_ptr: int, nbytes: int) -> None:
        self._check(self._lib.dino_module_set_encoded_constant(self._handle, name.encode(), ctypes.c_void_p(device_ptr), nbytes))

    def set_constant_torch(self, name: str, tensor) -> None:
        keep: list = []
        dtype = str(tensor.dtype).replace("torch.", "")
        t = _tensor_struct(tensor.data_ptr(), tuple(tensor.shape), dtype, keep)
        self._check(self._lib.dino_module_set_constant(self._handle, name.encode(), ctypes.byref(t)))

    # -- sessions
    def create_session(self) -> "Session":
        s = Session(self)
        self._sessions.add(s)
        return s

    def close(self) -> None:
        for s in list(self._sessions):
            s.close()
        if getattr(self, "_handle", None):
            self._lib.dino_module_free(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Session:
    def __init__(self, module: RuntimeModule):
        self.module = module
        self._lib = module._lib
        self._handle = ctypes.c_void_p()
        module._check(self._lib.dino_session_create(module._handle, ctypes.byref(self._handle)))
        self._pinned: dict[str, Any] = {}
        self._numpy_plans: dict[Any, dict[str, Any]] = {}
        self._user_stream = 0
        self._graph_replay = False
        self.numpy_graph_replay = True        # run_numpy keeps its arenas, so its launch sequences are replayed as CUDA graphs
        self.numpy_zero_copy_bytes = 65536    # run_numpy: results up to this size are stored by the kernels into pinned host memory

    def close(self) -> None:
        if self._handle:
            self._lib.dino_session_destroy(self._handle)
            self._handle = None

    def set_stream(self, stream_ptr: int | None) -> None:
        self._user_stream = stream_ptr or 0
        self._set_stream_raw(self._user_stream)

    def _set_stream_raw(self, stream_ptr: int) -> None:
        self.module._check(self._lib.dino_session_set_stream(self._handle, ctypes.c_void_p(stream_ptr)))

    def set_graph_replay(self, enabled: bool) -> None:
        """Steady-state replay for run_device_pointers / run_torch: a combination of shapes and device pointers seen twice is
        captured as a CUDA graph and replayed afterwards.  Keep the buffers you pass stable while it is on."""
        self._graph_replay = bool(enabled)
        self.module._check(self._lib.dino_session_set_graph_replay(self._handle, int(self._graph_replay)))

    def graph_stats(self) -> dict[str, int]:
        cached, launches = ctypes.c_size_t(), ctypes.c_size_t()
        self.module._check(self._lib.dino_session_get_graph_stats(self._handle, ctypes.byref(cached), ctypes.byref(launches)))
        return {"cached_graphs": int(cached.value), "graph_launches": int(launches.value)}

    # -- shapes
    def _output_shapes(self, in_shapes: Mapping[str, tuple[int, ...]]) -> dict[str, tuple[int, ...]]:
        """Output shapes from the graph (each gemm output is a.shape[:-1] + [N])."""
        graph = json.loads((self.module.path / "graph.dinoir.json").read_text()) if not hasattr(self, "_graph") else self._graph
        self._graph = graph
        shapes = dict(in_shapes)
        consts = {c["name"]: c for c in graph["constants"]}
        for node in graph["nodes"]:
            a = shapes[node["inputs"][0]]
            rows = consts[node["inputs"][1]]["shape"][0]
            shapes[node["outputs"][0]] = tuple(a[:-1]) + (rows // 2 if node["op"].startswith("dual_gemm_rcr_") else rows,)
        return {o["name"]: shapes[o["name"]] for o in graph["outputs"]}

    def _pack(self, inputs: Mapping[str, tuple[int, tuple[int, ...], str]], outputs: Mapping[str, tuple[int, tuple[int, ...], str]]):
        keep: list = []
        meta = self.module.metadata
        ins = (_DinoTensor * len(meta["inputs"]))(*[_tensor_struct(*inputs[i["name"]], keep) for i in meta["inputs"]])
        outs = (_DinoTensor * len(meta["outputs"]))(*[_tensor_struct(*outputs[o["name"]], keep) for o in meta["outputs"]])
        return ins, outs, keep

    # -- run
    def run_device_pointers(self, inputs, outputs) -> None:
        """inputs / outputs: name -> (device pointer, shape, dtype name).  Zero-copy."""
        ins, outs, keep = self._pack(inputs, outputs)
        self.module._check(self._lib.dino_session_run(self._handle, ins, len(ins), outs, len(outs)))

    def run_torch(self, inputs: Mapping[str, Any], outputs: Mapping[str, Any] | None = None) -> dict[str, Any]:
        import torch
        meta = self.module.metadata
        out_shapes = self._output_shapes({k: tuple(v.shape) for k, v in inputs.items()})
        if outputs is None:
            dev = next(iter(inputs.values())).device
            outputs = {o["name"]: torch.empty(out_shapes[o["name"]], dtype=getattr(torch, o["dtype"]), device=dev) for o in meta["outputs"]}
        dt = lambda t: str(t.dtype).replace("torch.", "")
        self.run_device_pointers({k: (v.data_ptr(), tuple(v.shape), dt(v)) for k, v in inputs.items()},
                                 {k: (v.data_ptr(), tuple(v.shape), dt(v)) for k, v in outputs.items()})
        return dict(outputs)

    def run_numpy(self, inputs: Mapping[str, np.ndarray]) -> dict[str, np.ndarray]:
        """Host arrays in, host arrays out.  All inputs of a call are packed into ONE pinned arena and go to the device
        in one copy, the module runs on the same stream, all outputs come back in one copy from one device arena, and
        the host waits once.  Arenas, tensor descriptors and the stream are cached per set of input shapes.
        bfloat16 travels as uint16 bit patterns or as float32 arrays (rounded to nearest even), and comes back as
        float32; float16 / float32 keep their numpy dtypes."""
        meta = self.module.metadata
        arrays = {spec["name"]: np.asarray(inputs[spec["name"]]) for spec in meta["inputs"]}
        key = tuple((name, arr.shape) for name, arr in arrays.items())
        plan = self._numpy_plans.get(key)
        if plan is None:
            plan = self._numpy_plans[key] = self._make_numpy_plan(arrays)
        lib = self._lib
        for spec in meta["inputs"]:
            arr, view = arrays[spec["name"]], plan["in_views"][spec["name"]]
            if spec["dtype"] == "bfloat16":
                if arr.dtype == np.float32 and arr.flags.c_contiguous:      # rounded natively, straight into the pinned arena
                    lib.dino_convert_f32_to_bf16(arr.ctypes.data, plan["in_ptrs"][spec["name"]], arr.size)
                else:
                    view[...] = arr if arr.dtype == np.uint16 else _f32_to_bf16_bits(arr)
            else:
                view[...] = arr                                   # numpy converts to the view's dtype
        # one native call: H2D of the input arena, the launches (a replayed graph in steady state), D2H of the output arena
        # (none when the outputs are small: the kernels then store straight into the pinned arena), one wait - all on the
        # plan's stream, with graph replay on for this call unless the user switched it on for the session anyway
        self.module._check(lib.dino_session_run_staged_on(
            self._handle, plan["stream_ptr"], int(self.numpy_graph_replay or self._graph_replay), plan["pin_in_ptr"], plan["dev_in_ptr"],
            plan["in_bytes"], plan["ins"], len(plan["ins"]), plan["outs"], len(plan["outs"]), plan["dev_out_ptr"], plan["pin_out_ptr"],
            plan["copy_out_bytes"]))
        out = {}
        if plan["all_bf16_out"]:
            # the whole pinned arena widens in ONE native call into one float32 buffer; the results are views of it
            wide = np.empty(plan["out_bytes"] // 2, dtype=np.float32)
            lib.dino_convert_bf16_to_f32(plan["pin_out_ptr"], wide.ctypes.data, wide.size)
            for name, (first, count, shape) in plan["out_slices"].items():
                out[name] = wide[first:first + count].reshape(shape)
            return out
        for o in meta["outputs"]:
            view = plan["out_views"][o["name"]]
            if o["dtype"] == "bfloat16":
                res = np.empty(view.shape, dtype=np.float32)      # the 16 bits become the high half of each float
                lib.dino_convert_bf16_to_f32(plan["out_ptrs"][o["name"]], res.ctypes.data, res.size)
                out[o["name"]] = res
            else:
                out[o["name"]] = view.copy()
        return out

    def _make_numpy_plan(self, arrays: Mapping[str, np.ndarray]) -> dict[str, Any]:
        import torch
        meta = self.module.metadata
        np_dt = {"bfloat16": np.uint16, "float16": np.float16, "float32": np.float32}
        esize = {"bfloat16": 2, "float16": 2, "float32": 4}
        out_shapes = self._output_shapes({k: tuple(v.shape) for k, v in arrays.items()})

        def layout(entries):
            offs, total = {}, 0
            for name, shape, dtype in entries:
                offs[name] = total
                total += -(-int(np.prod(shape)) * esize[dtype] // 256) * 256      # 256-byte aligned slices
            return offs, max(total, 256)

        in_entries = [(i["name"], tuple(arrays[i["name"]].shape), i["dtype"]) for i in meta["inputs"]]
        out_entries = [(o["name"], tuple(out_shapes[o["name"]]), o["dtype"]) for o in meta["outputs"]]
        in_off, in_bytes = layout(in_entries)
        out_off, out_bytes = layout(out_entries)
        dev = torch.device("cuda", torch.cuda.current_device())
        plan = {"pin_in": torch.empty(in_bytes, dtype=torch.uint8).pin_memory(), "dev_in": torch.empty(in_bytes, dtype=torch.uint8, device=dev),
                "pin_out": torch.empty(out_bytes, dtype=torch.uint8).pin_memory(), "dev_out": torch.empty(out_bytes, dtype=torch.uint8, device=dev),
                "stream": torch.cuda.Stream(device=dev), "keep": []}
        host_in, host_out = plan["pin_in"].numpy(), plan["pin_out"].numpy()

        def views(entries, offs, host):
            return {name: host[offs[name]:offs[name] + int(np.prod(shape)) * esize[dtype]].view(np_dt[dtype]).reshape(shape)
                    for name, shape, dtype in entries}

        plan["in_views"], plan["out_views"] = views(in_entries, in_off, host_in), views(out_entries, out_off, host_out)
        plan.update(in_bytes=in_bytes, out_bytes=out_bytes, out_off=out_off, pin_in_ptr=plan["pin_in"].data_ptr(),
                    dev_in_ptr=plan["dev_in"].data_ptr(), pin_out_ptr=plan["pin_out"].data_ptr(), dev_out_ptr=plan["dev_out"].data_ptr(),
                    any_bf16=any(o["dtype"] == "bfloat16" for o in meta["outputs"]))
        plan["ins"] = (_DinoTensor * len(in_entries))(*[_tensor_struct(plan["dev_in"].data_ptr() + in_off[n], s, d, plan["keep"])
                                                        for n, s, d in in_entries])
        # Decode-sized results (up to 64 KB in all) are written by the kernels straight into the pinned host arena (mapped into
        # the device's address space at the same address): no device-to-host copy node, one hop less before the host may read.
        zero_copy = out_bytes <= self.numpy_zero_copy_bytes
        out_base = plan["pin_out"].data_ptr() if zero_copy else plan["dev_out"].data_ptr()
        plan["outs"] = (_DinoTensor * len(out_entries))(*[_tensor_struct(out_base + out_off[n], s, d, plan["keep"]) for n, s, d in out_entries])
        plan.update(copy_out_bytes=0 if zero_copy else out_bytes, stream_ptr=plan["stream"].cuda_stream,
                    in_ptrs={n: plan["pin_in"].data_ptr() + in_off[n] for n, _, _ in in_entries},
                    out_ptrs={n: plan["pin_out"].data_ptr() + out_off[n] for n, _, _ in out_entries})
        plan["all_bf16_out"] = bool(out_entries) and all(d == "bfloat16" for _, _, d in out_entries)
        plan["out_slices"] = {n: (out_off[n] // 2, int(np.prod(sh)), tuple(sh)) for n, sh, _ in out_entries}
        return plan

    # -- benchmark
    def benchmark_torch(self, inputs: Mapping[str, Any], warmup: int = 5, iterations: int = 20) -> dict[str, Any]:
        """Native benchmark loop (CUDA-graph replay + events per iteration); summary like src/dinoml/runtime.py:1854-1866."""
        import torch
        meta = self.module.metadata
        out_shapes = self._output_shapes({k: tuple(v.shape) for k, v in inputs.items()})
        dev = next(iter(inputs.values())).device
        outputs = {o["name"]: torch.empty(out_shapes[o["name"]], dtype=getattr(torch, o["dtype"]), device=dev) for o in meta["outputs"]}
        dt = lambda t: str(t.dtype).replace("torch.", "")
        ins, outs, keep = self._pack({k: (v.data_ptr(), tuple(v.shape), dt(v)) for k, v in inputs.items()},
                                     {k: (v.data_ptr(), tuple(v.shape), dt(v)) for k, v in outputs.items()})
        ms = (ctypes.c_double * iterations)()
        self.module._check(self._lib.dino_session_benchmark(self._handle, ins, len(ins), outs, len(outs), warmup, iterations, ms, iterations))
        return summarize_ms(list(ms), native_entrypoint="dino_session_benchmark", timing_source="cuda_events", graph_replay=True,
                            warmup=warmup)


    def benchmark_device_pointers(self, inputs, outputs, *, warmup: int = 5, iterations: int = 20) -> dict[str, Any]:
        """Native benchmark on caller-owned device buffers: name -> (device pointer, shape, dtype name), as run_device_pointers
        (src/dinoml/runtime.py:1194-1217)."""
        ins, outs, keep = self._pack(inputs, outputs)
        ms = (ctypes.c_double * iterations)()
        self.module._check(self._lib.dino_session_benchmark(self._handle, ins, len(ins), outs, len(outs), warmup, iterations, ms, iterations))
        return summarize_ms(list(ms), native_entrypoint="dino_session_benchmark", timing_source="cuda_events", graph_replay=True, warmup=warmup)

    def benchmark_numpy(self, inputs: Mapping[str, np.ndarray], *, warmup: int = 5, iterations: int = 20) -> dict[str, Any]:
        """Host arrays in: they are uploaded once (the arenas of run_numpy), then the native benchmark loop runs on the device
        copies - device time per run, without the host copies (src/dinoml/runtime.py:966-977)."""
        meta = self.module.metadata
        arrays = {spec["name"]: np.asarray(inputs[spec["name"]]) for spec in meta["inputs"]}
        key = tuple((name, arr.shape) for name, arr in arrays.items())
        plan = self._numpy_plans.get(key)
        if plan is None:
            plan = self._numpy_plans[key] = self._make_numpy_plan(arrays)
        for spec in meta["inputs"]:
            arr, view = arrays[spec["name"]], plan["in_views"][spec["name"]]
            view[...] = (arr if arr.dtype == np.uint16 else _f32_to_bf16_bits(arr)) if spec["dtype"] == "bfloat16" else arr
        plan["dev_in"].copy_(plan["pin_in"])
        import torch
        torch.cuda.synchronize()
        ms = (ctypes.c_double * iterations)()
        self.module._check(self._lib.dino_session_benchmark(self._handle, plan["ins"], len(plan["ins"]), plan["outs"], len(plan["outs"]),
                                                            warmup, iterations, ms, iterations))
        return summarize_ms(list(ms), native_entrypoint="dino_session_benchmark", timing_source="cuda_events", graph_replay=True, warmup=warmup)


def _f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bfloat16 storage of a float array (src/dinoml/ir.py:68-73)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def summarize_ms(values: list[float], **metadata) -> dict[str, Any]:
    out = {"iterations": len(values), "mean_ms": statistics.fmean(values), "median_ms": statistics.median(values),
           "min_ms": min(values), "max_ms": max(values), "stddev_ms": statistics.pstdev(values) if len(values) > 1 else 0.0,
           "elapsed_ms": values}
    out.update(metadata)
    return out
