"""Thin tracing frontend for the quantized-linear path: the slice of the reference's `dml.trace` API
(src/dinoml/frontend.py:517-532, src/dinoml/nn/__init__.py:46-79, src/dinoml/shapes.py:7-47) that a
`gemm_rcr` / `gemm_rcr_bias` graph needs - Dim, TensorSpec, Parameter, Module, Tensor, trace, ModelSpec.
The IR is the reference's JSON dictionary shape: nodes `{"id","op","inputs","outputs","attrs"}`,
constants with `layout` / `storage` metadata (src/dinoml/ir.py:117-170)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

import numpy as np

from .constant_sources import GGUFConstant, materialize_gguf_encoded_constant

# runtime dtype enums of ABI v7 (src/dinoml/ir.py:30-39, runtime/include/dinoml/abi.h:14-23)
DTYPE_ENUM = {"float16": 1, "float32": 2, "int32": 3, "int64": 4, "bool": 5, "bfloat16": 6}
DTYPE_NBYTES = {"float16": 2, "float32": 4, "int32": 4, "int64": 8, "bool": 1, "bfloat16": 2}
RUNTIME_ABI_VERSION = 7


def normalize_dtype(dtype: str) -> str:
    alias = {"half": "float16", "fp16": "float16", "f16": "float16", "float": "float32", "fp32": "float32", "f32": "float32",
             "bf16": "bfloat16"}
    name = alias.get(str(dtype), str(dtype))
    if name not in DTYPE_ENUM:
        raise ValueError(f"Unsupported dtype {dtype!r}")
    return name


@dataclass(frozen=True)
class Dim:
    """Dynamic dimension with profiling buckets (src/dinoml/shapes.py:7-14)."""
    name: str
    min: int
    max: int
    typical: int | None = None
    buckets: tuple[int, ...] = ()

    def __post_init__(self):
        if not (0 <= self.min <= self.max):
            raise ValueError(f"Dim {self.name!r} needs 0 <= min <= max")
        for b in self.buckets:
            if not (self.min <= b <= self.max):
                raise ValueError(f"Dim {self.name!r} bucket {b} outside [{self.min}, {self.max}]")


def dim_spec(d) -> dict[str, Any]:
    if isinstance(d, Dim):
        return {"kind": "dynamic", "name": d.name, "min": d.min, "max": d.max, "typical": d.typical, "buckets": list(d.buckets)}
    return {"kind": "static", "value": int(d)}


@dataclass(frozen=True)
class TensorSpec:
    shape: Sequence[Any]
    dtype: str = "float16"


@dataclass
class Parameter:
    shape: Sequence[int]
    dtype: str = "float16"
    name: str | None = None


@dataclass(frozen=True)
class Tensor:
    """Symbolic tensor flowing through a trace."""
    name: str
    shape: tuple[Any, ...]
    dtype: str
    kind: str = "tensor"          # "input" | "constant" | "tensor"


class Module:
    def parameters(self) -> dict[str, Parameter]:
        out: dict[str, Parameter] = {}
        for key, value in vars(self).items():
            if isinstance(value, Parameter):
                out[key] = value
            elif isinstance(value, Module):
                for sub, p in value.parameters().items():
                    out[f"{key}.{sub}"] = p
        return out

    def forward(self, *args, **kwargs):  # pragma: no cover - interface
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)


class GraphBuilder:
    _active: "GraphBuilder | None" = None

    def __init__(self):
        self.nodes: list[dict[str, Any]] = []
        self.tensors: dict[str, Tensor] = {}

    def add_node(self, op: str, inputs: Sequence[Tensor], out_shape: tuple[Any, ...], dtype: str, attrs=None) -> Tensor:
        out = Tensor(f"t{len(self.nodes)}", out_shape, dtype)
        self.nodes.append({"id": f"n{len(self.nodes)}", "op": op, "inputs": [t.name for t in inputs], "outputs": [out.name],
                           "attrs": dict(attrs or {})})
        self.tensors[out.name] = out
        return out


def current_builder() -> GraphBuilder:
    if GraphBuilder._active is None:
        raise RuntimeError("dml.ops functions can only be called while tracing (inside dml.trace)")
    return GraphBuilder._active


@dataclass
class ModelSpec:
    """Traced graph + bound constants.  `graph` is JSON-serialisable; `constant_arrays` holds the bytes that go
    to constants.bin (dense storage arrays, or uint8 encoded GGUF bytes)."""
    graph: dict[str, Any]
    constant_arrays: dict[str, np.ndarray] = field(default_factory=dict)

    def constant(self, name: str) -> dict[str, Any]:
        for c in self.graph["constants"]:
            if c["name"] == name:
                return c
        raise KeyError(name)


def _to_storage(value: np.ndarray, dtype: str) -> np.ndarray:
    value = np.asarray(value)
    if dtype == "bfloat16":
        if value.dtype == np.uint16:
            return np.ascontiguousarray(value)
        bits = np.ascontiguousarray(value, dtype=np.float32).view(np.uint32)   # RNE, src/dinoml/ir.py:68-73
        return ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    return np.ascontiguousarray(value, dtype={"float16": np.float16, "float32": np.float32}[dtype])


def _fuse_dual_gemm_weights(nodes: list[dict[str, Any]], bound: dict[str, tuple]) -> None:
    """A dual GEMM node reads its two GGUF weights as ONE constant whose rows alternate in groups of 8 (rows 16t..16t+7 from
    B0, 16t+8..16t+15 from B1): that order puts a gate row and its up row into the same thread of the fused kernels.  The
    node is rewritten to [a, fused]; source constants no other node reads are dropped from the artifact."""
    for node in nodes:
        if not node["op"].startswith("dual_gemm_rcr_"):
            continue
        n0, n1 = node["inputs"][1], node["inputs"][2]
        (dt0, sh0, a0, st0), (dt1, sh1, a1, st1) = bound[n0], bound[n1]
        if not (st0 and st1 and st0.get("kind") == "gguf" and st1.get("kind") == "gguf"):
            raise NotImplementedError(f"{node['op']}: both weights must be GGUF-encoded constants")
        broadcast = tuple(sh1) == (1, sh0[1]) and sh0[0] != 1           # B1 [1, K]: its one row is repeated for every output column
        if st0["qtype"] != st1["qtype"] or (tuple(sh0) != tuple(sh1) and not broadcast) or dt0 != dt1 or sh0[0] % 8:
            raise NotImplementedError(f"{node['op']}: the two weights need one qtype, one shape (or B1 [1, K]) and N % 8 == 0")
        n, k = sh0
        rb = a0.size // n
        rows1 = np.broadcast_to(a1.reshape(1, rb), (n, rb)) if broadcast else a1.reshape(n, rb)
        fused = np.ascontiguousarray(np.stack((a0.reshape(n // 8, 8, rb), rows1.reshape(n // 8, 8, rb)), axis=1).reshape(-1))
        storage = dict(st0)
        storage.update({"tensor": f"{st0['tensor']}+{st1['tensor']}", "shape": [2 * n, k], "encoded_nbytes": int(fused.nbytes),
                        "gguf_shape": [k, 2 * n], "derived": {"kind": "interleave_rows8", "sources": [n0, n1],
                                                               "source_paths": [st0.get("path"), st1.get("path")]}})
        name = f"{n0}+{n1}.rows8"
        bound[name] = (dt0, (2 * n, k), fused, storage)
        sources = [n0, n1]
        fused_inputs = [node["inputs"][0], name]
        if len(node["inputs"]) == 5:          # the _bias_ forms: bias0 [N] and bias1 [N] (or [1]) become ONE dense vector in the same order
            nb0, nb1 = node["inputs"][3], node["inputs"][4]
            (bdt0, _, v0, bst0), (bdt1, _, v1, bst1) = bound[nb0], bound[nb1]
            if bst0 or bst1 or bdt0 != dt0 or bdt1 != dt0:
                raise NotImplementedError(f"{node['op']}: bias0 / bias1 must be dense constants of the activation dtype")
            v0, v1 = np.asarray(v0).reshape(-1), np.asarray(v1).reshape(-1)
            if v0.size != n or v1.size != (1 if broadcast else n):
                raise ValueError(f"{node['op']}: bias0 needs {n} elements and bias1 {1 if broadcast else n}")
            v1 = np.broadcast_to(v1, (n,))
            bias_name = f"{nb0}+{nb1}.rows8"
            bound[bias_name] = (dt0, (2 * n,), np.ascontiguousarray(np.stack((v0.reshape(n // 8, 8), v1.reshape(n // 8, 8)), axis=1).reshape(-1)), None)
            fused_inputs.append(bias_name)
            sources += [nb0, nb1]
        node["inputs"] = fused_inputs
        node["attrs"]["sources"] = sources
    used = {name for node in nodes for name in node["inputs"]}
    for node in nodes:
        for src in node["attrs"].get("sources", []):
            if src not in used:
                bound.pop(src, None)


def trace(module: Module, inputs: Mapping[str, TensorSpec], constants: Mapping[str, Any] | None = None,
          name: str = "model") -> ModelSpec:
    """Runs `module.forward` on symbolic tensors and binds constants.  A constant may be a numpy array (dense) or a
    GGUFConstant (bound encoded: ModelSpec.bind_constants GGUF branch, src/dinoml/ir.py:133-158)."""
    constants = dict(constants or {})
    builder = GraphBuilder()
    sym_inputs = {k: Tensor(k, tuple(v.shape), normalize_dtype(v.dtype), "input") for k, v in inputs.items()}
    params = module.parameters()
    missing = sorted(set(params) - set(constants))
    if missing:
        raise ValueError(f"no value bound for parameters {missing}")
    sym_params = {}
    for key, p in params.items():
        p.name = key
        sym_params[key] = Tensor(key, tuple(int(d) for d in p.shape), normalize_dtype(p.dtype), "constant")
    builder.tensors.update({t.name: t for t in list(sym_inputs.values()) + list(sym_params.values())})

    # parameters are read through attribute access: swap Parameter objects for their symbolic tensors during forward
    saved = []

    def swap(mod: Module, prefix: str):
        for key, value in list(vars(mod).items()):
            if isinstance(value, Parameter):
                saved.append((mod, key, value))
                setattr(mod, key, sym_params[prefix + key])
            elif isinstance(value, Module):
                swap(value, f"{prefix}{key}.")

    GraphBuilder._active = builder
    try:
        swap(module, "")
        outputs = module.forward(**sym_inputs)
    finally:
        GraphBuilder._active = None
        for mod, key, value in saved:
            setattr(mod, key, value)
    if isinstance(outputs, Tensor):
        outputs = [outputs]
    outputs = list(outputs)

    bound = {}                                                # name -> (dtype, shape, array, storage)
    for key, p in params.items():
        dtype, shape = normalize_dtype(p.dtype), tuple(int(d) for d in p.shape)
        value = constants[key]
        if isinstance(value, GGUFConstant):
            mat = materialize_gguf_encoded_constant(value, dtype, shape)
            arr, storage = mat.array, mat.storage
        else:
            arr = _to_storage(value, dtype)
            if tuple(arr.shape) != shape:
                raise ValueError(f"constant {key!r} has shape {tuple(arr.shape)}, expected {shape}")
            storage = None
        bound[key] = (dtype, shape, arr, storage)
    _fuse_dual_gemm_weights(builder.nodes, bound)

    const_entries, arrays, offset = [], {}, 0
    for key, (dtype, shape, arr, storage) in bound.items():
        strides, acc = [], 1
        for d in reversed(shape):
            strides.insert(0, acc)
            acc *= d
        offset = (offset + 255) // 256 * 256
        const_entries.append({"name": key, "tensor": key, "shape": list(shape), "shape_spec": [dim_spec(d) for d in shape],
                              "layout": {"schema_version": 1, "kind": "dense", "order": "row_major", "strides": strides,
                                         "storage_offset": 0},
                              "dtype": dtype, "offset": offset, "nbytes": int(arr.nbytes), "storage": storage})
        arrays[key] = arr
        offset += int(arr.nbytes)
    graph = {
        "name": name, "schema_version": 1,
        "inputs": [{"name": t.name, "dtype": t.dtype, "shape_spec": [dim_spec(d) for d in t.shape]} for t in sym_inputs.values()],
        "outputs": [{"name": t.name, "dtype": t.dtype, "shape_spec": [dim_spec(d) for d in t.shape]} for t in outputs],
        "nodes": builder.nodes,
        "tensors": [{"name": t.name, "dtype": t.dtype, "shape_spec": [dim_spec(d) for d in t.shape]} for t in builder.tensors.values()
                    if t.kind == "tensor"],
        "constants": const_entries,
    }
    return ModelSpec(graph, arrays)
