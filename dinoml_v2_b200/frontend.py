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

    const_entries, arrays, offset = [], {}, 0
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
