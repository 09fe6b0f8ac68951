"""GGUF constant descriptor and policies - the same public surface as the reference's
src/dinoml/constant_sources.py (GGUFConstant :43-126, gguf_constant :128-150, policy tables :13-34,
validate_gguf_constant_policy :211-239, materialize_gguf_encoded_constant :165-180), with the policy
the reference only declares as "future" - `direct_dequantize_in_kernel` - implemented: the weight
stays GGUF-encoded on the device and the matmul kernels read the blocks directly.

Differences from the reference, all on purpose:
* tensor bytes come from this package's own `.gguf` reader (gguf_file.py) instead of libgguf;
* there is no host dequantization here at all (the reference's `materialize()` needs
  libgguf.dequantize_rows; the CPU target is out of scope and the GPU path never needs dense weights);
* `GGUFConstant.from_blocks` binds in-memory encoded bytes (synthetic benchmarks, tests).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Sequence

import numpy as np

from .gguf_blocks import QTYPES, qtype_of, row_bytes
from .gguf_file import open_gguf

GGUF_MATERIALIZATION_DEQUANTIZE_FULL_BEFORE_LAUNCH = "dequantize_full_before_launch"
GGUF_MATERIALIZATION_DEQUANTIZE_ON_GPU_BEFORE_LAUNCH = "dequantize_on_gpu_before_launch"
GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL = "direct_dequantize_in_kernel"

GGUF_RESIDENCY_EAGER_DENSE_DEVICE = "eager_dense_device"
GGUF_RESIDENCY_CPU_UNTIL_FIRST_USE = "cpu_until_first_use"
GGUF_RESIDENCY_SEQUENTIAL_OFFLOAD = "sequential_offload"
GGUF_RESIDENCY_GROUPED_OFFLOAD = "grouped_offload"
GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD = "manual_runtime_load"
GGUF_RESIDENCY_EAGER_ENCODED_DEVICE = "eager_encoded_device"   # new: encoded bytes uploaded with the other constants

# Status strings keep the reference's vocabulary ("runtime_supported" / "future").
GGUF_MATERIALIZATION_POLICIES: Mapping[str, str] = {
    GGUF_MATERIALIZATION_DEQUANTIZE_FULL_BEFORE_LAUNCH: "future",      # needs a host dequantizer: CPU target only
    GGUF_MATERIALIZATION_DEQUANTIZE_ON_GPU_BEFORE_LAUNCH: "future",    # superseded by the fused kernels
    GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL: "runtime_supported",
}
# The three host-residency policies are only declared by the reference ("future", src/dinoml/constant_sources.py:29-33); here
# they are implemented in the native runtime (csrc/runtime.cu): the encoded bytes live in pinned host memory and reach the
# device on first use (cpu_until_first_use) or are streamed through two device slots ahead of their launches, one
# constant (sequential_offload) or one group of constants (grouped_offload) at a time.
GGUF_RESIDENCY_POLICIES: Mapping[str, str] = {
    GGUF_RESIDENCY_EAGER_DENSE_DEVICE: "future",       # a dense device copy: what the fused kernels make unnecessary
    GGUF_RESIDENCY_CPU_UNTIL_FIRST_USE: "runtime_supported",
    GGUF_RESIDENCY_SEQUENTIAL_OFFLOAD: "runtime_supported",
    GGUF_RESIDENCY_GROUPED_OFFLOAD: "runtime_supported",
    GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD: "runtime_supported",
    GGUF_RESIDENCY_EAGER_ENCODED_DEVICE: "runtime_supported",
}
HOST_RESIDENCIES = (GGUF_RESIDENCY_CPU_UNTIL_FIRST_USE, GGUF_RESIDENCY_SEQUENTIAL_OFFLOAD, GGUF_RESIDENCY_GROUPED_OFFLOAD)


def validate_gguf_constant_policy(materialization: str, residency: str, *, require_runtime_supported: bool = False) -> None:
    if materialization not in GGUF_MATERIALIZATION_POLICIES:
        raise ValueError(f"Unsupported GGUF materialization policy {materialization!r}; "
                         f"expected one of {sorted(GGUF_MATERIALIZATION_POLICIES)}")
    if residency not in GGUF_RESIDENCY_POLICIES:
        raise ValueError(f"Unsupported GGUF residency policy {residency!r}; expected one of {sorted(GGUF_RESIDENCY_POLICIES)}")
    if require_runtime_supported:
        if GGUF_MATERIALIZATION_POLICIES[materialization] != "runtime_supported":
            raise NotImplementedError(f"GGUF materialization policy {materialization!r} is not supported by the B200 runtime; "
                                      f"use {GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL!r}")
        if GGUF_RESIDENCY_POLICIES[residency] != "runtime_supported":
            raise NotImplementedError(f"GGUF residency policy {residency!r} is not supported by the B200 runtime; use "
                                      f"{GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD!r} or {GGUF_RESIDENCY_EAGER_ENCODED_DEVICE!r}")


def gguf_constant_policy_status(materialization: str, residency: str) -> dict[str, str]:
    validate_gguf_constant_policy(materialization, residency)
    return {"materialization": GGUF_MATERIALIZATION_POLICIES[materialization], "residency": GGUF_RESIDENCY_POLICIES[residency]}


@dataclass(frozen=True)
class MaterializedConstant:
    array: np.ndarray
    storage: dict[str, Any] | None = None


@dataclass(frozen=True)
class GGUFConstant:
    """Same fields as the reference descriptor (src/dinoml/constant_sources.py:43-53); the defaults are the
    policies this runtime implements."""
    path: str | Path
    tensor: str
    logical_dtype: str | None = None
    shape: Sequence[int] | None = None
    qtype: str | None = None
    encoded_nbytes: int | None = None
    n_per_row: int | None = None
    materialization: str = GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL
    residency: str = GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD
    offload_group: int | None = None      # grouped_offload: constants with the same number travel to the device together
    _blocks: np.ndarray | None = field(default=None, repr=False, compare=False)   # in-memory source (from_blocks)

    def __post_init__(self) -> None:
        validate_gguf_constant_policy(self.materialization, self.residency)
        if self.offload_group is not None and (self.residency != GGUF_RESIDENCY_GROUPED_OFFLOAD or int(self.offload_group) < 0):
            raise ValueError("offload_group is a non-negative group number for residency 'grouped_offload' only")

    @staticmethod
    def from_blocks(blocks: np.ndarray, qtype, shape: Sequence[int], *, tensor: str = "weight", logical_dtype: str | None = None,
                    materialization: str = GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL,
                    residency: str = GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD, offload_group: int | None = None) -> "GGUFConstant":
        q = qtype_of(qtype)
        n, k = (int(d) for d in shape)
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(n, row_bytes(q, k))
        return GGUFConstant(path="<memory>", tensor=tensor, logical_dtype=logical_dtype, shape=(n, k), qtype=q.name,
                            encoded_nbytes=int(blocks.nbytes), n_per_row=k, materialization=materialization, residency=residency,
                            offload_group=offload_group, _blocks=blocks)

    def materialize(self, dtype: str, shape: Sequence[int]) -> MaterializedConstant:
        """The reference dequantizes on the host here (src/dinoml/constant_sources.py:58-79).  This runtime has no
        host dequantizer and never needs dense weights, so it refuses loudly instead of falling back."""
        raise NotImplementedError("host dequantization of GGUF constants is not part of the B200 runtime; GGUF constants are "
                                  "bound encoded (materialize_gguf_encoded_constant) and dequantized inside the kernels")

    def read_encoded(self, expected_shape: Sequence[int]) -> tuple[np.ndarray, dict[str, Any]]:
        """Raw encoded bytes + observed metadata; mirrors _read_gguf_encoded_constant
        (src/dinoml/constant_sources.py:303-333)."""
        expected = tuple(int(d) for d in expected_shape)
        if self._blocks is not None:
            q = qtype_of(self.qtype)
            raw, gguf_shape, offset = self._blocks.reshape(-1), tuple(reversed(expected)), 0
        else:
            with open_gguf(self.path) as f:
                info = f.get_tensor(self.tensor)
                if info is None:
                    raise ValueError(f"GGUF tensor not found: {self.tensor!r}")
                if info.qtype not in QTYPES:
                    raise ValueError(f"GGUF tensor {self.tensor!r} has qtype {info.qtype}; supported: {sorted(QTYPES)}")
                q = qtype_of(info.qtype)
                gguf_shape = info.shape
                offset = info.data_offset
                raw = np.frombuffer(f.read_tensor_bytes(info), dtype=np.uint8).copy()
        logical = tuple(reversed(gguf_shape))
        if logical != expected:
            raise ValueError(f"GGUF tensor {self.tensor!r} has logical shape {logical}, expected {expected} "
                             f"(stored GGUF shape {tuple(gguf_shape)})")
        observed = {"qtype": q.name, "qtype_value": q.value, "encoded_nbytes": int(raw.nbytes), "gguf_shape": list(gguf_shape),
                    "data_offset": int(offset), "n_per_row": int(gguf_shape[0]) if gguf_shape else 1}
        self._validate_observed_hints(observed)
        return raw, observed

    def _metadata(self, dtype: str, shape: tuple[int, ...], observed: Mapping[str, Any]) -> dict[str, Any]:
        """Storage dict with the reference's keys (src/dinoml/constant_sources.py:81-108)."""
        metadata: dict[str, Any] = {
            "kind": "gguf", "path": str(self.path), "tensor": self.tensor, "logical_dtype": dtype, "shape": list(shape),
            "materialization": self.materialization, "residency": self.residency,
        }
        for key in ("qtype", "qtype_value", "encoded_nbytes", "gguf_shape", "data_offset", "n_per_row"):
            if observed.get(key) is not None:
                metadata[key] = observed[key]
        if self.offload_group is not None:
            metadata["offload_group"] = int(self.offload_group)
        return metadata

    def _validate_observed_hints(self, observed: Mapping[str, Any]) -> None:
        for key, label in (("qtype", "qtype"), ("encoded_nbytes", "encoded bytes"), ("n_per_row", "n_per_row")):
            want = getattr(self, key)
            if want is not None and want != observed.get(key):
                raise ValueError(f"GGUF constant {self.tensor!r} expected {label} {want}, observed {observed.get(key)}")


def gguf_constant(path: str | Path, tensor: str, *, logical_dtype: str | None = None, shape: Sequence[int] | None = None,
                  qtype: str | None = None, encoded_nbytes: int | None = None, n_per_row: int | None = None,
                  materialization: str = GGUF_MATERIALIZATION_DIRECT_DEQUANTIZE_IN_KERNEL,
                  residency: str = GGUF_RESIDENCY_MANUAL_RUNTIME_LOAD, offload_group: int | None = None) -> GGUFConstant:
    return GGUFConstant(path=path, tensor=tensor, logical_dtype=logical_dtype, shape=shape, qtype=qtype,
                        encoded_nbytes=encoded_nbytes, n_per_row=n_per_row, materialization=materialization, residency=residency,
                        offload_group=offload_group)


def materialize_gguf_encoded_constant(source: GGUFConstant, dtype: str, shape: Sequence[int]) -> MaterializedConstant:
    """Encoded bytes (uint8) + storage metadata, as src/dinoml/constant_sources.py:165-180."""
    expected = tuple(int(d) for d in shape)
    if source.logical_dtype is not None and source.logical_dtype != dtype:
        raise ValueError(f"GGUF constant {source.tensor!r} has logical dtype {source.logical_dtype}, expected {dtype}")
    if source.shape is not None and tuple(int(d) for d in source.shape) != expected:
        raise ValueError(f"GGUF constant {source.tensor!r} has shape {tuple(source.shape)}, expected {expected}")
    if len(expected) != 2:
        raise ValueError("GGUF-encoded constants must be rank-2 [N, K] weights")
    raw, observed = source.read_encoded(expected)
    want = expected[0] * row_bytes(observed["qtype"], expected[1])
    if raw.nbytes != want:
        raise ValueError(f"GGUF tensor {source.tensor!r}: {raw.nbytes} encoded bytes, expected {want} for shape {expected}")
    return MaterializedConstant(raw, source._metadata(dtype, expected, observed))
