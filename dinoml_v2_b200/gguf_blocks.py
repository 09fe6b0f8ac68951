"""GGUF block-layout tables: the three quantization types of the benchmark configurations (Q8_0, Q4_K, Q6_K) and the six
further ones the reference's fused prototype decodes (Q4_0, Q5_K, Q2_K, Q3_K, MXFP4, NVFP4).

The byte layouts are the ones the reference declares in
kernels/rocm/src/ck_gguf_q8_gemm.hip:20-25 (Q8_0), :27-32 (Q4_0), :34-41 (Q4_K), :43-51 (Q5_K), :53-60 (Q2_K),
:62-69 (Q3_K), :71-78 (Q6_K), :80-85 (MXFP4), :87-92 (NVFP4);
`qtype_value` is the ggml type id the reference records in constant storage
metadata (src/dinoml/constant_sources.py:88-108).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class QType:
    name: str          # "Q8_0", "Q4_K", ...
    value: int         # ggml enum
    block_size: int    # weights per block
    block_bytes: int   # bytes per block
    symbol: str        # lower-case tag used in kernel symbol names


Q8_0 = QType("Q8_0", 8, 32, 34, "q8_0")
Q4_K = QType("Q4_K", 12, 256, 144, "q4_k")
Q6_K = QType("Q6_K", 14, 256, 210, "q6_k")
Q4_0 = QType("Q4_0", 2, 32, 18, "q4_0")
Q2_K = QType("Q2_K", 10, 256, 84, "q2_k")
Q3_K = QType("Q3_K", 11, 256, 110, "q3_k")
Q5_K = QType("Q5_K", 13, 256, 176, "q5_k")
MXFP4 = QType("MXFP4", 39, 32, 17, "mxfp4")
NVFP4 = QType("NVFP4", 40, 64, 36, "nvfp4")

QTYPES = {q.name: q for q in (Q8_0, Q4_K, Q6_K, Q4_0, Q5_K, Q2_K, Q3_K, MXFP4, NVFP4)}
# every type has tensor-core kernels (a decode GEMV and the tcgen05 GEMM); float32 activations and weight rows that are not
# multiples of 16 bytes run on the CUDA-core kernel
TENSOR_CORE_QTYPES = tuple(QTYPES)
QTYPES_BY_VALUE = {q.value: q for q in QTYPES.values()}


def qtype_of(which) -> QType:
    """Accepts a QType, a name ("Q4_K", case-insensitive) or a ggml enum value."""
    if isinstance(which, QType):
        return which
    if isinstance(which, str):
        key = which.upper()
        if key in QTYPES:
            return QTYPES[key]
    elif int(which) in QTYPES_BY_VALUE:
        return QTYPES_BY_VALUE[int(which)]
    raise ValueError(f"unsupported GGUF qtype {which!r}; supported: {sorted(QTYPES)}")


def row_bytes(qtype, n_per_row: int) -> int:
    q = qtype_of(qtype)
    if n_per_row <= 0 or n_per_row % q.block_size:
        raise ValueError(f"n_per_row={n_per_row} is not a positive multiple of the {q.name} block size {q.block_size}")
    return n_per_row // q.block_size * q.block_bytes


def encoded_nbytes(qtype, rows: int, n_per_row: int) -> int:
    return int(rows) * row_bytes(qtype, n_per_row)
