"""TEST INFRASTRUCTURE ONLY - CPU oracle for the GGUF quantized-linear path.

Two restatements of the reference's CPU arithmetic:

* `gguf_oracle.c` (loaded here through ctypes as `libgguf_oracle.so`) - scalar C
  compiled with ``-ffp-contract=off``;
* `dequantize_numpy` - a vectorised numpy twin of the same formulas.

Both follow tools/bench_ck_gguf_q8_gemm.hip:2028-2036, 2078-2082, 2093-2107,
2156-2171 (decode) and :2589-2615 (`reference_gemm_quant`).  The reference's
real dequantizer (third_party/libgguf, un-vendored, no version pin) is absent, so
parity at that boundary is "unpinned"; the oracle is instead pinned bit-for-bit
to the independent `gguf` 0.19.0 package and, for the matmul, to the reference's
CPU artifact (fixtures under tests/golden/).

Only tests, the smoke check and the benchmark's CPU-baseline / reference arm may
import this package.  The shipped package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libgguf_oracle.so"
_lib = None

QTYPE_VALUE = {"Q4_0": 2, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "MXFP4": 39, "NVFP4": 40}
BLOCK = {2: (32, 18), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 39: (32, 17), 40: (64, 36)}
DTYPE_CODE = {"float32": 0, "float16": 1, "bfloat16": 2}


def build(force: bool = False) -> Path:
    """Compile gguf_oracle.c with the committed Makefile (gcc, -ffp-contract=off)."""
    src = _HERE / "gguf_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libgguf_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL, env={**os.environ, "CC": "gcc"})
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.oracle_dequantize_rows.argtypes = [vp, i64, i64, i64, ci, vp]
        L.oracle_dequantize_rows.restype = ci
        L.oracle_gemm_quant.argtypes = [vp, vp, i64, i64, i64, i64, ci, vp]
        L.oracle_gemm_quant.restype = ci
        L.oracle_gemm_rcr_dense.argtypes = [vp, vp, vp, vp, ci, i64, i64, i64]
        L.oracle_gemm_rcr_dense.restype = ci
        L.oracle_set_threads.argtypes = [ci]
        L.oracle_max_threads.restype = ci
        _lib = L
    return _lib


def _qv(qtype) -> int:
    return QTYPE_VALUE[qtype.upper()] if isinstance(qtype, str) else int(qtype)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def dequantize(blocks: np.ndarray, qtype, n_per_row: int, dtype: str = "float32") -> np.ndarray:
    """uint8 [rows, row_bytes] -> [rows, n_per_row]; float32, float16, or bfloat16 (uint16 storage)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rows = blocks.shape[0]
    out = np.empty((rows, n_per_row), dtype={"float32": np.float32, "float16": np.float16, "bfloat16": np.uint16}[dtype])
    rc = lib().oracle_dequantize_rows(_ptr(blocks), _qv(qtype), rows, n_per_row, DTYPE_CODE[dtype], _ptr(out))
    if rc:
        raise ValueError(f"oracle_dequantize_rows failed with code {rc}")
    return out


def gemm_quant(a: np.ndarray, blocks: np.ndarray, qtype, n: int, k: int, round_w: int = 0) -> np.ndarray:
    """fp32 a[m,k] x GGUF blocks [n, row_bytes] -> fp32 [m,n]; single fp32 accumulator in k order."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    m = a.shape[0]
    c = np.empty((m, n), dtype=np.float32)
    rc = lib().oracle_gemm_quant(_ptr(a), _ptr(blocks), _qv(qtype), m, n, k, int(round_w), _ptr(c))
    if rc:
        raise ValueError(f"oracle_gemm_quant failed with code {rc}")
    return c


def gemm_rcr_dense(a: np.ndarray, b: np.ndarray, dtype: str, bias: np.ndarray | None = None) -> np.ndarray:
    """Dense gemm_rcr[_bias] in storage dtype (float32 arrays, float16 arrays, or uint16 bf16 bits)."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), dtype=a.dtype)
    bias_p = _ptr(np.ascontiguousarray(bias)) if bias is not None else None
    rc = lib().oracle_gemm_rcr_dense(_ptr(a), _ptr(b), bias_p, _ptr(c), DTYPE_CODE[dtype], m, n, k)
    if rc:
        raise ValueError(f"oracle_gemm_rcr_dense failed with code {rc}")
    return c


# ----------------------------------------------------------------------------- numpy twin
def _f16(raw: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(raw).view(np.float16).astype(np.float32)[..., 0]


def dequantize_numpy(blocks: np.ndarray, qtype, n_per_row: int) -> np.ndarray:
    """Vectorised fp32 dequantization; every product is a separate fp32 operation (no FMA)."""
    qv = _qv(qtype)
    bs, bb = BLOCK[qv]
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    rows = blocks.shape[0]
    nb = n_per_row // bs
    b = blocks.reshape(rows, nb, bb)
    if qv == 8:
        d = _f16(b[..., 0:2])
        w = d[..., None] * b[..., 2:34].view(np.int8).astype(np.float32)
    elif qv == 12:
        d, dmin = _f16(b[..., 0:2]), _f16(b[..., 2:4])
        s = b[..., 4:16]
        sc = np.concatenate([s[..., 0:4] & 63, (s[..., 8:12] & 0x0F) | ((s[..., 0:4] >> 6) << 4)], axis=-1)
        mn = np.concatenate([s[..., 4:8] & 63, (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)], axis=-1)
        qs = b[..., 16:144].reshape(rows, nb, 4, 32)
        q = np.stack([qs & 0x0F, qs >> 4], axis=3).reshape(rows, nb, 8, 32).astype(np.float32)
        ds = (d[..., None] * sc.astype(np.float32))[..., None]
        dm = (dmin[..., None] * mn.astype(np.float32))[..., None]
        w = ds * q - dm
    elif qv == 14:
        ql = b[..., 0:128].reshape(rows, nb, 2, 2, 32)
        qh = b[..., 128:192].reshape(rows, nb, 2, 1, 32)
        sc = b[..., 192:208].view(np.int8).astype(np.float32).reshape(rows, nb, 2, 4, 2, 1)
        d = _f16(b[..., 208:210])
        low = np.concatenate([ql & 0x0F, ql >> 4], axis=3)                       # [.., hb, quad, l]
        shifts = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 1, 4, 1)
        high = ((qh >> shifts) & 3) << 4
        q = (low | high).astype(np.int32) - 32
        ds = d[..., None, None, None, None] * sc
        w = ds * q.astype(np.float32).reshape(rows, nb, 2, 4, 2, 16)
    else:
        raise ValueError(f"unsupported qtype {qtype}")
    return np.ascontiguousarray(w.reshape(rows, n_per_row), dtype=np.float32)


def max_errors(expected: np.ndarray, actual: np.ndarray) -> tuple[float, float, float]:
    """(max_abs, reference-style max_rel = |d|/max(1,|e|), normalised max|d|/max|e|).

    The middle figure is the reference's own metric, tools/bench_ck_gguf_q8_gemm.hip:798-808."""
    e = np.asarray(expected, dtype=np.float64)
    a = np.asarray(actual, dtype=np.float64)
    diff = np.abs(e - a)
    max_abs = float(diff.max()) if diff.size else 0.0
    rel = float((diff / np.maximum(1.0, np.abs(e))).max()) if diff.size else 0.0
    norm = float(max_abs / max(np.abs(e).max(), 1e-30)) if diff.size else 0.0
    return max_abs, rel, norm


def dot_noise(a: np.ndarray, blocks: np.ndarray, qtype, k: int) -> np.ndarray:
    """sqrt(sum_k (a[m,k] * w[n,k])^2) per output [m, n]: the scale of what rounding every weight (or product) by a
    relative u adds to a dot product, u * dot_noise for independent roundings.  Tests use it as the element-wise noise
    floor of kernels whose tensor-core operands are 16-bit (the reference's own CPU path multiplies weights rounded to
    the storage dtype too, src/dinoml/constant_sources.py:72)."""
    w = dequantize(blocks, qtype, k).astype(np.float64)
    a = np.asarray(a, dtype=np.float64)
    return np.sqrt((a * a) @ (w * w).T)


OPERAND_ULP = {"bfloat16": 2.0 ** -8, "float16": 2.0 ** -11}


def within_operand_noise(expected, actual, noise, dtype: str, tol: float, sigmas: float = 6.0) -> bool:
    """|d| <= tol * max(1, |e|) + sigmas * ulp(dtype) * noise, element-wise: the reference harness metric
    (tools/bench_ck_gguf_q8_gemm.hip:798-808) plus the noise floor of 16-bit operand rounding."""
    e = np.asarray(expected, dtype=np.float64)
    d = np.abs(e - np.asarray(actual, dtype=np.float64))
    return bool(np.all(d <= tol * np.maximum(1.0, np.abs(e)) + sigmas * OPERAND_ULP[dtype] * np.asarray(noise)))


def dual_gemm_quant(a, blocks0, blocks1, qtype, n: int, k: int, activation: str = "silu", bias0=None, bias1=None):
    """CPU restatement of the reference's dual GEMM on dequantized weights
    (src/dinoml/lowering/ops/templates/dual_gemm_cpu.cpp.j2:52-75): two fp32-accumulated products (plus bias0 / bias1,
    :66-69), the left one through silu / fast_gelu, multiplied, all in float32.  blocks1 (and bias1) may hold ONE row:
    the right factor is then the same for every column (:58-59, the [1, K] broadcast)."""
    left = gemm_quant(a, blocks0, qtype, n, k).astype(np.float32)
    right = gemm_quant(a, blocks1, qtype, int(np.asarray(blocks1).shape[0]), k).astype(np.float32)
    if bias0 is not None:
        left = left + np.asarray(bias0, dtype=np.float32).reshape(1, -1)
        right = right + np.asarray(bias1, dtype=np.float32).reshape(1, -1)
    if activation == "silu":
        with np.errstate(over="ignore"):                 # exp(-left) may be inf for very negative left: the quotient is then -0
            act = left / (np.float32(1.0) + np.exp(-left, dtype=np.float32))
    elif activation == "fast_gelu":
        inner = np.float32(0.7978845608) * left * (np.float32(1.0) + np.float32(0.044715) * left * left)
        act = np.float32(0.5) * left * (np.float32(1.0) + np.tanh(inner, dtype=np.float32))
    else:
        raise ValueError(activation)
    return (act * right).astype(np.float32)
