"""`dml.ops.gemm_rcr` / `gemm_rcr_bias` - the operator the quantized linear rides on.  Same signature and
shape / dtype rules as the reference (src/dinoml/ops/gemm.py:46-60, 681-690;
src/dinoml/kernels/families/gemm.py:67-92): a [..., K], b [N, K] ("rcr": row-major A, column-major B),
bias [N] or [1, N], out [..., N]; all operands share one dtype in {float16, float32, bfloat16}."""
from __future__ import annotations

from .frontend import Tensor, current_builder

GEMM_SUPPORTED_DTYPES = ("float16", "float32", "bfloat16")     # src/dinoml/kernels/families/gemm.py:10


def _static(d) -> int | None:
    return d if isinstance(d, int) else None


def _gemm(op: str, a: Tensor, b: Tensor, bias: Tensor | None) -> Tensor:
    if len(a.shape) < 1 or len(b.shape) != 2:
        raise ValueError(f"{op} expects a [..., K] and b [N, K], got {a.shape} and {b.shape}")
    if a.dtype not in GEMM_SUPPORTED_DTYPES:
        raise ValueError(f"{op} does not support dtype {a.dtype}")
    if a.dtype != b.dtype or (bias is not None and bias.dtype != a.dtype):
        raise ValueError(f"{op} operands must share one dtype, got {a.dtype}, {b.dtype}" + (f", {bias.dtype}" if bias else ""))
    k_a, k_b = _static(a.shape[-1]), _static(b.shape[1])
    if k_a is None or k_b is None or k_a != k_b:
        raise ValueError(f"{op} K dimensions differ or are dynamic: a {a.shape}, b {b.shape}")
    n = b.shape[0]
    if bias is not None and tuple(bias.shape) not in ((n,), (1, n)):
        raise ValueError(f"{op} bias must be [N] or [1, N], got {bias.shape}")
    return current_builder().add_node(op, [a, b] + ([bias] if bias is not None else []), tuple(a.shape[:-1]) + (n,), a.dtype)


def gemm_rcr(a: Tensor, b: Tensor) -> Tensor:
    return _gemm("gemm_rcr", a, b, None)


def gemm_rcr_bias(a: Tensor, b: Tensor, bias: Tensor) -> Tensor:
    return _gemm("gemm_rcr_bias", a, b, bias)
