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


DUAL_GEMM_ACTIVATIONS = ("silu", "fast_gelu")     # the two the reference's CPU template implements (dual_gemm_cpu.cpp.j2:66-70)


def _dual_gemm(activation: str, a: Tensor, b0: Tensor, b1: Tensor) -> Tensor:
    """act(a @ b0^T) * (a @ b1^T) - dml.ops.dual_gemm_rcr_<activation> (src/dinoml/ops/gemm.py:63-121,
    src/dinoml/kernels/families/dual_gemm.py:36-76).  Here b0 and b1 must both be [N, K] (no [1, K] broadcast)."""
    op = f"dual_gemm_rcr_{activation}"
    if len(a.shape) < 1 or len(b0.shape) != 2 or len(b1.shape) != 2:
        raise ValueError(f"{op} expects A[..., K] and rank-2 B0 / B1 tensors")
    if a.dtype not in GEMM_SUPPORTED_DTYPES or a.dtype != b0.dtype or a.dtype != b1.dtype:
        raise ValueError(f"{op} operands must share one supported dtype, got {a.dtype}, {b0.dtype}, {b1.dtype}")
    k = _static(a.shape[-1])
    if k is None or k != _static(b0.shape[1]) or k != _static(b1.shape[1]):
        raise ValueError(f"{op} expected B0[N, K] and B1[N, K] with K = {a.shape[-1]}, got {b0.shape} and {b1.shape}")
    if tuple(b0.shape) != tuple(b1.shape):
        raise ValueError(f"{op} expected B1 to match B0 {list(b0.shape)}, got {list(b1.shape)}")
    return current_builder().add_node(op, [a, b0, b1], tuple(a.shape[:-1]) + (b0.shape[0],), a.dtype, {"activation": activation})


def dual_gemm_rcr_silu(a: Tensor, b0: Tensor, b1: Tensor) -> Tensor:
    return _dual_gemm("silu", a, b0, b1)


def dual_gemm_rcr_fast_gelu(a: Tensor, b0: Tensor, b1: Tensor) -> Tensor:
    return _dual_gemm("fast_gelu", a, b0, b1)
