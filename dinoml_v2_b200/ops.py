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


def _dual_gemm(activation: str, a: Tensor, b0: Tensor, b1: Tensor, bias0: Tensor | None = None, bias1: Tensor | None = None) -> Tensor:
    """act(a @ b0^T [+ bias0]) * (a @ b1^T [+ bias1]) - dml.ops.dual_gemm_rcr_[bias_]<activation> (src/dinoml/ops/gemm.py:63-121,
    src/dinoml/kernels/families/dual_gemm.py:36-76).  b1 is [N, K] or [1, K] (then bias1 has one element): the shape rules
    of DualGemmOpSpec.validate_shapes."""
    has_bias = bias0 is not None or bias1 is not None
    op = f"dual_gemm_rcr_{'bias_' if has_bias else ''}{activation}"
    if len(a.shape) < 1 or len(b0.shape) != 2 or len(b1.shape) != 2:
        raise ValueError(f"{op} expects A[..., K] and rank-2 B0 / B1 tensors")
    if a.dtype not in GEMM_SUPPORTED_DTYPES or a.dtype != b0.dtype or a.dtype != b1.dtype:
        raise ValueError(f"{op} operands must share one supported dtype, got {a.dtype}, {b0.dtype}, {b1.dtype}")
    k = _static(a.shape[-1])
    if k is None or k != _static(b0.shape[1]) or k != _static(b1.shape[1]):
        raise ValueError(f"{op} expected B0[N, K] and B1[N, K] with K = {a.shape[-1]}, got {b0.shape} and {b1.shape}")
    n, b1_n = _static(b0.shape[0]), _static(b1.shape[0])
    if b1_n != n and b1_n != 1:
        raise ValueError(f"{op} expected B1[N, K] or B1[1, K] matching N={n}, got {list(b1.shape)}")
    inputs = [a, b0, b1]
    if has_bias:
        if bias0 is None or bias1 is None:
            raise ValueError(f"{op} expects both bias0 and bias1")
        for name, bias, want in (("bias0", bias0, n), ("bias1", bias1, b1_n)):
            if bias.dtype != a.dtype or _static(bias.shape[-1]) != want or any(_static(d) != 1 for d in bias.shape[:-1]):
                raise ValueError(f"{op} expected {name} with {want} elements of dtype {a.dtype}, got {list(bias.shape)} {bias.dtype}")
        inputs += [bias0, bias1]
    return current_builder().add_node(op, inputs, tuple(a.shape[:-1]) + (b0.shape[0],), a.dtype, {"activation": activation})


def dual_gemm_rcr_silu(a: Tensor, b0: Tensor, b1: Tensor) -> Tensor:
    return _dual_gemm("silu", a, b0, b1)


def dual_gemm_rcr_fast_gelu(a: Tensor, b0: Tensor, b1: Tensor) -> Tensor:
    return _dual_gemm("fast_gelu", a, b0, b1)


def dual_gemm_rcr_bias_silu(a: Tensor, b0: Tensor, b1: Tensor, bias0: Tensor, bias1: Tensor) -> Tensor:
    return _dual_gemm("silu", a, b0, b1, bias0, bias1)


def dual_gemm_rcr_bias_fast_gelu(a: Tensor, b0: Tensor, b1: Tensor, bias0: Tensor, bias1: Tensor) -> Tensor:
    return _dual_gemm("fast_gelu", a, b0, b1, bias0, bias1)
