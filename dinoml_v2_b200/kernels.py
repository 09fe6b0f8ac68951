"""Tensor-level wrappers over the C-ABI kernels (torch is used for device memory and streams only)."""
from __future__ import annotations

import torch

from . import _native
from .gguf_blocks import qtype_of, row_bytes

_TORCH_DTYPE = {"float16": torch.float16, "float32": torch.float32, "bfloat16": torch.bfloat16}
_DTYPE_NAME = {v: k for k, v in _TORCH_DTYPE.items()}


def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (the GGUF quantized-linear path has no CPU implementation)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def dequantize_rows(blocks: torch.Tensor, qtype, n_per_row: int, dtype: str = "float32", out: torch.Tensor | None = None,
                    stream=None) -> torch.Tensor:
    """uint8 [rows, row_bytes] GGUF blocks -> dense [rows, n_per_row] (bit-exact dequantization)."""
    q = qtype_of(qtype)
    _require_cuda(blocks, "blocks")
    if blocks.dtype != torch.uint8 or blocks.dim() != 2 or blocks.shape[1] != row_bytes(q, n_per_row):
        raise ValueError(f"blocks must be uint8 [rows, {row_bytes(q, n_per_row)}] for {q.name} with n_per_row={n_per_row}")
    rows = blocks.shape[0]
    if out is None:
        out = torch.empty((rows, n_per_row), dtype=_TORCH_DTYPE[dtype], device=blocks.device)
    _require_cuda(out, "out")
    rc = _native.lib().libgguf_cuda_dequantize_rows_on_stream(
        blocks.data_ptr(), q.value, rows, n_per_row, _native.DEQUANT_DTYPE[dtype], out.data_ptr(), _stream_ptr(stream))
    _native.check(rc, "libgguf_cuda_dequantize_rows_on_stream")
    return out


def gemm_rcr(a: torch.Tensor, b_quant: torch.Tensor, qtype, bias: torch.Tensor | None = None, *, variant: str = "auto",
             out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """a [..., K] x GGUF-encoded weight (uint8 [N, row_bytes]) -> [..., N], same dtype as `a`."""
    q = qtype_of(qtype)
    _require_cuda(a, "a")
    _require_cuda(b_quant, "b_quant")
    k = a.shape[-1]
    m = a.numel() // k
    n = b_quant.shape[0]
    if b_quant.dtype != torch.uint8 or b_quant.dim() != 2 or b_quant.shape[1] != row_bytes(q, k):
        raise ValueError(f"b_quant must be uint8 [N, {row_bytes(q, k)}] for {q.name} with K={k}")
    dtype = _DTYPE_NAME[a.dtype]
    if bias is not None:
        _require_cuda(bias, "bias")
        if bias.dtype != a.dtype or bias.numel() != n:
            raise ValueError("bias must have the activation dtype and N elements")
    if out is None:
        out = torch.empty(a.shape[:-1] + (n,), dtype=a.dtype, device=a.device)
    _require_cuda(out, "out")
    rc = _native.lib().dinoml_b200_gguf_gemm_rcr(
        a.data_ptr(), b_quant.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(), q.value,
        _native.DINO_DTYPE[dtype], m, n, k, _native.variant_code(variant), _stream_ptr(stream))
    _native.check(rc, "dinoml_b200_gguf_gemm_rcr")
    return out


def interleave_rows8(b0, b1):
    """Row order the gated dual GEMM expects: rows 16t..16t+7 = rows 8t..8t+7 of b0, rows 16t+8..16t+15 = of b1.
    b0, b1: [N, row_bytes] (torch tensors or numpy arrays), N % 8 == 0; a b1 of ONE row (the reference's [1, K] broadcast,
    src/dinoml/kernels/families/dual_gemm.py:60-66) is repeated N times.  Blocks are not touched."""
    if b1.shape[0] == 1 and b0.shape[0] != 1 and b1.shape[1:] == b0.shape[1:]:
        b1 = b1.expand(b0.shape[0], -1) if isinstance(b1, torch.Tensor) else __import__("numpy").broadcast_to(b1, b0.shape)
    if b0.shape != b1.shape or b0.shape[0] % 8:
        raise ValueError("both weights must have the same shape (or b1 one row) and a row count that is a multiple of 8")
    n, rb = b0.shape
    if isinstance(b0, torch.Tensor):
        return torch.stack((b0.reshape(n // 8, 8, rb), b1.reshape(n // 8, 8, rb)), dim=1).reshape(2 * n, rb).contiguous()
    import numpy as np
    return np.ascontiguousarray(np.stack((b0.reshape(n // 8, 8, rb), b1.reshape(n // 8, 8, rb)), axis=1).reshape(2 * n, rb))


def interleave_bias8(bias0, bias1):
    """[2N] bias vector of the gated dual GEMM with bias: 8 values of bias0, the 8 matching values of bias1, ... - the order of
    `interleave_rows8`.  bias1 of one element (B1 [1, K]) is repeated."""
    return interleave_rows8(bias0.reshape(-1, 1), bias1.reshape(-1, 1)).reshape(-1)


def dual_gemm_rcr(a: torch.Tensor, b01_interleaved: torch.Tensor, qtype, activation: str = "silu", *, variant: str = "auto",
                  out: torch.Tensor | None = None, stream=None, bias01_interleaved: torch.Tensor | None = None) -> torch.Tensor:
    """act(a @ dequant(B0)^T [+ bias0]) * (a @ dequant(B1)^T [+ bias1]) in one launch; `b01_interleaved` =
    interleave_rows8(B0, B1), `bias01_interleaved` = interleave_bias8(bias0, bias1) in the activation dtype.
    a [..., K] -> [..., N] with N = rows of each matrix.  Mirrors dml.ops.dual_gemm_rcr_silu / _fast_gelu and their
    _bias_ forms of the reference (src/dinoml/ops/gemm.py:63-121) for GGUF weights."""
    q = qtype_of(qtype)
    _require_cuda(a, "a")
    _require_cuda(b01_interleaved, "b01_interleaved")
    k = a.shape[-1]
    m = a.numel() // k
    rows = b01_interleaved.shape[0]
    if b01_interleaved.dtype != torch.uint8 or b01_interleaved.dim() != 2 or b01_interleaved.shape[1] != row_bytes(q, k) or rows % 16:
        raise ValueError(f"b01_interleaved must be uint8 [2N, {row_bytes(q, k)}] with N % 8 == 0 for {q.name} with K={k}")
    n = rows // 2
    if activation not in _native.ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(_native.ACTIVATIONS)}")
    if out is None:
        out = torch.empty(a.shape[:-1] + (n,), dtype=a.dtype, device=a.device)
    _require_cuda(out, "out")
    if bias01_interleaved is not None:
        _require_cuda(bias01_interleaved, "bias01_interleaved")
        if bias01_interleaved.dtype != a.dtype or bias01_interleaved.numel() != 2 * n:
            raise ValueError("bias01_interleaved must have the activation dtype and 2N elements")
    rc = _native.lib().dinoml_b200_gguf_dual_gemm_rcr_bias(
        a.data_ptr(), b01_interleaved.data_ptr(), bias01_interleaved.data_ptr() if bias01_interleaved is not None else None,
        out.data_ptr(), None, 0, q.value, _native.DINO_DTYPE[_DTYPE_NAME[a.dtype]], m, n, k,
        _native.ACTIVATIONS[activation], _native.variant_code(variant), _stream_ptr(stream))
    _native.check(rc, "dinoml_b200_gguf_dual_gemm_rcr")
    return out


def profile_gemm_rcr(a, b_quant, qtype, out, *, variant: str, iterations: int, bias=None, stream=None) -> float:
    """Milliseconds per launch of one candidate (negative on failure), timed by the library with CUDA events."""
    q = qtype_of(qtype)
    k = a.shape[-1]
    return float(_native.lib().dinoml_profile_b200_gguf_gemm_rcr(
        a.data_ptr(), b_quant.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(), q.value,
        _native.DINO_DTYPE[_DTYPE_NAME[a.dtype]], a.numel() // k, b_quant.shape[0], k, _native.variant_code(variant),
        int(iterations), _stream_ptr(stream)))


def select_variant(qtype, dtype: str, m: int, n: int, k: int) -> str:
    q = qtype_of(qtype)
    return _native.VARIANT_NAMES[_native.lib().dinoml_b200_gguf_gemm_rcr_select(q.value, _native.DINO_DTYPE[dtype], m, n, k)]


def variant_supports(variant: str, qtype, dtype: str, m: int, n: int, k: int) -> bool:
    """The library's own predicate: does this variant family serve the problem?"""
    q = qtype_of(qtype)
    family = _native.variant_code(variant) & 0xff
    return bool(_native.lib().dinoml_b200_gguf_variant_supports(family, q.value, _native.DINO_DTYPE[dtype], m, n, k))


def variant_configs(variant: str) -> int:
    """Number of tuning configurations of a variant family (valid: "family:1" .. "family:N")."""
    return int(_native.lib().dinoml_b200_gguf_variant_configs(_native.variant_code(variant) & 0xff))


def device_status() -> int:
    """Synchronizes and returns the status word written by bounded device-side waits (0 = none gave up)."""
    return int(_native.lib().dinoml_b200_gguf_device_status())
