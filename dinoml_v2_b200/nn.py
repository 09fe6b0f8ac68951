"""`dml.nn.Linear` (src/dinoml/nn/__init__.py:46-79): weight [out_features, in_features], optional bias."""
from __future__ import annotations

from . import ops
from .frontend import Module, Parameter


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype: str = "float16"):
        self.in_features, self.out_features, self.dtype = int(in_features), int(out_features), dtype
        self.weight = Parameter([self.out_features, self.in_features], dtype=dtype)
        self.bias = Parameter([self.out_features], dtype=dtype) if bias else None

    def forward(self, x):
        if self.bias is None:
            return ops.gemm_rcr(x, self.weight)
        return ops.gemm_rcr_bias(x, self.weight, self.bias)
