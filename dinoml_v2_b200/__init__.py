"""B200-native implementation of DinoML v2's GGUF quantized-linear path.

Public surface mirrors `import dinoml as dml` for this path: `dml.trace`, `dml.compile`, `dml.Target`,
`dml.ops.gemm_rcr[_bias]`, `dml.nn.Linear`, `dml.gguf_constant`, `dml.runtime.load` (src/dinoml/__init__.py:1-26)."""
from . import nn, ops, runtime  # noqa: F401
from .compiler import Artifact, Target, compile  # noqa: F401
from .constant_sources import GGUFConstant, MaterializedConstant, gguf_constant  # noqa: F401
from .frontend import Dim, Module, Parameter, Tensor, TensorSpec, trace  # noqa: F401

__all__ = ["Artifact", "Dim", "GGUFConstant", "MaterializedConstant", "Module", "Parameter", "Target", "Tensor", "TensorSpec",
           "compile", "gguf_constant", "nn", "ops", "runtime", "trace"]
