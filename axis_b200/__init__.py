"""axis_b200 — B200-native engine for the compiled training step.

Public surface mirrors the reference for this path: `compile_model`,
`CompiledTransformer`, `Engine`, `op` and the op-kind constants."""
from axis_b200 import checkpoint
from axis_b200.compile import CompiledTransformer, compile_model, greedy_owner
from axis_b200.engine import Engine, op
from axis_b200.model import Transformer

__all__ = ["CompiledTransformer", "compile_model", "greedy_owner", "Engine", "op", "Transformer", "checkpoint"]
__version__ = "0.1.0"
