from .base import MATRIX, TABLE, VECTOR, ParamSpec, Part
from .context import Runtime, StepContext
from .norm import RMSNorm
from .rope import RotaryEmbedding, inverse_frequencies
from .attention import Attention
from .mamba2 import Mamba2
from .mlp import GatedMLP
from .embedding import Embedding, LMHead
from .block import PreNormParallelBlock

__all__ = ["MATRIX", "TABLE", "VECTOR", "ParamSpec", "Part", "Runtime", "StepContext", "RMSNorm",
           "RotaryEmbedding", "inverse_frequencies", "Attention", "Mamba2", "GatedMLP", "Embedding", "LMHead",
           "PreNormParallelBlock"]
