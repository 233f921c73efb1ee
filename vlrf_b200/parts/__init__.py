from .block import PreNormBlock
from .context import StepContext, Workspace
from .embedding import LMHead, TokenEmbedding
from .feed_forward import DenseMLP
from .mixer import CausalSelfAttention
from .norm import LayerNorm
from .position import LearnedAbsolutePositions
from .registry import get_part, part_names, register_part, unregister_part

__all__ = ["PreNormBlock", "StepContext", "Workspace", "LMHead", "TokenEmbedding", "DenseMLP",
           "CausalSelfAttention", "LayerNorm", "LearnedAbsolutePositions", "get_part", "part_names",
           "register_part", "unregister_part"]
