from .base import Part, Runtime, build_part, register_part
from .linear import gated_linear, linear
from . import norm, position, attention, mlp, block, embedding  # noqa: F401  (registers the built-in parts)
from .attention import Attention
from .embedding import OutputHead, TokenEmbedding
from .block import PreNormBlock
from .mlp import GatedMLP
from .norm import RMSNorm
from .position import NoPosition, Rotary

__all__ = ["Part", "Runtime", "build_part", "register_part", "linear", "gated_linear", "Attention", "PreNormBlock",
           "GatedMLP", "RMSNorm", "NoPosition", "Rotary", "TokenEmbedding", "OutputHead"]
