from .qwen3 import Qwen3Config
from .specs import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, ModelPlan, NoPositionSpec,
                    OrderEntry, PreNormBlockSpec, RMSNormSpec, RotarySpec, names)

__all__ = ["Qwen3Config", "AttentionSpec", "EmbeddingSpec", "GatedMLPSpec", "HeadSpec", "ModelPlan",
           "NoPositionSpec", "OrderEntry", "PreNormBlockSpec", "RMSNormSpec", "RotarySpec", "names"]
