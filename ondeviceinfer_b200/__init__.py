"""ondeviceinfer_b200: a small Qwen3 dense inference library for one NVIDIA B200.

From a model folder (``config.json`` + safetensors) to generated tokens: typed
configuration and architecture registry, weights by checkpoint name, layers composed
from parts, a paged cache with a slot per sequence, one step function over batches of
unequal lengths, a generation loop with greedy and temperature sampling, and
hand-written sm_100a CUDA kernels underneath (bfloat16 for serving, true float32 as the
reference path).  There is no CPU execution path.
"""

from . import api
from .api import (GenerationResult, ResidentModel, generate, greedy_generate, load_resident_model,
                  random_resident_model)
from .cache import CacheCapacityError, KVNeed, SequenceCache, StateNeed
from .config import Qwen3Config
from .parts import register_part
from .registry import register_architecture
from .sampling import Sampler
from .weights import WeightsError, write_random_model

__all__ = ["GenerationResult", "ResidentModel", "generate", "greedy_generate", "load_resident_model",
           "random_resident_model", "CacheCapacityError", "KVNeed", "SequenceCache", "StateNeed",
           "Qwen3Config", "register_part", "register_architecture", "Sampler", "WeightsError",
           "write_random_model"]
