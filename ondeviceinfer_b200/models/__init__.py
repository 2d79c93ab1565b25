"""Architectures known to the registry.  Importing this package registers them."""

from ..config.qwen3 import Qwen3Config
from ..registry import register_architecture

register_architecture("Qwen3ForCausalLM", Qwen3Config, model_type="qwen3")
