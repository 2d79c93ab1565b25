"""Typed configuration of the Qwen3 dense decoder, read from its own ``config.json`` keys.

Fields, defaults and required keys follow ondeviceinfer/config.py:15-66 of
UESlubei/ondeviceinfer.  Two deliberate differences:

* the reference also demands ``hidden_size == num_attention_heads * head_dim``
  (ondeviceinfer/config.py:73-74); its model code works without that
  (ondeviceinfer/attention.py:106-129: q_proj is [nq*d, H], o_proj is [H, nq*d]) and
  Qwen3-32B has a query width of 8192 against a hidden size of 5120, so the rule is
  not carried;
* keys that the reference ignores but that would change the mathematics if honoured
  (``hidden_act``, ``rope_scaling``, ``use_sliding_window``) are checked, so that a
  checkpoint that needs them fails with a clear error instead of computing something else.

``attention_bias`` gives the four attention projections a bias each, as the reference's
modules do (ondeviceinfer/attention.py:106-129: ``bias=config.attention_bias``).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Mapping, Optional

from .specs import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, ModelPlan, OrderEntry,
                    PreNormBlockSpec, RMSNormSpec, RotarySpec, names)

_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
             "rms_norm_eps", "rope_theta", "tie_word_embeddings")


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    attention_bias: bool = False
    attention_dropout: float = 0.0
    bos_token_id: int = 151643
    eos_token_id: int = 151645
    pad_token_id: Optional[int] = None
    hidden_act: str = "silu"

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        if raw.get("model_type", cls.model_type) != cls.model_type:
            raise ValueError(f"Expected a Qwen3 config, got model_type={raw.get('model_type')!r}")
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise KeyError(f"config.json lacks required key(s): {', '.join(missing)}")
        if raw.get("rope_scaling") not in (None, {}):
            raise ValueError(f"rope_scaling={raw['rope_scaling']!r} is not supported: "
                             "this decoder applies plain rotary embeddings")
        if raw.get("use_sliding_window", False):
            raise ValueError("use_sliding_window=true is not supported for Qwen3 dense checkpoints")
        config = cls(
            vocab_size=int(raw["vocab_size"]),
            hidden_size=int(raw["hidden_size"]),
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=int(raw["num_attention_heads"]),
            num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=int(raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"]),
            max_position_embeddings=int(raw["max_position_embeddings"]),
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=float(raw["rope_theta"]),
            tie_word_embeddings=bool(raw["tie_word_embeddings"]),
            attention_bias=bool(raw.get("attention_bias", False)),
            attention_dropout=float(raw.get("attention_dropout", 0.0)),
            bos_token_id=raw.get("bos_token_id", 151643),
            eos_token_id=raw.get("eos_token_id", 151645),
            pad_token_id=raw.get("pad_token_id"),
            hidden_act=raw.get("hidden_act", "silu"),
        )
        config.validate()
        return config

    @classmethod
    def from_json(cls, path) -> "Qwen3Config":
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))

    def to_dict(self) -> dict:
        """A ``config.json`` dictionary that reads back as the same configuration."""
        raw = {f.name: getattr(self, f.name) for f in fields(self)}
        raw["architectures"] = [self.architecture]
        raw["model_type"] = self.model_type
        return raw

    # ------------------------------------------------------------------ checks

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim"):
            if getattr(self, key) <= 0:
                raise ValueError(f"{key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ValueError("Q heads must be divisible by KV heads for GQA")
        if self.head_dim % 2 != 0:
            raise ValueError("RoPE requires an even head dimension")
        if self.hidden_act != "silu":
            raise ValueError(f"hidden_act={self.hidden_act!r}: the Qwen3 feed-forward uses silu")
        if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
            raise ValueError("rms_norm_eps and rope_theta must be positive")

    @property
    def num_key_value_groups(self) -> int:
        """Query heads per key/value head (ondeviceinfer/config.py:76-79)."""
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def stop_token_ids(self) -> tuple:
        eos = self.eos_token_id
        if eos is None:
            return ()
        return tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)

    # ------------------------------------------------------------------ the plan

    def to_plan(self) -> ModelPlan:
        """Layer table of the Qwen3 dense decoder (ondeviceinfer/model.py:27-38,77-89,137-144):
        every layer is a pre-norm block of grouped-query attention with per-head Q/K
        RMSNorm and rotary embeddings, then a SiLU-gated feed-forward; layers run once
        each, in index order; the head is tied to the embedding when configured."""
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            attention = AttentionSpec(
                hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                position=RotarySpec(head_dim=self.head_dim, theta=self.rope_theta),
                prefix=p + "self_attn.",
                names=names(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight",
                            q_norm="q_norm.weight", k_norm="k_norm.weight",
                            **({"q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                                "o_bias": "o_proj.bias"} if self.attention_bias else {})),
                qk_norm_eps=self.rms_norm_eps, window=None, scale=None)
            mlp = GatedMLPSpec(
                hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
                activation=self.hidden_act, prefix=p + "mlp.",
                names=names(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight"))
            layers.append(PreNormBlockSpec(
                mixer_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps, p + "input_layernorm.weight"),
                mixer=attention,
                ffn_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps, p + "post_attention_layernorm.weight"),
                ffn=mlp))
        plan = ModelPlan(
            embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, "model.embed_tokens.weight"),
            layers=tuple(layers),
            order=tuple(OrderEntry(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
            head=HeadSpec(self.vocab_size, self.hidden_size,
                          None if self.tie_word_embeddings else "lm_head.weight"),
            # a tied checkpoint may still carry a copy of the head; it is not read
            ignored_tensors=("lm_head.weight",) if self.tie_word_embeddings else ())
        plan.validate()
        return plan
