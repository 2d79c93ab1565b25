"""Configuration and registry (no GPU)."""

import json

import pytest

import ondeviceinfer_b200  # noqa: F401  (registers the architectures)
import plain_qwen3 as plain
from ondeviceinfer_b200.config import AttentionSpec, GatedMLPSpec, ModelPlan, OrderEntry, Qwen3Config
from ondeviceinfer_b200.registry import (architecture_name, config_from_dict, config_from_folder,
                                         known_architectures, register_architecture)

RAW_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
    "intermediate_size": 12288, "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000,
    "tie_word_embeddings": False, "hidden_act": "silu", "sliding_window": None, "use_sliding_window": False,
    "rope_scaling": None, "torch_dtype": "bfloat16",
}


def test_config_reads_its_own_keys_and_derives_groups(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(RAW_8B))
    config = config_from_folder(tmp_path)
    assert isinstance(config, Qwen3Config)
    assert config.num_key_value_groups == 4
    assert (config.q_size, config.kv_size) == (4096, 1024)
    assert config.eos_token_id == 151645 and config.bos_token_id == 151643 and config.pad_token_id is None
    assert config.stop_token_ids == (151645,)


def test_head_dim_defaults_to_hidden_over_heads():
    raw = {k: v for k, v in RAW_8B.items() if k != "head_dim"}
    raw.update(hidden_size=2048, num_attention_heads=16)
    assert config_from_dict(raw).head_dim == 128


def test_query_width_may_differ_from_hidden_size():
    config = config_from_dict(plain.TINY_B)
    assert config.q_size == 192 and config.hidden_size == 96
    raw = dict(RAW_8B, hidden_size=5120, num_attention_heads=64, num_hidden_layers=64, intermediate_size=25600)
    assert config_from_dict(raw).q_size == 8192


def test_missing_keys_are_named_together():
    raw = {k: v for k, v in RAW_8B.items() if k not in ("rope_theta", "rms_norm_eps")}
    with pytest.raises(KeyError) as error:
        config_from_dict(raw)
    assert "rope_theta" in str(error.value) and "rms_norm_eps" in str(error.value)


@pytest.mark.parametrize("change,exc", [
    ({"num_key_value_heads": 5}, ValueError),
    ({"head_dim": 127}, ValueError),
    ({"hidden_act": "gelu"}, ValueError),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, ValueError),
    ({"use_sliding_window": True, "sliding_window": 4096}, ValueError),
    ({"model_type": "llama"}, ValueError),
    ({"num_hidden_layers": 0}, ValueError),
])
def test_what_would_change_the_mathematics_is_refused(change, exc):
    with pytest.raises(exc):
        config_from_dict(dict(RAW_8B, **change))


def test_registry_chooses_by_architecture_name_and_falls_back_to_model_type():
    assert architecture_name(RAW_8B) == "Qwen3ForCausalLM"
    assert architecture_name({k: v for k, v in RAW_8B.items() if k != "architectures"}) == "Qwen3ForCausalLM"
    with pytest.raises(KeyError) as error:
        architecture_name(dict(RAW_8B, architectures=["LlamaForCausalLM"]))
    assert "Qwen3ForCausalLM" in str(error.value)
    with pytest.raises(KeyError):
        architecture_name({"hidden_size": 8})
    assert "Qwen3ForCausalLM" in known_architectures()


def test_register_architecture_checks_the_interface():
    class Incomplete:
        pass

    with pytest.raises(TypeError):
        register_architecture("IncompleteLM", Incomplete)


def test_round_trip_through_config_json(tmp_path):
    config = config_from_dict(plain.TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    assert config_from_folder(tmp_path) == config


@pytest.mark.parametrize("raw", [plain.TINY_A, plain.TINY_B, RAW_8B])
def test_plan_carries_every_size_and_constant(raw):
    config = config_from_dict(raw)
    plan = config.to_plan()
    assert isinstance(plan, ModelPlan)
    assert len(plan.layers) == config.num_hidden_layers
    assert plan.order == tuple(OrderEntry(i) for i in range(config.num_hidden_layers))
    block = plan.layers[-1]
    attention, mlp = block.mixer, block.ffn
    assert isinstance(attention, AttentionSpec) and isinstance(mlp, GatedMLPSpec)
    assert (attention.num_heads, attention.num_kv_heads, attention.head_dim) == (
        config.num_attention_heads, config.num_key_value_heads, config.head_dim)
    assert attention.qk_norm_eps == config.rms_norm_eps and attention.position.theta == config.rope_theta
    assert attention.window is None and attention.scale is None
    assert mlp.intermediate_size == config.intermediate_size
    assert block.mixer_norm.eps == config.rms_norm_eps and plan.final_norm.size == config.hidden_size
    last = config.num_hidden_layers - 1
    assert attention.name("q_norm") == f"model.layers.{last}.self_attn.q_norm.weight"
    assert mlp.name("down") == f"model.layers.{last}.mlp.down_proj.weight"
    assert (plan.head.weight_name is None) == config.tie_word_embeddings


def test_plan_order_is_checked():
    plan = config_from_dict(plain.TINY_A).to_plan()
    bad = ModelPlan(plan.embedding, plan.layers, (OrderEntry(0), OrderEntry(5)), plan.final_norm, plan.head)
    with pytest.raises(ValueError):
        bad.validate()
    forward_ref = ModelPlan(plan.embedding, plan.layers, (OrderEntry(0, cache_from=1), OrderEntry(1)),
                            plan.final_norm, plan.head)
    with pytest.raises(ValueError):
        forward_ref.validate()
    ok = ModelPlan(plan.embedding, plan.layers, (OrderEntry(0), OrderEntry(1), OrderEntry(0), OrderEntry(1, cache_from=1)),
                   plan.final_norm, plan.head)
    ok.validate()


def test_attention_bias_gives_the_four_projections_a_bias_each():
    """ondeviceinfer/attention.py:106-129 builds q, k, v and o projections with bias=config.attention_bias."""
    from ondeviceinfer_b200.engine.model import DecoderModel

    plain_plan = config_from_dict(RAW_8B).to_plan()
    biased_plan = config_from_dict(dict(RAW_8B, attention_bias=True)).to_plan()
    assert not any(plain_plan.layers[0].mixer.has(role) for role in ("q_bias", "k_bias", "v_bias", "o_bias"))
    mixer = biased_plan.layers[3].mixer
    assert mixer.name("q_bias") == "model.layers.3.self_attn.q_proj.bias"
    assert mixer.name("o_bias") == "model.layers.3.self_attn.o_proj.bias"
    small = dict(RAW_8B, attention_bias=True, num_hidden_layers=1)
    shapes = {d.name: d.shape for d in DecoderModel(config_from_dict(small).to_plan()).tensor_decls()}
    assert shapes["model.layers.0.self_attn.q_proj.bias"] == (4096,)
    assert shapes["model.layers.0.self_attn.k_proj.bias"] == (1024,)
    assert shapes["model.layers.0.self_attn.v_proj.bias"] == (1024,)
    assert shapes["model.layers.0.self_attn.o_proj.bias"] == (4096,)
    assert config_from_dict(small).to_dict()["attention_bias"] is True
