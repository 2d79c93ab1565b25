"""Weights: binding by name, one error for everything that does not fit, random-weights mode (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import save_file

import plain_qwen3 as plain
from helpers import write_model_folder
from ondeviceinfer_b200 import WeightsError, write_random_model
from ondeviceinfer_b200.engine.model import DecoderModel
from ondeviceinfer_b200.registry import config_from_dict, config_from_folder
from ondeviceinfer_b200.weights import Fetcher, RandomSource, SafetensorsSource, check


def decls_of(cfg):
    plan = config_from_dict(cfg).to_plan()
    return DecoderModel(plan).tensor_decls(), plan


@pytest.mark.parametrize("cfg", [plain.TINY_A, plain.TINY_B])
def test_declared_tensors_are_the_checkpoint_names(cfg):
    decls, _ = decls_of(cfg)
    assert {d.name: tuple(d.shape) for d in decls} == plain.tensor_shapes(cfg)


def test_folder_loads_by_name(tmp_path):
    weights = plain.random_weights(plain.TINY_B, 1)
    write_model_folder(tmp_path, plain.TINY_B, weights)
    source = SafetensorsSource(tmp_path)
    decls, plan = decls_of(plain.TINY_B)
    check(decls, source.stored(), plan.ignored_tensors)
    name = "model.layers.2.self_attn.k_norm.weight"
    assert torch.equal(source.fetch(name), weights[name])
    with pytest.raises(KeyError):
        source.fetch("model.layers.9.self_attn.k_norm.weight")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    weights = plain.random_weights(plain.TINY_B, 1)
    del weights["model.layers.1.mlp.up_proj.weight"]
    del weights["model.norm.weight"]
    weights["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    weights["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(96, 96, dtype=torch.bfloat16)
    write_model_folder(tmp_path, plain.TINY_B, weights)
    decls, plan = decls_of(plain.TINY_B)
    with pytest.raises(WeightsError) as error:
        check(decls, SafetensorsSource(tmp_path).stored(), plan.ignored_tensors)
    e = error.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(e.wrong_shape) == 1 and "(192, 96)" in e.wrong_shape[0] and "(96, 96)" in e.wrong_shape[0]
    text = str(e)
    for piece in ("model.norm.weight", "rotary_emb.inv_freq", "q_proj.weight"):
        assert piece in text


def test_tied_head_is_not_required_and_ignored_if_present(tmp_path):
    weights = plain.random_weights(plain.TINY_A, 0)
    assert "lm_head.weight" not in weights
    decls, plan = decls_of(plain.TINY_A)
    write_model_folder(tmp_path / "without", plain.TINY_A, weights)
    check(decls, SafetensorsSource(tmp_path / "without").stored(), plan.ignored_tensors)
    weights["lm_head.weight"] = weights["model.embed_tokens.weight"].clone()
    write_model_folder(tmp_path / "with", plain.TINY_A, weights)
    check(decls, SafetensorsSource(tmp_path / "with").stored(), plan.ignored_tensors)


def test_untied_head_is_required(tmp_path):
    weights = plain.random_weights(plain.TINY_B, 1)
    del weights["lm_head.weight"]
    write_model_folder(tmp_path, plain.TINY_B, weights)
    decls, plan = decls_of(plain.TINY_B)
    with pytest.raises(WeightsError) as error:
        check(decls, SafetensorsSource(tmp_path).stored(), plan.ignored_tensors)
    assert error.value.missing == ["lm_head.weight"]


def test_sharded_folder_with_index(tmp_path):
    weights = plain.random_weights(plain.TINY_B, 1)
    names = sorted(weights)
    halves = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    weight_map = {}
    for file, members in halves.items():
        save_file({n: weights[n].contiguous() for n in members}, str(tmp_path / file))
        weight_map.update({n: file for n in members})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    (tmp_path / "config.json").write_text(json.dumps(plain.TINY_B))
    source = SafetensorsSource(tmp_path)
    decls, plan = decls_of(plain.TINY_B)
    check(decls, source.stored(), plan.ignored_tensors)
    assert torch.equal(source.fetch(names[-1]), weights[names[-1]])


def test_folder_without_safetensors(tmp_path):
    with pytest.raises(FileNotFoundError):
        SafetensorsSource(tmp_path)
    with pytest.raises(FileNotFoundError):
        config_from_folder(tmp_path)


def test_held_precisions():
    """Matrices in the compute dtype; small floating tensors in fp32 (a tensor stored in
    32-bit stays so); integer tables as int32."""
    class Source:
        tensors = {"m": torch.randn(4, 4, dtype=torch.bfloat16), "v16": torch.randn(4, dtype=torch.bfloat16),
                   "v32": torch.randn(4, dtype=torch.float32) * 1.000001, "i": torch.arange(5, dtype=torch.int64)}

        def fetch(self, name):
            return self.tensors[name]

    fetch = Fetcher(Source(), torch.bfloat16, "cpu")
    assert fetch.matrix("m").dtype == torch.bfloat16
    assert fetch.vector("v16").dtype == torch.float32 and torch.equal(fetch.vector("v16"), Source.tensors["v16"].float())
    assert fetch.vector("v32").dtype == torch.float32 and torch.equal(fetch.vector("v32"), Source.tensors["v32"])
    assert fetch.integer("i").dtype == torch.int32
    assert Fetcher(Source(), torch.float32, "cpu").matrix("m").dtype == torch.float32
    with pytest.raises(TypeError):
        fetch.matrix("i")
    with pytest.raises(TypeError):
        fetch.integer("m")


def test_random_model_folder_is_complete_and_repeatable(tmp_path):
    a = write_random_model(tmp_path / "a", plain.TINY_B, seed=7)
    b = write_random_model(tmp_path / "b", config_from_dict(plain.TINY_B), seed=7)
    c = write_random_model(tmp_path / "c", plain.TINY_B, seed=8)
    sa, sb, sc = SafetensorsSource(a), SafetensorsSource(b), SafetensorsSource(c)
    assert {n: s.shape for n, s in sa.stored().items()} == plain.tensor_shapes(plain.TINY_B)
    assert all(s.dtype == torch.bfloat16 for s in sa.stored().values())
    for name in sa.stored():
        assert torch.equal(sa.fetch(name), sb.fetch(name))
    assert not torch.equal(sa.fetch("lm_head.weight"), sc.fetch("lm_head.weight"))
    assert config_from_folder(a) == config_from_dict(plain.TINY_B)
    matrix = sa.fetch("model.layers.0.mlp.gate_proj.weight").float()
    norm = sa.fetch("model.layers.0.input_layernorm.weight").float()
    assert abs(float(matrix.std()) - 0.02) < 0.002 and abs(float(matrix.mean())) < 0.002
    assert abs(float(norm.mean()) - 1.0) < 0.01 and 0.003 < float(norm.std()) < 0.02


def test_random_source_is_order_independent():
    decls, _ = decls_of(plain.TINY_A)
    one, two = RandomSource(decls, 3), RandomSource(decls, 3)
    names = [d.name for d in decls]
    forward = {n: one.fetch(n) for n in names}
    backward = {n: two.fetch(n) for n in reversed(names)}
    assert all(torch.equal(forward[n], backward[n]) for n in names)
