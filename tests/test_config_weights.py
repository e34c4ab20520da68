"""Configuration, registry, checkpoint reading, weight errors and the random-weights mode (CPU)."""

import json

import pytest
import torch
from safetensors.torch import save_file

from mini_llm_runtime_b200.config import (ModelSpec, PartSpec, Qwen2Config, RunStep, config_from_dict,
                                          known_architectures, load_config, qwen2_model_spec,
                                          register_architecture, unregister_architecture)
from mini_llm_runtime_b200.models import build_model, load_model, write_random_model_dir
from mini_llm_runtime_b200.weights import WeightError, check_tensors, random_tensors, read_checkpoint
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_config_round_trip_and_derived_sizes():
    data = TINY_A.to_dict()
    assert data["architectures"] == ["Qwen2ForCausalLM"] and data["model_type"] == "qwen2"
    again = config_from_dict(data)
    assert again == TINY_A and again.head_dim == 16 and again.gqa_group_size == 2
    assert TINY_C.head_dim == 48 and TINY_C.layer_window(1) is None and TINY_C.layer_window(2) == 21


def test_config_requires_every_key_and_lists_the_missing_ones():
    data = TINY_A.to_dict()
    del data["rope_theta"], data["rms_norm_eps"]
    with pytest.raises(KeyError) as error:
        Qwen2Config.from_dict(data)
    assert "rope_theta" in str(error.value) and "rms_norm_eps" in str(error.value)


@pytest.mark.parametrize("change,message", [
    ({"model_type": "llama"}, "model_type"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "silu"),
    ({"num_key_value_heads": 3}, "divisible"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"head_dim": 15}, "even"),
])
def test_config_rejects(change, message):
    with pytest.raises((ValueError, KeyError)) as error:
        Qwen2Config.from_dict(dict(TINY_A.to_dict(), **change))
    assert message in str(error.value)


def test_registry_picks_by_architecture_name_and_lists_known_names():
    assert "Qwen2ForCausalLM" in known_architectures()
    with pytest.raises(KeyError) as error:
        config_from_dict(dict(TINY_A.to_dict(), architectures=["MysteryForCausalLM"]))
    assert "Qwen2ForCausalLM" in str(error.value)
    with pytest.raises(KeyError):
        config_from_dict({k: v for k, v in TINY_A.to_dict().items() if k != "architectures"})
    register_architecture("OtherQwen", Qwen2Config.from_dict, qwen2_model_spec)
    try:
        assert config_from_dict(dict(TINY_A.to_dict(), architectures=["OtherQwen"])) == TINY_A
        with pytest.raises(ValueError):
            register_architecture("OtherQwen", Qwen2Config.from_dict, qwen2_model_spec)
    finally:
        unregister_architecture("OtherQwen")


def test_model_spec_is_data():
    spec = qwen2_model_spec(TINY_C)
    assert len(spec.layers) == 4 and spec.cache_entries == 4
    assert [layer.mixer.args["window"] for layer in spec.layers] == [None, None, 21, 21]
    assert spec.layers[1].mixer.prefix == "model.layers.1.self_attn."
    assert spec.head.kind == "linear_head" and qwen2_model_spec(TINY_A).head.kind == "tied_head"
    needs = build_model(TINY_C, "float32").cache_needs()
    assert needs[0] == needs[1] and needs[2] == needs[3] and needs[0] != needs[2]


def test_run_order_validation():
    spec = qwen2_model_spec(TINY_A)

    def with_order(order):
        return ModelSpec(spec.architecture, spec.vocab_size, spec.hidden_size, spec.max_positions,
                         spec.embedding, spec.layers, tuple(order), spec.final_norm, spec.head)

    twice = with_order([RunStep(0, 0), RunStep(1, 1), RunStep(1, 2), RunStep(0, 0, writes_cache=False)])
    assert twice.cache_entries == 3
    with pytest.raises(ValueError):
        with_order([RunStep(0, 0), RunStep(1, 0)])             # two writers of one entry
    with pytest.raises(ValueError):
        with_order([RunStep(0, 1, writes_cache=False), RunStep(1, 1)])   # read before write
    with pytest.raises(ValueError):
        with_order([RunStep(0, 0), RunStep(5, 1)])             # no such layer
    with pytest.raises(ValueError):
        with_order([RunStep(0, 0), RunStep(1, 2)])             # gap in the entries


def test_random_weights_are_reproducible_and_follow_the_distributions():
    expected = build_model(TINY_B, "float32").expected_tensors()
    first = random_tensors(expected, 3)
    again = random_tensors(expected, 3)
    other = random_tensors(expected, 4)
    assert all(torch.equal(first[k], again[k]) for k in first)
    assert not torch.equal(first["model.embed_tokens.weight"], other["model.embed_tokens.weight"])
    assert all(t.dtype == torch.bfloat16 for t in first.values())
    matrix = first["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(float(matrix.std()) - 0.02) < 0.002 and abs(float(matrix.mean())) < 0.002
    norm = first["model.layers.2.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.02
    assert "lm_head.weight" in first
    assert "lm_head.weight" not in random_tensors(build_model(TINY_A, "float32").expected_tensors(), 3)


def test_model_folder_round_trip(tmp_path):
    write_random_model_dir(tmp_path, TINY_B, seed=9)
    entry, config = load_config(tmp_path)
    assert entry.name == "Qwen2ForCausalLM" and config == TINY_B
    stored = read_checkpoint(tmp_path)
    expected = build_model(TINY_B, "float32").expected_tensors()
    assert set(stored) == {name for name, spec in expected.items() if not spec.optional}
    generated = random_tensors(expected, 9)
    assert all(torch.equal(stored[k], generated[k]) for k in stored)
    assert all(t.dtype == torch.bfloat16 for t in stored.values())


def test_32_bit_tensors_stay_32_bit_and_integer_tables_become_int32(tmp_path):
    tensors = {"a": torch.ones(3, dtype=torch.float32), "b": torch.ones(3, dtype=torch.bfloat16),
               "c": torch.arange(4, dtype=torch.int64)}
    save_file(tensors, str(tmp_path / "model.safetensors"))
    stored = read_checkpoint(tmp_path)
    assert stored["a"].dtype == torch.float32 and stored["b"].dtype == torch.bfloat16
    assert stored["c"].dtype == torch.int32
    model = build_model(TINY_A, "bfloat16")
    weights = random_tensors(model.expected_tensors(), 1)
    weights["model.norm.weight"] = weights["model.norm.weight"].float()
    model.load(weights, "cpu")
    assert model.final_norm.weight.dtype == torch.float32
    assert model.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    model = build_model(TINY_A, "float32")
    tensors = random_tensors(model.expected_tensors(), 1)
    del tensors["model.layers.0.self_attn.k_proj.bias"], tensors["model.norm.weight"]
    tensors["model.layers.1.mlp.up_proj.weight"] = torch.zeros(7, 7)
    tensors["model.layers.9.extra.weight"] = torch.zeros(1)
    tensors["stray"] = torch.zeros(1)
    with pytest.raises(WeightError) as error:
        model.load(tensors, "cpu")
    text = str(error.value)
    for name in ("model.layers.0.self_attn.k_proj.bias", "model.norm.weight", "model.layers.9.extra.weight",
                 "stray", "model.layers.1.mlp.up_proj.weight", "(7, 7)", "(128, 64)"):
        assert name in text
    assert error.value.missing == ("model.layers.0.self_attn.k_proj.bias", "model.norm.weight")
    assert error.value.unexpected == ("model.layers.9.extra.weight", "stray")
    assert error.value.wrong_shape[0][0] == "model.layers.1.mlp.up_proj.weight"


def test_tied_checkpoint_may_repeat_the_embedding_but_not_change_it():
    model = build_model(TINY_A, "float32")
    tensors = random_tensors(model.expected_tensors(), 1)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    model.load(tensors, "cpu")
    tensors["lm_head.weight"] = tensors["lm_head.weight"] + 1
    with pytest.raises(ValueError):
        build_model(TINY_A, "float32").load(tensors, "cpu")
    untied = build_model(TINY_B, "float32")
    weights = random_tensors(untied.expected_tensors(), 1)
    del weights["lm_head.weight"]
    with pytest.raises(WeightError) as error:
        untied.load(weights, "cpu")
    assert error.value.missing == ("lm_head.weight",)


def test_sharded_checkpoints(tmp_path):
    expected = build_model(TINY_A, "float32").expected_tensors()
    tensors = random_tensors(expected, 2)
    names = sorted(tensors)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    save_file({n: tensors[n] for n in first}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n] for n in second}, str(tmp_path / "model-00002-of-00002.safetensors"))
    with pytest.raises(FileNotFoundError):
        read_checkpoint(tmp_path)   # shards without an index
    weight_map = {n: "model-00001-of-00002.safetensors" for n in first}
    weight_map.update({n: "model-00002-of-00002.safetensors" for n in second})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    stored = read_checkpoint(tmp_path)
    assert all(torch.equal(stored[n], tensors[n]) for n in names)
    weight_map[first[0]] = "model-00002-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(ValueError):
        read_checkpoint(tmp_path)   # the index disagrees with the shards
    weight_map[first[0]] = "model-00003-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(FileNotFoundError):
        read_checkpoint(tmp_path)   # a shard named by the index is missing


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path)
    with pytest.raises(FileNotFoundError):
        read_checkpoint(tmp_path)
