"""Configuration and registry (no GPU)."""
import pytest

from rustyllm_b200 import (ConfigError, LlamaConfig, UnknownArchitecture, known_architectures,
                           resolve_architecture)
from rustyllm_b200.models.llama import llama_spec
from tiny_configs import TINY


def test_reads_its_own_keys_and_derives_sizes():
    c = LlamaConfig.from_dict(TINY["A"]["config"])
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (64, 4, 2, 16)
    assert c.q_size == 64 and c.kv_size == 32 and c.group_size == 2
    assert c.eos_token_id == (255,) and c.rope_scaling is None
    b = LlamaConfig.from_dict(TINY["B"]["config"])
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.factor == 8.0
    assert b.eos_token_id == (382, 383) and b.tie_word_embeddings


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict({"vocab_size": 10, "hidden_size": 32, "intermediate_size": 48,
                               "num_hidden_layers": 1, "num_attention_heads": 4})
    assert c.num_key_value_heads == 4          # default = heads
    assert c.head_dim == 8                     # hidden / heads
    assert c.max_position_embeddings == 2048   # src/model.rs:105
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5


def test_head_dim_need_not_divide_hidden():
    c = LlamaConfig.from_dict(TINY["C"]["config"])
    assert c.q_size == 240 and c.hidden_size == 80


def test_rope_parameters_object_is_understood():
    d = dict(TINY["B"]["config"])
    sc = d.pop("rope_scaling")
    d.pop("rope_theta")
    d["rope_parameters"] = dict(sc, rope_theta=500000.0)
    c = LlamaConfig.from_dict(d)
    assert c.rope_theta == 500000.0 and c.rope_scaling.original_max_position_embeddings == 64


@pytest.mark.parametrize("patch, msg", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_attention_heads": 0}, "num_attention_heads"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "lacks"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"eos_token_id": 999}, "vocabulary"),
    ({"vocab_size": "many"}, "integer"),
])
def test_bad_configs_are_refused(patch, msg):
    d = dict(TINY["A"]["config"])
    d.update(patch)
    with pytest.raises(ConfigError, match=msg):
        LlamaConfig.from_dict(d)


def test_registry_resolves_by_architecture_then_model_type():
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    assert "llama" in known_architectures()
    with pytest.raises(UnknownArchitecture, match="known"):
        resolve_architecture({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})


def test_spec_is_data_and_names_every_tensor():
    c = LlamaConfig.from_dict(TINY["B"]["config"])
    spec = llama_spec(c)
    assert spec.schedule == (0, 1, 2) and len(spec.layers) == 3
    assert spec.layers[1].mixer.params["names"]["q"] == "model.layers.1.self_attn.q_proj"
    assert spec.head.params["tied_to"] == "embedding.weight"
    assert spec.layers[0].mixer.params["position"].params["scaling"]["factor"] == 8.0


def test_round_trip_to_dict():
    for t in TINY.values():
        c = LlamaConfig.from_dict(t["config"])
        assert LlamaConfig.from_dict(c.to_dict()) == c


def test_generation_config_adds_its_stop_ids(tmp_path):
    """Instruction-tuned folders name their end-of-turn ids in generation_config.json."""
    import json
    from rustyllm_b200.config.files import read_config_json, read_generation_stop_ids
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(dict(TINY["A"]["config"])))
    assert read_config_json(str(d))["eos_token_id"] == 255
    assert read_generation_stop_ids(str(d), 256) == ()            # no such file: nothing to add
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": [255, 7, 9], "temperature": 0.6}))
    assert read_generation_stop_ids(str(d), 256) == (255, 7, 9)
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": 3}))
    assert read_generation_stop_ids(str(d), 256) == (3,)
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": 256}))
    with pytest.raises(ConfigError, match="outside the vocabulary"):
        read_generation_stop_ids(str(d), 256)
    (d / "generation_config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError, match="object"):
        read_generation_stop_ids(str(d), 256)


def test_keys_of_other_architectures_that_would_change_the_arithmetic_are_refused():
    base = dict(vocab_size=32, hidden_size=16, intermediate_size=24, num_hidden_layers=1, num_attention_heads=2)
    assert LlamaConfig.from_dict(dict(base, partial_rotary_factor=1.0, sliding_window=None, use_cache=True)).head_dim == 8
    for extra in (dict(partial_rotary_factor=0.5), dict(sliding_window=4096)):
        with pytest.raises(ConfigError):
            LlamaConfig.from_dict(dict(base, **extra))
