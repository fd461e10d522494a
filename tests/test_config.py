"""Typed configuration and the architecture registry."""
import json
import os

import pytest

from helpers import TINY_A, TINY_B
from inference_engine_rust_b200 import (ConfigError, MistralConfig, config_from_dict,
                                        known_architectures, load_config, spec_of)
from inference_engine_rust_b200.config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def test_fields_come_from_config_json_keys():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, MistralConfig)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.rope_theta, a.sliding_window, a.rms_norm_eps) == \
        (2, 64, 4, 2, 16, 192, 256, 10000.0, 16, 1e-5)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size, b.rope_theta, b.sliding_window, b.rms_norm_eps) == \
        (3, 96, 6, 1, 32, 160, 384, 1e6, None, 1e-6)
    assert b.num_attention_heads * b.head_dim != b.hidden_size


def test_defaults_follow_the_reference():
    raw = dict(TINY_A)
    for k in ("head_dim", "num_key_value_heads", "rope_theta", "bos_token_id", "eos_token_id"):
        raw.pop(k)
    c = config_from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 10000.0
    assert (c.bos_token_id, c.eos_token_id) == (1, 2)


@pytest.mark.parametrize("change,needle", [
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"sliding_window": 0}, "sliding_window"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"eos_token_id": 256}, "eos_token_id"),
    ({"attention_bias": True}, "attention_bias"),
    ({"architectures": ["NoSuchModel"]}, "NoSuchModel"),
    ({"architectures": []}, "architectures"),
])
def test_bad_configurations_are_refused(change, needle):
    raw = dict(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert needle in str(e.value)


def test_head_dim_must_be_derivable():
    raw = dict(TINY_A, hidden_size=66)
    raw.pop("head_dim")
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(TINY_A, architectures=["GemmaForCausalLM"]))
    assert "MistralForCausalLM" in str(e.value) and known_architectures() == ["MistralForCausalLM"]


def test_round_trip_through_a_folder(tmp_path):
    c = config_from_dict(TINY_B)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.to_dict(), f)
    assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "bad"))


def test_spec_is_layer_by_layer_data():
    spec = spec_of(config_from_dict(TINY_A))
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 2
    assert [e.layer for e in spec.schedule] == [0, 1] and all(e.writes_cache for e in spec.schedule)
    l1 = spec.layers[1]
    assert l1.mixer.kind == "attention" and l1.ffn.kind == "swiglu" and l1.norm.kind == "rmsnorm"
    assert l1.mixer["window"] == 16 and l1.mixer["position"].kind == "rope"
    assert l1.mixer["position"]["pairing"] == "half" and l1.mixer["position"]["theta"] == 10000.0
    assert l1.mixer_prefix == "model.layers.1.self_attn." and spec.lm_head_name == "lm_head.weight"
    assert spec_of(config_from_dict(dict(TINY_A, tie_word_embeddings=True))).lm_head_name is None


def test_schedule_validation():
    spec = spec_of(config_from_dict(TINY_A))

    def with_schedule(s):
        return ModelSpec(**{**spec.__dict__, "schedule": tuple(s)})

    with_schedule([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)]).validate()       # a layer twice
    with_schedule([ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=0)]).validate()        # shared cache
    for bad in ([ScheduleEntry(2)], [ScheduleEntry(0, reads_cache_of=0)],
                [ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=0), ScheduleEntry(0, reads_cache_of=1)], []):
        with pytest.raises(ValueError):
            with_schedule(bad).validate()
