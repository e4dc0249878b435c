"""Configuration parsing and the registries (no GPU)."""
import json

import pytest

from dispec_b200.config import ConfigError, Qwen2Config, load_model_config
from dispec_b200.registry import RegistryError, architecture_entry, architectures, part_class
from dispec_b200.weights import build_model

import replay_util as ru


def test_reads_both_layouts_of_rope_theta_and_head_dim_fallback():
    a = load_model_config(ru.CONFIG_A)
    b = load_model_config(ru.CONFIG_B)  # rope_theta nested under rope_parameters
    assert isinstance(a, Qwen2Config) and a.rope_theta == 10000.0 and b.rope_theta == 1e6
    d = dict(ru.CONFIG_A)
    del d["head_dim"]
    assert load_model_config(d).head_dim == 16  # hidden_size // num_attention_heads
    assert a.layer_windows == (0, 0)


def test_window_layers_from_layer_types_and_from_max_window_layers():
    c = load_model_config(ru.CONFIG_C)
    assert c.layer_windows == (0, 24, 24, 0)
    d = dict(ru.CONFIG_C)
    del d["layer_types"]
    d["max_window_layers"] = 3
    assert load_model_config(d).layer_windows == (0, 0, 0, 24)
    d["use_sliding_window"] = False
    assert load_model_config(d).layer_windows == (0, 0, 0, 0)


def test_round_trip_through_to_dict():
    for cfg in (ru.CONFIG_A, ru.CONFIG_B, ru.CONFIG_C):
        c = load_model_config(cfg)
        assert load_model_config(json.loads(json.dumps(c.to_dict()))) == c


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps",
                                 "rope_theta", "hidden_act", "tie_word_embeddings"])
def test_missing_key_is_named(key):
    d = dict(ru.CONFIG_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        load_model_config(d)


def test_rejections_are_clear():
    with pytest.raises(ConfigError, match="multiple"):
        load_model_config(dict(ru.CONFIG_A, num_attention_heads=5))
    with pytest.raises(ConfigError, match="hidden_act"):
        load_model_config(dict(ru.CONFIG_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="rotary type"):
        load_model_config(dict(ru.CONFIG_A, rope_scaling={"rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="even"):
        load_model_config(dict(ru.CONFIG_A, head_dim=15))
    # a layer marked as sliding in a file that switches windows off contradicts itself
    with pytest.raises(ConfigError, match="use_sliding_window is false"):
        load_model_config(dict(ru.CONFIG_C, use_sliding_window=False))
    with pytest.raises(ConfigError, match="sliding_window is missing"):
        load_model_config(dict(ru.CONFIG_C, sliding_window=None))
    with pytest.raises(RegistryError, match="Qwen2ForCausalLM"):
        load_model_config(dict(ru.CONFIG_A, architectures=["NoSuchModel"]))
    with pytest.raises(ConfigError, match="architectures"):
        load_model_config({k: v for k, v in ru.CONFIG_A.items() if k != "architectures"})


def test_registry_lists_names():
    assert "Qwen2ForCausalLM" in architectures()
    assert architecture_entry("Qwen2ForCausalLM").config_class is Qwen2Config
    with pytest.raises(RegistryError, match="gqa_attention"):
        part_class("mixer", "no_such_mixer")
    with pytest.raises(RegistryError, match="role"):
        part_class("no_such_role", "x")


def test_model_is_assembled_layer_by_layer_from_the_configuration():
    m = build_model(load_model_config(ru.CONFIG_C))
    assert [blk.mixer.window for blk in m.layers] == [0, 24, 24, 0]
    assert [(g.window, g.num_slots) for g in m.cache_groups] == [(0, 2), (24, 2)]
    assert m.layers[0].mixer.num_heads == 10 and m.layers[0].mixer.num_kv_heads == 2
    assert m.layers[0].mixer.head_dim == 48 and m.layers[0].feed_forward.intermediate_size == 176
    assert m.layers[0].mixer_norm.eps == 3e-6
    # the rotary part is one object shared by all mixers
    assert len({id(blk.mixer.position_encoding) for blk in m.layers}) == 1
    a = build_model(load_model_config(ru.CONFIG_A))
    req = a.tensor_requirements()
    assert "lm_head.weight" not in req and len(req) == 2 * 12 + 2
    assert a.head.tensor_specs()["weight"].shape == (256, 64)
