"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from airframe_b200.config import (ConfigError, Gemma2Config, config_from_dict, config_from_folder,
                                  known_architectures, register_architecture)
from airframe_b200.config.base import ModelSpec, PartSpec, ScheduleEntry, LayerSpec
from tiny import TINY_A, TINY_B, TINY_C


def test_reads_every_key_of_tiny_a():
    c = config_from_dict(TINY_A)
    assert isinstance(c, Gemma2Config)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (2, 64, 4, 2)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (16, 128, 256)
    assert (c.rope_theta, c.sliding_window, c.query_pre_attn_scalar) == (10000.0, 8, 16.0)
    assert (c.attn_logit_softcapping, c.final_logit_softcapping) == (50.0, 30.0)
    assert c.max_position_embeddings == 64 and c.rms_norm_eps == 1e-6
    assert c.eos_token_ids == [1] and c.layer_types == [True, False]


def test_tiny_b_differs_in_every_size():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                "intermediate_size", "vocab_size", "rope_theta", "sliding_window", "query_pre_attn_scalar",
                "attn_logit_softcapping", "final_logit_softcapping", "max_position_embeddings",
                "rms_norm_eps"):
        assert getattr(a, key) != getattr(b, key), key
    assert b.eos_token_ids == [3, 7]
    assert b.head_dim * b.num_attention_heads != b.hidden_size


def test_model_spec_carries_sizes_per_layer():
    spec = config_from_dict(TINY_B).model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    windows = [l.mixer.params["window"] for l in spec.layers]
    assert windows == [16, None, 16]
    m = spec.layers[0].mixer.params
    assert m["scale"] == pytest.approx(24 ** -0.5) and m["softcap"] == 20.0
    assert m["position"].params == {"theta": 100000.0, "rotary_dim": 32, "pairing": "half"}
    assert spec.layers[1].norms["post_mixer"].params["weight"] == "model.layers.1.post_attention_layernorm.weight"
    assert spec.layers[1].norms["post_mixer"].params["eps"] == 1e-5
    assert spec.embedding.params["scale"] == pytest.approx(96 ** 0.5)
    assert spec.head.params["softcap"] == 15.0 and spec.head.params["tied_to"] == "model.embed_tokens.weight"
    assert spec.stop_token_ids == [3, 7]


def test_layer_types_key_wins_over_alternation():
    d = dict(TINY_B, layer_types=["full_attention", "full_attention", "sliding_attention"])
    assert config_from_dict(d).layer_types == [False, False, True]
    with pytest.raises(ConfigError, match="layer_types"):
        config_from_dict(dict(TINY_B, layer_types=["full_attention"]))
    with pytest.raises(ConfigError, match="unknown kind"):
        config_from_dict(dict(TINY_B, layer_types=["full_attention", "x", "full_attention"]))


def test_softcaps_may_be_null_but_not_absent():
    d = dict(TINY_A, attn_logit_softcapping=None, final_logit_softcapping=None)
    c = config_from_dict(d)
    assert c.attn_logit_softcapping is None and c.final_logit_softcapping is None
    spec = c.model_spec()
    assert spec.layers[0].mixer.params["softcap"] == 0.0 and spec.head.params["softcap"] == 0.0
    # an absent key is no answer: neither "off" nor some other model's value is assumed
    for key in ("attn_logit_softcapping", "final_logit_softcapping"):
        d = dict(TINY_A)
        del d[key]
        with pytest.raises(ConfigError, match=key):
            config_from_dict(d)


def test_written_config_keeps_integers_integer():
    d = config_from_dict(TINY_A).to_dict()
    assert d["query_pre_attn_scalar"] == 16 and isinstance(d["query_pre_attn_scalar"], int)
    assert config_from_dict(d) == config_from_dict(TINY_A)
    d = config_from_dict(dict(TINY_A, query_pre_attn_scalar=12.5)).to_dict()
    assert d["query_pre_attn_scalar"] == 12.5


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "intermediate_size", "num_attention_heads",
                                 "head_dim", "vocab_size", "rms_norm_eps", "rope_theta", "sliding_window",
                                 "max_position_embeddings"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("key,value,word", [
    ("hidden_size", "64", "integer"), ("hidden_size", 0, ">= 1"), ("rms_norm_eps", -1.0, "> 0"),
    ("num_key_value_heads", 3, "multiple"), ("head_dim", 15, "even"), ("hidden_activation", "relu", "not supported"),
    ("attention_bias", True, "attention_bias"), ("tie_word_embeddings", "yes", "true or false"),
    ("eos_token_id", 999, "outside"), ("eos_token_id", "x", "integer ids"), ("sliding_window", 0, ">= 1"),
    ("attn_logit_softcapping", -2.0, ">= 0"),
])
def test_bad_values_are_refused(key, value, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY_A, **{key: value}))


def test_registry_names_the_known_architectures():
    assert "Gemma2ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*Gemma2ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_registering_another_architecture():
    class Other(Gemma2Config):
        architecture = "OtherForCausalLM"
    register_architecture("OtherForCausalLM", Other)
    try:
        assert isinstance(config_from_dict(dict(TINY_A, architectures=["OtherForCausalLM"])), Other)
        with pytest.raises(ConfigError, match="registered already"):
            register_architecture("OtherForCausalLM", Gemma2Config)
    finally:
        from airframe_b200.config import registry
        registry._ARCHITECTURES.pop("OtherForCausalLM")


def test_round_trip_through_a_folder(tmp_path):
    c = config_from_dict(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert config_from_folder(tmp_path) == c
    with pytest.raises(ConfigError, match="no such file"):
        config_from_folder(tmp_path / "nowhere")
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        config_from_folder(tmp_path)


def test_schedule_validation():
    spec = config_from_dict(TINY_A).model_spec()
    s = copy.deepcopy(spec)
    s.schedule = [ScheduleEntry(0), ScheduleEntry(0), ScheduleEntry(1, cache_from=0)]
    s.validate()
    s.schedule = [ScheduleEntry(5)]
    with pytest.raises(ConfigError, match="names layer 5"):
        s.validate()
    s.schedule = [ScheduleEntry(0, cache_from=0)]
    with pytest.raises(ConfigError, match="does not come before"):
        s.validate()
    s.schedule = [ScheduleEntry(0), ScheduleEntry(1, cache_from=0), ScheduleEntry(0, cache_from=1)]
    with pytest.raises(ConfigError, match="keeps none"):
        s.validate()


def test_presets_parse_and_match_the_test_configurations():
    from airframe_b200.config import config_from_dict
    from airframe_b200.config.presets import PRESETS, preset
    import tiny
    for name in PRESETS:
        cfg = config_from_dict(preset(name))
        cfg.model_spec().validate()
    for name, ref in (("tinyA", tiny.TINY_A), ("tinyB", tiny.TINY_B)):
        p = preset(name)
        for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "rope_theta", "sliding_window", "query_pre_attn_scalar",
                    "attn_logit_softcapping", "final_logit_softcapping", "max_position_embeddings"):
            assert p[key] == ref[key], (name, key)
    with pytest.raises(KeyError, match="unknown preset"):
        preset("70b")
