"""Configuration: typed reading of the architecture's config.json keys, and the registry."""
import copy

import pytest

import helpers as H
from infer_b200.config import ConfigError, parse_config, registered_architectures
import infer_b200.models  # noqa: F401


def test_registry_has_the_architecture():
    assert "Qwen2ForCausalLM" in registered_architectures()


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_parse_and_spec(name):
    cfg = H.TINY[name]
    arch, typed = parse_config(cfg)
    spec = arch.to_spec(typed)
    assert len(spec.layers) == cfg["num_hidden_layers"] == len(spec.schedule)
    assert spec.vocab_size == cfg["vocab_size"] and spec.hidden_size == cfg["hidden_size"]
    m = spec.layers[0].part("mixer")
    assert m.kind == "attention" and m["num_heads"] == cfg["num_attention_heads"]
    assert m["head_dim"] == cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    assert spec.head["tied"] == cfg["tie_word_embeddings"] and spec.embedding.prefix == "model.embed_tokens."
    assert spec.layers[0].part("mixer_norm")["eps"] == cfg["rms_norm_eps"]
    assert m["position"]["theta"] == cfg["rope_theta"]
    # the dictionary written back parses to the same typed configuration
    assert parse_config(arch.to_dict(typed))[1] == typed


def test_window_is_chosen_layer_by_layer():
    spec = H.spec_of(H.TINY["c"])
    assert [l.part("mixer")["window"] for l in spec.layers] == [None, None, 40, 40]


def test_defaults_follow_the_reference():
    cfg = copy.deepcopy(H.TINY["a"])
    del cfg["tie_word_embeddings"]
    _, typed = parse_config(cfg)
    assert typed.tie_word_embeddings is False          # src/model_config.cpp:30
    assert typed.attention_bias is True                # src/model_config.cpp:41-42
    assert typed.head_dim == 16                        # hidden / heads


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
                                 "max_position_embeddings"])
def test_missing_key_is_named(key):
    cfg = copy.deepcopy(H.TINY["b"])
    del cfg[key]
    with pytest.raises(ConfigError, match=key):
        parse_config(cfg)


@pytest.mark.parametrize("patch, match", [
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"hidden_size": "64"}, "integer"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "positive"),
])
def test_bad_values_are_refused(patch, match):
    cfg = copy.deepcopy(H.TINY["a"])
    cfg.update(patch)
    with pytest.raises(ConfigError, match=match):
        parse_config(cfg)
