"""Configuration: typed reading of config.json keys, defaults, refusals, the registry."""

import pytest

import tiny
from sleuth_b200.config import (ConfigError, Qwen3Config, parse_config, register_architecture,
                                registered_architectures, unregister_architecture)
from sleuth_b200.parts.spec import ModelSpec


def test_reads_every_key_and_keeps_unknown_ones_aside():
    arch, cfg, unread = parse_config(dict(tiny.B, torch_dtype="bfloat16", transformers_version="x"))
    assert arch.name == "Qwen3ForCausalLM" and isinstance(cfg, Qwen3Config)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (503, 96, 160, 3)
    assert (cfg.num_attention_heads, cfg.kv_heads, cfg.head_size) == (6, 3, 24)
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and cfg.attention_bias and not cfg.tie_word_embeddings
    assert unread == ["torch_dtype", "transformers_version"]


def test_defaults_follow_the_reference():
    _, cfg, _ = parse_config(dict(model_type="qwen3", vocab_size=10, hidden_size=32, intermediate_size=8,
                                  num_hidden_layers=1, num_attention_heads=4))
    assert cfg.kv_heads == 4 and cfg.head_size == 8 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert not cfg.attention_bias and not cfg.tie_word_embeddings and cfg.windows == (0,)


def test_model_spec_carries_all_sizes():
    arch, cfg, _ = parse_config(tiny.C)
    spec = arch.model_spec(cfg)
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    m = spec.layers[1].mixer
    assert (m.hidden, m.heads, m.kv_heads, m.head_dim, m.window, m.qkv_bias, m.qk_norm) == (80, 5, 1, 64, 40, True, True)
    assert spec.layers[0].mixer.window == 0 and m.position.theta == 50000.0 and m.qk_norm_eps == 3e-6
    assert spec.layers[0].ffn.intermediate == 136 and spec.head.tied and spec.embedding.vocab == 311
    assert spec.layers[2].names["mixer.q_proj.weight"] == "model.layers.2.self_attn.q_proj.weight"


def test_tying_rule_with_tensor_names():
    arch, cfg, _ = parse_config(tiny.B)
    assert not arch.model_spec(cfg).head.tied
    assert arch.model_spec(cfg, tensor_names={"model.embed_tokens.weight"}).head.tied       # no lm_head.weight in the file


@pytest.mark.parametrize("patch,word", [
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(num_key_value_heads=4), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["full_attention", "sliding_attention", "banded"]), "layer_types"),
    (dict(layer_types=["sliding_attention"] * 3, sliding_window=None), "sliding_window"),
])
def test_refusals(patch, word):
    with pytest.raises(ConfigError, match=word):
        parse_config(dict(tiny.B, **patch))


def test_wrong_types_and_missing_keys_are_named():
    with pytest.raises(ConfigError, match="hidden_size"):
        parse_config(dict(tiny.A, hidden_size="64"))
    with pytest.raises(ConfigError, match="attention_bias"):
        parse_config(dict(tiny.A, attention_bias=1))
    bad = {k: v for k, v in tiny.A.items() if k != "intermediate_size"}
    bad["intermediate_sizes"] = 192
    with pytest.raises(ConfigError, match="intermediate_size.*misspelling"):
        parse_config(bad)


def test_unknown_architecture_lists_the_registered_ones():
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        parse_config(dict(tiny.A, architectures=["GPT2LMHeadModel"], model_type="gpt2"))


def test_model_type_alone_finds_the_architecture():
    cfg = {k: v for k, v in tiny.A.items() if k != "architectures"}
    assert parse_config(cfg)[0].name == "Qwen3ForCausalLM"


def test_registering_another_architecture():
    register_architecture("ToyForCausalLM", Qwen3Config, lambda cfg, tensor_names=None: "spec", model_types=("toy",))
    try:
        assert "ToyForCausalLM" in registered_architectures()
        arch, _, _ = parse_config(dict(tiny.A, architectures=["ToyForCausalLM"]))
        assert arch.model_spec(None) == "spec"
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "ToyForCausalLM" not in registered_architectures()


def test_config_round_trip_through_json_dict():
    _, cfg, _ = parse_config(tiny.C)
    _, again, _ = parse_config(cfg.to_json_dict())
    assert again.windows == cfg.windows == (0, 40, 0, 40) and again.head_size == 64
