"""Configuration and registry (no GPU)."""

import json

import pytest

import jax_llm_examples_b200 as J
from jax_llm_examples_b200.config import Llama4Config, load_config_json


def test_presets_differ_in_every_option():
    a = Llama4Config.from_dict(J.preset("tiny_a"))
    b = Llama4Config.from_dict(J.preset("tiny_b"))
    for field in ("num_hidden_layers", "hidden_size", "num_attention_heads", "head_dim", "num_local_experts",
                  "num_experts_per_tok", "intermediate_size", "vocab_size", "rope_theta", "rope_scaling",
                  "use_qk_norm", "attention_chunk_size", "floor_scale", "rms_norm_eps", "moe_layers", "no_rope_layers"):
        assert getattr(a, field) != getattr(b, field), field
    assert a.moe_layers == (0, 1, 2, 3) and b.moe_layers == (1, 3, 5, 7)
    assert a.no_rope_layers == (1, 1, 1, 0) and b.no_rope_layers == (1, 1, 1, 0, 1, 1, 1, 0)
    assert b.rope_scaling.factor == 8.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.hidden_size != b.num_attention_heads * b.head_dim


def test_text_config_nesting_and_round_trip(tmp_path):
    inner = {k: v for k, v in J.preset("tiny_b").items() if k != "architectures"}
    nested = {"architectures": ["Llama4ForConditionalGeneration"], "text_config": inner}
    cfg = J.resolve(nested).parse_config(nested)
    assert cfg.architecture == "Llama4ForConditionalGeneration" and cfg.hidden_size == 96
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_json_dict()))
    again = Llama4Config.from_dict(load_config_json(tmp_path))
    assert again == cfg


def test_layer_rules_from_intervals():
    d = J.preset("tiny_b")
    del d["no_rope_layers"]
    cfg = Llama4Config.from_dict(d)
    assert [cfg.layer_uses_rope(i) for i in range(8)] == [True, True, True, False] * 2
    assert [cfg.layer_is_moe(i) for i in range(8)] == [False, True] * 4
    d["moe_layers"] = [0, 5]
    assert Llama4Config.from_dict(d).moe_layers == (0, 5)


def test_temperature_switch():
    d = J.preset("tiny_a")
    d["attn_temperature_tuning"] = False
    assert not Llama4Config.from_dict(d).attn_temperature_tuning
    del d["attn_temperature_tuning"]
    assert Llama4Config.from_dict(d).attn_temperature_tuning  # both constants given
    del d["floor_scale"]
    assert not Llama4Config.from_dict(d).attn_temperature_tuning
    d["attn_temperature_tuning"] = True
    with pytest.raises(J.ConfigError, match="floor_scale"):
        Llama4Config.from_dict(d)


@pytest.mark.parametrize("edit, match", [
    (lambda d: d.pop("hidden_size"), "hidden_size"),
    (lambda d: d.update(num_key_value_heads=3), "multiple"),
    (lambda d: d.update(head_dim=15), "even"),
    (lambda d: d.update(num_experts_per_tok=9), "num_experts_per_tok"),
    (lambda d: d.update(no_rope_layers=[1, 0]), "no_rope_layers"),
    (lambda d: d.update(vocab_size="many"), "vocab_size"),
    (lambda d: d.update(rope_scaling={"rope_type": "yarn", "factor": 2.0}), "yarn"),
    (lambda d: d.update(rms_norm_eps=0.0), "rms_norm_eps"),
])
def test_bad_configs_name_the_key(edit, match):
    d = J.preset("tiny_a")
    edit(d)
    with pytest.raises(J.ConfigError, match=match):
        Llama4Config.from_dict(d)


def test_registry_names_and_errors():
    assert set(J.known_architectures()) >= {"Llama4ForCausalLM", "Llama4ForConditionalGeneration"}
    with pytest.raises(J.ConfigError, match="unknown architecture.*known"):
        J.resolve({"architectures": ["MysteryForCausalLM"]})
    with pytest.raises(J.ConfigError, match="architectures"):
        J.resolve({})
    with pytest.raises(J.ConfigError, match="no config.json"):
        load_config_json("/nonexistent/folder")


def test_layer_kinds_from_layer_types():
    """Newer HF files give ``layer_types`` instead of ``no_rope_layers``."""
    from jax_llm_examples_b200 import preset, resolve

    d = preset("tiny_a")
    d.pop("no_rope_layers", None)
    d["layer_types"] = ["chunked_attention", "full_attention", "chunked_attention", "chunked_attention"]
    cfg = resolve(d).parse_config(d)
    assert cfg.no_rope_layers == (1, 0, 1, 1) and not cfg.layer_uses_rope(1) and cfg.layer_uses_rope(0)
    d["layer_types"][0] = "sliding_attention"
    with pytest.raises(Exception, match="layer_types"):
        resolve(d).parse_config(d)
