"""Named configurations as data: the tiny test models and the benchmark layer sizes.

The reference keeps its two model sizes as constants in llama4/llama4_jax/configs.py:19-93.
Here a preset is a config.json dictionary, so it goes through the same reader as a file.
"""

from __future__ import annotations

from typing import Any


def _text(**kw: Any) -> dict[str, Any]:
    return {"architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text", **kw}


def _llama3(factor: float, low: float, high: float, orig: int) -> dict[str, Any]:
    return {"rope_type": "llama3", "factor": factor, "low_freq_factor": low, "high_freq_factor": high,
            "original_max_position_embeddings": orig}


def _every_nth_nope(layers: int, n: int) -> list[int]:
    return [int((i + 1) % n != 0) for i in range(layers)]


PRESETS: dict[str, dict[str, Any]] = {
    # Tiny A: MoE on every layer, top-1 of 4, qk-norm on, no rope scaling, last layer NoPE.
    "tiny_a": _text(
        num_hidden_layers=4, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        interleave_moe_layer_step=1, num_local_experts=4, num_experts_per_tok=1, intermediate_size=128,
        intermediate_size_mlp=128, vocab_size=256, rope_theta=10000.0, rope_scaling=None, use_qk_norm=True,
        attention_chunk_size=32, no_rope_layers=[1, 1, 1, 0], attn_temperature_tuning=True, floor_scale=16.0,
        attn_scale=0.1, rms_norm_eps=1e-5, tie_word_embeddings=False),
    # Tiny B: MoE on odd layers, top-2 of 8, dense SwiGLU on even layers, llama3 rope scaling, no qk-norm.
    "tiny_b": _text(
        num_hidden_layers=8, hidden_size=96, num_attention_heads=6, num_key_value_heads=2, head_dim=24,
        interleave_moe_layer_step=2, num_local_experts=8, num_experts_per_tok=2, intermediate_size=64,
        intermediate_size_mlp=192, vocab_size=384, rope_theta=500000.0, rope_scaling=_llama3(8.0, 1.0, 4.0, 64),
        use_qk_norm=False, attention_chunk_size=48, no_rope_layers=_every_nth_nope(8, 4),
        attn_temperature_tuning=True, floor_scale=24.0, attn_scale=0.1, rms_norm_eps=1e-6,
        tie_word_embeddings=False),
    # Scout layer sizes, 16 layers (the benchmark configuration).
    "scout16": _text(
        num_hidden_layers=16, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
        interleave_moe_layer_step=1, num_local_experts=16, num_experts_per_tok=1, intermediate_size=8192,
        intermediate_size_mlp=16384, vocab_size=202048, rope_theta=500000.0,
        rope_scaling=_llama3(16.0, 1.0, 1.0, 8192), use_qk_norm=True, attention_chunk_size=8192,
        no_rope_layers=_every_nth_nope(16, 4), attn_temperature_tuning=True, floor_scale=8192.0, attn_scale=0.1,
        rms_norm_eps=1e-5, tie_word_embeddings=False),
    # Maverick layer sizes, 4 layers: dense layers 0 and 2, 128 experts on layers 1 and 3.
    "maverick4": _text(
        num_hidden_layers=4, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
        interleave_moe_layer_step=2, num_local_experts=128, num_experts_per_tok=1, intermediate_size=8192,
        intermediate_size_mlp=16384, vocab_size=202048, rope_theta=500000.0, rope_scaling=None,
        use_qk_norm=False, attention_chunk_size=8192, no_rope_layers=[1, 1, 1, 0], attn_temperature_tuning=True,
        floor_scale=8192.0, attn_scale=0.1, rms_norm_eps=1e-5, tie_word_embeddings=False),
}
PRESETS["scout8_long"] = {**PRESETS["scout16"], "num_hidden_layers": 8, "no_rope_layers": _every_nth_nope(8, 4)}


def preset(name: str, **overrides: Any) -> dict[str, Any]:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {', '.join(sorted(PRESETS))}")
    d = dict(PRESETS[name])
    d.update(overrides)
    if "num_hidden_layers" in overrides and "no_rope_layers" not in overrides:
        n = overrides["num_hidden_layers"]
        base = PRESETS[name]["no_rope_layers"]
        d["no_rope_layers"] = [base[i % len(base)] for i in range(n)]
    return d
