"""Llama 4 text decoder: its tensors by name and how its layers are put together from parts.

Tensor names and orientations are those of the HF checkpoint that the reference converts
(llama4/llama4_jax/chkpt_utils.py:161-196 names, :80-159 shapes, :198-205 the gate_up split), read
with or without the ``language_model.`` prefix (llama4/scripts/convert_weights.py:41).

Layer rules (config: :class:`..config.llama4.Llama4Config`):
* rotary layers: interleaved RoPE, the weightless q/k norm if ``use_qk_norm``, and attention
  within chunks of ``attention_chunk_size``;
* the other layers: no position encoding, no q/k norm, attention over all keys, queries scaled
  by the attention temperature if ``attn_temperature_tuning``;
* feed-forward: routed experts plus a shared expert on ``moe_layers``, dense SwiGLU elsewhere.
The reference differs in two points: it has no attention temperature, and it passes the chunk
size on the layers WITHOUT rotary embeddings (model.py:944); this model chunks the rotary layers.
"""

from __future__ import annotations

import re
from typing import Mapping

import torch

from ..config.llama4 import Llama4Config
from ..config.registry import Architecture, register_architecture
from ..parts import DecoderModel, Runtime, llama3_scaled_frequencies, make_part
from ..weights.loader import TensorSpec

_SKIP = re.compile(r"^(vision_model\.|multi_modal_projector\.)")


def canonical_name(file_name: str) -> str | None:
    if _SKIP.match(file_name):
        return None
    return file_name[len("language_model."):] if file_name.startswith("language_model.") else file_name


def tensor_specs(cfg: Llama4Config) -> dict[str, TensorSpec]:
    D, V = cfg.hidden_size, cfg.vocab_size
    Hq, Hkv, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    F, Fm, E = cfg.intermediate_size, cfg.intermediate_size_mlp, cfg.num_local_experts
    specs: list[TensorSpec] = [TensorSpec("model.embed_tokens.weight", (V, D))]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        specs += [
            TensorSpec(p + "input_layernorm.weight", (D,), "norm"),
            TensorSpec(p + "self_attn.q_proj.weight", (Hq * dh, D)),
            TensorSpec(p + "self_attn.k_proj.weight", (Hkv * dh, D)),
            TensorSpec(p + "self_attn.v_proj.weight", (Hkv * dh, D)),
            TensorSpec(p + "self_attn.o_proj.weight", (D, Hq * dh)),
            TensorSpec(p + "post_attention_layernorm.weight", (D,), "norm"),
        ]
        if cfg.layer_is_moe(i):
            specs += [
                TensorSpec(p + "feed_forward.router.weight", (E, D)),
                TensorSpec(p + "feed_forward.experts.gate_up_proj", (E, D, 2 * F)),
                TensorSpec(p + "feed_forward.experts.down_proj", (E, F, D)),
                TensorSpec(p + "feed_forward.shared_expert.gate_proj.weight", (F, D)),
                TensorSpec(p + "feed_forward.shared_expert.up_proj.weight", (F, D)),
                TensorSpec(p + "feed_forward.shared_expert.down_proj.weight", (D, F)),
            ]
        else:
            specs += [
                TensorSpec(p + "feed_forward.gate_proj.weight", (Fm, D)),
                TensorSpec(p + "feed_forward.up_proj.weight", (Fm, D)),
                TensorSpec(p + "feed_forward.down_proj.weight", (D, Fm)),
            ]
    specs.append(TensorSpec("model.norm.weight", (D,), "norm"))
    specs.append(TensorSpec("lm_head.weight", (V, D), optional=cfg.tie_word_embeddings))
    return {s.name: s for s in specs}


def build(cfg: Llama4Config, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> DecoderModel:
    """Puts the decoder together.  ``tensors`` (by spec name, already on the device) is consumed:
    entries are removed as they are fused into the layouts the kernels read."""
    t = dict(tensors) if not isinstance(tensors, dict) else tensors
    dev = runtime.device
    Hq, Hkv, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    scaling = None
    if cfg.rope_scaling is not None:
        rs = cfg.rope_scaling
        scaling = {"factor": rs.factor, "low_freq_factor": rs.low_freq_factor, "high_freq_factor": rs.high_freq_factor,
                   "original_max_position_embeddings": rs.original_max_position_embeddings}
    # Which part serves which layer is decided here, layer by layer, by name from the parts registry.
    rope = make_part("position", "interleaved_rope", inv_freq=llama3_scaled_frequencies(dh, cfg.rope_theta, scaling), device=dev)
    nope = make_part("position", "none_with_temperature",
                     attn_scale=cfg.attn_scale if cfg.attn_temperature_tuning else 0.0, floor_scale=cfg.floor_scale)

    def take(name: str) -> torch.Tensor:
        return t.pop(name).to(dev)

    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        w_qkv = torch.cat([take(p + "self_attn.q_proj.weight"), take(p + "self_attn.k_proj.weight"),
                           take(p + "self_attn.v_proj.weight")], dim=0).contiguous()
        uses_rope = cfg.layer_uses_rope(i)
        mixer = make_part(
            "mixer", "paged_attention", w_qkv=w_qkv, w_o=take(p + "self_attn.o_proj.weight").contiguous(),
            n_heads=Hq, n_kv_heads=Hkv, head_dim=dh, position=rope if uses_rope else nope,
            qk_norm_eps=cfg.rms_norm_eps if (cfg.use_qk_norm and uses_rope) else None,
            chunk=cfg.attention_chunk_size if uses_rope else None,
        )
        if cfg.layer_is_moe(i):
            shared = make_part(
                "feed_forward", "dense_swiglu",
                w_gate_up=torch.cat([take(p + "feed_forward.shared_expert.gate_proj.weight"),
                                     take(p + "feed_forward.shared_expert.up_proj.weight")], dim=0).contiguous(),
                w_down=take(p + "feed_forward.shared_expert.down_proj.weight").contiguous())
            # HF keeps expert matrices as [in, out] (chkpt_utils.py:110-115); the kernels read [out, in]
            gate_up = take(p + "feed_forward.experts.gate_up_proj").transpose(1, 2).contiguous()
            down = take(p + "feed_forward.experts.down_proj").transpose(1, 2).contiguous()
            ffn = make_part("feed_forward", "routed_experts", w_router=take(p + "feed_forward.router.weight"),
                            we_gate_up=gate_up, we_down=down, top_k=cfg.num_experts_per_tok, shared=shared)
        else:
            ffn = make_part(
                "feed_forward", "dense_swiglu",
                w_gate_up=torch.cat([take(p + "feed_forward.gate_proj.weight"), take(p + "feed_forward.up_proj.weight")],
                                    dim=0).contiguous(),
                w_down=take(p + "feed_forward.down_proj.weight").contiguous())
        blocks.append(make_part(
            "block", "pre_norm",
            norm1=make_part("norm", "rms", weight=take(p + "input_layernorm.weight"), eps=cfg.rms_norm_eps), mixer=mixer,
            norm2=make_part("norm", "rms", weight=take(p + "post_attention_layernorm.weight"), eps=cfg.rms_norm_eps),
            feed_forward=ffn))
    embedding = take("model.embed_tokens.weight").contiguous()
    lm_head = take("lm_head.weight").contiguous() if "lm_head.weight" in t else embedding
    final_norm = make_part("norm", "rms", weight=take("model.norm.weight"), eps=cfg.rms_norm_eps)
    return DecoderModel(runtime, embedding, blocks, final_norm, lm_head, config=cfg)


LLAMA4 = Architecture(
    name="Llama4ForCausalLM",
    parse_config=Llama4Config.from_dict,
    tensor_specs=tensor_specs,
    build=build,
    canonical_name=canonical_name,
)
register_architecture(LLAMA4, "Llama4ForConditionalGeneration")
