"""Typed configuration of the Llama 4 text decoder, read from config.json keys.

The reference reads ``config.json["text_config"]`` (llama4/llama4_jax/model.py:229-231)
and maps a fixed set of keys (model.py:199-226).  This class reads the same keys and
also the ones the reference fixes in code: ``rope_scaling`` (model.py:160-163 hard-codes
factor 8 / low 1 / high 4 / 8192), ``no_rope_layers`` (model.py:201-203 hard-codes every
fourth layer), ``moe_layers``, and the attention-temperature keys ``attn_temperature_tuning``,
``floor_scale`` and ``attn_scale`` which the reference does not implement.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .base import ConfigError, read_key, require


@dataclasses.dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency correction (llama4/llama4_jax/model.py:654-672)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "RopeScaling":
        kind = d.get("rope_type", d.get("type"))
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (only 'llama3')")
        rs = RopeScaling(
            factor=read_key(d, "factor", float),
            low_freq_factor=read_key(d, "low_freq_factor", float),
            high_freq_factor=read_key(d, "high_freq_factor", float),
            original_max_position_embeddings=read_key(d, "original_max_position_embeddings", int),
        )
        require(rs.factor > 0, "rope_scaling.factor must be positive")
        require(rs.high_freq_factor >= rs.low_freq_factor > 0, "rope_scaling needs high_freq_factor >= low_freq_factor > 0")
        require(rs.original_max_position_embeddings > 0, "rope_scaling.original_max_position_embeddings must be positive")
        return rs

    def to_dict(self) -> dict[str, Any]:
        return {"rope_type": "llama3", **dataclasses.asdict(self)}


@dataclasses.dataclass(frozen=True)
class Llama4Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int  # width of each routed expert and of the shared expert
    intermediate_size_mlp: int  # width of the dense SwiGLU on non-MoE layers
    num_local_experts: int
    num_experts_per_tok: int
    moe_layers: tuple[int, ...]  # indices of layers whose feed-forward is routed experts
    no_rope_layers: tuple[int, ...]  # per layer: 1 = rotary layer, 0 = no position encoding
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None
    use_qk_norm: bool
    attention_chunk_size: int | None  # chunked causal attention on rotary layers; None = global
    attn_temperature_tuning: bool
    floor_scale: float
    attn_scale: float
    tie_word_embeddings: bool
    max_position_embeddings: int | None = None
    bos_token_id: int | None = None
    eos_token_ids: tuple[int, ...] = ()
    pad_token_id: int | None = None
    interleave_moe_layer_step: int | None = None
    architecture: str = "Llama4ForCausalLM"

    # ------------------------------------------------------------------ reading
    @staticmethod
    def from_dict(cfg_json: Mapping[str, Any]) -> "Llama4Config":
        arch = (cfg_json.get("architectures") or ["Llama4ForCausalLM"])[0]
        d = cfg_json.get("text_config", cfg_json)  # model.py:231 reads text_config
        n_layers = read_key(d, "num_hidden_layers", int)
        hidden = read_key(d, "hidden_size", int)
        n_heads = read_key(d, "num_attention_heads", int)
        head_dim = read_key(d, "head_dim", int, hidden // n_heads if n_heads else 0)
        n_kv = read_key(d, "num_key_value_heads", int, n_heads)

        step = read_key(d, "interleave_moe_layer_step", int, None)
        if d.get("moe_layers") is not None:
            moe_layers = tuple(int(i) for i in read_key(d, "moe_layers", list))
        else:
            if step is None:
                raise ConfigError("config.json: need 'moe_layers' or 'interleave_moe_layer_step'")
            require(step >= 1, "interleave_moe_layer_step must be >= 1")
            # model.py:558: layer i is MoE iff (i + 1) % interval == 0
            moe_layers = tuple(i for i in range(n_layers) if (i + 1) % step == 0)

        if d.get("no_rope_layers"):
            no_rope = tuple(int(v) for v in read_key(d, "no_rope_layers", list))
        elif d.get("layer_types"):
            # newer HF files name the layer kinds instead: "chunked_attention" = a rotary layer, "full_attention" = none
            kinds = read_key(d, "layer_types", list)
            require(all(k in ("chunked_attention", "full_attention") for k in kinds),
                    f"layer_types may hold 'chunked_attention' and 'full_attention', found {sorted(set(map(str, kinds)))}")
            no_rope = tuple(int(k == "chunked_attention") for k in kinds)
        else:
            # model.py:203 fixes the interval at 4; the commented lines 201-202 show that
            # no_rope_layers[i] == 1 marks a layer that does use rotary embeddings.
            interval = read_key(d, "no_rope_layer_interval", int, read_key(d, "nope_layer_interval", int, 4))
            require(interval >= 1, "no_rope_layer_interval must be >= 1")
            no_rope = tuple(int((i + 1) % interval != 0) for i in range(n_layers))

        rs = d.get("rope_scaling")
        # Temperature tuning is on when its switch says so; a file that gives both constants
        # but no switch means it too.  The constants are required whenever it is on.
        switch = d.get("attn_temperature_tuning")
        tuning = bool(switch) if switch is not None else (d.get("floor_scale") is not None and d.get("attn_scale") is not None)
        eos = d.get("eos_token_id", cfg_json.get("eos_token_id"))
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        n_moe = len(moe_layers)
        n_dense = n_layers - n_moe
        cfg = Llama4Config(
            vocab_size=read_key(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=n_layers,
            num_attention_heads=n_heads,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            intermediate_size=read_key(d, "intermediate_size", int, *(() if n_moe else (0,))),
            intermediate_size_mlp=read_key(d, "intermediate_size_mlp", int, *(() if n_dense else (0,))),
            num_local_experts=read_key(d, "num_local_experts", int, *(() if n_moe else (0,))),
            num_experts_per_tok=read_key(d, "num_experts_per_tok", int, *(() if n_moe else (0,))),
            moe_layers=moe_layers,
            no_rope_layers=no_rope,
            rms_norm_eps=read_key(d, "rms_norm_eps", float),
            rope_theta=read_key(d, "rope_theta", float),
            rope_scaling=None if rs is None else RopeScaling.from_dict(rs),
            use_qk_norm=read_key(d, "use_qk_norm", bool, False),
            attention_chunk_size=read_key(d, "attention_chunk_size", int, None),
            attn_temperature_tuning=tuning,
            floor_scale=read_key(d, "floor_scale", float, *(() if tuning else (1.0,))),
            attn_scale=read_key(d, "attn_scale", float, *(() if tuning else (0.0,))),
            tie_word_embeddings=read_key(d, "tie_word_embeddings", bool, cfg_json.get("tie_word_embeddings", False) or False),
            max_position_embeddings=read_key(d, "max_position_embeddings", int, None),
            bos_token_id=read_key(d, "bos_token_id", int, None),
            eos_token_ids=eos_ids,
            pad_token_id=read_key(d, "pad_token_id", int, None),
            interleave_moe_layer_step=step,
            architecture=arch,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        L = self.num_hidden_layers
        require(L >= 1, "num_hidden_layers must be >= 1")
        require(self.hidden_size >= 1 and self.vocab_size >= 1, "hidden_size and vocab_size must be positive")
        require(self.num_attention_heads >= 1 and self.num_key_value_heads >= 1, "head counts must be positive")
        require(
            self.num_attention_heads % self.num_key_value_heads == 0,
            f"num_attention_heads ({self.num_attention_heads}) must be a multiple of num_key_value_heads ({self.num_key_value_heads})",
        )
        require(self.head_dim >= 2 and self.head_dim % 2 == 0, f"head_dim ({self.head_dim}) must be even (rotary pairs)")
        require(len(self.no_rope_layers) == L, f"no_rope_layers has {len(self.no_rope_layers)} entries for {L} layers")
        require(all(v in (0, 1) for v in self.no_rope_layers), "no_rope_layers entries must be 0 or 1")
        require(all(0 <= i < L for i in self.moe_layers), "moe_layers holds an index outside the model")
        require(len(set(self.moe_layers)) == len(self.moe_layers), "moe_layers names a layer twice")
        if self.moe_layers:
            require(self.num_local_experts >= 1, "num_local_experts must be >= 1")
            require(
                1 <= self.num_experts_per_tok <= self.num_local_experts,
                f"num_experts_per_tok ({self.num_experts_per_tok}) must be in 1..num_local_experts ({self.num_local_experts})",
            )
            require(self.intermediate_size >= 1, "intermediate_size must be positive")
        if len(self.moe_layers) < L:
            require(self.intermediate_size_mlp >= 1, "intermediate_size_mlp must be positive")
        require(self.rms_norm_eps > 0, "rms_norm_eps must be positive")
        require(self.rope_theta > 0, "rope_theta must be positive")
        if self.attention_chunk_size is not None:
            require(self.attention_chunk_size >= 1, "attention_chunk_size must be positive")
        require(self.floor_scale > 0, "floor_scale must be positive")

    # ---------------------------------------------------------------- per layer
    def layer_uses_rope(self, i: int) -> bool:
        return bool(self.no_rope_layers[i])

    def layer_is_moe(self, i: int) -> bool:
        return i in self.moe_layers

    # ------------------------------------------------------------------ writing
    def to_json_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        t: dict[str, Any] = {
            "model_type": "llama4_text",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "intermediate_size_mlp": self.intermediate_size_mlp,
            "num_local_experts": self.num_local_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "moe_layers": list(self.moe_layers),
            "no_rope_layers": list(self.no_rope_layers),
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "use_qk_norm": self.use_qk_norm,
            "attention_chunk_size": self.attention_chunk_size,
            "attn_temperature_tuning": self.attn_temperature_tuning,
            "floor_scale": self.floor_scale,
            "attn_scale": self.attn_scale,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.interleave_moe_layer_step is not None:
            t["interleave_moe_layer_step"] = self.interleave_moe_layer_step
        for k in ("max_position_embeddings", "bos_token_id", "pad_token_id"):
            if getattr(self, k) is not None:
                t[k] = getattr(self, k)
        if self.eos_token_ids:
            t["eos_token_id"] = list(self.eos_token_ids)
        if self.architecture == "Llama4ForConditionalGeneration":
            return {"architectures": [self.architecture], "model_type": "llama4", "text_config": t}
        return {"architectures": [self.architecture], **t}
