"""Plain, slow implementation of the Llama 4 text decoder: the oracle of the tests.

It rests on the formulas of the reference, not on a run of it: the reference's model code
needs JAX, which is not installed where these tests run, so no golden output of it exists.
Each function cites the lines of the reference (paths within jax-ml/jax-llm-examples) that
it restates.  Two behaviours differ from the reference on purpose and are marked DEVIATION:
chunked attention is applied on rotary layers (the reference applies it on the NoPE layers,
llama4/llama4_jax/model.py:944), and NoPE layers scale their queries by the attention
temperature, which the reference does not have.

Whole sequences, no cache, materialised masks, Python loops over experts, one function for
each part.  Nothing here imports the engine's package.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ----------------------------------------------------------------------------- configuration
def text_config(config_json: dict) -> dict:
    """llama4/llama4_jax/model.py:229-231: the text decoder's keys live under text_config."""
    return config_json.get("text_config", config_json)


def layer_uses_rope(cfg: dict, i: int) -> bool:
    """model.py:913 (every 4th layer is NoPE) and model.py:201-202 (no_rope_layers[i]==1: rotary)."""
    if cfg.get("no_rope_layers"):
        return bool(cfg["no_rope_layers"][i])
    return (i + 1) % cfg.get("no_rope_layer_interval", 4) != 0


def layer_is_moe(cfg: dict, i: int) -> bool:
    """model.py:558: MoE iff (idx + 1) % moe_layer_interval == 0."""
    if cfg.get("moe_layers") is not None:
        return i in cfg["moe_layers"]
    return (i + 1) % cfg["interleave_moe_layer_step"] == 0


def temperature_on(cfg: dict) -> bool:
    sw = cfg.get("attn_temperature_tuning")
    if sw is None:
        return cfg.get("floor_scale") is not None and cfg.get("attn_scale") is not None
    return bool(sw)


# ------------------------------------------------------------------------------------- parts
def rms_norm(x: torch.Tensor, gamma: torch.Tensor | None, eps: float) -> torch.Tensor:
    """model.py:885-888: gamma * x / sqrt(mean(x^2) + eps); gamma None = weightless (L2 qk-norm)."""
    rms = torch.sqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps)
    return (gamma if gamma is not None else 1) * x / rms


def rope_inverse_frequencies(cfg: dict, dtype=torch.float32) -> torch.Tensor:
    """model.py:706-709 with the llama3 correction of model.py:654-672.

    The correction's constants come from config.json's rope_scaling (the reference fixes them
    in code, model.py:160-163); without rope_scaling there is no correction.  When
    high_freq_factor == low_freq_factor there is no medium band, and the smooth factor of
    model.py:668 (a division by zero there) is never used.
    """
    dh = cfg["head_dim"]
    fraction = torch.arange(0, dh, 2, dtype=torch.float32) / dh
    timescale = torch.tensor(float(cfg["rope_theta"]), dtype=torch.float32) ** fraction
    freq = (1.0 / timescale).to(dtype)
    rs = cfg.get("rope_scaling")
    if rs is None:
        return freq
    factor, low, high = float(rs["factor"]), float(rs["low_freq_factor"]), float(rs["high_freq_factor"])
    old_len = float(rs["original_max_position_embeddings"])
    low_freq_wavelen, high_freq_wavelen = old_len / low, old_len / high
    wavelen = 2 * math.pi / freq
    out = torch.where(wavelen > low_freq_wavelen, freq / factor, freq)
    if high != low:
        smooth = (old_len / wavelen - low) / (high - low)
        smoothed = (1 - smooth) * out / factor + smooth * out
        medium = ~(wavelen < high_freq_wavelen) & ~(wavelen > low_freq_wavelen)
        out = torch.where(medium, smoothed, out)
    return out


def apply_rope_interleaved(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """model.py:712-728: angle = position * frequency; adjacent pairs (2j, 2j+1) are rotated.

    x: [T, H, dh]; positions: [T].
    """
    angle = positions.to(inv_freq.dtype)[:, None] * inv_freq[None, :]  # [T, dh/2]
    sin, cos = torch.sin(angle)[:, None, :], torch.cos(angle)[:, None, :]
    sin, cos = sin.to(x.dtype), cos.to(x.dtype)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).reshape(x.shape)


def attention_temperature(positions: torch.Tensor, floor_scale: float, attn_scale: float) -> torch.Tensor:
    """DEVIATION (the reference has no temperature): query scale on NoPE layers,
    1 + attn_scale * ln(1 + floor((p + 1) / floor_scale)), p the query's absolute position.
    Where the definition comes from: this build's task statement names attention-temperature tuning on the NoPE
    layers with the constants floor_scale and attn_scale (config.json's ``attn_temperature_tuning``,
    ``floor_scale``, ``attn_scale``; Llama 4 Scout ships 8192 and 0.1); the formula is the one published with the
    Llama 4 models for those keys.  No line of jax-ml/jax-llm-examples states it, so nothing there can be cited."""
    p = positions.to(torch.float32)
    return torch.log1p(torch.floor((p + 1.0) / floor_scale)) * attn_scale + 1.0


def attention_mask(positions: torch.Tensor, chunk: int | None, window: int | None = None) -> torch.Tensor:
    """model.py:731-742: causal, and (if chunked) query and key in the same chunk.  [T, T] bool.

    ``window`` (keys within the last `window` positions) is not Llama 4; it serves the tests of
    the cache manager's windowed group."""
    q, k = positions[:, None], positions[None, :]
    mask = q >= k
    if chunk is not None:
        mask = mask & (q // chunk == k // chunk)
    if window is not None:
        mask = mask & (q - k < window)
    return mask


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """model.py:774-794: query head h uses KV head h // G; scores * dh^-0.5; masked to -1e30;
    softmax; weighted sum of values.  q: [T, Hq, dh]; k, v: [T, Hkv, dh]; returns [T, Hq, dh]."""
    T, Hq, dh = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    scale = dh ** -0.5
    q_ = q.reshape(T, Hkv, G, dh)
    scores = torch.einsum("thgd,shd->hgts", q_, k) * scale
    scores = torch.where(mask[None, None], scores, torch.full_like(scores, -1e30))
    p = torch.softmax(scores, dim=-1)
    out = torch.einsum("hgts,shd->thgd", p, v)
    return out.reshape(T, Hq, dh)


def swiglu(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """model.py:1142-1153: down(silu(h gate) * (h up)).  Weights in [in, out] orientation."""
    return (torch.nn.functional.silu(h @ w_gate) * (h @ w_up)) @ w_down


def route(h: torch.Tensor, w_router: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """model.py:965-967: scores = h W; top-k of the raw scores; weights = sigmoid of the chosen.
    Ties go to the lower expert index (the order of jax.lax.top_k).  Returns (weights [T,k],
    experts [T,k], the gap between the k-th and (k+1)-th score [T])."""
    scores = h @ w_router  # [T, E]
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    vals, idx = order.values[:, :k], order.indices[:, :k]
    if scores.shape[1] > k:
        gap = order.values[:, k - 1] - order.values[:, k]
    else:
        gap = torch.full((scores.shape[0],), float("inf"), dtype=scores.dtype)
    return torch.sigmoid(vals), idx, gap


def moe(h, w_router, we_gate_up, we_down, ws_gate, ws_up, ws_down, k: int, forced_idx=None):
    """model.py:999-1139 on one device: each chosen expert gets the token scaled by its router
    weight (model.py:1071), the routed outputs are summed (model.py:1111), and the shared expert
    runs on the unscaled token (model.py:1137-1139).  we_gate_up: [E, D, 2F], first half gate
    (chkpt_utils.py:198-205); we_down: [E, F, D].

    ``forced_idx`` [T, k] replaces the router's own choice of experts (the weights are still the
    sigmoid of this implementation's scores).  It exists for comparing with an implementation in
    lower precision, whose choice may rightly differ where two scores are nearly equal.  Returns
    (output, by how much each forced expert's score lies below the k-th best score, as a fraction of the
    router's typical score size, the RMS of all scores of the sequence [T]).  Rounding noise in a score is
    proportional to that size, not to the size of the token's own scores."""
    T, D = h.shape
    F = we_down.shape[1]
    w, idx, _ = route(h, w_router, k)
    scores = h @ w_router
    kth = torch.sort(scores, dim=-1, descending=True).values[:, k - 1]
    if forced_idx is not None:
        idx = torch.as_tensor(forced_idx, dtype=torch.long)
        w = torch.sigmoid(torch.gather(scores, 1, idx))
    shortfall = (kth[:, None] - torch.gather(scores, 1, idx)).max(dim=-1).values / scores.pow(2).mean().sqrt()
    routed = torch.zeros_like(h)
    for t in range(T):
        for j in range(k):
            e = int(idx[t, j])
            u = h[t] * w[t, j]
            routed[t] += swiglu(u[None], we_gate_up[e][:, :F], we_gate_up[e][:, F:], we_down[e])[0]
    return routed + swiglu(h, ws_gate, ws_up, ws_down), shortfall


# ------------------------------------------------------------------------------------ weights
def load_weights(model_dir: str | Path, dtype=torch.float32) -> dict[str, torch.Tensor]:
    """Reads model.safetensors by HF tensor name (chkpt_utils.py:161-196), dropping the
    ``language_model.`` prefix (scripts/convert_weights.py:41) when the file has it."""
    from safetensors import safe_open

    out = {}
    with safe_open(str(Path(model_dir) / "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            key = name[len("language_model."):] if name.startswith("language_model.") else name
            out[key] = f.get_tensor(name).to(dtype)
    return out


def load_config(model_dir: str | Path) -> dict:
    return text_config(json.loads((Path(model_dir) / "config.json").read_text()))


# -------------------------------------------------------------------------------------- model
def layer_forward(cfg: dict, w: dict[str, torch.Tensor], i: int, x: torch.Tensor, positions: torch.Tensor,
                  inv_freq: torch.Tensor, stats: dict | None = None, forced_routing: dict | None = None) -> torch.Tensor:
    """model.py:1156-1183 with attention_block model.py:891-955."""
    p = f"model.layers.{i}."
    eps = float(cfg["rms_norm_eps"])
    T = x.shape[0]
    Hq, Hkv, dh = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"]), cfg["head_dim"]

    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)  # model.py:1170
    # HF stores Linear weights as [out, in] (chkpt_utils.py:84-92)
    q = (h @ w[p + "self_attn.q_proj.weight"].T).reshape(T, Hq, dh)
    k = (h @ w[p + "self_attn.k_proj.weight"].T).reshape(T, Hkv, dh)
    v = (h @ w[p + "self_attn.v_proj.weight"].T).reshape(T, Hkv, dh)
    if layer_uses_rope(cfg, i):  # model.py:913-917
        q, k = apply_rope_interleaved(q, positions, inv_freq), apply_rope_interleaved(k, positions, inv_freq)
        if cfg.get("use_qk_norm", False):
            q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
        chunk = cfg.get("attention_chunk_size")  # DEVIATION: chunked on rotary layers
    else:
        chunk = None
        if temperature_on(cfg):
            q = q * attention_temperature(positions, float(cfg["floor_scale"]), float(cfg["attn_scale"]))[:, None, None].to(q.dtype)
    a = gqa_attention(q, k, v, attention_mask(positions, chunk))
    x = x + a.reshape(T, Hq * dh) @ w[p + "self_attn.o_proj.weight"].T  # model.py:952-954, 1173

    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)  # model.py:1177
    if layer_is_moe(cfg, i):
        f, gap = moe(
            h,
            w[p + "feed_forward.router.weight"].T,
            w[p + "feed_forward.experts.gate_up_proj"],
            w[p + "feed_forward.experts.down_proj"],
            w[p + "feed_forward.shared_expert.gate_proj.weight"].T,
            w[p + "feed_forward.shared_expert.up_proj.weight"].T,
            w[p + "feed_forward.shared_expert.down_proj.weight"].T,
            cfg["num_experts_per_tok"],
            None if forced_routing is None else forced_routing[i],
        )
        if stats is not None:
            stats.setdefault("router_shortfall", {})[i] = gap
    else:
        f = swiglu(h, w[p + "feed_forward.gate_proj.weight"].T, w[p + "feed_forward.up_proj.weight"].T,
                   w[p + "feed_forward.down_proj.weight"].T)
    return x + f  # model.py:1181


def forward(cfg: dict, w: dict[str, torch.Tensor], tokens, stats: dict | None = None,
            forced_routing: dict | None = None) -> torch.Tensor:
    """model.py:1186-1204: embedding, the layers in order, final norm, lm_head.  One whole
    sequence from position 0; returns logits [T, V] at every position.  ``forced_routing``:
    {layer index: expert choices [T, k]}, see :func:`moe`."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    dtype = w["model.embed_tokens.weight"].dtype
    x = w["model.embed_tokens.weight"][tokens]
    positions = torch.arange(tokens.shape[0])
    inv_freq = rope_inverse_frequencies(cfg, dtype)
    for i in range(cfg["num_hidden_layers"]):
        x = layer_forward(cfg, w, i, x, positions, inv_freq, stats, forced_routing)
    x = rms_norm(x, w["model.norm.weight"], float(cfg["rms_norm_eps"]))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return x @ head.T


def greedy_generate(cfg: dict, w: dict[str, torch.Tensor], prompt, steps: int) -> list[int]:
    """llama4/main.py:69-74: argmax at the last position, append, repeat (whole sequence each time)."""
    toks = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward(cfg, w, toks)
        nxt = int(torch.argmax(logits[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


# ----------------------------------------------------------------------------------- sampling
def philox4x32(counter: tuple[int, int, int, int], key: tuple[int, int], rounds: int = 10) -> tuple[int, ...]:
    """Philox-4x32 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = list(counter)
    k0, k1 = key
    for _ in range(rounds):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k0, p1 & 0xFFFFFFFF, (p0 >> 32) ^ c[3] ^ k1, p0 & 0xFFFFFFFF]
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return tuple(c)


def uniform_from_bits(bits: int) -> float:
    """24 high bits -> [0, 1)."""
    return (bits >> 8) * (1.0 / 16777216.0)


def sample_top(logits: torch.Tensor, temperature: float, top_k: int, u: float) -> int:
    """gpt_oss/gpt_oss_jax/model.py:1125-1147: softmax(logits / temp), keep the k most likely
    (all, in index order, when k = 0), normalised cumulative sum, first index whose cumulative value is >= u;
    temp <= 1e-3 means argmax."""
    if temperature <= 1e-3:
        return int(torch.argmax(logits))
    probs = torch.softmax(logits.to(torch.float32) / temperature, dim=-1)
    if top_k <= 0:  # whole vocabulary: cumulative sum in index order, no sort
        top_p, top_i = probs, torch.arange(probs.shape[-1])
    else:
        order = torch.sort(probs, descending=True, stable=True)
        k = min(top_k, probs.shape[-1])
        top_p, top_i = order.values[:k], order.indices[:k]
    cum = torch.cumsum(top_p.double(), dim=-1) / torch.sum(top_p.double())
    hit = torch.nonzero(u <= cum)
    j = int(hit[0]) if hit.numel() else top_p.shape[-1] - 1
    return int(top_i[j])
