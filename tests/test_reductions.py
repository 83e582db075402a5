"""Reduction invariants: configurations of the architecture under which its special parts fall away must give
what a plain dense decoder gives.

* No MoE layer, every layer rotary, no q/k norm, no temperature, a chunk longer than the sequence: a plain
  pre-norm decoder with grouped-query attention, rotary pairs and SwiGLU.
* MoE layers with k = E: every token takes every expert, so routing, sorting and gathering must change nothing:
  the layer is the dense sum over e of SwiGLU_e(sigmoid(score_e) * h), plus the shared expert on h.

The dense decoder below is written on its own (it shares no code with the plain implementation, which it
checks here, nor with the engine, which the GPU test checks)."""

import math
import random

import pytest
import torch

from tests import helpers as H

REDUCED = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "num_hidden_layers": 4, "hidden_size": 80, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 32,
    "moe_layers": [1, 3], "num_local_experts": 3, "num_experts_per_tok": 3, "intermediate_size": 48,
    "intermediate_size_mlp": 112, "vocab_size": 200, "rope_theta": 10000.0, "rope_scaling": None,
    "use_qk_norm": False, "attention_chunk_size": 4096, "no_rope_layers": [1, 1, 1, 1],
    "attn_temperature_tuning": False, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}


def dense_decoder(w: dict, c: dict, toks: list[int]) -> torch.Tensor:
    """Logits [T, V] of a plain dense decoder, float64 inside."""
    w = {k: v.double() for k, v in w.items()}
    T, Hq, Hkv, dh, eps = len(toks), c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], c["rms_norm_eps"]
    norm = lambda x, g: g * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    act = lambda x, gate, up, down: (torch.nn.functional.silu(x @ gate.T) * (x @ up.T)) @ down.T
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    pos = torch.arange(T, dtype=torch.float64)
    theta = torch.tensor([c["rope_theta"] ** (-2.0 * j / dh) for j in range(dh // 2)], dtype=torch.float64)
    cos, sin = torch.cos(pos[:, None] * theta)[:, None], torch.sin(pos[:, None] * theta)[:, None]

    def turn(z):  # pairs (2j, 2j + 1) as complex numbers times e^{i angle}
        zc = torch.view_as_complex(z.reshape(*z.shape[:-1], dh // 2, 2).contiguous()) * torch.complex(cos, sin)
        return torch.view_as_real(zc).reshape(z.shape)

    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = norm(x, w[p + "input_layernorm.weight"])
        q = turn((h @ w[p + "self_attn.q_proj.weight"].T).reshape(T, Hq, dh))
        k = turn((h @ w[p + "self_attn.k_proj.weight"].T).reshape(T, Hkv, dh)).repeat_interleave(Hq // Hkv, 1)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).reshape(T, Hkv, dh).repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,shd->hts", q, k) / math.sqrt(dh)
        a = torch.einsum("hts,shd->thd", torch.softmax(s.masked_fill(~causal, -math.inf), -1), v)
        x = x + a.reshape(T, Hq * dh) @ w[p + "self_attn.o_proj.weight"].T
        h = norm(x, w[p + "post_attention_layernorm.weight"])
        f = p + "feed_forward."
        if i in c["moe_layers"]:
            gate_w = torch.sigmoid(h @ w[f + "router.weight"].T)  # [T, E]: every expert, weight on the INPUT
            F = w[f + "experts.down_proj"].shape[1]
            y = act(h, w[f + "shared_expert.gate_proj.weight"], w[f + "shared_expert.up_proj.weight"], w[f + "shared_expert.down_proj.weight"])
            for e in range(c["num_local_experts"]):
                gu = w[f + "experts.gate_up_proj"][e]  # [D, 2F], gate columns first
                y = y + act(h * gate_w[:, e:e + 1], gu[:, :F].T, gu[:, F:].T, w[f + "experts.down_proj"][e].T)
        else:
            y = act(h, w[f + "gate_proj.weight"], w[f + "up_proj.weight"], w[f + "down_proj.weight"])
        x = x + y
    return (norm(x, w["model.norm.weight"]) @ w["lm_head.weight"].T).float()


@pytest.fixture(scope="module")
def reduced_dir(tmp_path_factory):
    import jax_llm_examples_b200 as J

    return J.write_random_model(tmp_path_factory.mktemp("reduced") / "m", REDUCED, seed=4, norm_noise=0.1, dtype=torch.float32, std=0.1)


def _weights(folder):
    from safetensors.torch import load_file

    return load_file(str(folder / "model.safetensors"))


def test_the_plain_implementation_reduces_to_a_dense_decoder(reduced_dir):
    toks = [random.Random(1).randrange(200) for _ in range(70)]
    ref = dense_decoder(_weights(reduced_dir), REDUCED, toks).numpy()
    got, _ = H.plain_logits(reduced_dir, toks)
    assert H.rel_err(got, ref) < 2e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_engine_reduces_to_a_dense_decoder(reduced_dir, dtype):
    import jax_llm_examples_b200 as J

    rng = random.Random(2)
    reqs = H.random_requests(rng, 200, [70, 33, 9])
    eng = J.Engine(J.load_model(reduced_dir, dtype, "cuda"), max_tokens=192, page_size=16, max_slots=4)
    w = _weights(reduced_dir)
    for steps in (H.trace_whole(reqs), H.trace_mixed(reqs, rng, max_live=3)):
        got, _ = H.run_trace(eng, steps)
        for rid, toks in reqs.items():
            ref = dense_decoder(w, REDUCED, toks).numpy()
            worst = max(H.rel_err(got[(rid, p)], ref[p]) for p in range(len(toks)))
            assert worst < H.TOL[dtype], (rid, worst)
