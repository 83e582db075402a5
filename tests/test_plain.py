"""The plain implementation checked against itself: properties that any right implementation of the
reference's formulas has (no GPU).  It cannot be compared with a run of the reference: JAX is not
installed here, so tests/golden/ holds no outputs of it."""

import math

import numpy as np
import pytest
import torch

import jax_llm_examples_b200 as J
from tests import helpers as H
from tests.plain import llama4_plain as plain


def test_philox_known_answers():
    assert plain.philox4x32((0, 0, 0, 0), (0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    ones = 0xFFFFFFFF
    assert plain.philox4x32((ones,) * 4, (ones, ones)) == (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)


def test_rope_is_a_rotation_and_depends_on_relative_position():
    cfg = plain.text_config(J.preset("tiny_b"))
    f = plain.rope_inverse_frequencies(cfg)
    assert f.shape == (12,) and torch.isfinite(f).all()
    q, k = torch.randn(5, 2, 24), torch.randn(5, 2, 24)
    p0, p1 = torch.arange(5), torch.arange(5) + 37
    q0, k0 = plain.apply_rope_interleaved(q, p0, f), plain.apply_rope_interleaved(k, p0, f)
    q1, k1 = plain.apply_rope_interleaved(q, p1, f), plain.apply_rope_interleaved(k, p1, f)
    assert torch.allclose(q0.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    s0 = torch.einsum("thd,shd->hts", q0, k0)
    s1 = torch.einsum("thd,shd->hts", q1, k1)
    assert torch.allclose(s0, s1, atol=1e-3)
    # pairs are adjacent: rotating only dims (0, 1) by the first frequency
    x = torch.zeros(1, 1, 24)
    x[0, 0, 0] = 1
    y = plain.apply_rope_interleaved(x, torch.tensor([3]), f)
    assert torch.allclose(y[0, 0, :2], torch.tensor([math.cos(3 * float(f[0])), math.sin(3 * float(f[0]))]), atol=1e-6)
    assert torch.all(y[0, 0, 2:] == 0)


def test_llama3_scaling_bands_and_equal_factors():
    cfg = plain.text_config(J.preset("tiny_b"))
    base = plain.rope_inverse_frequencies({**cfg, "rope_scaling": None})
    scaled = plain.rope_inverse_frequencies(cfg)
    wavelen = 2 * math.pi / base
    high, low = wavelen < 64 / 4, wavelen > 64 / 1
    assert torch.equal(scaled[high], base[high]) and torch.allclose(scaled[low], base[low] / 8)
    mid = ~high & ~low
    assert mid.any() and torch.all(scaled[mid] < base[mid]) and torch.all(scaled[mid] > base[mid] / 8)
    scout = plain.text_config(J.preset("scout16"))
    f = plain.rope_inverse_frequencies(scout)  # high == low: no medium band, nothing divides by zero
    assert torch.isfinite(f).all()


def test_masks():
    pos = torch.arange(10)
    m = plain.attention_mask(pos, 4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 4
    assert m[4].tolist() == [False] * 4 + [True] + [False] * 5
    assert plain.attention_mask(pos, None)[9].all()
    assert plain.attention_mask(pos, None, 3)[9].tolist() == [False] * 7 + [True] * 3


def test_temperature_steps_at_multiples_of_the_floor():
    t = plain.attention_temperature(torch.tensor([0, 14, 15, 30, 31, 47]), 16.0, 0.1)
    want = [1.0, 1.0, 1 + 0.1 * math.log(2), 1 + 0.1 * math.log(2), 1 + 0.1 * math.log(3), 1 + 0.1 * math.log(4)]
    assert torch.allclose(t, torch.tensor(want), atol=1e-6)


def test_router_ties_go_to_the_lower_index_and_weights_are_sigmoids():
    h = torch.tensor([[1.0, 0.0]])
    w = torch.tensor([[0.5, 2.0, 2.0, -1.0], [0, 0, 0, 0]])
    wt, idx, gap = plain.route(h, w, 2)
    assert idx.tolist() == [[1, 2]] and torch.allclose(wt, torch.sigmoid(torch.tensor([[2.0, 2.0]])))
    assert float(gap) == pytest.approx(1.5)


def test_permuting_the_experts_changes_nothing(tmp_path):
    folder = H.make_model_dir(tmp_path / "m", "tiny_b", seed=3)
    cfg, w = plain.load_config(folder), plain.load_weights(folder)
    toks = list(range(3, 60))
    ref = plain.forward(cfg, w, toks)
    perm = torch.randperm(8)
    w2 = dict(w)
    for i in range(8):
        if plain.layer_is_moe(cfg, i):
            p = f"model.layers.{i}.feed_forward."
            w2[p + "router.weight"] = w[p + "router.weight"][perm]
            w2[p + "experts.gate_up_proj"] = w[p + "experts.gate_up_proj"][perm]
            w2[p + "experts.down_proj"] = w[p + "experts.down_proj"][perm]
    assert torch.allclose(plain.forward(cfg, w2, toks), ref, atol=1e-5)


@pytest.mark.parametrize("name, n", [("tiny_a", 80), ("tiny_b", 130)])
def test_token_by_token_with_a_naive_cache_equals_the_whole_sequence(tmp_path, name, n):
    """A second, independent evaluation order: one token at a time over a contiguous cache of keys
    and values, written here without the functions of the whole-sequence path's layer loop."""
    folder = H.make_model_dir(tmp_path / "m", name, seed=4, norm_noise=0.1)
    cfg, w = plain.load_config(folder), plain.load_weights(folder)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg["vocab_size"], n).tolist()
    ref = plain.forward(cfg, w, toks)
    L, Hq, Hkv, dh = cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    G, eps, f = Hq // Hkv, cfg["rms_norm_eps"], plain.rope_inverse_frequencies(cfg)
    keys = [[] for _ in range(L)]
    vals = [[] for _ in range(L)]
    worst = 0.0
    for p, tok in enumerate(toks):
        x = w["model.embed_tokens.weight"][tok][None]
        pos = torch.tensor([p])
        for i in range(L):
            pre = f"model.layers.{i}."
            h = plain.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
            q = (h @ w[pre + "self_attn.q_proj.weight"].T).reshape(1, Hq, dh)
            k = (h @ w[pre + "self_attn.k_proj.weight"].T).reshape(1, Hkv, dh)
            v = (h @ w[pre + "self_attn.v_proj.weight"].T).reshape(1, Hkv, dh)
            first = 0
            if plain.layer_uses_rope(cfg, i):
                q, k = plain.apply_rope_interleaved(q, pos, f), plain.apply_rope_interleaved(k, pos, f)
                if cfg["use_qk_norm"]:
                    q, k = plain.rms_norm(q, None, eps), plain.rms_norm(k, None, eps)
                first = (p // cfg["attention_chunk_size"]) * cfg["attention_chunk_size"]
            else:
                q = q * (1 + cfg["attn_scale"] * math.log1p(math.floor((p + 1) / cfg["floor_scale"])))
            keys[i].append(k[0])
            vals[i].append(v[0])
            K_, V_ = torch.stack(keys[i][first:]), torch.stack(vals[i][first:])  # [S, Hkv, dh]
            out = torch.empty(Hq, dh)
            for hq in range(Hq):
                s = (K_[:, hq // G] @ q[0, hq]) * dh ** -0.5
                out[hq] = torch.softmax(s, 0) @ V_[:, hq // G]
            x = x + out.reshape(1, -1) @ w[pre + "self_attn.o_proj.weight"].T
            h = plain.rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps)
            if plain.layer_is_moe(cfg, i):
                ff, _ = plain.moe(h, w[pre + "feed_forward.router.weight"].T, w[pre + "feed_forward.experts.gate_up_proj"],
                                  w[pre + "feed_forward.experts.down_proj"],
                                  w[pre + "feed_forward.shared_expert.gate_proj.weight"].T,
                                  w[pre + "feed_forward.shared_expert.up_proj.weight"].T,
                                  w[pre + "feed_forward.shared_expert.down_proj.weight"].T, cfg["num_experts_per_tok"])
            else:
                ff = plain.swiglu(h, w[pre + "feed_forward.gate_proj.weight"].T, w[pre + "feed_forward.up_proj.weight"].T,
                                  w[pre + "feed_forward.down_proj.weight"].T)
            x = x + ff
        logits = plain.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T
        worst = max(worst, H.rel_err(logits[0].numpy(), ref[p].numpy()))
    assert worst < 2e-5, worst


def test_sample_top():
    logits = torch.tensor([0.0, 3.0, 1.0, 3.0, -2.0])
    assert plain.sample_top(logits, 0.0, 0, 0.7) == 1  # argmax, lower index on a tie
    p = torch.softmax(logits / 0.5, 0)
    assert plain.sample_top(logits, 0.5, 2, 0.49) == 1 and plain.sample_top(logits, 0.5, 2, 0.51) == 3
    cum = torch.cumsum(p, 0)
    for u in (0.01, 0.3, 0.6, 0.99):
        assert plain.sample_top(logits, 0.5, 0, u) == int(torch.nonzero(u <= cum)[0])
