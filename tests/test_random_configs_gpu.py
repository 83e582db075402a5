"""Random tiny configurations of the architecture, every size and option drawn anew (head sizes from 16 to 256 in
steps of 16, 1 to 20 query heads per KV head, widths and vocabularies that are no power of two or no multiple of
8, 1 to 40 experts, top-k up to all of them, layer kinds given as lists), through the engine in both precisions:
a mixed trace with so few pages that they are used again, and most of each request at once with the last 32
tokens one by one, against the plain implementation."""

import random

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random, wide: bool = False) -> dict:
    dh = rng.choice([16, 32, 48, 64, 64, 96, 112, 128, 128, 144, 256])
    hkv = rng.choice([1, 2, 3, 4])
    group = rng.choice([1, 2, 3, 5, 8, 10, 16, 20]) if dh in (64, 128) else rng.choice([1, 2, 3])
    layers = rng.randint(2, 5)
    experts = rng.choice([1, 2, 3, 5, 8, 16, 40])
    top_k = min(rng.choice([1, 1, 2, 3, experts if experts <= 8 else 1]), experts)
    cfg = {
        "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text", "num_hidden_layers": layers,
        "hidden_size": rng.choice([60, 64, 100, 96, 136, 250, 256, 1024]), "num_attention_heads": hkv * group,
        "num_key_value_heads": hkv, "head_dim": dh, "moe_layers": [i for i in range(layers) if rng.random() < 0.6],
        "num_local_experts": experts, "num_experts_per_tok": top_k, "intermediate_size": rng.choice([24, 32, 40, 64, 96, 128]),
        "intermediate_size_mlp": rng.choice([64, 80, 160]), "vocab_size": rng.choice([100, 257, 321, 1000, 5003]),
        "rope_theta": rng.choice([10000.0, 500000.0]), "use_qk_norm": rng.random() < 0.5,
        "attention_chunk_size": rng.choice([32, 48, 64, 80, 128, 200]),
        "no_rope_layers": [1 if rng.random() < 0.7 else 0 for _ in range(layers)],
        "attn_temperature_tuning": rng.random() < 0.5, "floor_scale": float(rng.choice([16, 24, 100])), "attn_scale": 0.1,
        "rms_norm_eps": rng.choice([1e-5, 1e-6]), "tie_word_embeddings": rng.random() < 0.2,
    }
    if rng.random() < 0.5:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                               "high_freq_factor": rng.choice([1.0, 4.0]), "original_max_position_embeddings": rng.choice([32, 64])}
    if wide:
        # widths from 1024 on take the kernels that a decode step of the real sizes takes (a cluster of blocks per row
        # for the norms, the norm that also sorts and gathers); a shared expert of the experts' shape rides as a group
        # of the experts' products when a step has one row
        cfg["hidden_size"] = rng.choice([1024, 1032, 1280, 2048])
        cfg["intermediate_size"] = rng.choice([32, 64, 96, 128])
        if rng.random() < 0.6:
            cfg["intermediate_size_mlp"] = cfg["intermediate_size"]
    return cfg


@pytest.mark.parametrize("seed", [202, 207, 211, 214, 216, 219, 226, 229, 301, 302])
def test_a_random_configuration(tmp_path, seed):
    import jax_llm_examples_b200 as J

    rng = random.Random(seed)
    cfg = random_config(rng)
    page = rng.choice([16, 64])
    folder = J.write_random_model(tmp_path / "m", cfg, seed, dtype=torch.bfloat16, norm_noise=0.1)
    lengths = [rng.randint(1, 150) for _ in range(5)] + [rng.choice([129, 200, 260])]
    reqs = H.random_requests(rng, cfg["vocab_size"], lengths)
    for dtype in ("float32", "bfloat16"):
        model = J.load_model(folder, dtype, "cuda")
        need = sum(-(-n // page) * page for n in sorted(lengths)[-4:])  # the four longest may be live together
        eng = J.Engine(model, max_tokens=need, page_size=page, max_slots=4)
        got, routing = H.run_trace(eng, H.trace_mixed(reqs, random.Random(seed), max_live=4))
        H.compare_with_plain(folder, reqs, got, routing, dtype)
        got, routing = H.run_trace(eng, H.trace_tail_decode(reqs, 32))
        H.compare_with_plain(folder, reqs, got, routing, dtype)
        assert all(eng.manager.free_pages(g) == eng.num_pages for g in range(len(eng.manager.groups)))


@pytest.mark.parametrize("seed", [500, 503, 511, 517])
def test_a_random_wide_configuration(tmp_path, seed):
    import jax_llm_examples_b200 as J

    rng = random.Random(seed)
    cfg = random_config(rng, wide=True)
    page = 64
    folder = J.write_random_model(tmp_path / "m", cfg, seed, dtype=torch.bfloat16, norm_noise=0.1)
    lengths = [rng.randint(1, 200) for _ in range(4)] + [rng.choice([129, 300])]
    reqs = H.random_requests(rng, cfg["vocab_size"], lengths)
    for dtype in ("float32", "bfloat16"):
        model = J.load_model(folder, dtype, "cuda")
        need = sum(-(-n // page) * page for n in sorted(lengths)[-4:])
        eng = J.Engine(model, max_tokens=need, page_size=page, max_slots=4)
        got, routing = H.run_trace(eng, H.trace_mixed(reqs, random.Random(seed), max_live=4, portions=H.LONG_PORTIONS))
        H.compare_with_plain(folder, reqs, got, routing, dtype)
        got, routing = H.run_trace(eng, H.trace_tail_decode(reqs, 32))
        H.compare_with_plain(folder, reqs, got, routing, dtype)


def test_forty_experts_top_two_and_prompts_of_hundreds_of_tokens(tmp_path):
    """More groups than a warp has lanes, two choices per token, and hundreds of (token, choice) pairs in a step: the
    sort's list of row tiles is long here, and once ran past its end."""
    import jax_llm_examples_b200 as J

    rng = random.Random(232)
    cfg = random_config(rng)
    cfg.update(num_hidden_layers=2, hidden_size=64, num_attention_heads=5, num_key_value_heads=1, head_dim=128, moe_layers=[0, 1],
               num_local_experts=40, num_experts_per_tok=2, intermediate_size=40, intermediate_size_mlp=64, no_rope_layers=[1, 1])
    folder = J.write_random_model(tmp_path / "m", cfg, 232, dtype=torch.bfloat16, norm_noise=0.1)
    reqs = H.random_requests(rng, cfg["vocab_size"], [353, 202, 144])
    for dtype in ("float32", "bfloat16"):
        eng = J.Engine(J.load_model(folder, dtype, "cuda"), max_tokens=1024, page_size=64, max_slots=3)
        got, routing = H.run_trace(eng, H.trace_whole(reqs))
        H.compare_with_plain(folder, reqs, got, routing, dtype)
