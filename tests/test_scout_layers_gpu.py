"""Layers of Llama 4 Scout's sizes (width 5120, 40 query / 8 KV heads of 128, expert width 8192) against
the plain implementation: two layers (one rotary and chunked, one NoPE with temperature), 4 experts and a small
vocabulary so that the plain implementation stays affordable on the CPU; the chunk (256) and the temperature
floor (128) are small so that a 600-token prompt crosses them.  Whole, with the tail decoded one by one, and
mixed (decoded tokens beside portions of up to 300 tokens); in 32-bit and in bfloat16.  And, on four such layers,
one 4096-token prompt in 32-bit, whole and in portions of 512."""

import random

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

SCOUT_LAYERS = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "num_hidden_layers": 2, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128,
    "interleave_moe_layer_step": 1, "num_local_experts": 4, "num_experts_per_tok": 1, "intermediate_size": 8192,
    "intermediate_size_mlp": 16384, "vocab_size": 1000, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "use_qk_norm": True, "attention_chunk_size": 256, "no_rope_layers": [1, 0], "attn_temperature_tuning": True,
    "floor_scale": 128.0, "attn_scale": 0.1, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}


@pytest.fixture(scope="module")
def scout_dir(tmp_path_factory):
    import jax_llm_examples_b200 as J

    return J.write_random_model(tmp_path_factory.mktemp("scout") / "m", SCOUT_LAYERS, seed=7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scout_sized_layers_under_every_cut(scout_dir, dtype):
    import jax_llm_examples_b200 as J

    rng = random.Random(1)
    reqs = H.random_requests(rng, 1000, [600, 130, 257])
    model = J.load_model(scout_dir, dtype)
    eng = J.Engine(model, max_tokens=1024, page_size=64, max_slots=4, use_graphs=False)
    traces = {"whole": H.trace_whole(reqs), "tail": H.trace_tail_decode(reqs, 32), "mixed": H.trace_mixed(reqs, rng, max_live=3, portions=H.LONG_PORTIONS)}
    results = {}
    for name, steps in traces.items():
        got, routing = H.run_trace(eng, steps)
        worst = H.compare_with_plain(scout_dir, reqs, got, routing, dtype)
        results[name] = got
        print(f"scout layers {dtype} {name}: worst relative error {worst:.2e}")
    if dtype == "float32":
        for name in ("tail", "mixed"):
            assert max(H.rel_err(results[name][k], results["whole"][k]) for k in results["whole"]) < 2e-6
    else:
        assert any("tc" in k and "split_kv" in k for k in eng.attention_kernels_seen), eng.attention_kernels_seen


@pytest.fixture(scope="module")
def scout4_dir(tmp_path_factory):
    import jax_llm_examples_b200 as J

    four = dict(SCOUT_LAYERS, num_hidden_layers=4, no_rope_layers=[1, 1, 0, 1])
    return J.write_random_model(tmp_path_factory.mktemp("scout4") / "m", four, seed=8)


def test_scout_sized_layers_4096_tokens_in_float32(scout4_dir):
    scout_dir = scout4_dir
    """The 32-bit path at length: one 4096-token prompt whole and in portions of 512 tokens (sixteen chunks, the
    temperature factor up to ln(33)), every position against the plain implementation."""
    import jax_llm_examples_b200 as J

    reqs = H.random_requests(random.Random(2), 1000, [4096])
    toks = reqs["r0"]
    model = J.load_model(scout_dir, "float32")
    eng = J.Engine(model, max_tokens=4096, page_size=64, max_slots=2)
    portions = [{"entries": [{"id": "r0", "tokens": toks[a:a + 512], "want": list(range(512))}], "end": ["r0"] if a + 512 == 4096 else []}
                for a in range(0, 4096, 512)]
    whole, routing = H.run_trace(eng, H.trace_whole(reqs))
    worst = H.compare_with_plain(scout_dir, reqs, whole, routing, "float32")
    print(f"scout layers float32, 4096 tokens whole: worst relative error {worst:.2e}")
    cut, _ = H.run_trace(eng, portions)
    assert max(H.rel_err(cut[k], whole[k]) for k in whole) < 2e-6
