"""The step shape a serving run produces most often, on the kernels that serve it at head size 128: decoded
single tokens beside prompt portions of 64 tokens and more.  The attention part then sends one step's rows to
three kernels that write disjoint rows of one output (split-KV for the single tokens, the tcgen05 flash kernel
for long portions, the mma.sync flash kernel for short ones).  Tiny widths, head size 128, against the plain
implementation in 32-bit and in bfloat16: by traces (portion sizes around 64 and 128, pages reused) and once
through the real scheduler."""

import random

import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

# tiny_a with head size 128: one query head per KV head pair (G = 2), and five (G = 5, as in Llama 4 Scout); the
# chunk of the second (192) is no multiple of the tile height (128), so that tiles straddle chunk starts anywhere
HEAD128 = {
    "g2": dict(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, head_dim=128, attention_chunk_size=128),
    "g5": dict(hidden_size=320, num_attention_heads=10, num_key_value_heads=2, head_dim=128, attention_chunk_size=192,
               num_hidden_layers=3, no_rope_layers=[1, 0, 1], floor_scale=100.0),
}
PAGE = 64


@pytest.fixture(scope="module")
def head128_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("head128")
    return {name: H.make_model_dir(root / name, "tiny_a", seed=10 + i, norm_noise=0.1, **over)
            for i, (name, over) in enumerate(HEAD128.items())}


def _engine(folder, dtype, max_tokens, **kw):
    import jax_llm_examples_b200 as J

    return J.Engine(J.load_model(folder, dtype, "cuda"), max_tokens=max_tokens, page_size=PAGE, max_slots=8, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(HEAD128))
def test_mixed_steps_with_long_portions(head128_dirs, name, dtype):
    rng = random.Random(31)
    lengths = [520, 330, 700, 129, 64, 411, 257, 600, 90, 385]
    reqs = H.random_requests(rng, 256, lengths)
    longest = -(-max(lengths) // PAGE) * PAGE
    eng = _engine(head128_dirs[name], dtype, max_tokens=4 * longest)
    steps = H.trace_mixed(reqs, rng, max_live=4, portions=H.LONG_PORTIONS)
    got, routing = H.run_trace(eng, steps)
    worst = H.compare_with_plain(head128_dirs[name], reqs, got, routing, dtype)
    print(f"{name} {dtype} mixed with long portions: worst relative error {worst:.2e}")
    assert sum(-(-n // PAGE) for n in lengths) > eng.num_pages, "the trace must need more pages than the pool has"
    if dtype == "bfloat16":
        # the composition under test really occurred: all three attention kernels in one step
        assert ("tc", "flash", "split_kv") in eng.attention_kernels_seen, eng.attention_kernels_seen
        assert ("tc", "split_kv") in eng.attention_kernels_seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_agree_with_whole_prompts(head128_dirs, dtype):
    """Whole prompts, the tail decoded, and portions around the kernels' sizes give the same logits (32-bit: to
    rounding of the sums' order; bfloat16: within its tolerance of the plain implementation)."""
    rng = random.Random(32)
    reqs = H.random_requests(rng, 256, [450, 128, 321])
    eng = _engine(head128_dirs["g5"], dtype, max_tokens=1024)
    results = {}
    for kind, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail_decode(reqs, 32)),
                        ("mixed", H.trace_mixed(reqs, rng, max_live=3, portions=H.LONG_PORTIONS))):
        got, routing = H.run_trace(eng, steps)
        H.compare_with_plain(head128_dirs["g5"], reqs, got, routing, dtype)
        results[kind] = got
    if dtype == "float32":
        for kind in ("tail", "mixed"):
            assert max(H.rel_err(results[kind][k], results["whole"][k]) for k in results["whole"]) < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_scheduler_mixes_decoding_with_long_portions(head128_dirs, dtype):
    """Eight staggered prompts of 100 to 400 tokens under a budget of 192 tokens a step: the scheduler's own steps
    hold decoded tokens beside portions of up to 192 tokens.  Greedy tokens against the plain implementation."""
    import jax_llm_examples_b200 as J

    folder = head128_dirs["g2"]
    model = J.load_model(folder, dtype, "cuda")
    rng = random.Random(33)
    prompts = [[rng.randrange(256) for _ in range(rng.randrange(100, 401))] for _ in range(8)]
    gen = J.Generator(model, max_tokens=8 * 448, page_size=PAGE, max_slots=8, max_tokens_per_step=192)
    seen = set()
    step = gen.engine.step

    def watched(entries):
        out = step(entries)
        seen.update(gen.engine.last_scratch.get("attention_kernels", ()))
        return out

    gen.engine.step = watched
    outs = gen.generate(prompts, J.SamplingParams(max_new_tokens=40))
    gen.engine.check_status()
    assert [len(o) for o in outs] == [40] * 8
    if dtype == "bfloat16":
        assert any("tc" in k and "split_kv" in k for k in seen), seen
    for p, o in zip(prompts, outs):
        H.plain_greedy_checked(folder, p, o, dtype)
