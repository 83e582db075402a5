"""Generation through the Python entry point and the command line: greedy tokens against the plain
implementation, long decoding (through the replayed CUDA graphs), the first tokens of a sequence,
sampling with a temperature, and what happens when the cache is too small for everyone."""

import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.plain import llama4_plain as plain

pytestmark = pytest.mark.gpu


_plain_greedy_checked = H.plain_greedy_checked


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_c"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs[name], dtype)
    rng = random.Random(4)
    prompts = [[rng.randrange(model.vocab_size) for _ in range(n)] for n in (1, 2, 31, 77)]
    outs = J.generate(model, prompts, J.SamplingParams(max_new_tokens=12), page_size=16, max_tokens_per_step=48)
    assert [len(o) for o in outs] == [12] * 4
    for p, o in zip(prompts, outs):
        _plain_greedy_checked(model_dirs[name], p, o, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_right(model_dirs, dtype):
    """200 tokens decoded one by one (crossing chunks, pages and the temperature floor), batch of 3; in
    bfloat16 the steps run as replayed CUDA graphs."""
    import jax_llm_examples_b200 as J

    folder = model_dirs["tiny_c"]
    model = J.load_model(folder, dtype)
    gen = J.Generator(model, max_tokens=3 * 240, page_size=16, max_slots=3, max_tokens_per_step=64)
    prompts = [[5, 6, 7], [9] * 17, [200, 100]]
    outs = gen.generate(prompts, J.SamplingParams(max_new_tokens=200))
    if dtype == "bfloat16":
        assert gen.engine.graph_replays > 150
    for p, o in zip(prompts, outs):
        assert len(o) == 200
        _plain_greedy_checked(folder, p, o[:60], dtype)
    # logits at the far end, teacher-forced through the engine's own tokens, against the plain implementation
    eng = J.Engine(model, max_tokens=256, page_size=16, max_slots=1, use_graphs=False)
    seq = prompts[0] + outs[0]
    got, routing = H.run_trace(eng, H.trace_tail_decode({"r": seq}, 32))
    H.compare_with_plain(folder, {"r": seq}, got, routing, dtype)


def test_replayed_graphs_follow_the_growing_context(model_dirs):
    """A captured decode step is planned for a bucket of context lengths; as the requests grow the engine moves
    from one bucket's graph to the next.  With buckets made small, 150 decoded tokens cross many of them."""
    import jax_llm_examples_b200 as J

    folder = model_dirs["tiny_c"]
    model = J.load_model(folder, "bfloat16")
    gen = J.Generator(model, max_tokens=3 * 256, page_size=16, max_slots=3, max_tokens_per_step=64)
    gen.engine.KV_BUCKET_MIN = 32
    assert [gen.engine.kv_bucket(n) for n in (1, 32, 33, 36, 37, 64, 65, 100, 128, 129, 700)] == [32, 32, 40, 40, 40, 64, 80, 112, 128, 160, 768]
    prompts = [[5, 6, 7], [9] * 40, [200, 100] * 9]
    outs = gen.generate(prompts, J.SamplingParams(max_new_tokens=150))
    buckets = {key[2] for key, g in gen.engine._graphs.items() if "graph" in g}
    assert len(buckets) >= 8 and gen.engine.graph_replays > 100, (buckets, gen.engine.graph_replays)
    for p, o in zip(prompts, outs):
        H.plain_greedy_checked(folder, p, o, "bfloat16")
    # a wide engine (the default when the pool is sized from free memory) plans for the context in use all the same
    wide = J.Engine(model, max_tokens=4096, page_size=16, max_slots=2, max_seq_len=131072)
    assert wide.kv_bucket(700) == 1024 and wide.kv_bucket(9000) == 10240 and wide.kv_bucket(131072) == 131072


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """Positions 0, 1, 2 alone and together: the shortest contexts (one key, a fresh page, no history)."""
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs[name], dtype)
    eng = J.Engine(model, max_tokens=64, page_size=16, max_slots=4)
    reqs = {"a": [3], "b": [4, 5], "c": [6, 7, 8]}
    steps = [{"entries": [{"id": "a", "tokens": [3], "want": [0]}, {"id": "b", "tokens": [4], "want": [0]},
                          {"id": "c", "tokens": [6, 7, 8], "want": [0, 1, 2]}], "end": ["a", "c"]},
             {"entries": [{"id": "b", "tokens": [5], "want": [0]}], "end": ["b"]}]
    got, routing = H.run_trace(eng, steps)
    H.compare_with_plain(model_dirs[name], reqs, got, routing, dtype)


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch(model_dirs):
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs["tiny_b"], "float32")
    params = J.SamplingParams(temperature=0.8, top_k=16, max_new_tokens=10)
    prompts = [[1, 2, 3, 4], [7] * 30, [11, 12]]

    def run(which, **kw):
        gen = J.Generator(model, max_tokens=512, page_size=16, max_slots=4, seed=3, **kw)
        reqs = [gen.submit(prompts[i], params) for i in which]
        for r, i in zip(reqs, which):
            r.request_id = i  # the request's random stream is its id: keep it whatever the batch
        gen.scheduler.run()
        return {i: r.output for r, i in zip(reqs, which)}

    together = run([0, 1, 2])
    assert together == run([0, 1, 2])
    alone = {**run([0]), **run([1]), **run([2])}
    assert alone == together
    assert run([0, 1, 2], max_tokens_per_step=7) == together
    greedy = J.generate(model, prompts, J.SamplingParams(max_new_tokens=10), page_size=16)
    assert any(g != together[i] for i, g in enumerate(greedy))  # the draws are not just the argmax


def test_too_few_pages_preempts_and_still_gives_the_same_tokens(model_dirs):
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs["tiny_a"], "float32")
    prompts = [[i + 1] * 20 for i in range(4)]
    params = J.SamplingParams(max_new_tokens=40)
    roomy = J.Generator(model, max_tokens=4 * 64, page_size=16, max_slots=4).generate(prompts, params)
    tight_gen = J.Generator(model, max_tokens=7 * 16, page_size=16, max_slots=4)  # 7 pages for 4 x 60 tokens
    tight = tight_gen.generate(prompts, params)
    assert tight == roomy
    assert sum(r.preemptions for r in tight_gen.scheduler.finished) > 0
    tight_gen.engine.manager.check()
    with pytest.raises(ValueError, match="does not fit the cache"):
        J.Generator(model, max_tokens=32, page_size=16, max_slots=2).generate([[1] * 40], params)


def test_command_line(model_dirs):
    cmd = [sys.executable, "-m", "jax_llm_examples_b200.main", "--model", str(model_dirs["tiny_a"]), "--dtype", "float32",
           "--prompt-ids", "5,6,7,8", "--prompt-ids", "9", "--max-new-tokens", "6", "--page-size", "16"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=H.ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln and ln[0].isdigit()]
    assert len(lines) == 2 and all(len(ln.split()) == 6 for ln in lines)
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs["tiny_a"], "float32")
    want = J.generate(model, [[5, 6, 7, 8], [9]], J.SamplingParams(max_new_tokens=6), page_size=16)
    assert [list(map(int, ln.split())) for ln in lines] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_decode_steps_as_the_reference_calls_them(model_dirs, dtype):
    """The reference's offline loop (llama4/main.py:68-75): prefill, then decode_step over the same batch.
    The tokens are those of the scheduler's path."""
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs["tiny_b"], dtype, "cuda")
    rng = random.Random(21)
    prompts = [[rng.randrange(384) for _ in range(n)] for n in (37, 5, 64)]
    want = J.generate(model, prompts, J.SamplingParams(max_new_tokens=9), page_size=16)
    tokens, logits, batch = J.prefill(model, prompts, page_size=16, max_new_tokens=9)
    assert logits.shape == (3, 384) and logits.dtype == torch.float32
    got = [[t] for t in tokens]
    for _ in range(8):
        tokens, batch = J.decode_step(batch, tokens)
        for g, t in zip(got, tokens):
            g.append(t)
    batch.release()
    assert got == want
    eng = batch.engine
    assert all(eng.manager.free_pages(g) == eng.num_pages for g in range(len(eng.manager.groups)))


def test_engine_sizes_its_pool_from_free_memory(model_dirs):
    import jax_llm_examples_b200 as J

    model = J.load_model(model_dirs["tiny_a"], "bfloat16", "cuda")
    fit = J.Engine.tokens_that_fit(model, page_size=16, memory_fraction=0.001)
    assert fit > 0 and fit % 16 == 0
    eng = J.Engine(model, max_tokens=None, page_size=16, max_slots=2, memory_fraction=0.001)
    assert eng.num_pages * 16 <= fit + 16 and eng.max_seq_len <= J.Engine.DEFAULT_MAX_SEQ_LEN
    s = eng.new_request()
    logits = eng.step([J.StepEntry(s, [1, 2, 3], [2])])
    assert logits.shape == (1, 256)
    eng.finish(s)


def test_kernel_timer_and_named_ranges(model_dirs):
    """``Generator(profile="kernels")`` times every launch by kernel and by op group (under the reference's scope
    names) and gives the same tokens; NVTX ranges can be switched on around the same scopes."""
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200 import tracing

    model = J.load_model(model_dirs["tiny_c"], "float32")  # 32-bit: the same sums in the same order, traced or not
    prompts = [[3, 4, 5] * 30, [7, 8]]
    params = J.SamplingParams(max_new_tokens=6)
    want = J.generate(model, prompts, params, page_size=16)
    gen = J.Generator(model, max_tokens=512, page_size=16, max_slots=2, profile="kernels")
    gen.engine.use_graphs = True
    assert gen.generate(prompts, params) == want
    assert gen.engine.graph_replays == 0  # a replayed graph would hide its launches from the timer
    t = gen.kernel_timer
    assert t.by_kernel["jlx_add_rmsnorm"][0] > 0 and t.by_kernel["jlx_add_rmsnorm"][1] > 0
    for name in ("qkv_matmul", "rope", "attention", "projection", "attn_pre_norm", "attn_post_norm", "we_gate_up", "we_down", "permute"):
        assert t.by_scope[name][0] > 0, name
    assert "jlx_embed" in t.report() and "attention" in t.report("scope")
    assert not tracing.active()
    tracing.enable_nvtx(True)
    try:
        assert tracing.active()
        assert J.generate(model, prompts, params, page_size=16) == want
    finally:
        tracing.enable_nvtx(False)


def test_device_timeline_of_a_replayed_decode_step():
    """``python -m jax_llm_examples_b200.timeline`` builds the kernels with their time stamps, replays decode steps
    from a graph and lays their launches out in stream order: every kernel of a layer is there, and each ends after
    it could start."""
    import os
    import subprocess
    import sys

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "jax_llm_examples_b200.timeline", "--preset", "tiny_a", "--batch", "2",
                          "--context", "96", "--steps", "3", "--repeat", "3"], cwd=repo, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = out.stdout.strip().splitlines()
    assert lines[0].startswith("# one decode step, tiny_a, 4 layers, batch 2") and "medians of 3 steps" in lines[0]
    rows = [ln.split() for ln in lines[2:]]
    names = [r[0] for r in rows]
    for kernel, at_least in (("embed", 1), ("add_rmsnorm", 4), ("rope_kv_store", 4), ("expert_sort", 4), ("argmax", 2)):
        assert names.count(kernel) >= at_least, (kernel, names)
    assert sum(n.startswith("attention") for n in names) >= 4 and sum(n.startswith("gemm") for n in names) >= 16, names
    assert "?" not in names
    assert names[0] == "embed" and names[-1] == "argmax"
    ats = [float(r[2]) for r in rows]
    assert ats == sorted(ats)
    assert all(float(r[4]) > 0 for r in rows)  # busy: every launch ends after it was ready
